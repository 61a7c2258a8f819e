"""Host packer: round trips, shards, ragged shapes, blob validation (no GPU)."""
import numpy as np
import pytest

from oracle import oracle as O


@pytest.mark.parametrize("N,K", [(16, 64), (1, 16), (100, 448), (17, 1040), (256, 4096), (33, 80)])
def test_nvfp4_roundtrip(qg, N, K):
    codes, scales, ts = O.make_nvfp4(N, K, seed=N * 7 + K, ts=0.625)
    blob = qg.pack(qg.FMT_NVFP4, codes, scales, ts)
    assert blob.size == qg.packed_size(qg.FMT_NVFP4, N, K)
    assert blob.size == 256 + ((N + 15) // 16) * ((K + 63) // 64) * 576
    assert qg.blob_info(blob) == (qg.FMT_NVFP4, N, K)
    assert qg.blob_verify(blob) == 0
    c2, s2, ts2 = qg.unpack(blob)
    assert np.array_equal(c2, codes) and np.array_equal(s2, scales) and ts2 == np.float32(0.625)


@pytest.mark.parametrize("N,K", [(16, 64), (50, 128), (31, 208)])
def test_fp8_roundtrip(qg, N, K):
    codes, scales = O.make_fp8(N, K, seed=N + K)
    blob = qg.pack(qg.FMT_FP8, codes, scales)
    assert qg.blob_verify(blob) == 0
    c2, s2, _ = qg.unpack(blob)
    assert np.array_equal(c2, codes) and np.array_equal(s2, scales)


def test_adversarial_patterns(qg):
    """All-ones codes, zero / subnormal / maximal scales: the packer moves bytes, never values."""
    N, K = 48, 256
    for fill_c, fill_s in [(0xFF, 0x00), (0x00, 0x7E), (0x8F, 0x01), (0xF8, 0x07)]:
        codes = np.full((N, K // 2), fill_c, dtype=np.uint8)
        scales = np.full((N, K // 16), fill_s, dtype=np.uint8)
        c2, s2, _ = qg.unpack(qg.pack(qg.FMT_NVFP4, codes, scales, 1.0))
        assert np.array_equal(c2, codes) and np.array_equal(s2, scales)


def test_every_code_lands_once(qg):
    """A single non-zero code moves exactly one nibble of the payload."""
    N, K = 16, 64
    zero = qg.pack(qg.FMT_NVFP4, np.zeros((N, K // 2), np.uint8), np.zeros((N, K // 16), np.uint8), 1.0)
    seen = set()
    for n in range(N):
        for k in range(K):
            codes = np.zeros((N, K // 2), np.uint8)
            codes[n, k // 2] = 0xF << (4 * (k & 1))
            blob = qg.pack(qg.FMT_NVFP4, codes, np.zeros((N, K // 16), np.uint8), 1.0)
            diff = np.nonzero(blob[256:] != zero[256:])[0]
            assert diff.size == 1 and diff[0] < 512
            v = int(blob[256 + diff[0]])
            assert v in (0x0F, 0xF0)
            key = (int(diff[0]), v)
            assert key not in seen
            seen.add(key)
    assert len(seen) == N * K


def test_shards(qg):
    """Column-parallel (rows) and row-parallel (K) tensor-parallel shards are sub-matrices."""
    N, K = 96, 512
    codes, scales, ts = O.make_nvfp4(N, K, seed=3)
    for world in (2, 4):
        for r in range(world):
            sh = qg.Shard(r * N // world, (r + 1) * N // world, 0, K)
            c, s, _ = qg.unpack(qg.pack(qg.FMT_NVFP4, codes, scales, ts, shard=sh))
            assert np.array_equal(c, codes[sh.n0:sh.n1]) and np.array_equal(s, scales[sh.n0:sh.n1])
            sh = qg.Shard(0, N, r * K // world, (r + 1) * K // world)
            c, s, _ = qg.unpack(qg.pack(qg.FMT_NVFP4, codes, scales, ts, shard=sh))
            assert np.array_equal(c, codes[:, sh.k0 // 2:sh.k1 // 2])
            assert np.array_equal(s, scales[:, sh.k0 // 16:sh.k1 // 16])
    fc, fs = O.make_fp8(64, 256, 4)
    c, s, _ = qg.unpack(qg.pack(qg.FMT_FP8, fc, fs, shard=qg.Shard(16, 48, 64, 192)))
    assert np.array_equal(c, fc[16:48, 64:192]) and np.array_equal(s, fs[16:48])


def test_rejects(qg):
    codes, scales, ts = O.make_nvfp4(16, 64, seed=1)
    assert qg.packed_size(qg.FMT_NVFP4, 16, 72) == 0          # K not a multiple of 16
    assert qg.packed_size(7, 16, 64) == 0                      # unknown format
    assert qg.packed_size(qg.FMT_NVFP4, 16, 64, qg.Shard(0, 16, 8, 64)) == 0  # shard cuts a scale block
    assert qg.packed_size(qg.FMT_NVFP4, 16, 64, qg.Shard(0, 17, 0, 64)) == 0
    blob = qg.pack(qg.FMT_NVFP4, codes, scales, ts)
    bad = blob.copy()
    bad[300] ^= 0x10
    assert qg.blob_verify(bad) == qg.ERR_BAD_BLOB
    with pytest.raises(qg.QgemvError):
        qg.unpack(bad)
    bad = blob.copy()
    bad[0] ^= 1                                                # magic
    assert qg.blob_verify(bad) == qg.ERR_BAD_BLOB
    assert qg.blob_verify(blob[:-16].copy()) == qg.ERR_BAD_BLOB  # truncated
    bad = blob.copy()
    bad[4] += 1                                                # version of a stale layout
    with pytest.raises(qg.QgemvError):
        qg.blob_info(bad)


# ---- tensor-core layout (QGEMV_FMT_NVFP4_TC) ------------------------------------------------------
@pytest.mark.parametrize("N,K", [(128, 64), (1, 16), (100, 448), (17, 1040), (256, 4096), (300, 80)])
def test_tc_roundtrip(qg, N, K):
    codes, scales, ts = O.make_nvfp4(N, K, seed=N * 7 + K, ts=0.625)
    blob = qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts)
    assert blob.size == qg.packed_size(qg.FMT_NVFP4_TC, N, K)
    assert blob.size == 256 + ((N + 127) // 128) * ((K + 63) // 64) * 4608
    assert qg.blob_info(blob) == (qg.FMT_NVFP4_TC, N, K)
    assert qg.blob_verify(blob) == 0
    c2, s2, ts2 = qg.unpack(blob)
    assert np.array_equal(c2, codes) and np.array_equal(s2, scales) and ts2 == np.float32(0.625)
    bad = blob.copy()
    bad[300] ^= 1
    assert qg.blob_verify(bad) != 0


def test_tc_item_order(qg):
    """The item is the MMA operand itself: codes as 8-row x 16-byte core matrices (K-major, no
    swizzle), scales in the 32-lane x 4-column order of the tensor-memory copy."""
    N, K = 256, 192
    codes, scales, ts = O.make_nvfp4(N, K, seed=9)
    payload = qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts)[256:]
    items_per_tile = K // 64
    for n in (0, 7, 8, 31, 32, 127, 128, 200, 255):
        for k in (0, 1, 31, 32, 63, 64, 130, 191):
            item = payload[((n // 128) * items_per_tile + k // 64) * 4608:][:4608]
            r, kk = n % 128, k % 64
            byte = item[(r // 8) * 256 + (kk // 32) * 128 + (r % 8) * 16 + (kk % 32) // 2]
            code = (byte >> 4) if kk & 1 else (byte & 15)
            want = codes[n, k // 2]
            assert code == ((want >> 4) if k & 1 else (want & 15))
            assert item[4096 + (r % 32) * 16 + (r // 32) * 4 + kk // 16] == scales[n, k // 16]


def test_tc_shards(qg):
    N, K = 384, 512
    codes, scales, ts = O.make_nvfp4(N, K, seed=3)
    for world in (2, 4):
        for r in range(world):
            sh = qg.Shard(r * N // world, (r + 1) * N // world, 0, K)
            c, s, _ = qg.unpack(qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts, shard=sh))
            assert np.array_equal(c, codes[sh.n0:sh.n1]) and np.array_equal(s, scales[sh.n0:sh.n1])
            sh = qg.Shard(0, N, r * K // world, (r + 1) * K // world)
            c, s, _ = qg.unpack(qg.pack(qg.FMT_NVFP4_TC, codes, scales, ts, shard=sh))
            assert np.array_equal(c, codes[:, sh.k0 // 2:sh.k1 // 2])
            assert np.array_equal(s, scales[:, sh.k0 // 16:sh.k1 // 16])
