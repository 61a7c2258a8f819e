"""The safetensors reader: container parsing on CPU, and (GPU) a checkpoint's NVFP4 layer loaded
straight into the packed tensor-core layout."""
import numpy as np
import pytest

from oracle import oracle as O
from st_writer import write_safetensors


def _checkpoint(tmp_path, N=272, K=2112, ts=0.375):
    codes, scales, _ = O.make_nvfp4(N, K, seed=N + K)
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, {
        "layers.0.proj.weight": ("U8", codes),
        "layers.0.proj.weight_scale": ("F8_E4M3", scales),
        "layers.0.proj.weight_scale_2": ("F32", np.array(ts, dtype=np.float32)),
        "norm.weight": ("BF16", np.arange(8, dtype=np.uint16)),
    }, metadata={"format": "pt"})
    return path, codes, scales, ts


def test_header_and_views(tmp_path):
    from crit_hub_b200.loader import SafetensorsFile, nvfp4_linear_arrays
    path, codes, scales, ts = _checkpoint(tmp_path)
    f = SafetensorsFile(path)
    assert f.metadata == {"format": "pt"}
    assert f.tensors["layers.0.proj.weight"].shape == codes.shape and f.tensors["norm.weight"].dtype == "BF16"
    c, s, t = nvfp4_linear_arrays(f, "layers.0.proj")
    assert np.array_equal(c, codes) and np.array_equal(s, scales) and t == np.float32(ts)
    with pytest.raises(KeyError):
        nvfp4_linear_arrays(f, "layers.1.proj")
    f.close()


def test_bad_files_are_refused(tmp_path):
    from crit_hub_b200.loader import SafetensorsFile
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(ValueError):
        SafetensorsFile(str(p))
    p = tmp_path / "len.safetensors"
    p.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(ValueError):
        SafetensorsFile(str(p))
    path = str(tmp_path / "off.safetensors")
    write_safetensors(path, {"a": ("F32", np.zeros(4, dtype=np.float32))})
    raw = bytearray(open(path, "rb").read())
    open(path, "wb").write(bytes(raw[:-4]))          # data shorter than the offsets say
    with pytest.raises(ValueError):
        SafetensorsFile(path)


@pytest.mark.gpu
def test_checkpoint_layer_to_device(tmp_path, qg, handle):
    import gpu_util as U
    from crit_hub_b200.loader import SafetensorsFile, load_nvfp4_linear
    path, codes, scales, ts = _checkpoint(tmp_path, N=1000, K=4112)
    f = SafetensorsFile(path)
    w = load_nvfp4_linear(handle, f, "layers.0.proj")
    assert (w.N, w.K) == (1000, 4112)
    x = O.make_x(3, 4112, seed=3)
    assert O.rel_l2(U.run_gemv(qg, handle, w, x), O.gemv_nvfp4_f64(codes, scales, ts, x)) < 5e-5
    U.assert_bits_equal(U.dequant(qg, handle, w), O.dequant_nvfp4(codes, scales, ts))
    ws = load_nvfp4_linear(handle, f, "layers.0.proj", shard=qg.Shard(0, 1000, 2048, 4112))   # a row-parallel rank's columns
    xs = np.ascontiguousarray(x[:, 2048:])
    cs, ss, t2 = qg.unpack(qg.pack(qg.FMT_NVFP4, codes, scales, ts, shard=qg.Shard(0, 1000, 2048, 4112)))
    assert O.rel_l2(U.run_gemv(qg, handle, ws, xs), O.gemv_nvfp4_f64(cs, ss, t2, xs)) < 5e-5
    w.unload()
    ws.unload()
    f.close()


@pytest.mark.gpu
def test_checkpoint_experts_to_device(tmp_path, qg, handle):
    """The experts of an MoE layer: one tensor triple each in the file -> one stacked weight laid out on the device,
    byte for byte the stack of host-packed blobs (checksums aside); and the expert list computes with it."""
    import torch
    import gpu_util as U
    from crit_hub_b200.loader import SafetensorsFile, load_nvfp4_experts
    E, N, K, T, topk = 6, 256, 192, 5, 2
    mats = [O.make_nvfp4(N, K, seed=70 + e, ts=0.25 + e / 8.0) for e in range(E)]
    tensors = {}
    for e, (c, s, t) in enumerate(mats):
        tensors[f"mlp.experts.{e}.down.weight"] = ("U8", c)
        tensors[f"mlp.experts.{e}.down.weight_scale"] = ("F8_E4M3", s)
        tensors[f"mlp.experts.{e}.down.weight_scale_2"] = ("F32", np.array(t, dtype=np.float32))
    path = str(tmp_path / "experts.safetensors")
    write_safetensors(path, tensors)
    f = SafetensorsFile(path)
    w = load_nvfp4_experts(handle, f, [f"mlp.experts.{e}.down" for e in range(E)])
    assert (w.N, w.K) == (N, K)
    host = np.stack([qg.pack(qg.FMT_NVFP4_TC, c, s, t) for c, s, t in mats])
    got = w.read_blob().reshape(host.shape)
    # (the header's checksum field is the only difference: the device packer leaves it zero)
    diff = np.nonzero(got != host)
    assert diff[1].size == 0 or diff[1].max() < 256
    assert np.array_equal(got[:, 256:], host[:, 256:])
    rng = np.random.default_rng(5)
    ids = np.stack([rng.permutation(E)[:topk] for _ in range(T)]).astype(np.int32)
    x = O.make_x(T, K, seed=8)
    codes = np.stack([m[0] for m in mats]); scales = np.stack([m[1] for m in mats]); ts = np.array([m[2] for m in mats], dtype=np.float32)
    ref = O.moe_gemv_nvfp4_f64(codes, scales, ts, ids, x, per_slot_input=False)
    xd, idd = U.dev_u16(x), torch.from_numpy(ids).cuda()
    out = torch.full((T * topk, N), float("nan"), dtype=torch.float32, device="cuda")
    handle.moe_gemv(w, idd.data_ptr(), xd.data_ptr(), T, topk, False, out.data_ptr(), qg.OUT_F32)
    torch.cuda.synchronize()
    U.status_ok(handle)
    assert O.rel_l2(out.cpu().numpy(), ref) < 5e-5
    w.unload()
    f.close()
