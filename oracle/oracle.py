"""ctypes front-end of the CPU oracle (test infrastructure, never shipped).

Only `tests/`, the smoke check and the CPU-baseline / reference legs of the
benchmark may import this module.  The shipped package must never do so.

Besides the C++ oracle (`qgemv_oracle.cpp`) this module holds
  * a small, independent numpy restatement of the codecs (`np_*`), used to
    cross-check the C++ code, and
  * the seeded synthetic-input generators shared by tests and fixtures.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                        -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "_build", "libqgemv_oracle.so")
        src = os.path.join(_HERE, "qgemv_oracle.cpp")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            import importlib.util
            spec = importlib.util.spec_from_file_location("_oracle_build", os.path.join(_HERE, "build.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            path = mod.build()
        L = C.CDLL(path)
        L.orc_e2m1_decode.restype = C.c_float
        L.orc_e2m1_decode.argtypes = [C.c_uint32]
        L.orc_e4m3_decode.restype = C.c_float
        L.orc_e4m3_decode.argtypes = [C.c_uint32]
        L.orc_e4m3_encode.restype = C.c_uint32
        L.orc_e4m3_encode.argtypes = [C.c_float]
        L.orc_bf16_decode.restype = C.c_float
        L.orc_bf16_decode.argtypes = [C.c_uint32]
        L.orc_bf16_encode.restype = C.c_uint32
        L.orc_bf16_encode.argtypes = [C.c_float]
        L.orc_num_threads.restype = C.c_int
        L.orc_gemv_nvfp4_fast.restype = C.c_int
        L.orc_gemv_fp8_fast.restype = C.c_int
        _LIB = L
    return _LIB


_FAST = None


def fast_lib() -> C.CDLL:
    """The library the TIMED fp32 baseline runs from: this machine's own build (-O3 -march=native)
    when it can be compiled here, else the portable one.  Parity checks always use lib()."""
    global _FAST
    if _FAST is None:
        import importlib.util
        spec = importlib.util.spec_from_file_location("_oracle_build", os.path.join(_HERE, "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        path = mod.build_native()
        if path is None:
            _FAST = lib()
        else:
            _FAST = C.CDLL(path)
            _FAST.orc_num_threads.restype = C.c_int
            _FAST.orc_gemv_nvfp4_fast.restype = C.c_int
            _FAST.orc_gemv_fp8_fast.restype = C.c_int
    return _FAST


def set_threads(n: int) -> None:
    """Host threads of the OpenMP loops (both builds): launchers may have exported OMP_NUM_THREADS=1."""
    lib().orc_set_threads(C.c_int(int(n)))
    if fast_lib() is not lib():
        fast_lib().orc_set_threads(C.c_int(int(n)))


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


# ---- array codecs ------------------------------------------------------------------------------
def e4m3_encode(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint8)
    lib().orc_e4m3_encode_array(_p(a), _p(out), C.c_int64(a.size))
    return out


def bf16_encode(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().orc_bf16_encode_array(_p(a), _p(out), C.c_int64(a.size))
    return out


def bf16_decode(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().orc_bf16_decode_array(_p(a), _p(out), C.c_int64(a.size))
    return out


# ---- dequant / gemv ----------------------------------------------------------------------------
def dequant_nvfp4(codes, scales, ts) -> np.ndarray:
    N, K = scales.shape[0], scales.shape[1] * 16
    out = np.empty((N, K), dtype=np.float32)
    lib().orc_dequant_nvfp4(_p(codes), _p(scales), C.c_float(ts), C.c_int64(N), C.c_int64(K), _p(out))
    return out


def dequant_fp8(codes, ch_scale) -> np.ndarray:
    N, K = codes.shape
    out = np.empty((N, K), dtype=np.float32)
    lib().orc_dequant_fp8(_p(codes), _p(ch_scale), C.c_int64(N), C.c_int64(K), _p(out))
    return out


def gemv_nvfp4_f64(codes, scales, ts, x_bf16) -> np.ndarray:
    N, K = scales.shape[0], scales.shape[1] * 16
    x_bf16 = np.ascontiguousarray(x_bf16.reshape(-1, K))
    B = x_bf16.shape[0]
    y = np.empty((B, N), dtype=np.float64)
    lib().orc_gemv_nvfp4_f64(_p(codes), _p(scales), C.c_float(ts), C.c_int64(N), C.c_int64(K),
                             _p(x_bf16), C.c_int64(B), _p(y))
    return y


def gemv_fp8_f64(codes, ch_scale, x_bf16) -> np.ndarray:
    N, K = codes.shape
    x_bf16 = np.ascontiguousarray(x_bf16.reshape(-1, K))
    B = x_bf16.shape[0]
    y = np.empty((B, N), dtype=np.float64)
    lib().orc_gemv_fp8_f64(_p(codes), _p(ch_scale), C.c_int64(N), C.c_int64(K), _p(x_bf16),
                           C.c_int64(B), _p(y))
    return y


def gemv_nvfp4_fast(codes, scales, ts, x_bf16, native: bool = False):
    """fp32-accumulated OpenMP GEMV (the timed CPU baseline). Returns (y fp32 [B][N], threads)."""
    N, K = scales.shape[0], scales.shape[1] * 16
    x_bf16 = np.ascontiguousarray(x_bf16.reshape(-1, K))
    B = x_bf16.shape[0]
    y = np.empty((B, N), dtype=np.float32)
    L = fast_lib() if native else lib()
    th = L.orc_gemv_nvfp4_fast(_p(codes), _p(scales), C.c_float(ts), C.c_int64(N), C.c_int64(K),
                               _p(x_bf16), C.c_int64(B), _p(y))
    return y, th


def gemv_fp8_fast(codes, ch_scale, x_bf16):
    N, K = codes.shape
    x_bf16 = np.ascontiguousarray(x_bf16.reshape(-1, K))
    B = x_bf16.shape[0]
    y = np.empty((B, N), dtype=np.float32)
    th = lib().orc_gemv_fp8_fast(_p(codes), _p(ch_scale), C.c_int64(N), C.c_int64(K), _p(x_bf16),
                                 C.c_int64(B), _p(y))
    return y, th


def moe_gemv_nvfp4_f64(codes, scales, ts, expert_ids, x_bf16, per_slot_input: bool) -> np.ndarray:
    """codes [E][N][K/2], scales [E][N][K/16], ts [E]; expert_ids i32 [T][topk]."""
    E, N, K16 = scales.shape
    K = K16 * 16
    T, topk = expert_ids.shape
    out = np.empty((T * topk, N), dtype=np.float64)
    ids = np.ascontiguousarray(expert_ids, dtype=np.int32)
    tsa = np.ascontiguousarray(ts, dtype=np.float32)
    lib().orc_moe_gemv_nvfp4_f64(_p(codes), _p(scales), _p(tsa), C.c_int64(N), C.c_int64(K), _p(ids),
                                 C.c_int64(T), C.c_int64(topk), _p(np.ascontiguousarray(x_bf16)),
                                 C.c_int(1 if per_slot_input else 0), _p(out))
    return out


def quantize_a4(x_bf16: np.ndarray):
    """bf16 activations [M][K] -> NVFP4 (codes u8 [M][K/2], block scales u8 [M][K/16], row scales f32 [M])
    by the stated quantiser of the skinny GEMM's A4 mode."""
    M, K = x_bf16.shape
    x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
    codes = np.empty((M, K // 2), dtype=np.uint8)
    scales = np.empty((M, K // 16), dtype=np.uint8)
    g = np.empty((M,), dtype=np.float32)
    lib().orc_quantize_a4(_p(x), C.c_int64(M), C.c_int64(K), _p(codes), _p(scales), _p(g))
    return codes, scales, g


def gemm_nvfp4_a4_f64(wcodes, wscales, ts, xcodes, xscales, g) -> np.ndarray:
    """fp64 Y[M][N] from NVFP4 weights and NVFP4-quantised activations."""
    N, K = wscales.shape[0], wscales.shape[1] * 16
    M = xcodes.shape[0]
    y = np.empty((M, N), dtype=np.float64)
    lib().orc_gemm_nvfp4_a4_f64(_p(wcodes), _p(wscales), C.c_float(ts), C.c_int64(N), C.c_int64(K), _p(xcodes),
                                _p(xscales), _p(np.ascontiguousarray(g, dtype=np.float32)), C.c_int64(M), _p(y))
    return y


def num_threads() -> int:
    return int(lib().orc_num_threads())


# ---- independent numpy restatement of the codecs ---------------------------------------------
def np_e2m1_decode(code: np.ndarray) -> np.ndarray:
    return E2M1_VALUES[np.asarray(code, dtype=np.int64) & 15]


def np_e4m3_decode(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, dtype=np.int64) & 255
    s = np.where(b & 0x80, -1.0, 1.0)
    e = (b >> 3) & 15
    m = b & 7
    mag = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * np.exp2(e.astype(np.float64) - 7.0))
    out = (s * mag).astype(np.float32)
    out[(e == 15) & (m == 7)] = np.nan
    return out


def np_dequant_nvfp4(codes, scales, ts) -> np.ndarray:
    N, K = scales.shape[0], scales.shape[1] * 16
    nib = np.empty((N, K), dtype=np.uint8)
    nib[:, 0::2] = codes & 15
    nib[:, 1::2] = codes >> 4
    w = np_e2m1_decode(nib) * np.repeat(np_e4m3_decode(scales), 16, axis=1)
    return (w.astype(np.float32) * np.float32(ts)).astype(np.float32)


# ---- seeded synthetic inputs -------------------------------------------------------------------
def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(seed))


def make_nvfp4(N: int, K: int, seed: int, ts: float = 1.0):
    """Codes uniform over the 16 E2M1 codes; scales = E4M3(|N(0,1)| * 0.05); fp32 tensor scale."""
    codes = _rng(seed * 3 + 1).integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    sc = np.abs(_rng(seed * 3 + 2).standard_normal((N, K // 16), dtype=np.float32)) * np.float32(0.05)
    return codes, e4m3_encode(sc), float(ts)


def make_fp8(N: int, K: int, seed: int):
    """Codes uniform over the 254 non-NaN E4M3 codes; channel scale = fp32(|N(0,1)| * 0.02)."""
    c = _rng(seed * 3 + 1).integers(0, 254, size=(N, K), dtype=np.uint8)
    c = np.where(c >= 127, c + 1, c).astype(np.uint8)      # skip 0x7F
    c = np.where(c == 255, 0x7E, c).astype(np.uint8)       # never 0xFF
    s = (np.abs(_rng(seed * 3 + 2).standard_normal(N, dtype=np.float32)) * np.float32(0.02)).astype(np.float32)
    return c, s


def make_x(B: int, K: int, seed: int) -> np.ndarray:
    """bf16 bit patterns of N(0,1) activations, shape [B][K]."""
    return bf16_encode(_rng(seed * 3 + 3).standard_normal((B, K), dtype=np.float32))


def rel_l2(got, want) -> float:
    got = np.asarray(got, dtype=np.float64).ravel()
    want = np.asarray(want, dtype=np.float64).ravel()
    den = float(np.linalg.norm(want))
    return float(np.linalg.norm(got - want)) / (den if den > 0 else 1.0)
