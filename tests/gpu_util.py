"""Helpers for the GPU parity tests: torch is used only for device memory."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O


def dev_u16(a: np.ndarray):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()


def run_gemv(qg, handle, w, x_bf16: np.ndarray, out_f32: bool = True, h=None):
    """x_bf16: u16 [B][K] host array -> y as float64-comparable numpy [B][N]."""
    import torch
    h = h or handle
    B = x_bf16.shape[0]
    xd = dev_u16(x_bf16)
    if out_f32:
        yd = torch.full((B, w.N), float("nan"), dtype=torch.float32, device="cuda")
        h.gemv(w, xd.data_ptr(), B, yd.data_ptr(), qg.OUT_F32)
        torch.cuda.synchronize()
        return yd.cpu().numpy()
    yd = torch.full((B, w.N), float("nan"), dtype=torch.bfloat16, device="cuda")
    h.gemv(w, xd.data_ptr(), B, yd.data_ptr(), qg.OUT_BF16)
    torch.cuda.synchronize()
    return yd.view(torch.int16).cpu().numpy().view(np.uint16)


def status_ok(handle):
    st = handle.device_status()
    assert st.code == 0, f"device status {st}"


def dequant(qg, handle, w, which: int = 0) -> np.ndarray:
    import torch
    out = torch.full((w.N, w.K), float("nan"), dtype=torch.float32, device="cuda")
    handle.dequant_f32(w, out.data_ptr(), which)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bits_equal(got, ref):
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(bits(got)[~nan], bits(ref)[~nan])
