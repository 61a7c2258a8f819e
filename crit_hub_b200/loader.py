"""Reading NVFP4 projections from a safetensors checkpoint into packed device weights.

The engines the registry lists load pre-quantised checkpoints through their own loaders
(engines/crit-labs/mtp5-nvfp4-drafts/card.yaml:69: "NVFP4 ... as stored").  The common on-disk form of
an NVFP4 linear layer is three tensors: `<name>.weight` (U8 [N][K/2], two E2M1 codes per byte, the
even element in the low nibble), `<name>.weight_scale` (F8_E4M3 [N][K/16]) and `<name>.weight_scale_2`
(F32 scalar, the per-tensor scale).  This module reads the safetensors container itself (an 8-byte
little-endian header length, a JSON header with dtype / shape / data_offsets per tensor, then the raw
bytes), memory-maps the file, copies the two arrays to the device and lets the library's kernel lay
them out (`qgemv_load_device`): no host-side packing pass.  Pure container parsing plus the C ABI;
no third-party reader is needed.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass

import numpy as np

from . import FMT_NVFP4_TC, QGemv, Shard, Weight

_ITEMSIZE = {"U8": 1, "I8": 1, "F8_E4M3": 1, "F8_E5M2": 1, "BF16": 2, "F16": 2, "F32": 4, "I32": 4, "I64": 8, "F64": 8}


@dataclass
class TensorInfo:
    dtype: str
    shape: tuple
    begin: int   # byte offsets inside the data section
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file: `tensors` maps names to TensorInfo, `raw(name)` is a u8 view."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError("not a safetensors file: shorter than its length field")
        (n,) = struct.unpack("<Q", head)
        size = self._f.seek(0, 2)
        if n < 2 or 8 + n > size:
            raise ValueError("not a safetensors file: header length out of range")
        self._f.seek(8)
        header = json.loads(self._f.read(n).decode("utf-8"))
        self.metadata = header.pop("__metadata__", {})
        self.data_start = 8 + n
        self.tensors: dict[str, TensorInfo] = {}
        for name, t in header.items():
            b, e = t["data_offsets"]
            shape = tuple(int(d) for d in t["shape"])
            want = int(np.prod(shape, dtype=np.int64)) * _ITEMSIZE.get(t["dtype"], 0) if shape else _ITEMSIZE.get(t["dtype"], 0)
            if t["dtype"] not in _ITEMSIZE or e - b != want or b < 0 or self.data_start + e > size:
                raise ValueError(f"tensor {name}: dtype / shape / offsets do not agree")
            self.tensors[name] = TensorInfo(t["dtype"], shape, int(b), int(e))
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def raw(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return np.frombuffer(self._map, dtype=np.uint8, count=t.end - t.begin, offset=self.data_start + t.begin)

    def close(self) -> None:
        try:
            self._map.close()
        except BufferError:      # views handed out by raw() are still alive: the mapping goes with the last of them
            pass
        self._f.close()


def nvfp4_linear_arrays(f: SafetensorsFile, name: str):
    """(codes u8 [N][K/2], scales u8 [N][K/16], tensor_scale) views of one NVFP4 linear layer."""
    w, s = f.tensors[f"{name}.weight"], f.tensors[f"{name}.weight_scale"]
    if w.dtype != "U8" or len(w.shape) != 2 or s.dtype not in ("F8_E4M3", "U8") or len(s.shape) != 2:
        raise ValueError(f"{name}: expected U8 [N][K/2] codes and F8_E4M3 [N][K/16] block scales")
    N, K = w.shape[0], w.shape[1] * 2
    if s.shape != (N, K // 16) or K % 16 != 0:
        raise ValueError(f"{name}: block scales of shape {s.shape} do not match codes of shape {w.shape}")
    ts = 1.0
    if f"{name}.weight_scale_2" in f.tensors:
        t2 = f.tensors[f"{name}.weight_scale_2"]
        if t2.dtype != "F32" or t2.end - t2.begin != 4:
            raise ValueError(f"{name}.weight_scale_2: expected one F32 value")
        ts = float(f.raw(f"{name}.weight_scale_2").view(np.float32)[0])
    return f.raw(f"{name}.weight").reshape(N, K // 2), f.raw(f"{name}.weight_scale").reshape(N, K // 16), ts


def load_nvfp4_linear(handle: QGemv, f: SafetensorsFile, name: str, shard: Shard | None = None) -> Weight:
    """One NVFP4 linear layer of the checkpoint as a packed weight in the tensor-core layout.  The arrays
    go to the device as they are in the file and are laid out there; `shard` cuts a tensor-parallel
    rank's rows or columns."""
    import torch

    codes, scales, ts = nvfp4_linear_arrays(f, name)
    N, K = scales.shape[0], scales.shape[1] * 16
    dev = torch.device("cuda", handle.device)
    cd = torch.from_numpy(np.ascontiguousarray(codes)).to(dev)
    sd = torch.from_numpy(np.ascontiguousarray(scales)).to(dev)
    return handle.load_device(FMT_NVFP4_TC, cd.data_ptr(), sd.data_ptr(), N, K, ts, shard=shard)


def load_nvfp4_experts(handle: QGemv, f: SafetensorsFile, names: list[str], shard: Shard | None = None) -> Weight:
    """The equally shaped NVFP4 linear layers `names` (the experts of an MoE layer, one tensor triple each:
    `<name>.weight`, `.weight_scale`, `.weight_scale_2`) as ONE stacked weight in the tensor-core layout, ready
    for `moe_gemv`; expert e of the stack is names[e].  The arrays go to the device as they are in the file and
    are laid out there."""
    import torch

    dev = torch.device("cuda", handle.device)
    keep, cps, sps, tss = [], [], [], []
    N = K = None
    for name in names:
        codes, scales, ts = nvfp4_linear_arrays(f, name)
        n, k = scales.shape[0], scales.shape[1] * 16
        if N is None:
            N, K = n, k
        elif (n, k) != (N, K):
            raise ValueError(f"{name}: {n} x {k}, the first expert is {N} x {K}")
        cd = torch.from_numpy(np.ascontiguousarray(codes)).to(dev)
        sd = torch.from_numpy(np.ascontiguousarray(scales)).to(dev)
        keep += [cd, sd]          # alive until the packing kernels have run (the call returns after them)
        cps.append(cd.data_ptr()), sps.append(sd.data_ptr()), tss.append(ts)
    return handle.load_stacked_device(FMT_NVFP4_TC, cps, sps, N, K, tss, shard=shard)
