"""Python binding of the qgemv C ABI (include/qgemv.h) -- a ctypes layer, no torch types.

Device buffers are passed as integer addresses (`tensor.data_ptr()` of a torch CUDA tensor, or
any other allocator's pointer); streams as integer `cudaStream_t` handles.  Every compute call
goes to the CUDA library; if it cannot be loaded the import of the binding fails loudly --
there is no CPU path in this package.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

from . import _build

FMT_NVFP4 = 1
FMT_FP8 = 2
FMT_NVFP4_TC = 3   # NVFP4 in the tile order the block-scaled tensor-core GEMV consumes as stored
JOB_AFTER_PREVIOUS = 1   # qgemv_job.flags: wait for the job before this one
JOB_ALLREDUCE = 2        # qgemv_job.flags: row-parallel projection, summed over the ranks inside the launch
JOB_X_SILU_MUL = 4       # qgemv_job.flags: the rows of x hold gate and up values; the GEMV multiplies silu(gate) * up
MOE_X_SILU_MUL = 1       # moe_gemv's x_act: the same for the experts' down stage
OUT_BF16 = 0
OUT_F32 = 1
ACT_A16_EXACT = 0
ACT_A4_BLOCKSCALED = 1
ACT_A8 = 2
MAX_BATCH = 8

ERR_INVALID_ARG = -1
ERR_BAD_BLOB = -2
ERR_UNSUPPORTED_SHAPE = -3
ERR_CUDA = -4
ERR_NCCL = -5
ERR_TIMEOUT = -6
ERR_BOUNDS = -7
ERR_NO_DEVICE = -8


class MoePlan(C.Structure):
    _fields_ = [("rows_per_problem", C.c_int32), ("plane_buffers", C.c_int32), ("plane_slots", C.c_int32),
                ("ring_stages", C.c_int32), ("stage_items", C.c_int32), ("max_problems", C.c_int32),
                ("table_offset", C.c_int32), ("smem_bytes", C.c_int32)]


class SkinnyPlan(C.Structure):
    """qgemv_skinny_plan: how qgemv_gemm_skinny would run a shape."""
    _fields_ = [("run_units", C.c_int32), ("x_stage_units", C.c_int32), ("x_stages", C.c_int32),
                ("p_stages", C.c_int32), ("a_stages", C.c_int32), ("tmem_columns", C.c_int32),
                ("smem_bytes", C.c_int32), ("ctas", C.c_int32), ("scratch_bytes", C.c_int64)]


class QgemvError(RuntimeError):
    def __init__(self, status: int, what: str):
        super().__init__(f"{what}: {status_string(status)} ({status})")
        self.status = status


class _Config(C.Structure):
    _fields_ = [("device", C.c_int32), ("use_pdl", C.c_int32), ("grid_override", C.c_int32),
                ("debug", C.c_int32), ("spin_limit", C.c_int64), ("tc_stage_items", C.c_int32),
                ("tc_smem_kb", C.c_int32)]


class Shard(C.Structure):
    """Rows [n0, n1) and columns [k0, k1) of the canonical matrix."""
    _fields_ = [("n0", C.c_int64), ("n1", C.c_int64), ("k0", C.c_int64), ("k1", C.c_int64)]


class _Job(C.Structure):
    _fields_ = [("w", C.c_void_p), ("x", C.c_void_p), ("y", C.c_void_p), ("y_dtype", C.c_int32), ("flags", C.c_int32),
                ("x_stride", C.c_int64), ("norm_weight", C.c_void_p), ("residual", C.c_void_p), ("norm_eps", C.c_float),
                ("reserved", C.c_int32)]


class _DevStatus(C.Structure):
    _fields_ = [("code", C.c_int32), ("where", C.c_int32), ("block", C.c_int32), ("extra", C.c_int32)]


@dataclass
class DeviceStatus:
    code: int
    where: int
    block: int
    extra: int


_LIB = None


def lib_path() -> str:
    return _build.LIB_PATH


def _load() -> C.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    path = _build.LIB_PATH
    if not os.path.exists(path):
        path = _build.build()
    L = C.CDLL(path)
    vp, i32, i64, sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
    L.qgemv_status_string.restype = C.c_char_p
    L.qgemv_status_string.argtypes = [i32]
    L.qgemv_last_cuda_error.restype = C.c_char_p
    L.qgemv_init.argtypes = [C.POINTER(_Config), C.POINTER(vp)]
    L.qgemv_destroy.argtypes = [vp]
    L.qgemv_sm_count.argtypes = [vp]
    L.qgemv_set_trace.argtypes = [vp, vp]
    L.qgemv_packed_size.restype = sz
    L.qgemv_packed_size.argtypes = [i32, i64, i64, C.POINTER(Shard)]
    L.qgemv_pack_host.argtypes = [i32, vp, vp, C.c_float, i64, i64, C.POINTER(Shard), vp]
    L.qgemv_unpack_host.argtypes = [vp, sz, vp, vp, C.POINTER(C.c_float)]
    L.qgemv_blob_info.argtypes = [vp, sz, C.POINTER(i32), C.POINTER(i64), C.POINTER(i64)]
    L.qgemv_blob_verify.argtypes = [vp, sz]
    L.qgemv_load.argtypes = [vp, vp, sz, C.POINTER(vp)]
    L.qgemv_load_stacked.argtypes = [vp, vp, sz, i32, C.POINTER(vp)]
    L.qgemv_unload.argtypes = [vp, vp]
    L.qgemv_load_device.argtypes = [vp, i32, vp, vp, C.c_float, i64, i64, C.POINTER(Shard), vp, C.POINTER(vp)]
    L.qgemv_load_stacked_device.argtypes = [vp, i32, C.POINTER(vp), C.POINTER(vp), C.POINTER(C.c_float), i32, i64, i64,
                                            C.POINTER(Shard), vp, C.POINTER(vp)]
    L.qgemv_weight_read.argtypes = [vp, vp, vp, sz]
    L.qgemv_pack_header.argtypes = [i32, C.c_float, i64, i64, C.POINTER(Shard), vp]
    L.qgemv_set_host_threads.argtypes = [i32]
    L.qgemv_weight_bytes.restype = i64
    L.qgemv_weight_bytes.argtypes = [vp]
    L.qgemv_gemv.argtypes = [vp, vp, vp, i32, vp, i32, vp]
    L.qgemv_sequence_create.argtypes = [vp, C.POINTER(_Job), i32, i32, C.POINTER(vp)]
    L.qgemv_sequence_run.argtypes = [vp, vp, vp]
    L.qgemv_sequence_destroy.argtypes = [vp, vp]
    L.qgemv_gemv_prefetch.argtypes = [vp, vp, vp, i32, vp, i32, vp, vp]
    L.qgemv_gemm_skinny.argtypes = [vp, vp, vp, i32, vp, i32, i32, vp]
    L.qgemv_quantize_a4.argtypes = [vp, vp, i32, i64, vp, vp, vp, vp]
    L.qgemv_gemm_skinny_plan.argtypes = [i32, i64, i64, i32, i32, C.POINTER(SkinnyPlan)]
    L.qgemv_moe_plan.argtypes = [i64, i64, i32, i32, i32, i32, i32, C.POINTER(MoePlan)]
    L.qgemv_tp_create.argtypes = [vp, i32, i32, i64, vp]
    L.qgemv_tp_connect.argtypes = [vp, vp]
    L.qgemv_tp_allreduce.argtypes = [vp, vp, i32, i64, vp]
    L.qgemv_tp_allgather.argtypes = [vp, vp, vp, i32, i64, vp]
    L.qgemv_tp_buffer.argtypes = [vp, C.POINTER(vp), C.POINTER(sz)]
    L.qgemv_tp_connect_ptrs.argtypes = [vp, C.POINTER(vp)]
    L.qgemv_gemv_noalloc.argtypes = [vp, vp, vp, i32, vp, i32, vp]
    L.qgemv_noalloc_last_status.argtypes = [vp, C.POINTER(_DevStatus)]
    L.qgemv_moe_gemv.argtypes = [vp, vp, vp, vp, i32, i32, i32, vp, i32, vp]
    L.qgemv_moe_gemv_act.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, vp, i32, vp]
    L.qgemv_moe_mlp.argtypes = [vp, vp, vp, vp, vp, i32, i32, vp, vp, i32, vp]
    L.qgemv_moe_combine.argtypes = [vp, vp, i32, vp, i32, i32, i64, vp, i32, vp]
    L.qgemv_dequant_f32.argtypes = [vp, vp, i32, vp, vp]
    L.qgemv_last_device_status.argtypes = [vp, vp, C.POINTER(_DevStatus)]
    _LIB = L
    return L


def status_string(status: int) -> str:
    return _load().qgemv_status_string(int(status)).decode()


def _check(status: int, what: str) -> None:
    if status != 0:
        if status == ERR_CUDA:
            what = f"{what} [{_load().qgemv_last_cuda_error().decode()}]"
        raise QgemvError(status, what)


def _np_ptr(a: np.ndarray) -> C.c_void_p:
    if not a.flags["C_CONTIGUOUS"]:
        raise ValueError("array must be C-contiguous")
    return a.ctypes.data_as(C.c_void_p)


# ---- host packer ---------------------------------------------------------------------------------
def set_host_threads(n: int) -> None:
    """Threads of the host packer (a launcher may have exported OMP_NUM_THREADS=1)."""
    _check(_load().qgemv_set_host_threads(int(n)), "set_host_threads")


def packed_size(fmt: int, N: int, K: int, shard: Shard | None = None) -> int:
    return int(_load().qgemv_packed_size(fmt, N, K, C.byref(shard) if shard else None))


def pack(fmt: int, codes: np.ndarray, scales: np.ndarray, tensor_scale: float = 1.0,
         shard: Shard | None = None, out: np.ndarray | None = None) -> np.ndarray:
    """Pack canonical codes / scales into the device layout; returns the blob as a u8 array.

    NVFP4: codes u8 [N][K/2], scales u8 [N][K/16].  FP8: codes u8 [N][K], scales f32 [N].
    """
    if fmt in (FMT_NVFP4, FMT_NVFP4_TC):
        N, K = scales.shape[0], scales.shape[1] * 16
        if codes.dtype != np.uint8 or scales.dtype != np.uint8 or codes.shape != (N, K // 2):
            raise ValueError("NVFP4 wants codes u8 [N][K/2] and scales u8 [N][K/16]")
    elif fmt == FMT_FP8:
        N, K = codes.shape
        if codes.dtype != np.uint8 or scales.dtype != np.float32 or scales.shape != (N,):
            raise ValueError("FP8 wants codes u8 [N][K] and scales f32 [N]")
    else:
        raise QgemvError(ERR_INVALID_ARG, "pack")
    size = packed_size(fmt, N, K, shard)
    if size == 0:
        raise QgemvError(ERR_UNSUPPORTED_SHAPE, "pack")
    blob = out if out is not None else np.empty(size, dtype=np.uint8)
    if blob.size != size or blob.dtype != np.uint8:
        raise ValueError("output blob has the wrong size")
    _check(_load().qgemv_pack_host(fmt, _np_ptr(codes), _np_ptr(scales), C.c_float(tensor_scale), N, K,
                                   C.byref(shard) if shard else None, _np_ptr(blob)), "pack")
    return blob


def blob_info(blob: np.ndarray):
    fmt, N, K = C.c_int(), C.c_int64(), C.c_int64()
    _check(_load().qgemv_blob_info(_np_ptr(blob), blob.size, C.byref(fmt), C.byref(N), C.byref(K)), "blob_info")
    return fmt.value, N.value, K.value


def blob_verify(blob: np.ndarray) -> int:
    return int(_load().qgemv_blob_verify(_np_ptr(blob), blob.size))


def unpack(blob: np.ndarray):
    """Inverse of pack(): returns (codes, scales, tensor_scale) of the sub-matrix in the blob."""
    fmt, N, K = blob_info(blob)
    if fmt in (FMT_NVFP4, FMT_NVFP4_TC):
        codes = np.empty((N, K // 2), dtype=np.uint8)
        scales = np.empty((N, K // 16), dtype=np.uint8)
    else:
        codes = np.empty((N, K), dtype=np.uint8)
        scales = np.empty((N,), dtype=np.float32)
    ts = C.c_float()
    _check(_load().qgemv_unpack_host(_np_ptr(blob), blob.size, _np_ptr(codes), _np_ptr(scales), C.byref(ts)),
           "unpack")
    return codes, scales, ts.value


# ---- device side -----------------------------------------------------------------------------------
class Weight:
    """A packed weight resident on the device (one matrix, or a stack of experts)."""

    def __init__(self, owner: "QGemv", ptr: int, fmt: int, N: int, K: int, n_stack: int):
        self._owner, self._ptr = owner, ptr
        self.fmt, self.N, self.K, self.n_stack = fmt, N, K, n_stack

    @property
    def weight_bytes(self) -> int:
        """Algorithmic weight bytes of one matrix (codes + scales)."""
        return int(_load().qgemv_weight_bytes(self._ptr))

    def read_blob(self) -> np.ndarray:
        """The packed blob(s) as they sit in device memory, copied back to the host."""
        out = np.empty(self.n_stack * packed_size(self.fmt, self.N, self.K), dtype=np.uint8)
        _check(_load().qgemv_weight_read(self._owner._ptr, self._ptr, _np_ptr(out), out.size), "weight_read")
        return out

    def unload(self) -> None:
        if self._ptr:
            _check(_load().qgemv_unload(self._owner._ptr, self._ptr), "unload")
            self._ptr = None


class Sequence:
    """A job list resident on the device (qgemv_sequence): run() launches it as one persistent kernel."""

    def __init__(self, owner: "QGemv", ptr: int, n_jobs: int, B: int):
        self._owner, self._ptr, self.n_jobs, self.B = owner, ptr, n_jobs, B

    def run(self, stream: int = 0) -> None:
        _check(_load().qgemv_sequence_run(self._owner._ptr, self._ptr, stream), "sequence_run")

    def destroy(self) -> None:
        if self._ptr:
            _load().qgemv_sequence_destroy(self._owner._ptr, self._ptr)
            self._ptr = None


class QGemv:
    """One library handle on one device."""

    def __init__(self, device: int = 0, use_pdl: bool = True, grid_override: int = 0, debug: bool = False,
                 spin_limit: int = 0, inject_drop_copies: bool = False, debug_bits: int = 0,
                 tc_stage_items: int = 0, tc_smem_kb: int = 0):
        L = _load()
        cfg = _Config(device, 1 if use_pdl else 0, grid_override,
                      (1 if debug else 0) | (2 if inject_drop_copies else 0) | debug_bits, spin_limit,
                      tc_stage_items, tc_smem_kb)
        h = C.c_void_p()
        _check(L.qgemv_init(C.byref(cfg), C.byref(h)), "init")
        self._ptr = h.value
        self.device = device

    def close(self) -> None:
        if self._ptr:
            _load().qgemv_destroy(self._ptr)
            self._ptr = None

    @property
    def sm_count(self) -> int:
        return int(_load().qgemv_sm_count(self._ptr))

    def set_trace(self, dev_ptr: int | None) -> None:
        """Phase timestamps of the tensor-core GEMV into a device buffer of 16 u64 per CTA (None: off)."""
        _check(_load().qgemv_set_trace(self._ptr, dev_ptr), "set_trace")

    def load(self, blob: np.ndarray) -> Weight:
        fmt, N, K = blob_info(blob)
        w = C.c_void_p()
        _check(_load().qgemv_load(self._ptr, _np_ptr(blob), blob.size, C.byref(w)), "load")
        return Weight(self, w.value, fmt, N, K, 1)

    def load_device(self, fmt: int, codes_ptr: int, scales_ptr: int, N: int, K: int, tensor_scale: float = 1.0,
                    shard: Shard | None = None, stream: int = 0) -> Weight:
        """Weight from canonical NVFP4 arrays in device memory (codes u8 [N][K/2], scales u8 [N][K/16]),
        packed by a kernel; NVFP4_TC only.  The arrays may be freed when this returns."""
        w = C.c_void_p()
        _check(_load().qgemv_load_device(self._ptr, fmt, codes_ptr, scales_ptr, C.c_float(tensor_scale), N, K,
                                         C.byref(shard) if shard else None, stream, C.byref(w)), "load_device")
        n = (shard.n1 - shard.n0) if shard else N
        k = (shard.k1 - shard.k0) if shard else K
        return Weight(self, w.value, fmt, n, k, 1)

    def load_stacked_device(self, fmt: int, codes_ptrs: list[int], scales_ptrs: list[int], N: int, K: int,
                            tensor_scales, shard: Shard | None = None, stream: int = 0) -> Weight:
        """The experts of an MoE layer from canonical NVFP4 arrays in device memory (one pair of device pointers
        and one tensor scale per expert), packed by a kernel into one stacked weight; NVFP4_TC only."""
        E = len(codes_ptrs)
        if E < 1 or len(scales_ptrs) != E or len(tensor_scales) != E:
            raise ValueError("one codes pointer, one scales pointer and one tensor scale per expert")
        cp = (C.c_void_p * E)(*codes_ptrs)
        sp = (C.c_void_p * E)(*scales_ptrs)
        ts = (C.c_float * E)(*[float(t) for t in tensor_scales])
        w = C.c_void_p()
        _check(_load().qgemv_load_stacked_device(self._ptr, fmt, cp, sp, ts, E, N, K, C.byref(shard) if shard else None,
                                                 stream, C.byref(w)), "load_stacked_device")
        n = (shard.n1 - shard.n0) if shard else N
        k = (shard.k1 - shard.k0) if shard else K
        return Weight(self, w.value, fmt, n, k, E)

    def load_stacked(self, blobs: np.ndarray) -> Weight:
        """blobs: u8 [E][bytes_each], every row a packed blob of the same shape and format."""
        if blobs.ndim != 2:
            raise ValueError("blobs must be [E][bytes_each]")
        fmt, N, K = blob_info(blobs[0])
        w = C.c_void_p()
        _check(_load().qgemv_load_stacked(self._ptr, _np_ptr(blobs), blobs.shape[1], blobs.shape[0], C.byref(w)),
               "load_stacked")
        return Weight(self, w.value, fmt, N, K, blobs.shape[0])

    def gemv(self, w: Weight, x_ptr: int, B: int, y_ptr: int, y_dtype: int = OUT_BF16, stream: int = 0,
             next_weight: Weight | None = None) -> None:
        """y = W x.  `next_weight`: the matrix the caller multiplies by next; it is prefetched into L2."""
        if next_weight is None:
            _check(_load().qgemv_gemv(self._ptr, w._ptr, x_ptr, B, y_ptr, y_dtype, stream), "gemv")
        else:
            _check(_load().qgemv_gemv_prefetch(self._ptr, w._ptr, x_ptr, B, y_ptr, y_dtype, next_weight._ptr,
                                               stream), "gemv")

    def sequence(self, jobs: list[tuple], B: int, chained: bool = False) -> "Sequence":
        """jobs: (weight, x_ptr, y_ptr, y_dtype) in execution order; one persistent launch runs them all.
        A job waits for the earlier jobs whose buffers it reads or overwrites; with `chained` every job
        also waits for the one before it, whatever the addresses say.  NVFP4_TC weights only."""
        arr = (_Job * len(jobs))()
        for i, jb in enumerate(jobs):   # (weight, x_ptr, y_ptr, y_dtype[, flags[, x_stride[, fused]]])
            w, x_ptr, y_ptr, y_dtype = jb[:4]
            flags = (jb[4] if len(jb) > 4 else 0) | (JOB_AFTER_PREVIOUS if chained else 0)
            fz = jb[6] if len(jb) > 6 and jb[6] else {}     # {"norm_weight": ptr, "norm_eps": e, "residual": ptr}
            arr[i] = _Job(w._ptr, x_ptr, y_ptr, y_dtype, flags, jb[5] if len(jb) > 5 else 0,
                          fz.get("norm_weight"), fz.get("residual"), float(fz.get("norm_eps", 0.0)), 0)
        q = C.c_void_p()
        _check(_load().qgemv_sequence_create(self._ptr, arr, len(jobs), B, C.byref(q)), "sequence_create")
        return Sequence(self, q.value, len(jobs), B)

    def gemm_skinny(self, w: Weight, x_ptr: int, M: int, y_ptr: int, y_dtype: int = OUT_BF16,
                    act_mode: int = ACT_A16_EXACT, stream: int = 0) -> None:
        """Y[M][N] = X[M][K] dequant(W)^T on the tcgen05 tensor cores, M = 16..256 (multiple of 16)."""
        _check(_load().qgemv_gemm_skinny(self._ptr, w._ptr, x_ptr, M, y_ptr, y_dtype, act_mode, stream),
               "gemm_skinny")

    def quantize_a4(self, x_ptr: int, M: int, K: int, codes_ptr: int, scales_ptr: int, row_scales_ptr: int,
                    stream: int = 0) -> None:
        """The A4 mode's activation quantiser alone: canonical codes [M][K/2], scales [M][K/16], row scales f32 [M]."""
        _check(_load().qgemv_quantize_a4(self._ptr, x_ptr, M, K, codes_ptr, scales_ptr, row_scales_ptr, stream),
               "quantize_a4")

    def moe_gemv(self, experts: Weight, expert_ids_ptr: int, x_ptr: int, T: int, topk: int,
                 per_slot_input: bool, out_ptr: int, out_dtype: int = OUT_F32, stream: int = 0, x_act: int = 0) -> None:
        """x_act = MOE_X_SILU_MUL: the rows of x hold gate and up values (2 K) and the experts multiply
        bf16(silu(gate) * up) -- the down stage fed straight from the gate/up stage's output rows."""
        if x_act:
            _check(_load().qgemv_moe_gemv_act(self._ptr, experts._ptr, expert_ids_ptr, x_ptr, T, topk,
                                              1 if per_slot_input else 0, x_act, out_ptr, out_dtype, stream), "moe_gemv_act")
            return
        _check(_load().qgemv_moe_gemv(self._ptr, experts._ptr, expert_ids_ptr, x_ptr, T, topk,
                                      1 if per_slot_input else 0, out_ptr, out_dtype, stream), "moe_gemv")

    def moe_mlp(self, gate_up: Weight, down: Weight, expert_ids_ptr: int, x_ptr: int, T: int, topk: int,
                gate_up_rows_ptr: int, out_ptr: int, out_dtype: int = OUT_F32, stream: int = 0) -> None:
        """Both stages of the experts' MLP as one launch (tensor-core layout): gate/up, silu(gate) * up, down."""
        _check(_load().qgemv_moe_mlp(self._ptr, gate_up._ptr, down._ptr, expert_ids_ptr, x_ptr, T, topk,
                                     gate_up_rows_ptr, out_ptr, out_dtype, stream), "moe_mlp")

    def moe_combine(self, slot_out_ptr: int, slot_dtype: int, expert_w_ptr: int, T: int, topk: int, N: int,
                    y_ptr: int, y_dtype: int = OUT_BF16, stream: int = 0) -> None:
        _check(_load().qgemv_moe_combine(self._ptr, slot_out_ptr, slot_dtype, expert_w_ptr, T, topk, N, y_ptr,
                                         y_dtype, stream), "moe_combine")

    def dequant_f32(self, w: Weight, out_ptr: int, which: int = 0, stream: int = 0) -> None:
        _check(_load().qgemv_dequant_f32(self._ptr, w._ptr, which, out_ptr, stream), "dequant_f32")

    # ---- tensor parallel --------------------------------------------------------------------------
    def tp_create(self, rank: int, world: int, max_elems: int) -> np.ndarray:
        """Allocates this rank's exchange buffer; returns its 64-byte CUDA IPC handle."""
        out = np.zeros(64, dtype=np.uint8)
        _check(_load().qgemv_tp_create(self._ptr, rank, world, max_elems, _np_ptr(out)), "tp_create")
        return out

    def tp_connect(self, all_handles: np.ndarray) -> None:
        """all_handles: u8 [world][64], the handles of every rank in rank order."""
        _check(_load().qgemv_tp_connect(self._ptr, _np_ptr(np.ascontiguousarray(all_handles, dtype=np.uint8))),
               "tp_connect")

    def tp_allreduce(self, y_ptr: int, y_dtype: int, n: int, stream: int = 0) -> None:
        _check(_load().qgemv_tp_allreduce(self._ptr, y_ptr, y_dtype, n, stream), "tp_allreduce")

    def tp_allgather(self, shard_ptr: int, y_ptr: int, y_dtype: int, n_shard: int, stream: int = 0) -> None:
        """y[r * n_shard + e] = rank r's shard[e]."""
        _check(_load().qgemv_tp_allgather(self._ptr, shard_ptr, y_ptr, y_dtype, n_shard, stream), "tp_allgather")

    def tp_buffer(self) -> tuple[int, int]:
        """(device pointer, bytes) of this rank's exchange buffer."""
        p, n = C.c_void_p(), C.c_size_t()
        _check(_load().qgemv_tp_buffer(self._ptr, C.byref(p), C.byref(n)), "tp_buffer")
        return int(p.value), int(n.value)

    def tp_connect_ptrs(self, peer_ptrs: list[int]) -> None:
        """Single process, several GPUs (or a test): the other ranks' buffers as device pointers, rank order."""
        arr = (C.c_void_p * len(peer_ptrs))(*[C.c_void_p(p) for p in peer_ptrs])
        _check(_load().qgemv_tp_connect_ptrs(self._ptr, arr), "tp_connect_ptrs")

    def device_status(self, stream: int = 0) -> DeviceStatus:
        st = _DevStatus()
        _check(_load().qgemv_last_device_status(self._ptr, stream, C.byref(st)), "device_status")
        return DeviceStatus(st.code, st.where, st.block, st.extra)


def gemv_noalloc(dev_blob_ptr: int, host_blob: np.ndarray, x_ptr: int, B: int, y_ptr: int,
                 y_dtype: int = OUT_BF16, stream: int = 0) -> None:
    """Allocation-free GEMV: `dev_blob_ptr` is the caller's device copy of the packed blob and
    `host_blob` the same blob (at least its first 256 bytes) in host memory.  Needs no handle; the
    kernel's scratch is a static array inside the library (see include/qgemv.h for the limits)."""
    _check(_load().qgemv_gemv_noalloc(dev_blob_ptr, _np_ptr(host_blob), x_ptr, B, y_ptr, y_dtype, stream),
           "gemv_noalloc")


def noalloc_last_status(stream: int = 0) -> DeviceStatus:
    """Synchronises `stream` and returns the status word of the last allocation-free GEMV on the
    current device (all zero when none has run, or when it ended without a report)."""
    st = _DevStatus()
    _check(_load().qgemv_noalloc_last_status(stream, C.byref(st)), "noalloc_last_status")
    return DeviceStatus(st.code, st.where, st.block, st.extra)


def moe_plan(K: int, n_experts: int, T: int, topk: int, K2: int = 0, ctas: int = 148, smem_kb: int = 0) -> MoePlan:
    """How an expert-list launch (moe_gemv / moe_mlp on tensor-core-layout experts) would be laid out; host arithmetic,
    no device needed.  K2: the second stage's K for moe_mlp.  Raises QgemvError where the launch would refuse."""
    plan = MoePlan()
    _check(_load().qgemv_moe_plan(K, K2, n_experts, T, topk, ctas, smem_kb, C.byref(plan)), "moe_plan")
    return plan


def gemm_skinny_plan(fmt: int, N: int, K: int, M: int, sm_count: int = 148) -> SkinnyPlan:
    """Pure host arithmetic: ring depths, tensor- and shared-memory use of a skinny GEMM shape."""
    plan = SkinnyPlan()
    _check(_load().qgemv_gemm_skinny_plan(fmt, N, K, M, sm_count, C.byref(plan)), "gemm_skinny_plan")
    return plan
