"""Layer-stack runner: a fixed list of projection GEMVs replayed as one CUDA graph.

A decode step of a dense model is, for this library, a sequence of weight-streaming GEMVs
(QKV, o_proj, gate/up, down per layer; "one CUDA graph per round",
tools/fixtures/engines/crit-labs/mtp4-nvfp4-mma/card.yaml:75).  The runner owns the activation
and output buffers of every call, captures the launches once, and replays the graph.  With
programmatic dependent launch enabled on the handle each kernel's weight prefetch overlaps the
tail of the one before it.

torch is used for device memory, streams and graph capture only; every kernel is the
library's own, reached through the C ABI.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from . import OUT_BF16, OUT_F32, QGemv, Weight


@dataclass
class _Call:
    weight: Weight
    x_off: int  # element offsets into the stack's activation / output arenas
    y_off: int


class LayerStack:
    """Owns an activation arena [sum B*K] bf16 and an output arena [sum B*N]; one GEMV per weight."""

    def __init__(self, handle: QGemv, weights: list[Weight], batch: int, out_dtype: int = OUT_BF16,
                 device: int = 0, prefetch_next: bool = False, after_call=None, fused: bool = False,
                 chained: bool = False, job_flags: list[int] | None = None, chain: bool = False,
                 job_opts: list[dict | None] | None = None):
        self.handle, self.batch, self.out_dtype = handle, batch, out_dtype
        # fused: the whole list as ONE persistent launch (qgemv_sequence_*; tensor-core layout only, no hooks)
        self.fused = fused and after_call is None
        # chained: every job of the fused launch waits for the one before it, as a decode step's
        # projections do (each consumes, through attention / activation / norm, what the previous produced)
        self.chained = chained
        self.job_flags = job_flags  # per-call qgemv_job flags of the fused launch (e.g. JOB_ALLREDUCE), or None
        # per-call element-wise options of the fused launch ({"norm_weight": ptr, "norm_eps": e, "residual": ptr}), or None
        self.job_opts = job_opts
        self.sequence = None
        # after_call(i): optional hook enqueued on the same stream right after GEMV i (and captured
        # with it), e.g. the all-reduce of a row-parallel projection's partial outputs
        self.after_call = after_call
        self.prefetch_next = prefetch_next  # name the following matrix in every call (L2 prefetch)
        self.device = torch.device("cuda", device)
        self.calls: list[_Call] = []
        # chain: call i reads the first K_i columns of call i - 1's output (a decode step's data flow with the
        # element-wise work between the projections left out); only the first call has an input of its own.
        # Needs the fused launch (rows of a column range are strided) and bf16 outputs.
        from . import JOB_X_SILU_MUL
        cols = lambda i: weights[i].K * (2 if job_flags and job_flags[i] & JOB_X_SILU_MUL else 1)   # columns of x call i reads
        self.chain = chain and self.fused and out_dtype == OUT_BF16 and all(
            cols(i) <= weights[i - 1].N and weights[i - 1].N % 8 == 0 for i in range(1, len(weights)))
        x_total = y_total = 0
        for i, w in enumerate(weights):
            self.calls.append(_Call(w, x_total, y_total))
            if not self.chain or i == 0:
                x_total += ((batch * w.K + 7) // 8) * 8      # keep every row block 16-byte aligned
            y_total += ((batch * w.N + 7) // 8) * 8
        self.x_dev = torch.zeros(x_total, dtype=torch.bfloat16, device=self.device)
        ydt = torch.bfloat16 if out_dtype == OUT_BF16 else torch.float32
        self.y_dev = torch.zeros(y_total, dtype=ydt, device=self.device)
        self.x_host = torch.zeros(x_total, dtype=torch.bfloat16).pin_memory()
        self.y_host = torch.zeros(y_total, dtype=ydt).pin_memory()
        self.stream = torch.cuda.Stream(device=self.device)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.weight_bytes = sum(w.weight_bytes for w in weights)

    # ---- buffers --------------------------------------------------------------------------
    def set_inputs(self, xs: list[torch.Tensor]) -> None:
        """xs[i]: bf16 [batch][K_i] activations of call i (host or device tensors)."""
        for c, x in zip(self.calls[:1] if self.chain else self.calls, xs):
            n = self.batch * c.weight.K
            self.x_host[c.x_off:c.x_off + n].copy_(x.reshape(-1).to(torch.bfloat16).cpu())
        self.x_dev.copy_(self.x_host, non_blocking=False)

    def input(self, i: int) -> torch.Tensor:
        """Host copy of call i's activations [batch][K] as of the last step_host()."""
        c = self.calls[i]
        if self.chain and i > 0:
            from . import JOB_X_SILU_MUL
            k = c.weight.K * (2 if self.job_flags and self.job_flags[i] & JOB_X_SILU_MUL else 1)
            return self.output(i - 1, host=True)[:, :k]
        return self.x_host[c.x_off:c.x_off + self.batch * c.weight.K].view(self.batch, c.weight.K)

    def output(self, i: int, host: bool = False) -> torch.Tensor:
        c = self.calls[i]
        src = self.y_host if host else self.y_dev
        return src[c.y_off:c.y_off + self.batch * c.weight.N].view(self.batch, c.weight.N)

    @property
    def h2d_bytes(self) -> int:
        return self.x_host.numel() * self.x_host.element_size()

    @property
    def d2h_bytes(self) -> int:
        return self.y_host.numel() * self.y_host.element_size()

    # ---- launches -------------------------------------------------------------------------
    def _enqueue(self, stream_handle: int) -> None:
        xe, ye = self.x_dev.element_size(), self.y_dev.element_size()
        xb, yb = self.x_dev.data_ptr(), self.y_dev.data_ptr()
        n = len(self.calls)
        if self.fused:
            if self.sequence is None:
                from . import ERR_UNSUPPORTED_SHAPE, QgemvError
                try:
                    jobs = []
                    for i, c in enumerate(self.calls):
                        fl = self.job_flags[i] if self.job_flags else 0
                        opts = self.job_opts[i] if self.job_opts else None
                        if self.chain and i > 0:
                            prev = self.calls[i - 1]
                            jobs.append((c.weight, yb + prev.y_off * ye, yb + c.y_off * ye, self.out_dtype, fl, prev.weight.N, opts))
                        else:
                            jobs.append((c.weight, xb + c.x_off * xe, yb + c.y_off * ye, self.out_dtype, fl, 0, opts))
                    self.sequence = self.handle.sequence(jobs, self.batch, chained=self.chained)
                except QgemvError as e:  # e.g. activations too large for the persistent kernel: one launch per GEMV
                    if e.status != ERR_UNSUPPORTED_SHAPE or self.chain:
                        raise
                    self.fused = False
            if self.fused:
                self.sequence.run(stream_handle)
                return
        for i, c in enumerate(self.calls):
            nxt = self.calls[(i + 1) % n].weight if self.prefetch_next and n > 1 else None
            self.handle.gemv(c.weight, xb + c.x_off * xe, self.batch, yb + c.y_off * ye, self.out_dtype,
                             stream_handle, next_weight=nxt)
            if self.after_call is not None:
                self.after_call(i)

    def capture(self) -> None:
        """Run once eagerly (loads modules, warms caches), then capture the stack into a graph."""
        with torch.cuda.stream(self.stream):
            self._enqueue(self.stream.cuda_stream)
        self.stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=self.stream):
            self._enqueue(torch.cuda.current_stream().cuda_stream)
        self.graph = g

    def step(self) -> None:
        """One pass over the stack, inputs and outputs resident on the device (asynchronous)."""
        with torch.cuda.stream(self.stream):
            if self.graph is not None:
                self.graph.replay()
            else:
                self._enqueue(self.stream.cuda_stream)

    def step_host(self) -> None:
        """One pass with host buffers: pinned activations in, pinned results out, then a sync."""
        with torch.cuda.stream(self.stream):
            self.x_dev.copy_(self.x_host, non_blocking=True)
            if self.graph is not None:
                self.graph.replay()
            else:
                self._enqueue(self.stream.cuda_stream)
            self.y_host.copy_(self.y_dev, non_blocking=True)
        self.stream.synchronize()

    @property
    def launches_per_step(self) -> int:
        return 1 if self.fused else len(self.calls)


def llama_layer_shapes(hidden: int, q_heads: int, kv_heads: int, head_dim: int, inter: int):
    """(name, N, K) of the four projections of one decoder layer (fused QKV and gate/up)."""
    return [("qkv", (q_heads + 2 * kv_heads) * head_dim, hidden), ("o", hidden, q_heads * head_dim),
            ("gate_up", 2 * inter, hidden), ("down", hidden, inter)]


def synth_nvfp4_dev(N: int, K: int, seed: int, device: torch.device):
    """Seeded synthetic NVFP4 matrix in device memory: codes uniform over the 16 E2M1 codes, E4M3
    scales of |N(0,1)| * 0.05 per 16-element block.  Returns device tensors (codes u8 [N][K/2],
    scales u8 [N][K/16]); the same seed gives the same matrix on every GPU."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    codes = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=device, generator=g)
    sc = torch.randn((N, K // 16), dtype=torch.float32, device=device, generator=g).abs_().mul_(0.05)
    return codes, sc.to(torch.float8_e4m3fn).view(torch.uint8)


def synth_nvfp4(N: int, K: int, seed: int, device: torch.device):
    """synth_nvfp4_dev copied to the host: numpy (codes, scales), tensor scale 1.0."""
    codes, scales = synth_nvfp4_dev(N, K, seed, device)
    return codes.cpu().numpy(), scales.cpu().numpy()


def synth_fp8(N: int, K: int, seed: int, device: torch.device):
    """Codes uniform over the 254 finite E4M3 codes; channel scales fp32 |N(0,1)| * 0.02."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    c = torch.randint(0, 254, (N, K), dtype=torch.int16, device=device, generator=g)
    c = torch.where(c >= 127, c + 1, c).to(torch.uint8)
    s = torch.randn((N,), dtype=torch.float32, device=device, generator=g).abs_().mul_(0.02)
    return c.cpu().numpy(), s.cpu().numpy().astype(np.float32)
