"""Benchmark of the NVFP4 decode GEMV path: weight GB/s over a Llama-shaped layer stack.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]
    python bench.py --workload prefill [--tokens M]      (one secondary workload alone: skinny GEMM)
    python bench.py --workload prefill_a4 [--tokens M]   (block-scaled prefill, NVFP4 activations)
    python bench.py --workload lmhead [--batch B]        (FP8 output head)
    python bench.py --workload moe [--tokens T]          (the experts' MLP of an MoE layer: gate/up, silu x up, down;
                                                          --moe-layout lane | --moe-two-launches for the other forms)

A "step" is one pass of the hot path over the whole layer stack (four weight-streaming GEMVs per
layer) at decode batch B.  By default the stack runs as ONE persistent launch per step
(qgemv_sequence_*), replayed from a CUDA graph.  `value` = algorithmic weight bytes of all ranks /
device time, inputs resident in HBM; `e2e` = the same metric with pinned host activations copied in
and results copied out inside the timed region.  One JSON line is printed by rank 0.

N = 1 runs the Llama-3-8B-shaped stack (32 layers, 3.9 GB of NVFP4 weights -- larger than L2, so
every step streams from HBM), verifies sampled rows of its outputs against the CPU oracle, and then
attaches the secondary workloads (batch 2/4/8, output head, MoE, prefill) under `secondary`, each
verified the same way.  N > 1 runs all 80 layers of the Llama-3-70B-shaped stack tensor-parallel
(column-parallel QKV and gate/up, row-parallel o and down whose partial sums are exchanged over
NVLink inside the same launch), total work fixed: strong scaling; the shards are cut from seeded
canonical matrices and one layer is checked against the unsharded oracle before timing.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "nvfp4_decode_gemv_weight_gbps"
UNIT = "GB/s"
LLAMA_8B = dict(name="llama-3-8b", hidden=4096, q_heads=32, kv_heads=8, head_dim=128, inter=14336, layers=32)
LLAMA_70B = dict(name="llama-3-70b", hidden=8192, q_heads=64, kv_heads=8, head_dim=128, inter=28672, layers=80)
TOL_BF16 = 2e-3   # relative L2 of bf16 outputs against the fp64 oracle
TOL_F32 = 5e-5    # of fp32 outputs


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def measured_peak_tflops():
    """Measured dense bf16 burst peak of this pool's B200s (TFLOP/s), else the stated fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period = index, period_s
        self.sm, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self.thread = None
        self.error = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # noqa: BLE001 - report, never fail the benchmark on telemetry
            self.error = f"nvml unavailable: {e}"
            return self
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except AttributeError:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception as e:  # noqa: BLE001
                self.error = str(e)
                break
            time.sleep(self.period)

    def stop(self):
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)
        out = {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.sm)}
        if self.error:
            out["note"] = self.error
        return out


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def u16(t):
    """bf16 torch tensor -> numpy uint16 bit patterns (host)."""
    import numpy as np
    import torch
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def sample_rows(N: int, count: int = 192):
    """Row indices of a sampled slice: the first, the last (a ragged tile's) and a middle stripe."""
    import numpy as np
    c = max(1, count // 3)
    idx = np.unique(np.concatenate([np.arange(min(c, N)), np.arange(max(0, N - c), N),
                                    np.arange(max(0, N // 2 - c // 2), min(N, N // 2 + c // 2))]))
    return idx


def tensor_scale_for(K: int) -> float:
    """Per-tensor scale that keeps the outputs of a synthetic matrix near the magnitude of its inputs
    (the codes are uniform over E2M1, the block scales |N(0,1)| * 0.05: an element's RMS is 0.1463),
    so that values stay in range when every GEMV of the stack feeds the next."""
    return float(1.0 / (0.1463 * K ** 0.5))


def timed(stream, fn, n, barrier=None):
    """Device time of n calls of fn on `stream` (CUDA events on that stream, a sync on both sides)."""
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    (barrier or torch.cuda.synchronize)()
    with torch.cuda.stream(stream):
        e0.record()
    for _ in range(n):
        fn()
    with torch.cuda.stream(stream):
        e1.record()
    (barrier or torch.cuda.synchronize)()
    return e0.elapsed_time(e1)


# ---- the decode stack --------------------------------------------------------------------------------
class DecodeStack:
    """The rank's share of the layer stack, its runners and the slices kept for verification.

    Tensor parallel: QKV and gate/up are column-parallel (this rank holds N/world output rows), o
    and down are row-parallel (K/world input columns; their outputs are partial sums, summed over the
    ranks).  Every rank synthesises the same canonical matrix on its GPU (seeded by layer and
    projection) and packs its shard there (qgemv_load_device)."""

    def __init__(self, model, rank, world, dev_index, layout="tc", keep_full=False):
        import torch

        import crit_hub_b200 as qg
        from crit_hub_b200.stack import llama_layer_shapes, synth_nvfp4_dev

        self.qg, self.model, self.rank, self.world, self.layout = qg, model, rank, world, layout
        self.device = torch.device("cuda", dev_index)
        self.handle = qg.QGemv(device=dev_index, use_pdl=True)
        self.shapes = llama_layer_shapes(model["hidden"], model["q_heads"], model["kv_heads"], model["head_dim"], model["inter"])
        self.weights, self.full_weights, self.row_parallel, self.kept = [], [], [], {}
        self.bytes = 0
        n_calls = model["layers"] * 4
        keep_calls = {0, 1, 2, 3, n_calls - 2, n_calls - 1}
        for layer in range(model["layers"]):
            for mi, (name, N, K) in enumerate(self.shapes):
                codes, scales = synth_nvfp4_dev(N, K, 1000 * layer + mi, self.device)
                ts = tensor_scale_for(K)
                rowp = world > 1 and name in ("o", "down")
                shard = None
                if world > 1:
                    shard = (qg.Shard(0, N, rank * K // world, (rank + 1) * K // world) if rowp
                             else qg.Shard(rank * N // world, (rank + 1) * N // world, 0, K))
                if layout == "tc":
                    w = self.handle.load_device(qg.FMT_NVFP4_TC, codes.data_ptr(), scales.data_ptr(), N, K, ts, shard=shard)
                else:
                    w = self.handle.load(qg.pack(qg.FMT_NVFP4, codes.cpu().numpy(), scales.cpu().numpy(), ts, shard=shard))
                self.weights.append(w)
                self.row_parallel.append(rowp)
                self.bytes += w.weight_bytes
                if keep_full:
                    self.full_weights.append(self.handle.load_device(qg.FMT_NVFP4_TC, codes.data_ptr(), scales.data_ptr(), N, K, ts))
                call = layer * 4 + mi
                if call in keep_calls:
                    # rows of THIS rank's output (full N for row-parallel), all of its K columns
                    n0, n1 = (shard.n0, shard.n1) if shard else (0, N)
                    k0, k1 = (shard.k0, shard.k1) if shard else (0, K)
                    idx = sample_rows(n1 - n0, 768)
                    self.kept[call] = (idx, codes[n0:n1][idx][:, k0 // 2:k1 // 2].cpu().numpy().copy(),
                                       scales[n0:n1][idx][:, k0 // 16:k1 // 16].cpu().numpy().copy(), ts)
                del codes, scales
        torch.cuda.synchronize()

    def runner(self, batch, fused=True, chained=False, prefetch_next=True, after_call=None, weights=None, flags=None, chain=False,
               opts=None):
        import torch
        from crit_hub_b200.stack import LayerStack
        ws = weights if weights is not None else self.weights
        st = LayerStack(self.handle, ws, batch, self.qg.OUT_BF16, device=self.device.index, after_call=after_call,
                        prefetch_next=prefetch_next, fused=fused and self.layout == "tc", chained=chained, job_flags=flags, chain=chain, job_opts=opts)
        g = torch.Generator()
        g.manual_seed(7 + self.rank + 100 * batch)
        st.set_inputs([torch.randn((batch, w.K), generator=g).to(torch.bfloat16) for w in ws])
        return st

    def verify(self, stack):
        """Sampled rows of the kept calls of a (single-rank) runner against the fp64 oracle, from the
        host copies of one step_host()."""
        from oracle import oracle as O
        worst = 0.0
        for call, (idx, codes, scales, ts) in self.kept.items():
            x = u16(stack.input(call))
            got = stack.output(call, host=True).float().numpy()[:, idx]
            worst = max(worst, O.rel_l2(got, O.gemv_nvfp4_f64(codes, scales, ts, x)))
        return worst


def _verify_fused(self, stack, flags, opts, norm_w_bits, resid_bits):
    """Sampled rows of the kept calls of a runner whose jobs carry a norm, SiLU x up or a residual: the
    fp64 oracle applied to the device's own input of each call."""
    import numpy as np
    from oracle import oracle as O
    worst = 0.0
    for call, (idx, codes, scales, ts) in self.kept.items():
        x = O.bf16_decode(u16(stack.input(call))).astype(np.float64)
        K = stack.calls[call].weight.K
        if flags[call] & self.qg.JOB_X_SILU_MUL:
            g, u = x[:, :K], x[:, K:2 * K]
            x = O.bf16_decode(O.bf16_encode((g / (1.0 + np.exp(-g)) * u).astype(np.float32))).astype(np.float64)
        r = np.ones(x.shape[0])
        if "norm_weight" in opts[call]:
            r = 1.0 / np.sqrt((x ** 2).mean(axis=1) + opts[call]["norm_eps"])
            x = O.bf16_decode(O.bf16_encode((x.astype(np.float32) * O.bf16_decode(norm_w_bits)[None, :]))).astype(np.float64)
        ref = O.gemv_nvfp4_f64(codes, scales, ts, O.bf16_encode(x.astype(np.float32))) * r[:, None]
        if "residual" in opts[call]:
            ref = ref + O.bf16_decode(resid_bits)[:, idx]
        got = stack.output(call, host=True).float().numpy()[:, idx]
        worst = max(worst, O.rel_l2(got, ref))
    return worst


DecodeStack.verify_fused = _verify_fused


def cpu_reference_sample(model, batch, steps, warmup, threads):
    """Times the CPU restatement (fp32-accumulate OpenMP GEMV, this machine's own build) on one layer."""
    from crit_hub_b200.stack import llama_layer_shapes
    from oracle import oracle as O

    O.set_threads(threads)
    shapes = llama_layer_shapes(model["hidden"], model["q_heads"], model["kv_heads"], model["head_dim"], model["inter"])
    mats = []
    for mi, (name, N, K) in enumerate(shapes):
        codes, scales, ts = O.make_nvfp4(N, K, seed=mi)
        mats.append((codes, scales, ts, O.make_x(batch, K, seed=mi)))
    layer_bytes = sum(m[1].shape[0] * m[1].shape[1] * 16 * 9 // 16 + 4 for m in mats)
    used = threads
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        for codes, scales, ts, x in mats:
            _, used = O.gemv_nvfp4_fast(codes, scales, ts, x, native=True)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return layer_bytes / sec / 1e9, sec, used, layer_bytes


def cpu_baseline_entry(model, batch, steps=3, warmup=1):
    cg, sec, threads, layer_bytes = cpu_reference_sample(model, batch, steps, warmup, host_cores())
    return {"value": round(cg, 3), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"one {model['name']}-shaped layer ({layer_bytes} weight bytes), {steps} timed passes after {warmup}, "
                      f"fp32-accumulate OpenMP port of the host reference built with -O3 -march=native, {threads} threads"}


def run_reference(args):
    """The reference arm: the CPU restatement of the path on the host cores.  The registry holds
    no implementation of this arithmetic to install or compile, so the port is what runs."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    model = LLAMA_8B if args.gpus == 1 else LLAMA_70B
    steps, warmup = max(args.steps, 1), max(args.warmup, 0)
    gbs, sec, threads, layer_bytes = cpu_reference_sample(model, args.batch, steps, warmup, host_cores())
    sample = (f"one {model['name']}-shaped layer (4 GEMVs, {layer_bytes} weight bytes) per step, {steps} steps after "
              f"{warmup} warm-up, {threads} OpenMP threads, -O3 -march=native")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
        "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{model['name']} layer stack, NVFP4, batch {args.batch} (CPU port, bounded sample)"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---- secondary workloads (one GPU) ---------------------------------------------------------------------
def run_prefill(args, M=None):
    """The tcgen05 skinny GEMM over the four projections of one Llama-3-70B-shaped layer (481 MB of
    NVFP4 weights, larger than L2) at M rows.  One step = the four GEMMs; value = 2*M*N*K flops of the
    layer / device time.  Verified on sampled output rows of the QKV projection."""
    import torch

    import crit_hub_b200 as qg
    from crit_hub_b200.stack import llama_layer_shapes, synth_nvfp4
    from oracle import oracle as O

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    M = M or args.tokens
    model = LLAMA_70B
    h = qg.QGemv(device=0, use_pdl=True)
    shapes = llama_layer_shapes(model["hidden"], model["q_heads"], model["kv_heads"], model["head_dim"], model["inter"])
    ws, xs, ys, xh, yh = [], [], [], [], []
    g = torch.Generator()
    g.manual_seed(11)
    kept = None
    for mi, (name, N, K) in enumerate(shapes):
        codes, scales = synth_nvfp4(N, K, 77 + mi, dev)
        if mi == 0:
            idx = sample_rows(N, 96)
            kept = (idx, codes[idx].copy(), scales[idx].copy())
        ws.append(h.load(qg.pack(qg.FMT_NVFP4, codes, scales, 1.0)))
        xh.append(torch.randn((M, K), generator=g).to(torch.bfloat16).pin_memory())
        xs.append(xh[-1].to(dev))
        ys.append(torch.empty((M, N), dtype=torch.bfloat16, device=dev))
        yh.append(torch.empty((M, N), dtype=torch.bfloat16).pin_memory())
    flops = sum(2.0 * M * w.N * w.K for w in ws)
    wbytes = sum(w.weight_bytes for w in ws)
    stream = torch.cuda.Stream(device=dev)

    def dev_step():
        for w, x, y in zip(ws, xs, ys):
            h.gemm_skinny(w, x.data_ptr(), M, y.data_ptr(), qg.OUT_BF16, stream=stream.cuda_stream)

    def host_step():
        with torch.cuda.stream(stream):
            for x, xp in zip(xs, xh):
                x.copy_(xp, non_blocking=True)
        dev_step()
        with torch.cuda.stream(stream):
            for y, yp in zip(ys, yh):
                yp.copy_(y, non_blocking=True)
        stream.synchronize()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        dev_step()
    sampler = ClockSampler(0).start()
    ms = timed(stream, dev_step, args.steps)
    clocks = sampler.stop()
    host_step()
    ms_host = timed(stream, host_step, args.steps)
    st = h.device_status(stream.cuda_stream)
    if st.code != 0:
        raise SystemExit(f"kernel reported {st}")
    idx, codes, scales = kept
    err = O.rel_l2(yh[0].float().numpy()[:, idx], O.gemv_nvfp4_f64(codes, scales, 1.0, u16(xh[0])))
    tf = flops * args.steps / (ms * 1e-3) / 1e12
    tf_host = flops * args.steps / (ms_host * 1e-3) / 1e12
    peak, kind = measured_peak_tflops()
    act_bytes = sum(x.numel() * 2 for x in xh) + sum(y.numel() * 2 for y in yh)
    line = {
        "metric": "nvfp4_prefill_gemm_tflops", "value": round(tf, 1), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate in tensor memory)", "data": "synthetic",
        "config": {"workload": f"llama-3-70b-shaped layer (qkv, o, gate_up, down), NVFP4 weights, {M} tokens, "
                               "W4A16-exact tcgen05 skinny GEMM", "tokens": M, "flops_per_step": flops,
                   "weight_bytes_per_step": wbytes, "tokens_per_s_one_layer": round(M / (ms / args.steps * 1e-3), 1),
                   "cache": "weights per step (481 MB) exceed L2 (126 MB)"},
        "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": peak, "unit": "TFLOP/s",
                     "frac": round(tf / peak, 4), "traffic": round(0.956 * (wbytes + act_bytes) / 4),
                     "traffic_source": "ncu capture of the gate_up launch (DRAM read+write = 0.956 x weight+activation+result bytes), scaled by bytes to the average launch",
                     "peak_kind": kind + " bf16 burst",
                     "kernel": "gemm_skinny_kernel<NVFP4>", "flops_per_launch": flops / 4,
                     "us_per_launch": round(ms * 1e3 / (4 * args.steps), 2)},
        "e2e": {"value": round(tf_host, 1), "unit": "TFLOP/s",
                "h2d_bytes_per_step": sum(x.numel() * 2 for x in xh), "d2h_bytes_per_step": sum(y.numel() * 2 for y in yh),
                "ms_per_step": round(ms_host / args.steps, 5)},
        "gpu_launches": 8 * args.steps, "clocks": clocks,
        "verified": bool(err < TOL_BF16),
        "verify": {"rel_l2": float(f"{err:.3e}"), "tol": TOL_BF16, "checked": f"{len(idx)} sampled output rows of the qkv projection, all {M} tokens, fp64 oracle"},
    }
    for w in ws:
        w.unload()
    h.close()
    return line


def run_prefill_a4(args, M=None):
    """The block-scaled prefill: the same 70B-shaped layer with the activations quantised to NVFP4 by the
    library's stated quantiser and both operands consumed as stored by tcgen05 kind::mxf4nvf4
    (QGEMV_ACT_A4_BLOCKSCALED).  A different operator from the W4A16-exact GEMM: verified against an
    fp64 GEMM on the SAME quantised activations; the error against unquantised activations (FP4's own)
    is reported beside it."""
    import torch

    import crit_hub_b200 as qg
    from crit_hub_b200.stack import llama_layer_shapes, synth_nvfp4_dev
    from oracle import oracle as O

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    M = M or args.tokens
    model = LLAMA_70B
    h = qg.QGemv(device=0, use_pdl=True)
    shapes = llama_layer_shapes(model["hidden"], model["q_heads"], model["kv_heads"], model["head_dim"], model["inter"])
    ws, xs, ys, xh, yh = [], [], [], [], []
    g = torch.Generator()
    g.manual_seed(13)
    kept = None
    for mi, (name, N, K) in enumerate(shapes):
        codes, scales = synth_nvfp4_dev(N, K, 177 + mi, dev)
        if mi == 0:
            idx = sample_rows(N, 96)
            kept = (idx, codes[idx].cpu().numpy().copy(), scales[idx].cpu().numpy().copy())
        ws.append(h.load_device(qg.FMT_NVFP4_TC, codes.data_ptr(), scales.data_ptr(), N, K, 1.0))
        xh.append(torch.randn((M, K), generator=g).to(torch.bfloat16).pin_memory())
        xs.append(xh[-1].to(dev))
        ys.append(torch.empty((M, N), dtype=torch.bfloat16, device=dev))
        yh.append(torch.empty((M, N), dtype=torch.bfloat16).pin_memory())
        del codes, scales
    flops = sum(2.0 * M * w.N * w.K for w in ws)
    wbytes = sum(w.weight_bytes for w in ws)
    stream = torch.cuda.Stream(device=dev)

    def dev_step():
        for w, x, y in zip(ws, xs, ys):
            h.gemm_skinny(w, x.data_ptr(), M, y.data_ptr(), qg.OUT_BF16, qg.ACT_A4_BLOCKSCALED, stream=stream.cuda_stream)

    def host_step():
        with torch.cuda.stream(stream):
            for x, xp in zip(xs, xh):
                x.copy_(xp, non_blocking=True)
        dev_step()
        with torch.cuda.stream(stream):
            for y, yp in zip(ys, yh):
                yp.copy_(y, non_blocking=True)
        stream.synchronize()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        dev_step()
    sampler = ClockSampler(0).start()
    ms = timed(stream, dev_step, args.steps)
    clocks = sampler.stop()
    host_step()
    ms_host = timed(stream, host_step, args.steps)
    st = h.device_status(stream.cuda_stream)
    if st.code != 0:
        raise SystemExit(f"kernel reported {st}")
    idx, codes, scales = kept
    x0 = u16(xh[0])
    xc, xsc, xg = O.quantize_a4(x0)
    ref = O.gemm_nvfp4_a4_f64(codes, scales, 1.0, xc, xsc, xg)
    got = yh[0].float().numpy()[:, idx]
    err = O.rel_l2(got, ref)
    err_unq = O.rel_l2(got, O.gemv_nvfp4_f64(codes, scales, 1.0, x0))
    tf = flops * args.steps / (ms * 1e-3) / 1e12
    tf_host = flops * args.steps / (ms_host * 1e-3) / 1e12
    gbs = wbytes * args.steps / (ms * 1e-3) / 1e9
    peak, kind = measured_peak_gbs()
    line = {
        "metric": "nvfp4_a4_prefill_gemm_tflops", "value": round(tf, 1), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "e2m1 x ue4m3 block-scaled, both operands (tcgen05 kind::mxf4nvf4), fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"llama-3-70b-shaped layer (qkv, o, gate_up, down), NVFP4 weights and NVFP4-quantised activations, {M} tokens",
                   "tokens": M, "flops_per_step": flops, "weight_bytes_per_step": wbytes,
                   "launches_per_gemm": "zero-fill, activation quantiser, GEMM (+ chunk sum where row tiles are fewer than SMs)",
                   "cache": "weights per step (481 MB) exceed L2 (126 MB)"},
        "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": UNIT, "frac": round(gbs / peak, 4),
                     "traffic": None, "peak_kind": kind,
                     "note": "at the FP4 tensor rate this shape is bound by the weight stream, so the fraction is of HBM bandwidth; "
                             "no FP4 peak is in MEASURED_PEAKS.json (nominal dense 9 PFLOP/s)",
                     "kernel": "gemm_a4_kernel", "bytes_per_launch": wbytes // 4, "us_per_launch": round(ms * 1e3 / (4 * args.steps), 2)},
        "e2e": {"value": round(tf_host, 1), "unit": "TFLOP/s",
                "h2d_bytes_per_step": sum(x.numel() * 2 for x in xh), "d2h_bytes_per_step": sum(y.numel() * 2 for y in yh),
                "ms_per_step": round(ms_host / args.steps, 5)},
        "gpu_launches": 10 * args.steps, "clocks": clocks,
        "verified": bool(err < TOL_BF16),
        "verify": {"rel_l2_same_quantiser": float(f"{err:.3e}"), "tol": TOL_BF16, "rel_l2_vs_unquantised_activations": float(f"{err_unq:.3e}"),
                   "checked": f"{len(idx)} sampled output rows of the qkv projection, all {M} tokens, fp64 GEMM on the oracle's quantised activations"},
    }
    for w in ws:
        w.unload()
    h.close()
    return line


def run_lmhead(args, B=None):
    """The FP8-E4M3 output head (128256 x 4096, per-channel scales, fp32 logits) at decode batch B;
    two copies of the matrix alternate so every launch streams from HBM.  Verified on sampled rows."""
    import torch

    import crit_hub_b200 as qg
    from crit_hub_b200.stack import LayerStack, synth_fp8
    from oracle import oracle as O

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    N, K = 128256, 4096
    B = B or args.batch
    h = qg.QGemv(device=0, use_pdl=True)
    ws, kept = [], None
    for i in range(2):
        codes, scales = synth_fp8(N, K, 5 + i, dev)
        if i == 0:
            idx = sample_rows(N, 384)
            kept = (idx, codes[idx].copy(), scales[idx].copy())
        ws.append(h.load(qg.pack(qg.FMT_FP8, codes, scales)))
    stack = LayerStack(h, ws, B, qg.OUT_F32)
    g = torch.Generator()
    g.manual_seed(3)
    stack.set_inputs([torch.randn((B, K), generator=g).to(torch.bfloat16) for _ in ws])
    stack.capture()
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        stack.step()
    sampler = ClockSampler(0).start()
    ms = timed(stack.stream, stack.step, args.steps)
    clocks = sampler.stop()
    stack.step_host()
    ms_host = timed(stack.stream, stack.step_host, args.steps)
    st = h.device_status(stack.stream.cuda_stream)
    if st.code != 0:
        raise SystemExit(f"kernel reported {st}")
    idx, codes, scales = kept
    x0 = u16(stack.x_host[:B * K].view(B, K))
    err = O.rel_l2(stack.output(0, host=True).numpy()[:, idx], O.gemv_fp8_f64(codes, scales, x0))
    wbytes = sum(w.weight_bytes for w in ws)
    passes = 2 if B > 8 else 1      # batch 9..16 streams the matrix twice
    gbs = wbytes * args.steps / (ms * 1e-3) / 1e9
    peak, kind = measured_peak_gbs()
    line = {
        "metric": "fp8_lm_head_gemv_weight_gbps", "value": round(gbs, 2), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"FP8-E4M3 output head 128256 x 4096, per-channel scales, fp32 logits, batch {B}; two copies alternate",
                   "batch": B, "weight_bytes_per_step": wbytes, "us_per_launch": round(ms * 1e3 / (2 * passes * args.steps), 2),
                   "passes_over_the_matrix": passes,
                   "cache": "each copy (525 MB) exceeds L2 (126 MB)"},
        "roofline": {"bound": "hbm", "achieved": round(gbs * passes, 2), "peak": peak, "unit": UNIT, "frac": round(gbs * passes / peak, 4),
                     "traffic": int(1.0069 * (wbytes // 2)),
                     "traffic_source": "ncu capture of one launch: DRAM read+write 529.4 MB for 525.85 MB of weights",
                     "peak_kind": kind, "kernel": "gemv_stream_wp_kernel<FP8>",
                     "bytes_per_launch": wbytes // 2, "us_per_launch": round(ms * 1e3 / (2 * passes * args.steps), 2)},
        "e2e": {"value": round(wbytes * args.steps / (ms_host * 1e-3) / 1e9, 2), "unit": UNIT,
                "h2d_bytes_per_step": stack.h2d_bytes, "d2h_bytes_per_step": stack.d2h_bytes,
                "ms_per_step": round(ms_host / args.steps, 5)},
        "gpu_launches": 2 * passes * args.steps, "clocks": clocks,
        "verified": bool(err < TOL_F32),
        "verify": {"rel_l2": float(f"{err:.3e}"), "tol": TOL_F32, "checked": f"{len(idx)} sampled rows of the logits, fp64 oracle"},
    }
    for w in ws:
        w.unload()
    h.close()
    return line


def run_moe(args, T=None):
    """The grouped MoE GEMV -- 128 experts, top-8, hidden 2048, expert width 768 (gate/up 1536 x 2048
    and down 2048 x 768 per expert, NVFP4), T tokens per step, four layers of distinct experts in one
    CUDA graph.  value = bytes of the experts actually touched / device time.  Verified on sampled
    (token, expert) slots of the first layer."""
    import numpy as np
    import torch

    import crit_hub_b200 as qg
    from crit_hub_b200.stack import synth_nvfp4, synth_nvfp4_dev
    from oracle import oracle as O

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    E, topk, hidden, inter, L = 128, 8, 2048, 768, 4
    T = T or (args.tokens if args.tokens <= 512 and args.tokens != 256 else 8)
    tc = getattr(args, "moe_layout", "tc") == "tc"   # tensor-core layout: the expert list runs on the sequence kernel
    fmt = qg.FMT_NVFP4_TC if tc else qg.FMT_NVFP4
    one_launch = tc and not getattr(args, "moe_two_launches", False)
    h = qg.QGemv(device=0, use_pdl=True)
    host0 = {}

    def stacked(N, K, seed0, keep=None):
        """E seeded experts as one stacked weight: laid out on the device (tensor-core layout) or packed on the host."""
        if tc:
            mats = [synth_nvfp4_dev(N, K, seed0 + e, dev) for e in range(E)]
            if keep is not None:
                host0[keep] = [(c.cpu().numpy(), s.cpu().numpy()) for c, s in mats]
            return h.load_stacked_device(fmt, [c.data_ptr() for c, _ in mats], [s.data_ptr() for _, s in mats], N, K, [1.0] * E)
        blobs = []
        for e in range(E):
            c, s = synth_nvfp4(N, K, seed0 + e, dev)
            if keep is not None:
                host0.setdefault(keep, []).append((c, s))
            blobs.append(qg.pack(fmt, c, s, 1.0))
        return h.load_stacked(np.stack(blobs))

    gu = [stacked(2 * inter, hidden, 1000 * l, "gu" if l == 0 else None) for l in range(L)]
    dn = [stacked(hidden, inter, 1000 * l + 500, "dn" if l == 0 else None) for l in range(L)]
    per_expert = gu[0].weight_bytes + dn[0].weight_bytes
    g = torch.Generator(device=dev)
    g.manual_seed(T)
    ids = torch.topk(torch.randn(T, E, device=dev, generator=g), topk, dim=-1).indices.to(torch.int32).contiguous()
    distinct = int(torch.unique(ids).numel())
    x_host = torch.randn(T, hidden).to(torch.bfloat16).pin_memory()
    x = x_host.to(dev)
    hbufs = [torch.empty(T * topk, 2 * inter, device=dev, dtype=torch.bfloat16) for _ in range(L)]
    act = torch.randn(T * topk, inter, device=dev).to(torch.bfloat16)
    outs = [torch.empty(T * topk, hidden, device=dev, dtype=torch.float32) for _ in range(L)]
    out_host = torch.empty(T * topk, hidden, dtype=torch.float32).pin_memory()
    stream = torch.cuda.Stream()

    def layers(st):
        for l in range(L):
            if one_launch:   # both stages of the layer's expert MLP (gate/up, silu(gate) * up, down) as one launch
                h.moe_mlp(gu[l], dn[l], ids.data_ptr(), x.data_ptr(), T, topk, hbufs[l].data_ptr(), outs[l].data_ptr(), qg.OUT_F32, st)
                continue
            h.moe_gemv(gu[l], ids.data_ptr(), x.data_ptr(), T, topk, False, hbufs[l].data_ptr(), qg.OUT_BF16, st)
            if tc:   # the real data flow: the down stage reads the gate/up rows, silu(gate) * up applied inside the launch
                h.moe_gemv(dn[l], ids.data_ptr(), hbufs[l].data_ptr(), T, topk, True, outs[l].data_ptr(), qg.OUT_F32, st,
                           x_act=qg.MOE_X_SILU_MUL)
            else:    # (lane-order experts have no fused activation: a stand-in input for the down stage)
                h.moe_gemv(dn[l], ids.data_ptr(), act.data_ptr(), T, topk, True, outs[l].data_ptr(), qg.OUT_F32, st)

    with torch.cuda.stream(stream):
        layers(stream.cuda_stream)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        layers(torch.cuda.current_stream().cuda_stream)

    def dev_step():
        with torch.cuda.stream(stream):
            graph.replay()

    def host_step():
        with torch.cuda.stream(stream):
            x.copy_(x_host, non_blocking=True)
            graph.replay()
            out_host.copy_(outs[L - 1], non_blocking=True)
        stream.synchronize()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        dev_step()
    sampler = ClockSampler(0).start()
    ms = timed(stream, dev_step, args.steps)
    clocks = sampler.stop()
    host_step()
    ms_host = timed(stream, host_step, args.steps)
    st = h.device_status(stream.cuda_stream)
    if st.code != 0:
        raise SystemExit(f"kernel reported {st}")
    # sampled slots of layer 0: gate/up reads the token's row, down reads the slot's own row
    ids_h = ids.cpu().numpy()
    xs_h, act_h = u16(x_host), u16(act)
    hb, ob = hbufs[0].float().cpu().numpy(), outs[0].cpu().numpy()
    if tc:   # what the down stage multiplies: bf16(silu(gate) * up) of the gate/up rows the device produced (fp64 inside)
        v = hb.astype(np.float64)
        act_h = O.bf16_encode((v[:, :inter] / (1.0 + np.exp(-v[:, :inter])) * v[:, inter:]).astype(np.float32))
    # (the device's fast exponential rounds one bf16 product in several hundred the other way: an error of one bf16 ulp
    # in that share of the down stage's inputs, ~1.6e-4 at 64 tokens, well under the 2e-3 of bf16 results)
    tol_dn = 5e-4 if tc else TOL_F32
    rng = np.random.default_rng(T)
    slots = sorted(set(int(s) for s in rng.integers(0, T * topk, size=6)) | {0, T * topk - 1})
    err_gu = err_dn = 0.0
    for s in slots:
        t, e = s // topk, int(ids_h[s // topk, s % topk])
        c, sc = host0["gu"][e]
        err_gu = max(err_gu, O.rel_l2(hb[s], O.gemv_nvfp4_f64(c, sc, 1.0, xs_h[t:t + 1])[0]))
        c, sc = host0["dn"][e]
        err_dn = max(err_dn, O.rel_l2(ob[s], O.gemv_nvfp4_f64(c, sc, 1.0, act_h[s:s + 1])[0]))
    nbytes = distinct * per_expert * L
    gbs = nbytes * args.steps / (ms * 1e-3) / 1e9
    peak, kind = measured_peak_gbs()
    line = {
        "metric": "nvfp4_moe_gemv_touched_weight_gbps", "value": round(gbs, 2), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"MoE grouped GEMV: {E} experts, top-{topk}, hidden {hidden}, expert width {inter}, NVFP4, "
                               f"{T} tokens, {L} layers (gate/up + down) in one CUDA graph, {'tensor-core' if tc else 'lane-order'} layout"
                               + (", one launch per layer (gate/up, silu x up, down)" if one_launch else ""),
                   "tokens": T, "distinct_experts": distinct, "touched_weight_bytes_per_step": nbytes,
                   "us_per_layer": round(ms * 1e3 / args.steps / L, 2),
                   "cache": "four layers of distinct experts; at 1 token the touched experts (21 MB per layer) fit L2"},
        "roofline": {"bound": "hbm", "achieved": round(gbs, 2), "peak": peak, "unit": UNIT, "frac": round(gbs / peak, 4),
                     "traffic": int((1.04 if tc else 1.01) * (nbytes // ((1 if one_launch else 2) * L))),
                     "traffic_source": ("ncu capture at 8 tokens (profiles/moe_expert_list_128experts_t8_traffic.md): DRAM read+write = "
                                        "1.019-1.066 x the touched experts' bytes per launch; scaled by bytes") if tc else
                                       ("ncu capture at 8 tokens (profiles/moe_stream_128experts_t8_traffic.md): DRAM read+write = "
                                        "1.004-1.027 x the touched experts' bytes per launch; scaled by bytes"),
                     "peak_kind": kind, "kernel": "gemv_seq_kernel<4, expert list>" if tc else "moe_stream_kernel<NVFP4>",
                     "bytes_per_launch": nbytes // ((1 if one_launch else 2) * L),
                     "us_per_launch": round(ms * 1e3 / ((1 if one_launch else 2) * L * args.steps), 2)},
        "e2e": {"value": round(nbytes * args.steps / (ms_host * 1e-3) / 1e9, 2), "unit": UNIT,
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 4,
                "ms_per_step": round(ms_host / args.steps, 5)},
        "gpu_launches": (1 if one_launch else 2 if tc else 4) * L * args.steps, "clocks": clocks,
        "verified": bool(err_gu < TOL_BF16 and err_dn < tol_dn),
        "verify": {"rel_l2_gate_up_bf16": float(f"{err_gu:.3e}"), "rel_l2_down_f32": float(f"{err_dn:.3e}"),
                   "tol": [TOL_BF16, tol_dn], "checked": f"{len(slots)} sampled (token, expert) slots of layer 0, all rows, fp64 oracle"
                   + ("; the down stage reads the gate/up rows through silu(gate) * up inside its launch" if tc else "")},
    }
    for w in gu + dn:
        w.unload()
    h.close()
    return line


def brief(line):
    """The part of a secondary workload's line that goes under `secondary`."""
    keep = {k: line[k] for k in ("metric", "value", "unit", "ms_per_step", "verified", "verify") if k in line}
    keep["frac"] = line["roofline"]["frac"]
    keep["bound"] = line["roofline"]["bound"]
    keep["kernel"] = line["roofline"]["kernel"]
    keep["traffic"] = line["roofline"].get("traffic")
    keep["e2e"] = line["e2e"]["value"]
    keep["clocks"] = {k: line["clocks"].get(k) for k in ("sm_mhz", "reasons")}
    keep["workload"] = line["config"]["workload"]
    return keep


# ---- the headline --------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling small cases)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="N = 1: skip the secondary workloads")
    ap.add_argument("--no-tp1", action="store_true", help="N > 1: do not time the unsharded stack on rank 0")
    ap.add_argument("--moe-layout", default="tc", choices=["tc", "lane"],
                    help="MoE workload: tc = experts in the tensor-core layout (sequence kernel), lane = lane order (mma.sync streaming kernel)")
    ap.add_argument("--moe-two-launches", action="store_true",
                    help="MoE workload, tensor-core layout: gate/up and down as two launches per layer instead of one")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "prefill_a4", "lmhead", "moe"],
                    help="decode: the headline GEMV layer stack; prefill: the skinny GEMM over one 70B-shaped layer; "
                         "lmhead: the FP8 output head; moe: the grouped expert GEMV (--tokens 1/8/64)")
    ap.add_argument("--layout", default="tc", choices=["tc", "lane"],
                    help="stored form of the NVFP4 weights: tc = tile order consumed as stored by the block-scaled "
                         "tensor-core GEMV; lane = lane-ordered units for the CUDA-core GEMV")
    ap.add_argument("--no-fused", action="store_true", help="one launch per GEMV instead of one persistent launch per step")
    ap.add_argument("--no-prefetch", action="store_true", help="do not name the next matrix in each GEMV call (no L2 prefetch)")
    ap.add_argument("--exchange", default="fused", choices=["fused", "calls", "nccl"],
                    help="N > 1: fused = partial sums exchanged inside the persistent launch; calls = one launch per GEMV "
                         "plus qgemv_tp_allreduce, in a graph; nccl = one launch per GEMV plus an eager NCCL all-reduce")
    ap.add_argument("--tokens", type=int, default=256, help="rows of the prefill workload (16..256, multiple of 16)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload != "decode":
        if int(os.environ.get("WORLD_SIZE", "1")) != 1:
            raise SystemExit(f"--workload {args.workload} is a single-GPU workload")
        line = {"prefill": run_prefill, "prefill_a4": run_prefill_a4, "lmhead": run_lmhead, "moe": run_moe}[args.workload](args)
        print(json.dumps(line), flush=True)
        if not line["verified"]:
            raise SystemExit("verification against the oracle failed")
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    import crit_hub_b200 as qg
    from oracle import oracle as O

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        qg.set_host_threads(max(1, host_cores() // world))
    warmup = max(args.warmup, 3)
    model = dict(LLAMA_8B if world == 1 else LLAMA_70B)
    if args.layers > 0:
        model["layers"] = args.layers
    B = args.batch

    def note(msg):
        if os.environ.get("QGEMV_BENCH_VERBOSE"):
            print(f"[rank {rank}] {msg}", file=sys.stderr, flush=True)

    note("building the stack")
    fused = not args.no_fused and args.layout == "tc" and (world == 1 or args.exchange == "fused")
    want_tp1 = world > 1 and rank == 0 and not args.no_tp1 and args.layout == "tc"
    ds = DecodeStack(model, rank, world, local, args.layout, keep_full=want_tp1)
    handle = ds.handle
    hidden = model["hidden"]

    stack_ref = []
    flags = None
    after_call = None
    if world > 1:
        # exchange buffers: gather every rank's CUDA IPC handle.  Room for the all-reduce jobs of the
        # whole stack (B * hidden elements each) plus one stand-alone exchange.
        n_rowp = sum(ds.row_parallel)
        pool = (n_rowp + 8) * B * hidden + 4 * B * hidden + 4096
        mine = torch.from_numpy(handle.tp_create(rank, world, pool)).to(ds.device)
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        torch.cuda.synchronize()
        handle.tp_connect(torch.stack(gathered).cpu().numpy())
        dist.barrier()
        torch.cuda.synchronize()
        if fused:
            flags = [qg.JOB_ALLREDUCE if rp else 0 for rp in ds.row_parallel]
        elif args.exchange == "calls":
            def after_call(i):
                if ds.row_parallel[i]:
                    out = stack_ref[0].output(i)
                    handle.tp_allreduce(out.data_ptr(), qg.OUT_BF16, out.numel(), torch.cuda.current_stream().cuda_stream)
        else:
            def after_call(i):
                if ds.row_parallel[i]:
                    dist.all_reduce(stack_ref[0].output(i))

    # ---- N > 1: one layer against the UNSHARDED oracle before anything is timed ----
    verify = None
    if world > 1:
        note("verifying one tensor-parallel layer")
        from crit_hub_b200.stack import synth_nvfp4_dev
        g = torch.Generator()
        g.manual_seed(1234)
        attn = torch.randn((B, ds.shapes[1][2]), generator=g).to(torch.bfloat16)          # o's full input
        mlp = torch.randn((B, ds.shapes[3][2]), generator=g).to(torch.bfloat16)           # down's full input
        errs, got = [], {}
        same = True
        dist.barrier()
        torch.cuda.synchronize()
        for mi, xin in ((1, attn), (3, mlp)):
            name, N, K = ds.shapes[mi]
            k0, k1 = rank * K // world, (rank + 1) * K // world
            xd = xin[:, k0:k1].contiguous().to(ds.device)
            y = torch.zeros((B, N), dtype=torch.float32, device=ds.device)
            w = ds.weights[mi]
            if fused:
                seq = handle.sequence([(w, xd.data_ptr(), y.data_ptr(), qg.OUT_F32, qg.JOB_ALLREDUCE)], B)
                for _ in range(2):
                    seq.run()
                torch.cuda.synchronize()
                seq.destroy()
            else:
                handle.gemv(w, xd.data_ptr(), B, y.data_ptr(), qg.OUT_F32)
                if args.exchange == "calls":
                    handle.tp_allreduce(y.data_ptr(), qg.OUT_F32, y.numel())
                else:
                    dist.all_reduce(y)
                torch.cuda.synchronize()
            st = handle.device_status()
            if st.code != 0:
                raise SystemExit(f"kernel reported {st}")
            y0 = y.clone()
            dist.broadcast(y0, src=0)
            eq = torch.tensor([1 if torch.equal(y0.view(torch.int32), y.view(torch.int32)) else 0], device=ds.device)
            dist.all_reduce(eq, op=dist.ReduceOp.MIN)
            same = same and bool(eq.item())
            got[mi] = y.cpu().numpy()
        if rank == 0:   # (after the exchanges: the other ranks' kernels must not wait for this host work)
            for mi, xin in ((1, attn), (3, mlp)):
                name, N, K = ds.shapes[mi]
                codes, scales = synth_nvfp4_dev(N, K, mi, ds.device)       # layer 0's canonical matrix, unsharded
                idx = sample_rows(N)
                ref = O.gemv_nvfp4_f64(codes[idx].cpu().numpy(), scales[idx].cpu().numpy(), tensor_scale_for(K), u16(xin))
                errs.append(O.rel_l2(got[mi][:, idx], ref))
                del codes, scales
        ok_t = torch.tensor([1 if (rank != 0 or max(errs) < TOL_F32) else 0], device=ds.device)
        dist.all_reduce(ok_t, op=dist.ReduceOp.MIN)
        verify = {"ok": bool(ok_t.item()) and same, "rel_l2": [float(f"{e:.3e}") for e in errs], "tol": TOL_F32,
                  "same_bits_on_every_rank": same,
                  "checked": "o and down projections of layer 0, fp32 partial sums exchanged over the ranks, sampled rows of rank 0's "
                             "hidden vector against the unsharded fp64 oracle; every rank's bits against rank 0's"}
        if not verify["ok"]:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "verified": False, "verify": verify}), flush=True)
            raise SystemExit("tensor-parallel verification failed")

    # ---- the timed runner ----
    stack = ds.runner(B, fused=fused, prefetch_next=not args.no_prefetch, after_call=after_call, flags=flags)
    stack_ref.append(stack)
    eager = world > 1 and args.exchange == "nccl"
    note("capturing")
    if eager:
        stack.step()   # no graph: NCCL runs eagerly between the GEMVs, on the stack's stream
        torch.cuda.synchronize()
    else:
        stack.capture()
    st = handle.device_status(stack.stream.cuda_stream)
    if st.code != 0:
        raise SystemExit(f"kernel reported {st}")

    def barrier():
        # every NCCL operation of this process runs on the stack's stream: collectives of one
        # communicator must be issued in the same order on every rank
        torch.cuda.synchronize()
        if world > 1:
            with torch.cuda.stream(stack.stream):
                dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            with torch.cuda.stream(stack.stream):
                t = torch.tensor([ms], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            torch.cuda.synchronize()
            ms = float(t.item())
        return ms

    for _ in range(warmup):
        stack.step()
    note("warm-up done")
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = max_over_ranks(timed(stack.stream, stack.step, args.steps, barrier))
    clocks = sampler.stop() if rank == 0 else None
    for _ in range(2):
        stack.step_host()
    ms_host = max_over_ranks(timed(stack.stream, stack.step_host, args.steps, barrier))
    st = handle.device_status(stack.stream.cuda_stream)
    if st.code != 0:
        raise SystemExit(f"kernel reported {st}")

    extra = {}
    if world == 1:
        err = ds.verify(stack)            # the host copies of the last step_host()
        verify = {"ok": bool(err < TOL_BF16), "rel_l2": float(f"{err:.3e}"), "tol": TOL_BF16,
                  "checked": f"sampled rows (first, middle, last) of {len(ds.kept)} of the {len(stack.calls)} GEMVs of the timed stack, "
                             "bf16 outputs against the fp64 oracle"}
        if fused:
            # the same weights as a true chain: every GEMV reads the first K columns of the previous one's output
            chain = ds.runner(B, fused=True, chain=True)
            chain.capture()
            for _ in range(warmup):
                chain.step()
            ms_chain = timed(chain.stream, chain.step, args.steps)
            chain.step_host()
            extra["chained_gbs"] = round(ds.bytes * args.steps / (ms_chain * 1e-3) / 1e9, 2)
            extra["chained_us_per_layer"] = round(ms_chain * 1e3 / args.steps / model["layers"], 3)
            extra["chained_verify_rel_l2"] = float(f"{ds.verify(chain):.3e}")
            # ... and that chain with the element-wise work of a decoder layer folded into the jobs: RMS norm into
            # qkv and gate/up, residual added to o and down, SiLU(gate) * up into down (which then reads all 2 K
            # columns of gate/up's output)
            hid = model["hidden"]
            gnorm = torch.Generator()
            gnorm.manual_seed(99)
            norm_w = (1.0 + 0.1 * torch.randn(hid, generator=gnorm)).to(torch.bfloat16).to(ds.device)
            resid = torch.randn((B, hid), generator=gnorm).to(torch.bfloat16).to(ds.device)
            fl, op = [], []
            for i in range(len(ds.weights)):
                name = ds.shapes[i % 4][0]
                fl.append(qg.JOB_X_SILU_MUL if name == "down" else 0)
                op.append({"norm_weight": norm_w.data_ptr(), "norm_eps": 1e-5} if name in ("qkv", "gate_up") else {"residual": resid.data_ptr()})
            lay = ds.runner(B, fused=True, chain=True, flags=fl, opts=op)
            lay.capture()
            for _ in range(warmup):
                lay.step()
            ms_lay = timed(lay.stream, lay.step, args.steps)
            lay.step_host()
            extra["chained_fused_layer_gbs"] = round(ds.bytes * args.steps / (ms_lay * 1e-3) / 1e9, 2)
            extra["chained_fused_layer_verify_rel_l2"] = float(f"{ds.verify_fused(lay, fl, op, u16(norm_w), u16(resid)):.3e}")
            # ... and independent inputs with every job made to wait for the one before it all the same
            slow = ds.runner(B, fused=True, chained=True)
            slow.capture()
            for _ in range(warmup):
                slow.step()
            ms_slow = timed(slow.stream, slow.step, args.steps)
            extra["forced_order_gbs"] = round(ds.bytes * args.steps / (ms_slow * 1e-3) / 1e9, 2)
            # and one launch per GEMV (L2 prefetch of the next matrix), as a captured graph
            calls = ds.runner(B, fused=False, prefetch_next=True)
            calls.capture()
            for _ in range(warmup):
                calls.step()
            ms_calls = timed(calls.stream, calls.step, args.steps)
            extra["one_launch_per_gemv_gbs"] = round(ds.bytes * args.steps / (ms_calls * 1e-3) / 1e9, 2)
    total_bytes = float(ds.bytes)
    if world > 1:
        with torch.cuda.stream(stack.stream):
            t = torch.tensor([float(ds.bytes)], device="cuda", dtype=torch.float64)
            dist.all_reduce(t)
        torch.cuda.synchronize()
        total_bytes = float(t.item())

    # N > 1: the unsharded stack on rank 0's GPU (the same workload at TP = 1), the other ranks wait
    if want_tp1:
        note("timing the unsharded stack on rank 0")
        one = ds.runner(B, fused=True, weights=ds.full_weights)
        one.capture()
        for _ in range(warmup):
            one.step()
        ms_one = timed(one.stream, one.step, args.steps)
        one_bytes = sum(w.weight_bytes for w in ds.full_weights)
        extra["tp1_gbs"] = round(one_bytes * args.steps / (ms_one * 1e-3) / 1e9, 2)
        extra["tp1_us_per_layer"] = round(ms_one * 1e3 / args.steps / model["layers"], 3)
    if world > 1:
        barrier()

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        gbs = total_bytes * args.steps / (ms * 1e-3) / 1e9
        gbs_host = total_bytes * args.steps / (ms_host * 1e-3) / 1e9
        n_exchange = 0 if fused else sum(1 for rp in ds.row_parallel if rp)
        launches = (stack.launches_per_step + (n_exchange if args.exchange == "calls" else 0)) * args.steps
        per_launch_bytes = ds.bytes / stack.launches_per_step
        per_launch_us = ms * 1e3 / (stack.launches_per_step * args.steps)
        achieved = per_launch_bytes / (per_launch_us * 1e-6) / 1e9
        if fused:
            kernel = "gemv_seq_kernel<4>"
            order = ("every GEMV has an input buffer of its own, resident in HBM (the workload of the earlier records of this metric); "
                     "the job list orders jobs only where their buffers overlap, so here they may overlap in time.  "
                     "`chained_gbs`: the same weights with every GEMV reading the output of the one before it (its first K columns) -- a "
                     "decode step's data flow with the element-wise work left out, where each job waits for the last row of the one before; "
                     "`chained_fused_layer_gbs`: that chain with RMS norm (qkv, gate/up), SiLU x up (down) and residual adds (o, down) "
                     "folded into the jobs; `forced_order_gbs`: independent inputs, each job made to wait for the one before it")
            traffic, tsrc = int(per_launch_bytes * 1.032), ("ncu capture of a 2-layer launch of the same kernel (profiles/gemv_seq_llama8b_2layers.md): "
                                                             "DRAM read 1.001 x, read+write 1.032 x the algorithmic weight bytes; scaled by bytes")
        elif args.layout == "tc":
            kernel, order = "gemv_tc_kernel<4>", "stream order"
            traffic, tsrc = None, None
        else:
            kernel, order = "gemv_stream_wp_kernel<NVFP4>", "stream order"
            traffic, tsrc = int(per_launch_bytes * 1.002), "ncu capture of a 2-layer case: DRAM read+write = 1.002 x algorithmic bytes; scaled by bytes"
        exchange = {"fused": "fp32 partial sums of o and down pushed over NVLink and summed in rank order inside the persistent launch "
                             "(gemv_seq_kernel, FINISH warps)",
                    "calls": "qgemv_tp_allreduce (tp_exchange_kernel) after o and down, in the graph",
                    "nccl": "eager ncclAllReduce (torch.distributed) after o and down, no graph"}[args.exchange] if world > 1 else "none"
        line = {
            "metric": METRIC, "value": round(gbs, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True,
            "scaling": "weak" if world == 1 else "strong", "vs_baseline": None,
            "dtype": "e2m1 x ue4m3 block-scaled (tcgen05 kind::mxf4nvf4), fp32 accumulate" if args.layout == "tc" else "f16 (fp32 accumulate)",
            "data": "synthetic",
            "config": {
                "workload": f"{model['name']}-shaped decode layer stack, NVFP4 weights, batch {B}, "
                            f"{model['layers']} layers x (qkv, o, gate_up, down)",
                "batch": B, "layers": model["layers"], "tp": world, "exchange": exchange,
                "launch": "one persistent cooperative launch per step (qgemv_sequence_run), replayed from a CUDA graph" if fused
                          else ("one launch per GEMV, eager" if eager else "one launch per GEMV, replayed from a CUDA graph"),
                "order": order,
                "weight_bytes_per_step": int(total_bytes),
                "us_per_layer": round(ms * 1e3 / args.steps / model["layers"], 3),
                "cache": "weights per step exceed L2 (126 MB); every step streams from HBM",
                "pct_of_8TBps": round(gbs / world / 8000.0 * 100, 2),
                **extra,
            },
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "traffic": traffic, "traffic_source": tsrc,
                         "peak_kind": peak_kind, "kernel": kernel, "bytes_per_launch": int(per_launch_bytes),
                         "us_per_launch": round(per_launch_us, 3)},
            "e2e": {"value": round(gbs_host, 2), "unit": UNIT, "h2d_bytes_per_step": stack.h2d_bytes,
                    "d2h_bytes_per_step": stack.d2h_bytes, "ms_per_step": round(ms_host / args.steps, 5)},
            "gpu_launches": launches,
            "clocks": clocks,
            "verified": bool(verify["ok"]), "verify": verify,
        }
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_entry(LLAMA_8B if world == 1 else LLAMA_70B, B)
        if world == 1 and not args.no_secondary:
            sec = {}
            small = argparse.Namespace(**vars(args))
            small.steps, small.warmup = min(args.steps, 20), 3
            for b in (2, 4, 8):
                if b == B:
                    continue
                sb = ds.runner(b, fused=fused)
                sb.capture()
                for _ in range(3):
                    sb.step()
                msb = timed(sb.stream, sb.step, small.steps)
                sb.step_host()
                errb = ds.verify(sb)
                stb = handle.device_status(sb.stream.cuda_stream)
                v = ds.bytes * small.steps / (msb * 1e-3) / 1e9
                sec[f"decode_batch_{b}"] = {"metric": METRIC, "value": round(v, 2), "unit": UNIT, "frac": round(v / peak, 4),
                                            "us_per_layer": round(msb * 1e3 / small.steps / model["layers"], 3),
                                            "fused": bool(sb.fused), "verified": bool(errb < TOL_BF16 and stb.code == 0),
                                            "verify": {"rel_l2": float(f"{errb:.3e}"), "tol": TOL_BF16}}
                del sb
            for b in (1, 16):
                sec[f"lm_head_batch_{b}"] = brief(run_lmhead(small, b))
            for t in (1, 8, 64):
                sec[f"moe_tokens_{t}"] = brief(run_moe(small, t))
            for m in (128, 256):
                sec[f"prefill_tokens_{m}"] = brief(run_prefill(small, m))
            for m in (16, 128, 256):
                sec[f"prefill_a4_tokens_{m}"] = brief(run_prefill_a4(small, m))
            line["secondary"] = sec
            line["verified"] = bool(line["verified"] and all(s["verified"] for s in sec.values()))
        print(json.dumps(line), flush=True)
        if not line["verified"]:
            raise SystemExit("verification against the oracle failed")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
