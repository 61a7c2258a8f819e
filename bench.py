"""Benchmark of the NVFP4 decode GEMV path: weight GB/s over a Llama-shaped layer stack.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]
    python bench.py --workload prefill [--tokens M]      (secondary: tcgen05 skinny GEMM, one GPU)
    python bench.py --workload lmhead [--batch B]        (secondary: FP8 output head, one GPU)
    python bench.py --workload moe [--tokens T]          (secondary: grouped MoE GEMV, one GPU)

A "step" is one pass of the hot path over the whole layer stack (four weight-streaming GEMVs per
layer) at decode batch B, replayed as one CUDA graph.  `value` = algorithmic weight bytes of all
ranks / device time, inputs resident in HBM; `e2e` = the same metric with pinned host activations
copied in and results copied out inside the timed region.  One JSON line is printed by rank 0.

N = 1 runs the Llama-3-8B-shaped stack (32 layers, 3.9 GB of NVFP4 weights -- larger than L2, so
every replay streams from HBM).  N > 1 runs 16 layers of the Llama-3-70B-shaped stack tensor-parallel
(column-parallel QKV and gate/up, row-parallel o and down with an all-reduce of the partial
hidden vector), total work fixed: strong scaling.
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


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

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


def build_stack(model, batch, rank, world, dev_index, layout="tc", prefetch_next=True, fused=True):
    """The rank's share of the layer stack.  Tensor parallel: QKV and gate/up are column-parallel
    (this rank holds N/world output rows), o and down are row-parallel (K/world input columns; their
    outputs are partial sums that are all-reduced right after the GEMV, inside the captured graph).
    Each rank synthesises its own shard directly (seeded by layer, matrix and rank)."""
    import torch
    import torch.distributed as dist

    import crit_hub_b200 as qg
    from crit_hub_b200.stack import LayerStack, llama_layer_shapes, synth_nvfp4

    device = torch.device("cuda", dev_index)
    handle = qg.QGemv(device=dev_index, use_pdl=True)
    shapes = llama_layer_shapes(model["hidden"], model["q_heads"], model["kv_heads"], model["head_dim"],
                                model["inter"])
    weights, total_bytes, row_parallel = [], 0, []
    for layer in range(model["layers"]):
        for mi, (name, N, K) in enumerate(shapes):
            if world > 1:
                if name in ("qkv", "gate_up"):
                    N = N // world
                else:
                    K = K // world
            codes, scales = synth_nvfp4(N, K, (1000 * layer + mi) * 16 + rank, device)
            w = handle.load(qg.pack(qg.FMT_NVFP4_TC if layout == "tc" else qg.FMT_NVFP4, codes, scales, 1.0))
            weights.append(w)
            row_parallel.append(world > 1 and name in ("o", "down"))
            total_bytes += w.weight_bytes

    stack_ref = []
    if world > 1:
        # exchange buffers for the peer-memory all-reduce: gather every rank's CUDA IPC handle
        hidden_elems = batch * model["hidden"]
        mine = torch.from_numpy(handle.tp_create(rank, world, hidden_elems)).to(device)
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        torch.cuda.synchronize()
        handle.tp_connect(torch.stack(gathered).cpu().numpy())
        dist.barrier()
        torch.cuda.synchronize()

    def after_call(i):
        if row_parallel[i]:
            st = stack_ref[0]
            out = st.output(i)
            handle.tp_allreduce(out.data_ptr(), qg.OUT_BF16, out.numel(), torch.cuda.current_stream().cuda_stream)

    stack = LayerStack(handle, weights, batch, qg.OUT_BF16, device=dev_index,
                       after_call=after_call if world > 1 else None, prefetch_next=prefetch_next,
                       fused=fused and layout == "tc" and world == 1)
    stack_ref.append(stack)
    g = torch.Generator()
    g.manual_seed(7 + rank)
    stack.set_inputs([torch.randn((batch, w.K), generator=g).to(torch.bfloat16) for w in weights])
    return handle, stack, total_bytes


def cpu_reference_sample(model, batch, steps, warmup):
    """Times the CPU restatement (fp32-accumulate OpenMP GEMV) on one layer of the stack."""
    import numpy as np

    from crit_hub_b200.stack import llama_layer_shapes
    from oracle import oracle as O

    shapes = llama_layer_shapes(model["hidden"], model["q_heads"], model["kv_heads"], model["head_dim"],
                                model["inter"])
    mats = []
    for mi, (name, N, K) in enumerate(shapes):
        codes, scales, ts = O.make_nvfp4(N, K, seed=mi)
        mats.append((codes, scales, ts, O.make_x(batch, K, seed=mi)))
    layer_bytes = sum(m[1].shape[0] * m[1].shape[1] * 16 * 9 // 16 + 4 for m in mats)
    threads = O.num_threads()
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        for codes, scales, ts, x in mats:
            O.gemv_nvfp4_fast(codes, scales, ts, x)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return layer_bytes / sec / 1e9, sec, threads, layer_bytes


def run_reference(args):
    """The reference arm: the CPU restatement of the path on the host cores.  The registry holds
    no implementation of this arithmetic to install or compile, so the port is what runs."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    model = LLAMA_8B if args.gpus == 1 else LLAMA_70B
    steps, warmup = min(args.steps, 5), min(args.warmup, 2)
    gbs, sec, threads, layer_bytes = cpu_reference_sample(model, args.batch, max(steps, 1), warmup)
    sample = f"one {model['name']}-shaped layer (4 GEMVs, {layer_bytes} weight bytes) per step, {max(steps,1)} steps"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": max(steps, 1), "warmup": warmup, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
        "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{model['name']} layer stack, NVFP4, batch {args.batch} (CPU port, bounded sample)"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def measured_peak_tflops():
    """Measured dense bf16 burst peak of this pool's B200s (TFLOP/s), else the stated fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, "fallback"


def run_prefill(args):
    """Secondary workload: the tcgen05 skinny GEMM over the four projections of one
    Llama-3-70B-shaped layer (481 MB of NVFP4 weights, larger than L2) at --tokens rows.
    One step = the four GEMMs; value = 2*M*N*K flops of the layer / device time."""
    import numpy as np
    import torch

    import crit_hub_b200 as qg
    from crit_hub_b200.stack import llama_layer_shapes, synth_nvfp4

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise SystemExit("--workload prefill is a single-GPU workload")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    M = args.tokens
    model = LLAMA_70B
    h = qg.QGemv(device=0, use_pdl=True)
    shapes = llama_layer_shapes(model["hidden"], model["q_heads"], model["kv_heads"], model["head_dim"], model["inter"])
    ws, xs, ys, xh, yh = [], [], [], [], []
    g = torch.Generator()
    g.manual_seed(11)
    for mi, (name, N, K) in enumerate(shapes):
        codes, scales = synth_nvfp4(N, K, 77 + mi, dev)
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

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            e0.record()
        for _ in range(n):
            fn()
        with torch.cuda.stream(stream):
            e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        dev_step()
    sampler = ClockSampler(0)
    sampler.start()
    ms = timed(dev_step, args.steps)
    clocks = sampler.stop()
    host_step()
    ms_host = timed(host_step, args.steps)
    st = h.device_status(stream.cuda_stream)
    if st.code != 0:
        raise SystemExit(f"kernel reported {st}")
    tf = flops * args.steps / (ms * 1e-3) / 1e12
    tf_host = flops * args.steps / (ms_host * 1e-3) / 1e12
    peak, kind = measured_peak_tflops()
    line = {
        "metric": "nvfp4_prefill_gemm_tflops", "value": round(tf, 1), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate in tensor memory)", "data": "synthetic",
        "config": {"workload": f"llama-3-70b-shaped layer (qkv, o, gate_up, down), NVFP4 weights, {M} tokens, "
                               "W4A16-exact tcgen05 skinny GEMM", "tokens": M, "flops_per_step": flops,
                   "weight_bytes_per_step": wbytes, "tokens_per_s_one_layer": round(M / (ms / args.steps * 1e-3), 1),
                   "cache": "weights per step (481 MB) exceed L2 (126 MB)"},
        "roofline": {"bound": "tensor", "achieved": round(tf, 1), "peak": peak, "unit": "TFLOP/s",
                     "frac": round(tf / peak, 4), "traffic": round(0.956 * (wbytes + sum(x.numel() * 2 for x in xh) + sum(y.numel() * 2 for y in yh)) / 4),
                     "traffic_source": "ncu capture of the gate_up launch (DRAM read+write = 0.956 x weight+activation+result bytes), scaled by bytes to the average launch",
                     "peak_kind": kind + " bf16 burst",
                     "kernel": "gemm_skinny_kernel<NVFP4>", "flops_per_launch": flops / 4,
                     "us_per_launch": round(ms * 1e3 / (4 * args.steps), 2)},
        "e2e": {"value": round(tf_host, 1), "unit": "TFLOP/s",
                "h2d_bytes_per_step": sum(x.numel() * 2 for x in xh), "d2h_bytes_per_step": sum(y.numel() * 2 for y in yh),
                "ms_per_step": round(ms_host / args.steps, 5)},
        "gpu_launches": 8 * args.steps, "clocks": clocks,
    }
    if not args.no_cpu_baseline:
        from oracle import oracle as O
        codes, scales, ts = O.make_nvfp4(4096, 4096, seed=3)
        x = O.make_x(min(M, 128), 4096, seed=3)
        O.gemv_nvfp4_fast(codes, scales, ts, x)
        t0 = time.perf_counter()
        _, threads = O.gemv_nvfp4_fast(codes, scales, ts, x)
        sec = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": round(2.0 * x.shape[0] * 4096 * 4096 / sec / 1e12, 5), "unit": "TFLOP/s",
                                "cores": threads, "kind": "port",
                                "sample": f"4096x4096 NVFP4 matrix, {x.shape[0]} tokens, one pass of the fp32 OpenMP port"}
    print(json.dumps(line), flush=True)


def run_lmhead(args):
    """Secondary workload: the FP8-E4M3 output head (128256 x 4096, per-channel scales, fp32 logits)
    at decode batch --batch; two copies of the matrix alternate so every launch streams from HBM."""
    import torch

    import crit_hub_b200 as qg
    from crit_hub_b200.stack import LayerStack, synth_fp8

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise SystemExit("--workload lmhead is a single-GPU workload")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    N, K, B = 128256, 4096, args.batch
    h = qg.QGemv(device=0, use_pdl=True)
    ws = []
    for i in range(2):
        codes, scales = synth_fp8(N, K, 5 + i, dev)
        ws.append(h.load(qg.pack(qg.FMT_FP8, codes, scales)))
    stack = LayerStack(h, ws, B, qg.OUT_F32)
    g = torch.Generator()
    g.manual_seed(3)
    stack.set_inputs([torch.randn((B, K), generator=g).to(torch.bfloat16) for _ in ws])
    stack.capture()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        with torch.cuda.stream(stack.stream):
            e0.record()
        for _ in range(n):
            fn()
        with torch.cuda.stream(stack.stream):
            e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        stack.step()
    sampler = ClockSampler(0)
    sampler.start()
    ms = timed(stack.step, args.steps)
    clocks = sampler.stop()
    stack.step_host()
    ms_host = timed(stack.step_host, args.steps)
    st = h.device_status(stack.stream.cuda_stream)
    if st.code != 0:
        raise SystemExit(f"kernel reported {st}")
    wbytes = sum(w.weight_bytes for w in ws)
    gbs = wbytes * args.steps / (ms * 1e-3) / 1e9
    peak, kind = measured_peak_gbs()
    line = {
        "metric": "fp8_lm_head_gemv_weight_gbps", "value": round(gbs, 2), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"FP8-E4M3 output head 128256 x 4096, per-channel scales, fp32 logits, batch {B}; two copies alternate",
                   "batch": B, "weight_bytes_per_step": wbytes, "us_per_launch": round(ms * 1e3 / (2 * args.steps), 2),
                   "cache": "each copy (525 MB) exceeds L2 (126 MB)"},
        "roofline": {"bound": "hbm", "achieved": round(gbs, 2), "peak": peak, "unit": UNIT, "frac": round(gbs / peak, 4),
                     "traffic": int(1.0069 * (wbytes // 2)),
                     "traffic_source": "ncu capture of one launch: DRAM read+write 529.4 MB for 525.85 MB of weights",
                     "peak_kind": kind, "kernel": "gemv_stream_wp_kernel<FP8>",
                     "bytes_per_launch": wbytes // 2, "us_per_launch": round(ms * 1e3 / (2 * args.steps), 2)},
        "e2e": {"value": round(wbytes * args.steps / (ms_host * 1e-3) / 1e9, 2), "unit": UNIT,
                "h2d_bytes_per_step": stack.h2d_bytes, "d2h_bytes_per_step": stack.d2h_bytes,
                "ms_per_step": round(ms_host / args.steps, 5)},
        "gpu_launches": 2 * args.steps, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def run_moe(args):
    """Secondary workload: the grouped MoE GEMV -- 128 experts, top-8, hidden 2048, expert width 768
    (gate/up 1536 x 2048 and down 2048 x 768 per expert, NVFP4), --tokens tokens per step, four
    layers of distinct experts in one CUDA graph.  value = bytes of the experts actually touched /
    device time."""
    import numpy as np
    import torch

    import crit_hub_b200 as qg
    from crit_hub_b200.stack import synth_nvfp4

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise SystemExit("--workload moe is a single-GPU workload")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    E, topk, hidden, inter, L = 128, 8, 2048, 768, 4
    T = args.tokens if args.tokens <= 512 and args.tokens != 256 else 8
    h = qg.QGemv(device=0, use_pdl=True)

    def stacked(N, K, seed0):
        blobs = []
        for e in range(E):
            c, s = synth_nvfp4(N, K, seed0 + e, dev)
            blobs.append(qg.pack(qg.FMT_NVFP4, c, s, 1.0))
        return np.stack(blobs)

    gu = [h.load_stacked(stacked(2 * inter, hidden, 1000 * l)) for l in range(L)]
    dn = [h.load_stacked(stacked(hidden, inter, 1000 * l + 500)) for l in range(L)]
    per_expert = gu[0].weight_bytes + dn[0].weight_bytes
    g = torch.Generator(device=dev)
    g.manual_seed(T)
    ids = torch.topk(torch.randn(T, E, device=dev, generator=g), topk, dim=-1).indices.to(torch.int32).contiguous()
    distinct = int(torch.unique(ids).numel())
    x_host = torch.randn(T, hidden).to(torch.bfloat16).pin_memory()
    x = x_host.to(dev)
    hbuf = torch.empty(T * topk, 2 * inter, device=dev, dtype=torch.bfloat16)
    act = torch.randn(T * topk, inter, device=dev).to(torch.bfloat16)
    out = torch.empty(T * topk, hidden, device=dev, dtype=torch.float32)
    out_host = torch.empty(T * topk, hidden, dtype=torch.float32).pin_memory()
    stream = torch.cuda.Stream()

    def layers(st):
        for l in range(L):
            h.moe_gemv(gu[l], ids.data_ptr(), x.data_ptr(), T, topk, False, hbuf.data_ptr(), qg.OUT_BF16, st)
            h.moe_gemv(dn[l], ids.data_ptr(), act.data_ptr(), T, topk, True, out.data_ptr(), qg.OUT_F32, st)

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
            out_host.copy_(out, non_blocking=True)
        stream.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            e0.record()
        for _ in range(n):
            fn()
        with torch.cuda.stream(stream):
            e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        dev_step()
    sampler = ClockSampler(0)
    sampler.start()
    ms = timed(dev_step, args.steps)
    clocks = sampler.stop()
    host_step()
    ms_host = timed(host_step, args.steps)
    st = h.device_status(stream.cuda_stream)
    if st.code != 0:
        raise SystemExit(f"kernel reported {st}")
    nbytes = distinct * per_expert * L
    gbs = nbytes * args.steps / (ms * 1e-3) / 1e9
    peak, kind = measured_peak_gbs()
    line = {
        "metric": "nvfp4_moe_gemv_touched_weight_gbps", "value": round(gbs, 2), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"MoE grouped GEMV: {E} experts, top-{topk}, hidden {hidden}, expert width {inter}, NVFP4, "
                               f"{T} tokens, {L} layers (gate/up + down) in one CUDA graph",
                   "tokens": T, "distinct_experts": distinct, "touched_weight_bytes_per_step": nbytes,
                   "us_per_layer": round(ms * 1e3 / args.steps / L, 2),
                   "cache": "four layers of distinct experts; at 1 token the touched experts (21 MB per layer) fit L2"},
        "roofline": {"bound": "hbm", "achieved": round(gbs, 2), "peak": peak, "unit": UNIT, "frac": round(gbs / peak, 4),
                     "traffic": None, "peak_kind": kind, "kernel": "moe_stream_kernel<NVFP4>",
                     "bytes_per_launch": nbytes // (2 * L), "us_per_launch": round(ms * 1e3 / (2 * L * args.steps), 2)},
        "e2e": {"value": round(nbytes * args.steps / (ms_host * 1e-3) / 1e9, 2), "unit": UNIT,
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": out_host.numel() * 4,
                "ms_per_step": round(ms_host / args.steps, 5)},
        "gpu_launches": 4 * L * args.steps, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiling small cases)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "lmhead", "moe"],
                    help="decode: the headline GEMV layer stack; prefill: the skinny GEMM over one 70B-shaped layer; "
                         "lmhead: the FP8 output head; moe: the grouped expert GEMV (--tokens 1/8/64)")
    ap.add_argument("--layout", default="tc", choices=["tc", "lane"],
                    help="stored form of the NVFP4 weights: tc = tile order consumed as stored by the block-scaled "
                         "tensor-core GEMV; lane = lane-ordered units for the CUDA-core GEMV")
    ap.add_argument("--no-fused", action="store_true", help="one launch per GEMV instead of one persistent launch per step")
    ap.add_argument("--no-prefetch", action="store_true", help="do not name the next matrix in each GEMV call (no L2 prefetch)")
    ap.add_argument("--tokens", type=int, default=256, help="rows of the prefill workload (16..256, multiple of 16)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload == "prefill":
        run_prefill(args)
        return
    if args.workload == "lmhead":
        run_lmhead(args)
        return
    if args.workload == "moe":
        run_moe(args)
        return

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    warmup = max(args.warmup, 3)
    model = dict(LLAMA_8B if world == 1 else LLAMA_70B)
    if world > 1:
        # 16 of the 80 layers (7.7 GB of weights in all; >= 0.96 GB per GPU, well above L2): the
        # metric is a rate, and packing all 38.5 GB on the host would take minutes before the first
        # timed step
        model["layers"] = 16
    if args.layers > 0:
        model["layers"] = args.layers

    def note(msg):
        if os.environ.get("QGEMV_BENCH_VERBOSE"):
            print(f"[rank {rank}] {msg}", file=sys.stderr, flush=True)

    note("building the stack")
    handle, stack, rank_bytes = build_stack(model, args.batch, rank, world, local, args.layout,
                                            prefetch_next=not args.no_prefetch, fused=not args.no_fused)
    note("capturing")
    stack.capture()
    note("captured")
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

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with torch.cuda.stream(stack.stream):
            e0.record()
        for _ in range(n):
            fn()
        with torch.cuda.stream(stack.stream):
            e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            with torch.cuda.stream(stack.stream):
                t = torch.tensor([ms], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            torch.cuda.synchronize()
            ms = float(t.item())
        return ms

    def dev_step():
        stack.step()

    def host_step():
        stack.step_host()

    for _ in range(warmup):
        dev_step()
    note("warm-up done")
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(dev_step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    for _ in range(2):
        host_step()
    ms_host = timed(host_step, args.steps)
    st = handle.device_status(stack.stream.cuda_stream)
    if st.code != 0:
        raise SystemExit(f"kernel reported {st}")

    total_bytes = rank_bytes
    if world > 1:
        with torch.cuda.stream(stack.stream):
            t = torch.tensor([float(rank_bytes)], device="cuda", dtype=torch.float64)
            dist.all_reduce(t)
        torch.cuda.synchronize()
        total_bytes = float(t.item())
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        gbs = total_bytes * args.steps / (ms * 1e-3) / 1e9
        gbs_host = total_bytes * args.steps / (ms_host * 1e-3) / 1e9
        n_allreduce = sum(1 for i in range(stack.launches_per_step) if world > 1 and i % 4 in (1, 3))
        launches = (stack.launches_per_step + n_allreduce) * args.steps
        per_launch_bytes = rank_bytes / stack.launches_per_step
        per_launch_us = ms * 1e3 / (stack.launches_per_step * args.steps)
        achieved = per_launch_bytes / (per_launch_us * 1e-6) / 1e9
        line = {
            "metric": METRIC, "value": round(gbs, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": round(ms / args.steps, 5), "higher_is_better": True,
            "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)",
            "data": "synthetic",
            "config": {
                "workload": f"{model['name']}-shaped decode layer stack, NVFP4 weights, batch {args.batch}, "
                            f"{model['layers']} layers x (qkv, o, gate_up, down)",
                "batch": args.batch, "layers": model["layers"], "tp": world,
                "exchange": "none" if world == 1 else "peer-memory push all-reduce after o and down (tp_allreduce_kernel), in the graph",
                "weight_bytes_per_step": int(total_bytes),
                "us_per_layer": round(ms * 1e3 / args.steps / model["layers"], 3),
                "cache": "weights per step exceed L2 (126 MB); every replay streams from HBM",
                "pct_of_8TBps": round(gbs / world / 8000.0 * 100, 2),
            },
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "traffic": int(per_launch_bytes * 1.002),
                         "traffic_source": "ncu capture of a 2-layer case: DRAM read+write = 1.002 x algorithmic bytes for every shape; scaled by bytes",
                         "peak_kind": peak_kind,
                         "kernel": "gemv_stream_wp_kernel<NVFP4>", "bytes_per_launch": int(per_launch_bytes),
                         "us_per_launch": round(per_launch_us, 3)},
            "e2e": {"value": round(gbs_host, 2), "unit": UNIT, "h2d_bytes_per_step": stack.h2d_bytes,
                    "d2h_bytes_per_step": stack.d2h_bytes, "ms_per_step": round(ms_host / args.steps, 5)},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            cg, sec, threads, layer_bytes = cpu_reference_sample(LLAMA_8B, args.batch, 3, 1)
            line["cpu_baseline"] = {
                "value": round(cg, 3), "unit": UNIT, "cores": threads, "kind": "port",
                "sample": f"one llama-3-8b-shaped layer ({layer_bytes} weight bytes), 3 timed passes, fp32-accumulate "
                          f"OpenMP port of the host reference"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
