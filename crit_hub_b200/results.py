"""Results in the registry's vocabulary: the six headline stats, throughput levels, the headroom
block and the self-reported evidence file, built from measured layer-stack times.

The registry states a result as six stats in a fixed order (tools/card.py:34), optional `more`
figures (tools/card.py:36) and `throughput` levels (tools/card.py:39); a measurement that did not
come from its own evaluator is "self-reported": `track` must be `open`
(tools/check_engines.py:721-724), `measured_with` is free text, and an optional
`evidence/self-reported.json` must record every stated figure verbatim
(tools/check_engines.py:639-674).  The roofline block mirrors the evaluator's `headroom` object
(engines/crit-labs/mtp5-nvfp4-drafts/evidence/crit-eval.json:9582-9592).

A projection library measures projections only, so the mapping is: `decode_tok_s` = batch / layer-
stack GEMV time (an upper bound for a full model), `prefill_tok_s` = tokens / skinny-GEMM stack
time, `ttft_ms` = that stack time, `ppl` / `kld_mean` / `context_tokens` = null; the `settings`
text of the evidence says so.  Pure host code: nothing here touches the GPU.
"""
from __future__ import annotations

import datetime
import hashlib
import json
import re

STATS = ("decode_tok_s", "prefill_tok_s", "ttft_ms", "ppl", "kld_mean", "context_tokens")
MORE = ("greedy_decode_tok_s", "long_context_decode_tok_s", "heldout_decode_tok_s", "host_ram_gib",
        "quality_budget_pct")
THROUGHPUT = ("concurrency", "tok_s")
SELF_REPORTED = "evidence/self-reported.json"
_GPU = re.compile(r"[a-z0-9][a-z0-9.-]*")                       # tools/check_engines.py:44
_MODEL = re.compile(r"[a-z0-9][a-z0-9.-]*@[A-Za-z0-9.+-]+")     # tools/check_engines.py:45


def _positive(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0


def is_figure(v) -> bool:
    """A figure is a positive number or [low, high] with low <= high (tools/check_engines.py:90-96)."""
    if _positive(v):
        return True
    return isinstance(v, list) and len(v) == 2 and all(_positive(x) for x in v) and v[0] <= v[1]


def figure(values, digits: int = 1):
    """One measurement -> a number; several -> [low, high] across runs."""
    vals = [float(v) for v in (values if isinstance(values, (list, tuple)) else [values])]
    lo, hi = round(min(vals), digits), round(max(vals), digits)
    return lo if lo == hi else [lo, hi]


def make_stats(decode_tok_s, prefill_tok_s=None, ttft_ms=None) -> dict:
    """The six stats in the registry's order; what a projection library cannot measure is null."""
    return {"decode_tok_s": decode_tok_s, "prefill_tok_s": prefill_tok_s, "ttft_ms": ttft_ms,
            "ppl": None, "kld_mean": None, "context_tokens": None}


def make_throughput(levels: dict) -> list:
    """{batch: tok_s} -> ascending [{concurrency, tok_s}] (tools/check_engines.py:424-436)."""
    return [{"concurrency": int(c), "tok_s": levels[c]} for c in sorted(levels)]


def headroom(bytes_per_pass: int, bandwidth_gbs: float, step_ms: float) -> dict:
    """The evaluator's bytes-over-bandwidth floor: pass_floor_ms = bytes / bandwidth,
    pass_efficiency = floor / measured step."""
    floor_ms = bytes_per_pass / (bandwidth_gbs * 1e9) * 1e3
    return {"bytes_per_pass": int(bytes_per_pass), "bandwidth_gbs": float(bandwidth_gbs), "pass_floor_ms": floor_ms,
            "step_ms": float(step_ms), "pass_efficiency": floor_ms / step_ms}


def from_bench_line(line: dict, batch: int = 1) -> dict:
    """Stats and headroom from one JSON line of bench.py's decode workload."""
    layers = line["config"]["layers"]
    step_ms = line["ms_per_step"]
    stats = make_stats(figure(batch / (step_ms * 1e-3)))
    return {"stats": stats, "headroom": headroom(line["config"]["weight_bytes_per_step"], line["roofline"]["peak"], step_ms),
            "layers": layers}


def make_result(gpu: str, model: str, stats: dict, settings: str, method: str = "qgemv bench.py (CUDA events)",
                throughput: list | None = None, measured_on: str | None = None, hardware: str | None = None,
                quality_mode: str = "preserve"):
    """Returns (result, evidence_bytes): the `results[]` entry of a card and the bytes of its
    evidence/self-reported.json, whose sha256 the entry lists."""
    if not _GPU.fullmatch(gpu) or not _MODEL.fullmatch(model):
        raise ValueError("gpu / model do not match the registry's id patterns")
    figures = {k: v for k, v in stats.items() if v is not None}
    if throughput:
        figures["throughput"] = throughput
    evidence = {"results": [{"gpu": gpu, "model": model,
                             "measurements": [{"method": method, "settings": settings, "figures": figures}]}]}
    blob = (json.dumps(evidence, indent=1) + "\n").encode()
    result = {"gpu": gpu, "track": "open", "model": model, "measured_with": method,
              "measured_on": measured_on or datetime.date.today().isoformat(), "quality_mode": quality_mode}
    if hardware:
        result["hardware"] = hardware
    result["stats"] = {k: stats[k] for k in STATS}
    if throughput:
        result["throughput"] = throughput
    result["evidence"] = [{"file": SELF_REPORTED, "sha256": hashlib.sha256(blob).hexdigest()}]
    return result, blob
