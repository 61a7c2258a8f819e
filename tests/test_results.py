"""The result record in the registry's six-stat vocabulary (host logic only)."""
import json
import os
import sys

import pytest

from crit_hub_b200 import results as R

BENCH_LINE = {"metric": "nvfp4_decode_gemv_weight_gbps", "value": 2904.31, "ms_per_step": 1.35174,
              "config": {"layers": 32, "weight_bytes_per_step": 3925869056}, "roofline": {"peak": 6516.4}}


def test_stats_order_and_nulls():
    s = R.make_stats(R.figure(739.8), prefill_tok_s=None)
    assert list(s) == list(R.STATS)
    assert s["ppl"] is None and s["kld_mean"] is None and s["context_tokens"] is None
    assert s["decode_tok_s"] == 739.8 and s["prefill_tok_s"] is None and s["ttft_ms"] is None


def test_figures():
    assert R.figure([10.04, 10.04]) == 10.0
    assert R.figure([9.0, 11.26]) == [9.0, 11.3]
    assert R.is_figure(1.5) and R.is_figure([1, 2]) and not R.is_figure([2, 1]) and not R.is_figure(0)
    assert not R.is_figure(True) and not R.is_figure([1, 2, 3])


def test_headroom_matches_bytes_over_bandwidth():
    h = R.headroom(19257628032, 1392.5, 42.926346519608146)
    assert abs(h["pass_floor_ms"] - 13.82953539102334) < 1e-9            # the evaluator's own example
    assert abs(h["pass_efficiency"] - 0.32216893614988185) < 1e-12


def test_result_from_bench_line_round_trip():
    rec = R.from_bench_line(BENCH_LINE, batch=1)
    assert abs(rec["headroom"]["pass_efficiency"] - 2904.31 / 6516.4) < 2e-4
    tp = R.make_throughput({8: 5000.0, 1: rec["stats"]["decode_tok_s"], 4: [2700.0, 2750.5]})
    assert [t["concurrency"] for t in tp] == [1, 4, 8]
    result, blob = R.make_result("b200", "llama-3-8b@NVFP4", rec["stats"],
                                 settings="projection GEMVs only (4 per layer, 32 layers), batch 1, random-init weights",
                                 throughput=tp, measured_on="2026-01-01", hardware="1x NVIDIA B200")
    assert result["track"] == "open" and list(result["stats"]) == list(R.STATS)
    # the evidence file is the one the record points at, and it holds every stated figure verbatim
    import hashlib
    assert result["evidence"] == [{"file": R.SELF_REPORTED, "sha256": hashlib.sha256(blob).hexdigest()}]
    entry = json.loads(blob)["results"][0]
    assert (entry["gpu"], entry["model"]) == (result["gpu"], result["model"])
    recorded = [m["figures"] for m in entry["measurements"]]
    for key, value in result["stats"].items():
        assert value is None or any(f.get(key) == value for f in recorded), key
    for level in result["throughput"]:
        assert any(level in f.get("throughput", []) for f in recorded)
    with pytest.raises(ValueError):
        R.make_result("B200!", "llama", rec["stats"], settings="x")


def test_throughput_levels_are_sorted_and_unique():
    tp = R.make_throughput({4: 10.0, 1: 5.0, 2: [5.0, 6.0]})
    assert [t["concurrency"] for t in tp] == [1, 2, 4] and all(set(t) == set(R.THROUGHPUT) for t in tp)


# the registry checkout, when it sits next to this repository (or where CRIT_HUB_TOOLS points)
REF_TOOLS = os.environ.get("CRIT_HUB_TOOLS") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference", "tools")


@pytest.mark.skipif(not os.path.isdir(REF_TOOLS), reason="the registry's own checker is not on this machine")
def test_against_the_registrys_checker():
    """Where the registry's tools are present, its own functions accept the records built here."""
    sys.path.insert(0, REF_TOOLS)
    try:
        import check_engines as CE
    except Exception as e:  # missing optional dependency of the checker
        pytest.skip(f"cannot import the registry's checker: {e}")
    finally:
        sys.path.remove(REF_TOOLS)
    rec = R.from_bench_line(BENCH_LINE)
    tp = R.make_throughput({1: rec["stats"]["decode_tok_s"], 8: 4100.5})
    result, blob = R.make_result("b200", "llama-3-8b@NVFP4", rec["stats"], settings="projection GEMVs only", throughput=tp)
    assert CE.check_stats("r", result["stats"], {}) == []
    assert CE.check_throughput("r", result["throughput"]) == []
    assert CE.check_self_reported("r", result, json.loads(blob)) == []
    assert tuple(R.STATS) == tuple(CE.cardlib.STATS) and tuple(R.MORE) == tuple(CE.cardlib.MORE)
