"""The layout of an expert-list launch (tensor-core-layout MoE): host arithmetic, checked without a GPU."""
import pytest


def test_baseline_shape_plans(qg):
    # 128 experts, top-8, gate/up K = 2048 and down K = 768, as one launch
    for T, rows in ((1, 1), (3, 3), (8, 8), (64, 8)):
        p = qg.moe_plan(2048, 128, T, 8, K2=768)
        assert p.rows_per_problem == rows and p.plane_slots == 32 and p.stage_items == 4
        assert p.ring_stages >= 4 and p.plane_buffers in (1, 2)
        assert p.smem_bytes <= 227 * 1024 and p.table_offset % 128 == 0
        assert p.max_problems == min(128, T * 8) + (T * 8) // rows
    # few rows: two plane buffers and a deep ring; eight rows of K = 2048: still two buffers
    assert qg.moe_plan(2048, 128, 1, 8).plane_buffers == 2 and qg.moe_plan(2048, 128, 1, 8).ring_stages >= 10
    assert qg.moe_plan(2048, 128, 64, 8).plane_buffers == 2


def test_long_k_takes_fewer_rows(qg):
    assert qg.moe_plan(4096, 64, 64, 4).rows_per_problem == 8
    p = qg.moe_plan(7168, 64, 64, 4)
    assert p.rows_per_problem == 4 and p.plane_buffers == 1 and p.ring_stages >= 3
    p = qg.moe_plan(14336, 64, 64, 4)
    assert p.rows_per_problem == 2
    assert qg.moe_plan(21504, 16, 8, 2).rows_per_problem == 2      # (one row takes the same planes as two)
    with pytest.raises(qg.QgemvError) as e:
        qg.moe_plan(28672, 16, 8, 2)
    assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE


def test_refusals(qg):
    for kw in (dict(K=2048, n_experts=513, T=8, topk=2),          # more experts than the walk's tables hold
               dict(K=2048, n_experts=64, T=1024, topk=8),        # more than 4096 (token, choice) entries
               dict(K=2048, n_experts=256, T=512, topk=8, ctas=8)):   # too many problems per CTA for its table
        with pytest.raises(qg.QgemvError) as e:
            qg.moe_plan(**kw)
        assert e.value.status == qg.ERR_UNSUPPORTED_SHAPE
    with pytest.raises(qg.QgemvError) as e:
        qg.moe_plan(2000, 8, 1, 1)                                 # K not a multiple of 64
    assert e.value.status == qg.ERR_INVALID_ARG
