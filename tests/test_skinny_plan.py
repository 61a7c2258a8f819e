"""Host-side planning of the tcgen05 skinny GEMM: every supported shape must fit the SM's shared
and tensor memory, keep at least three packed stages (the parity waits rely on it) and two
activation stages.  No GPU involved."""
import pytest

SMEM_MAX = 227 * 1024


@pytest.mark.parametrize("fmt_name", ["NVFP4", "FP8"])
def test_every_token_count_fits(qg, fmt_name):
    fmt = getattr(qg, "FMT_" + fmt_name)
    for M in range(16, 257, 16):
        for K in (64, 128, 192, 256, 4096, 8192, 28672):
            p = qg.gemm_skinny_plan(fmt, 8192, K, M)
            units = K // 64
            assert p.run_units in (1, 2, 4) and units % p.run_units == 0
            assert p.x_stage_units <= p.run_units and p.run_units % p.x_stage_units == 0
            assert p.smem_bytes <= SMEM_MAX, (M, K, p.smem_bytes)
            assert p.p_stages >= 3 and p.p_stages <= 10
            assert 2 <= p.x_stages <= 16
            assert p.x_stage_units * M * 128 <= 32768 or p.x_stage_units == 1
            assert p.a_stages in (2, 3)
            assert p.tmem_columns in (32, 64, 128, 256, 512)
            assert M + p.a_stages * 32 * p.run_units <= p.tmem_columns
            assert 1 <= p.ctas <= 148


def test_cta_count_and_scratch(qg):
    p = qg.gemm_skinny_plan(qg.FMT_NVFP4, 128, 64, 16)      # one tile, one unit: one CTA
    assert p.ctas == 1 and p.run_units == 1
    p = qg.gemm_skinny_plan(qg.FMT_NVFP4, 57344, 8192, 256)
    assert p.ctas == 148 and p.run_units == 4 and p.a_stages == 2 and p.tmem_columns == 512
    assert qg.gemm_skinny_plan(qg.FMT_NVFP4, 8192, 8192, 256).ctas == 128    # 64 tiles x 2 K parts
    assert qg.gemm_skinny_plan(qg.FMT_NVFP4, 10240, 8192, 256).ctas == 80   # 80 tiles, one CTA each
    assert p.scratch_bytes >= 256 * 8192 * 2 + 2 * 148 * 256 * 128 * 4
    p = qg.gemm_skinny_plan(qg.FMT_NVFP4, 57344, 8192, 128)
    assert p.a_stages == 3 and p.tmem_columns == 512


def test_refused_shapes(qg):
    for args in [(qg.FMT_NVFP4, 100, 64, 16), (qg.FMT_NVFP4, 128, 96, 16), (qg.FMT_NVFP4, 128, 64, 8),
                 (qg.FMT_NVFP4, 128, 64, 272), (qg.FMT_NVFP4, 128, 64, 24), (7, 128, 64, 16)]:
        with pytest.raises(qg.QgemvError):
            qg.gemm_skinny_plan(*args)
