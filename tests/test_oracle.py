"""The oracle against the reference's own outputs (golden fixtures) and itself."""
import pytest
import torch

from conftest import golden_cases, load_golden
from oracle.attention_ref import (attention_flops, attention_fp32, attention_online,
                                  error_metrics, make_inputs)

ATOL = RTOL = 1e-2  # the reference's tolerance (flash_attention_forward.py:736-738)


@pytest.mark.parametrize("name", golden_cases())
def test_oracle_matches_reference_output(name):
    g = load_golden(name)
    ref = attention_fp32(g["q"], g["k"], g["v"], g["causal"], g["sm_scale"])
    m = error_metrics(g["o"], ref, ATOL, RTOL)
    assert m["finite"] and m["allclose"], m
    # the reference's recorded error magnitude is ~1e-3 (one fp16 ulp near 1)
    assert m["max_abs"] < 4e-3, m


@pytest.mark.parametrize("name", golden_cases())
def test_online_recurrence_matches_reference_output(name):
    g = load_golden(name)
    out = attention_online(g["q"], g["k"], g["v"], g["causal"], g["sm_scale"],
                           g["block_m"], g["block_n"])
    m = error_metrics(g["o"], out, ATOL, RTOL)
    assert m["finite"] and m["allclose"], m


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("bm,bn", [(16, 16), (64, 32), (32, 128), (128, 64), (48, 80)])
def test_result_independent_of_tiles(causal, bm, bn):
    q, k, v = make_inputs(1, 2, 200, 32, seed=3)
    ref, lse_ref = attention_fp32(q, k, v, causal, 0.3, return_lse=True)
    out, lse = attention_online(q, k, v, causal, 0.3, bm, bn, return_lse=True)
    assert error_metrics(out, ref, 2e-3, 2e-3)["allclose"]
    assert torch.allclose(lse, lse_ref, atol=1e-4, rtol=1e-4)


def test_causal_first_row_is_v0_and_rows_sum_to_one():
    q, k, v = make_inputs(1, 1, 64, 16, seed=5)
    out = attention_fp32(q, k, v, True, 0.5)
    assert torch.allclose(out[0, 0, 0], v[0, 0, 0].float(), atol=1e-6)
    ones = torch.ones_like(v)
    assert torch.allclose(attention_fp32(q, k, ones, False, 0.5), torch.ones(1, 1, 64, 16), atol=1e-5)


def test_chunking_does_not_change_result():
    q, k, v = make_inputs(2, 3, 96, 16, seed=9)
    a = attention_fp32(q, k, v, True, 0.25, heads_per_chunk=1)
    b = attention_fp32(q, k, v, True, 0.25, heads_per_chunk=6)
    assert torch.equal(a, b)


def test_flop_count():
    assert attention_flops(128, 8, 2048, 128, False) == pytest.approx(2.199e12, rel=1e-3)
    assert attention_flops(128, 8, 2048, 128, True) == pytest.approx(1.0995e12, rel=1e-3)
    assert attention_flops(1, 2, 128, 64, False) == 8388608
