"""Parity of the CUDA kernels with the fp32 oracle and the reference's own outputs, on a B200.

Every case calls through the C ABI (ctypes -> rsfa_fwd).  Tolerance is the reference's:
atol = rtol = 1e-2 (flash_attention_forward.py:736-738), plus a separate finiteness check
because the reference's equal_nan=True would let NaN == NaN pass.
"""
import ctypes
import math

import pytest
import torch

from conftest import golden_cases, load_golden
from oracle.attention_ref import CONFIGS, attention_fp32, error_metrics, make_inputs

pytestmark = pytest.mark.gpu

ATOL = RTOL = 1e-2


@pytest.fixture(scope="module")
def fa(cuda_device):
    import ascend_rsfa.flash_attention_forward as mod

    mod.set_option("force_path", -1)
    yield mod
    mod.set_option("force_path", -1)


def check(fa, q, k, v, causal, scale, bm, bn, dev, lse=True, tol=ATOL):
    o, M = fa.attention_with_lse(q.to(dev), k.to(dev), v.to(dev), causal, scale, bm, bn)
    torch.cuda.synchronize()
    fa.device_status()
    ref, lse_ref = attention_fp32(q, k, v, causal, scale, return_lse=True)
    m = error_metrics(o, ref, tol, tol)
    assert m["finite"], m
    assert m["allclose"], m
    if lse:
        assert torch.allclose(M.cpu(), lse_ref, atol=2e-3, rtol=2e-3)
    return m


@pytest.mark.parametrize("name", golden_cases())
def test_matches_reference_outputs(fa, cuda_device, name):
    g = load_golden(name)
    o = fa.attention(g["q"].to(cuda_device), g["k"].to(cuda_device), g["v"].to(cuda_device),
                     g["causal"], g["sm_scale"], g["block_m"], g["block_n"])
    torch.cuda.synchronize()
    m = error_metrics(o, g["o"].float(), ATOL, RTOL)
    assert m["finite"] and m["allclose"], m


@pytest.mark.parametrize("causal", [False, True])
def test_cfg1(fa, cuda_device, causal):
    B, H, S, D, scale, mult = CONFIGS["cfg1"]
    q, k, v = make_inputs(B, H, S, D, seed=42, std=mult)
    m = check(fa, q, k, v, causal, scale, 64, 64, cuda_device)
    assert m["max_abs"] < 4e-3


# The reference's own fp16 test shapes (flash_attention_forward.py:671-697; the bf16 one is in test_bf16),
# N(0, 0.5), sm_scale 0.5, with batch reduced where the oracle would take too long.
REFERENCE_SHAPES = [
    (1, 2, 1024, 64, False, 64, 32), (1, 1, 64, 64, False, 64, 16), (4, 32, 64, 64, False, 64, 32),
    (1, 1, 128, 128, False, 16, 16), (1, 1, 128, 128, False, 64, 64), (4, 32, 128, 128, False, 32, 64),
    (1, 2, 1024, 64, False, 128, 32), (1, 1, 64, 64, True, 64, 16), (4, 32, 64, 64, True, 64, 32),
    (1, 1, 128, 128, True, 16, 16), (1, 1, 128, 128, True, 64, 64), (1, 2, 1024, 64, True, 64, 32),
    (1, 1, 128, 128, True, 32, 32), (1, 2, 1024, 64, True, 128, 32), (2, 4, 2048, 128, False, 128, 128),
    (2, 4, 4096, 64, False, 128, 128), (4, 8, 1024, 128, False, 128, 128), (4, 8, 1024, 64, False, 128, 128),
    (2, 4, 2048, 64, True, 64, 64), (4, 8, 1024, 64, True, 64, 64), (4, 32, 512, 64, True, 64, 64),
    (4, 32, 256, 128, True, 64, 64), (4, 32, 64, 64, False, 64, 16), (4, 32, 64, 64, True, 64, 16),
]


@pytest.mark.parametrize("Z,H,N,D,causal,BM,BN", REFERENCE_SHAPES)
def test_reference_test_shapes(fa, cuda_device, Z, H, N, D, causal, BM, BN):
    q, k, v = make_inputs(Z, H, N, D, seed=20, std=0.5)
    m = check(fa, q, k, v, causal, 0.5, BM, BN, cuda_device)
    assert m["max_abs"] < 4e-3  # the reference records <= 9.8e-4 on its shapes


def test_bf16(fa, cuda_device):
    # the reference's one bf16 case is (128, 8, 1024, 64), non-causal, tile (128, 128) (:698); 16 of its heads here
    q, k, v = make_inputs(2, 8, 1024, 64, seed=20, std=0.5, dtype=torch.bfloat16)
    check(fa, q, k, v, False, 0.5, 128, 128, cuda_device, tol=2e-2)
    q, k, v = make_inputs(1, 2, 512, 128, seed=21, std=0.5, dtype=torch.bfloat16)
    check(fa, q, k, v, True, 0.5, 128, 128, cuda_device, tol=2e-2)
    q, k, v = make_inputs(1, 2, 100, 32, seed=22, std=0.5, dtype=torch.bfloat16)
    check(fa, q, k, v, True, 0.5, 64, 64, cuda_device, tol=2e-2)


@pytest.mark.parametrize("D", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("causal", [False, True])
def test_every_head_dim(fa, cuda_device, D, causal):
    q, k, v = make_inputs(1, 3, 384, D, seed=5)
    check(fa, q, k, v, causal, 1.0 / math.sqrt(D), 128, 128, cuda_device)


@pytest.mark.parametrize("D", [16, 32])
@pytest.mark.parametrize("variant", [0, 1, 2])
def test_small_head_dims_on_the_d64_kernels(fa, cuda_device, D, variant):
    # D = 16 and 32 run on the three D = 64 tcgen05 kernels (single-buffered S, double-buffered S,
    # separate P) with zero columns read past D: every kernel, ragged lengths, both masks, bf16.
    assert fa.select_path(300, D, True, 0.25)[0] == 1
    fa.set_option("tcgen05_variant", variant)
    try:
        for S in (129, 300, 1000, 2049):
            q, k, v = make_inputs(2, 2, S, D, seed=S + D)
            check(fa, q, k, v, False, 0.25, 128, 128, cuda_device)
            check(fa, q, k, v, True, 0.25, 128, 128, cuda_device)
        q, k, v = make_inputs(1, 3, 640, D, seed=23, std=0.5, dtype=torch.bfloat16)
        check(fa, q, k, v, True, 0.5, 128, 128, cuda_device, tol=2e-2)
    finally:
        fa.set_option("tcgen05_variant", -1)


@pytest.mark.parametrize("S", [1, 7, 63, 65, 127, 129, 255, 257, 300, 511, 640, 1000])
@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("causal", [False, True])
def test_ragged_sequence_lengths(fa, cuda_device, S, D, causal):
    q, k, v = make_inputs(1, 2, S, D, seed=S)
    check(fa, q, k, v, causal, 0.25, 128, 128, cuda_device)


@pytest.mark.parametrize("path", [0, 1])
@pytest.mark.parametrize("causal", [False, True])
def test_both_kernel_families_agree(fa, cuda_device, path, causal):
    fa.set_option("force_path", path)
    try:
        for S, D in [(128, 64), (128, 128), (96, 64), (768, 128), (1536, 64), (320, 256)]:
            q, k, v = make_inputs(2, 2, S, D, seed=9)
            check(fa, q, k, v, causal, 0.3, 128, 128, cuda_device)
    finally:
        fa.set_option("force_path", -1)


@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("causal", [False, True])
def test_both_tcgen05_variants(fa, cuda_device, variant, causal):
    """Single-buffered (128-key tiles), double-buffered (64-key tiles) and, at D = 64, separate-P kernels."""
    fa.set_option("tcgen05_variant", variant)
    assert fa.select_path(1024, 128, causal, 0.5)[2] == (64 if variant == 1 else 128)
    try:
        for B, H, S, D, scale in [(2, 2, 1024, 128, 0.5), (1, 3, 1536, 64, 0.125), (1, 2, 449, 128, 0.3),
                                  (1, 2, 191, 64, 0.3), (1, 1, 2048, 128, 2.0), (3, 5, 2304, 64, 0.125),
                                  (1, 2, 640, 64, 2.0)]:
            q, k, v = make_inputs(B, H, S, D, seed=S + D)
            check(fa, q, k, v, causal, scale, 128, 128, cuda_device)
    finally:
        fa.set_option("tcgen05_variant", -1)


@pytest.mark.parametrize("causal", [False, True])
def test_short_sequences_on_both_kernel_families(fa, cuda_device, causal):
    # Sequences of at most 128 keys run on the tcgen05 kernel, whatever the batch (one work item is a
    # single, partly empty pair of Q tiles; HBM-bound for large batches), except D = 16 and S <= 64 at
    # D <= 64, which stay on the short-sequence kernel.  The launch counter shows one launch either
    # way (a single key tile does not use the D = 64 two-launch scheme).
    for B, H, S, D, scale in [(40, 8, 128, 128, 0.3), (33, 8, 96, 64, 0.25), (32, 8, 128, 256, 0.0625),
                              (64, 4, 77, 128, 0.3), (64, 4, 64, 64, 0.25), (2, 4, 128, 128, 0.3),
                              (64, 4, 128, 32, 0.3), (33, 8, 100, 16, 0.5), (64, 4, 64, 32, 0.3), (1, 1, 128, 128, 0.3),
                              (1, 2, 17, 256, 0.3), (1, 3, 65, 64, 0.3)]:
        q, k, v = make_inputs(B, H, S, D, seed=S + D + B)
        n0 = fa.launch_count()
        check(fa, q, k, v, causal, scale, 128, 128, cuda_device)
        assert fa.launch_count() - n0 == 1, (B, H, S, D)
        on_tcgen05 = D >= 32 and not (S <= 64 and D <= 64)
        assert fa.select_path(S, D, causal, scale)[0] == (1 if on_tcgen05 else 0)
        assert fa.work_items(B, H, S, D, causal, scale) == B * H * (1 if on_tcgen05 else -(-S // 64))


def test_separate_p_kernel_repeats_items_whose_sum_check_failed(fa, cuda_device):
    # D = 64 with 128-key tiles: the fast loop of the separate-P kernel cannot repair a key tile; a work
    # item whose sum check failed is run again by the same CTA with the loop that can.  Near one-hot rows
    # with a growing maximum (sm_scale 3) fail in many items; flat rows in none.  Both must match the
    # oracle, and each call is one launch.
    q, k, v = make_inputs(2, 3, 1024, 64, seed=31)
    n0 = fa.launch_count()
    check(fa, q, k, v, False, 3.0, 128, 128, cuda_device)
    check(fa, q, k, v, True, 3.0, 128, 128, cuda_device)
    check(fa, q, k, v, False, 0.125, 128, 128, cuda_device)
    assert fa.launch_count() - n0 == 3


@pytest.mark.parametrize("shape", [(1, 1, 256, 64), (1, 1, 300, 64), (1, 2, 129, 32), (1, 1, 777, 64), (3, 1, 513, 16)])
def test_separate_p_kernel_repeats_on_the_smallest_grids(fa, cuda_device, shape):
    # One to nine work items, each on a CTA of its own: the item that fails is the CTA's first and last,
    # so the repeat is found by the look at the other ring slot that precedes the CTA's exit.
    B, H, S, D = shape
    q, k, v = make_inputs(B, H, S, D, seed=S + D)
    fa.set_option("tcgen05_variant", 2)     # the separate-P kernel also where a single key tile would not take it
    try:
        for causal in (False, True):
            check(fa, q, k, v, causal, 3.0 * (64.0 / D) ** 0.5, 128, 128, cuda_device)
    finally:
        fa.set_option("tcgen05_variant", -1)


def test_separate_p_kernel_gives_up_on_the_fast_loop_for_one_hot_rows(fa, cuda_device):
    # 512 work items, more than three per CTA: a CTA that has had to repeat more than one item in four
    # runs the rest of its items with the repairing loop at once.  Every item must still come out
    # right, whichever loop produced it; bf16 and a ragged length go through the same paths.
    q, k, v = make_inputs(4, 64, 512, 64, seed=37)
    check(fa, q, k, v, False, 3.0, 128, 128, cuda_device)
    check(fa, q, k, v, True, 3.0, 128, 128, cuda_device)
    q, k, v = make_inputs(2, 40, 1000, 64, seed=38, dtype=torch.bfloat16)
    check(fa, q, k, v, False, 3.0, 128, 128, cuda_device)
    check(fa, q, k, v, True, 3.0, 128, 128, cuda_device)


def test_repairing_loop_follows_a_maximum_that_keeps_growing(fa, cuda_device):
    # Keys sorted so that every row's largest scores come last, with a wide spread: the first attempt
    # fails early, and the repeat has to move its reference up again and again, in the first and in the
    # second half of a key tile, rescaling O each time.  D = 32 runs on the same kernel.
    for D in (64, 32):
        g = torch.Generator().manual_seed(5 + D)
        S = 2048
        k = torch.randn(1, 2, S, D, generator=g)
        ramp = torch.linspace(0.05, 3.0, S).view(1, 1, S, 1)
        k = (k.sign() * ramp).to(torch.float16)          # |k| grows with the key index
        q = (torch.randn(1, 2, S, D, generator=g).sign()).to(torch.float16)
        v = torch.randn(1, 2, S, D, generator=g).to(torch.float16)
        for causal in (False, True):
            check(fa, q, k, v, causal, 1.0, 128, 128, cuda_device)


def test_result_does_not_depend_on_requested_tile(fa, cuda_device):
    """Requests that resolve to the same instantiated tile are bit-identical; different tiles agree
    within the tolerance (the reference's results are tile-independent in the same sense)."""
    for D in (64, 128):
        q, k, v = [t.to(cuda_device) for t in make_inputs(1, 2, 512, D, seed=4)]
        outs = {}
        for bm, bn in [(16, 16), (64, 32), (128, 64), (128, 128), (128, 512), (256, 256)]:
            tile = fa.select_path(512, D, True, 0.5, bm, bn)[1:]
            o = fa.attention(q, k, v, True, 0.5, bm, bn)
            torch.cuda.synchronize()
            if tile in outs:
                assert torch.equal(o, outs[tile])
            outs[tile] = o
        assert set(outs) == {(128, 64), (128, 128)}      # both instantiated tiles were reached
        a, b = outs[(128, 64)].float(), outs[(128, 128)].float()
        assert torch.allclose(a, b, atol=ATOL, rtol=RTOL)


def test_wide_logits_online_softmax_stability(fa, cuda_device):
    # the cfg5 recipe: inputs x2 widen the logit range; also a huge-scale case that forces rescales
    q, k, v = make_inputs(1, 2, 2048, 64, seed=8, std=2.0)
    check(fa, q, k, v, True, 0.125, 128, 128, cuda_device)
    check(fa, q, k, v, False, 0.125, 128, 128, cuda_device)
    q, k, v = make_inputs(1, 1, 1024, 128, seed=8, std=1.0)
    check(fa, q, k, v, False, 3.0, 128, 128, cuda_device)   # near one-hot rows, max keeps growing
    # keys sorted so every tile raises the running max: exercises the in-TMEM rescale each step
    kn = k.float().norm(dim=-1)
    order = kn.argsort(dim=-1)
    k2 = torch.gather(k, 2, order[..., None].expand_as(k))
    q2 = k2.flip(2).contiguous()
    check(fa, q2, k2, v, False, 1.0, 128, 128, cuda_device)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("tile", [(128, 128), (128, 64)])
@pytest.mark.parametrize("D", [64, 128])
def test_sudden_growth_of_the_row_maximum(fa, cuda_device, causal, tile, D):
    # The kernels exponentiate a key tile against a reference fixed at the first tile and move
    # it only when a value might leave the 16-bit range of P.  Flat scores everywhere except a
    # few keys that beat everything before them by far more than that range: one in the second
    # half of a tile, one in the first half of a later tile, one in the last (diagonal) tile.
    B, H, S = 1, 2, 640
    g = torch.Generator().manual_seed(21)
    u = torch.ones(D) / math.sqrt(D)
    q = (0.3 * torch.randn(B, H, S, D, generator=g) + 2.0 * u).half()
    k = (0.3 * torch.randn(B, H, S, D, generator=g)).half()
    v = torch.randn(B, H, S, D, generator=g).half()
    for idx, c in ((128 + 70, 40.0), (256 + 10, 90.0), (512 + 100, 150.0)):
        k[:, :, idx, :] = (c * u).half()
    m = check(fa, q, k, v, causal, 0.5, tile[0], tile[1], cuda_device)
    assert m["max_abs"] < 4e-3, m
    # moderate growth (a few log2 units per tile) must stay on the fast path and stay exact too
    k2 = (0.3 * torch.randn(B, H, S, D, generator=g)).half()
    k2 *= torch.linspace(0.5, 3.0, S)[None, None, :, None].half()
    m = check(fa, q, k2, v, causal, 0.5, tile[0], tile[1], cuda_device)
    assert m["max_abs"] < 4e-3, m


@pytest.mark.parametrize("causal", [False, True])
def test_head_dim_256_shapes(fa, cuda_device, causal):
    # cfg3's per-head shape (S=1024, D=256, sm_scale=1/16) on a few heads, plus forced rescales
    q, k, v = make_inputs(2, 3, 1024, 256, seed=12)
    m = check(fa, q, k, v, causal, 1.0 / 16.0, 128, 64, cuda_device)
    assert m["max_abs"] < 4e-3
    q, k, v = make_inputs(1, 2, 704, 256, seed=13)
    check(fa, q, k, v, causal, 1.0, 64, 64, cuda_device)      # peaked rows: the running max keeps moving
    q, k, v = make_inputs(1, 1, 2048, 256, seed=14, std=0.5)
    check(fa, q, k, v, causal, 0.5, 64, 256, cuda_device)


# ---- the benchmark configurations' own per-head shapes (cfg4: S=4096, D=128, sm_scale=1/sqrt(128);
# cfg5: S=8192, D=64, inputs x 2.0, sm_scale=1/8), a few heads each, both masks.  The reference runs
# S=8192, D=64 among its paper shapes (flash_attention_forward.py:743-756,
# benchmarks/run_correctness_test.py:142-148).
_ORACLE_CACHE = {}


def _oracle(name, B, H, causal):
    key = (name, B, H, causal)
    if key not in _ORACLE_CACHE:
        _, _, S, D, scale, mult = CONFIGS[name]
        q, k, v = make_inputs(B, H, S, D, seed=42, std=mult)
        _ORACLE_CACHE[key] = (q, k, v) + attention_fp32(q, k, v, causal, scale, return_lse=True)
    return _ORACLE_CACHE[key]


def _check_config_shape(fa, dev, name, B, H, causal, bm, bn):
    _, _, S, D, scale, _ = CONFIGS[name]
    q, k, v, ref, lse_ref = _oracle(name, B, H, causal)
    o, M = fa.attention_with_lse(q.to(dev), k.to(dev), v.to(dev), causal, scale, bm, bn)
    torch.cuda.synchronize()
    fa.device_status()
    m = error_metrics(o, ref, ATOL, RTOL)
    # error relative to the magnitude of the output: with inputs x 2 (cfg5) rows are close to one-hot
    # and |O| reaches 8 and more, where one fp16 step of the OUTPUT is 2^-7 = 7.8e-3; the absolute
    # error then is a few 1e-3 although every element is within about one fp16 step of the oracle.
    scaled = float(((o.float().cpu() - ref).abs() / ref.abs().clamp_min(1.0)).max())
    print("%s S=%d D=%d causal=%s tile=(%d,%d): max_abs %.3e, max |err|/max(1,|ref|) %.3e, max |ref| %.2f"
          % (name, S, D, causal, bm, bn, m["max_abs"], scaled, float(ref.abs().max())))
    assert m["finite"] and m["allclose"], m
    assert scaled < 2e-3, (m, scaled)
    assert torch.allclose(M.cpu(), lse_ref, atol=2e-3, rtol=2e-3)
    return m


@pytest.mark.parametrize("causal", [False, True])
def test_cfg4_shape_long_sequence_d128(fa, cuda_device, causal):
    bm, bn = fa.get_tiling(16, 16, 4096, 128, causal)
    m = _check_config_shape(fa, cuda_device, "cfg4", 2, 4, causal, bm, bn)
    assert m["max_abs"] < 4e-3, m          # N(0,1) inputs: outputs of order 1
    _check_config_shape(fa, cuda_device, "cfg4", 2, 4, causal, 128, 64)   # the 64-key kernel at 64 key tiles per row


@pytest.mark.parametrize("variant", [-1, 0, 1, 2])
@pytest.mark.parametrize("causal", [False, True])
def test_cfg5_shape_very_long_small_head_wide_logits(fa, cuda_device, causal, variant):
    # 64 key tiles of 128 per row; variant -1 / 2 = separate-P kernel, 0 = 128-key kernel, 1 = 64-key
    # kernel: one launch each.  Inputs x 2.0 widen the logits (std 5.8 log2 units).
    fa.set_option("tcgen05_variant", variant)
    try:
        n0 = fa.launch_count()
        _check_config_shape(fa, cuda_device, "cfg5", 1, 4, causal, 128, 128)
        assert fa.launch_count() - n0 == 1
    finally:
        fa.set_option("tcgen05_variant", -1)


def test_more_heads_than_a_grid_dimension_on_the_short_sequence_kernel(fa, cuda_device):
    # 8192 x 16 = 131072 heads of S=64, D=64: the short-sequence kernel keeps its heads on grid.x
    # (gridDim.y would stop at 65535).  q = k = 0 gives uniform weights, v = 1 gives O = 1 everywhere.
    from ascend_rsfa import _capi

    B, H, S, D = 8192, 16, 64, 64
    assert fa.select_path(S, D, False, 0.5)[0] == _capi.RSFA_PATH_GENERIC
    items = ctypes.c_longlong(0)
    assert _capi.load().rsfa_work_items(B, H, S, D, 0, 0.5, ctypes.byref(items)) == 0 and items.value == B * H
    z = torch.zeros(B, H, S, D, dtype=torch.float16, device=cuda_device)
    v = torch.ones_like(z)
    v[-1, -1] = 3.0                      # the very last head is told apart
    for causal in (False, True):
        o = fa.attention(z, z, v, causal, 0.5, 64, 64)
        torch.cuda.synchronize()
        assert bool((o[:-1] == 1).all()) and bool((o[-1, :-1] == 1).all()) and bool((o[-1, -1] == 3).all())
    del z, v, o
    torch.cuda.empty_cache()


def test_bounded_wait_runs_out_and_is_reported(fa, cuda_device):
    """The wait-expired path on a healthy GPU: the producer leaves out one K/V tile load together
    with the barrier arrival that would announce it (the "test_drop_load" option), so nothing is in
    flight and no address is touched; the MMA warp's wait for that tile runs out after
    `wait_limit_ms`, every role of the CTA leaves, tensor memory is freed and the kernel returns by
    itself with (1 << 16) | tag in the status word."""
    from ascend_rsfa import _capi

    lib = _capi.load()
    q, k, v = [t.to(cuda_device) for t in make_inputs(1, 1, 256, 128, seed=3)]
    ref = attention_fp32(q.cpu(), k.cpu(), v.cpu(), False, 0.5)
    fa.device_status()                                   # clean before the experiment
    fa.set_option("wait_limit_ms", 1)
    fa.set_option("test_drop_load", 1)                   # load 0 = K_0, load 1 = V_0
    try:
        fa.attention(q, k, v, False, 0.5, 128, 128)      # returns normally: the launch is asynchronous
        torch.cuda.synchronize()
    finally:
        fa.set_option("test_drop_load", -1)
        fa.set_option("wait_limit_ms", 2000)
    raw = ctypes.c_int(0)
    rc = lib.rsfa_device_status(0, ctypes.byref(raw))
    assert rc == _capi.RSFA_ERR_DEVICE_STATUS
    assert (raw.value >> 16) == 1 and 1 <= (raw.value & 0xffff) <= 10, hex(raw.value)
    assert lib.rsfa_device_status(0, ctypes.byref(raw)) == _capi.RSFA_OK and raw.value == 0   # reading cleared it
    # the context is intact and the next ordinary calls are correct (the work queue was left clean)
    for _ in range(2):
        o = fa.attention(q, k, v, False, 0.5, 128, 128)
        torch.cuda.synchronize()
        m = error_metrics(o, ref)
        assert m["finite"] and m["allclose"], m
    fa.device_status()


def test_check_status_option_makes_the_next_call_fail(fa, cuda_device):
    """With "check_status" on, the status word travels to the host behind every call and the next
    call on the device refuses to launch once a non-zero word has arrived; device_status() raises
    with the word and clears it, after which calls work again."""
    q, k, v = [t.to(cuda_device) for t in make_inputs(1, 1, 256, 128, seed=4)]
    ref = attention_fp32(q.cpu(), k.cpu(), v.cpu(), True, 0.5)
    fa.device_status()
    fa.set_option("check_status", 1)
    fa.set_option("wait_limit_ms", 1)
    fa.set_option("test_drop_load", 1)
    try:
        fa.attention(q, k, v, True, 0.5, 128, 128)
        torch.cuda.synchronize()
        fa.set_option("test_drop_load", -1)
        fa.set_option("wait_limit_ms", 2000)
        with pytest.raises(RuntimeError, match="device status"):
            fa.attention(q, k, v, True, 0.5, 128, 128)
        with pytest.raises(RuntimeError, match="device status 0x1000"):
            fa.device_status()
        o = fa.attention(q, k, v, True, 0.5, 128, 128)
        torch.cuda.synchronize()
        m = error_metrics(o, ref)
        assert m["finite"] and m["allclose"], m
    finally:
        fa.set_option("test_drop_load", -1)
        fa.set_option("wait_limit_ms", 2000)
        fa.set_option("check_status", 0)
    fa.device_status()


def test_d64_calls_on_several_streams_keep_their_repeats_apart(fa, cuda_device):
    # Calls in flight at the same time on different streams, on data whose sum checks fail in many
    # work items (near one-hot rows, sm_scale 3): which items are repeated is known only inside each
    # CTA, so nothing is shared between the calls and every one must come out right.
    q, k, v = make_inputs(2, 3, 1024, 64, seed=31)
    ref = {c: attention_fp32(q, k, v, c, 3.0) for c in (False, True)}
    qd, kd, vd = [t.to(cuda_device) for t in (q, k, v)]
    streams = [torch.cuda.Stream(device=cuda_device) for _ in range(3)]
    torch.cuda.synchronize()
    outs = []
    for i in range(24):
        causal = bool(i & 1)
        with torch.cuda.stream(streams[i % 3]):
            outs.append((causal, fa.attention(qd, kd, vd, causal, 3.0, 128, 128)))
    torch.cuda.synchronize()
    fa.device_status()
    for causal, o in outs:
        m = error_metrics(o, ref[causal])
        assert m["finite"] and m["allclose"], m


def test_back_to_back_launches_of_mixed_shapes_on_two_streams(fa, cuda_device):
    """Sixty calls of different shapes, masks and kernel families issued without a synchronisation in
    between, alternating between two streams: every launch takes a work queue that the launch using it
    before must have left at zero, sets itself up under the tail of the launch in front of it on its
    stream (programmatic dependent launch) and must not touch memory before that launch is complete.
    All outputs are compared with the oracle at the end."""
    shapes = [(2, 3, 512, 128, 0.3), (1, 2, 300, 64, 0.25), (1, 2, 384, 256, 0.0625), (3, 4, 128, 128, 0.3),
              (2, 2, 64, 64, 0.5), (1, 5, 1024, 128, 0.2), (2, 2, 777, 64, 0.125), (1, 1, 130, 32, 0.3)]
    cases = []
    for i, (B, H, S, D, scale) in enumerate(shapes):
        q, k, v = make_inputs(B, H, S, D, seed=100 + i)
        for causal in (False, True):
            cases.append((q, k, v, causal, scale, attention_fp32(q, k, v, causal, scale)))
    dev = cuda_device
    on_dev = [tuple(t.to(dev) for t in c[:3]) for c in cases]
    streams = [torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)]
    torch.cuda.synchronize()
    outs = []
    for rep in range(4):
        for i, (c, d) in enumerate(zip(cases, on_dev)):
            if rep > 0 and i % 4 != rep:        # 16 + 3 x 4 = 28 calls per ... keep the total near sixty
                continue
            with torch.cuda.stream(streams[(i + rep) & 1]):
                outs.append((i, fa.attention(d[0], d[1], d[2], c[3], c[4], 128, 128)))
    for i, (c, d) in enumerate(zip(cases, on_dev)):  # and once more, all on one stream, back to back
        with torch.cuda.stream(streams[0]):
            outs.append((i, fa.attention(d[0], d[1], d[2], c[3], c[4], 128, 128)))
    torch.cuda.synchronize()
    fa.device_status()
    assert len(outs) >= 40
    for i, o in outs:
        m = error_metrics(o, cases[i][5])
        assert m["finite"] and m["allclose"], (i, m)


def test_strided_inputs_and_views(fa, cuda_device):
    B, H, S, D = 2, 3, 256, 64
    big = torch.randn(B, S, 3, H, D, generator=torch.Generator().manual_seed(1)).half()
    q, k, v = [big[:, :, i].permute(0, 2, 1, 3) for i in range(3)]   # [B,H,S,D] views, row stride 3*H*D
    dev = cuda_device
    bigd = big.to(dev)
    qd, kd, vd = [bigd[:, :, i].permute(0, 2, 1, 3) for i in range(3)]
    o = fa.attention(qd, kd, vd, True, 0.3, 128, 128)
    torch.cuda.synchronize()
    ref = attention_fp32(q.contiguous(), k.contiguous(), v.contiguous(), True, 0.3)
    m = error_metrics(o, ref)
    assert m["finite"] and m["allclose"], m
    assert o.shape == (B, H, S, D)
    # a batch of one whose (meaningless) batch stride is odd: PyTorch calls such a view contiguous and
    # passes it on unchanged; the tensor maps must not take that stride at face value
    base = torch.randn(1 * 2 * 300 * 128 + 3, generator=torch.Generator().manual_seed(2)).half().to(dev)
    for off in (0,):
        t = torch.as_strided(base, (1, 2, 300, 128), (2 * 300 * 128 + 3, 300 * 128, 128, 1), off)
        assert t.is_contiguous()
        o = fa.attention(t, t, t, False, 0.1, 128, 128)
        torch.cuda.synchronize()
        tc = t.cpu().contiguous()
        m = error_metrics(o, attention_fp32(tc, tc, tc, False, 0.1))
        assert m["finite"] and m["allclose"], m


def test_requires_grad_inputs_and_no_backward(fa, cuda_device):
    q, k, v = [t.to(cuda_device).requires_grad_() for t in make_inputs(1, 1, 256, 64, seed=2, std=0.5)]
    o = fa.attention(q, k, v, False, 0.5, 64, 64)
    assert o.shape == q.shape and o.dtype == q.dtype
    with pytest.raises(NotImplementedError):
        o.float().sum().backward()


def test_size_independent_properties_at_full_cfg2_heads(fa, cuda_device):
    """At benchmark configuration cfg2's per-head size (S=2048, D=128) on many heads: rows of P sum to one
    (V = ones -> O = ones), causal row 0 equals v[0], and a uniform shift of the logits
    (adding a constant vector to every key along q) leaves the output unchanged."""
    B, H, S, D = 4, 8, 2048, 128
    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(B, H, S, D, generator=g, device=dev).half()
    k = torch.randn(B, H, S, D, generator=g, device=dev).half()
    v = torch.randn(B, H, S, D, generator=g, device=dev).half()
    ones = torch.ones_like(v)
    for causal in (False, True):
        o = fa.attention(q, k, ones, causal, 0.5, 128, 128)
        assert torch.allclose(o.float(), torch.ones_like(o, dtype=torch.float32), atol=2e-3)
    o = fa.attention(q, k, v, True, 0.5, 128, 128)
    assert torch.allclose(o[:, :, 0].float(), v[:, :, 0].float(), atol=1e-3)
    # checksum of checksums against the oracle on a sample of heads
    sel = [(0, 0), (1, 3), (3, 7)]
    for b, h in sel:
        ref = attention_fp32(q[b:b + 1, h:h + 1].cpu(), k[b:b + 1, h:h + 1].cpu(), v[b:b + 1, h:h + 1].cpu(), True, 0.5)
        m = error_metrics(o[b:b + 1, h:h + 1], ref)
        assert m["finite"] and m["allclose"], m
    fa.device_status()


@pytest.mark.parametrize("name", ["cfg2", "cfg3", "cfg4", "cfg5"])
def test_full_size_configurations_through_size_independent_properties(fa, cuda_device, name):
    """Every benchmark configuration at its FULL size (all B x H heads in one launch, so every work item of
    the queue, the last partly filled wave included): with V = 1 every output element is the sum of a
    row of P and must be 1, whatever Q and K are; the log-sum-exp must be finite everywhere; and the two
    kernel families ((128,128) and (128,64) tiles, where both exist) must agree on random V within the
    tolerance.  The oracle cannot follow to these sizes; it checks the per-head shapes in the tests above."""
    B, H, S, D, scale, mult = CONFIGS[name]
    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(11)
    q = (torch.randn(B, H, S, D, generator=g, device=dev) * mult).half()
    k = (torch.randn(B, H, S, D, generator=g, device=dev) * mult).half()
    ones = torch.ones(B, H, S, D, dtype=torch.float16, device=dev)
    for causal in (False, True):
        bm, bn = fa.get_tiling(B, H, S, D, causal)
        o, lse = fa.attention_with_lse(q, k, ones, causal, scale, bm, bn)
        torch.cuda.synchronize()
        assert float((o.float() - 1.0).abs().max()) < 2e-3, (name, causal)
        assert bool(torch.isfinite(lse).all())
        del o, lse
    del ones
    v = (torch.randn(B, H, S, D, generator=g, device=dev) * mult).half()
    if D <= 128:
        for causal in (False, True):
            a = fa.attention(q, k, v, causal, scale, 128, 128)
            b = fa.attention(q, k, v, causal, scale, 128, 64)
            torch.cuda.synchronize()
            diff = (a.float() - b.float()).abs()
            assert bool((diff <= ATOL + RTOL * b.float().abs()).all()), (name, causal, float(diff.max()))
            del a, b, diff
    fa.device_status()
    del q, k, v
    torch.cuda.empty_cache()


def test_host_buffer_entry_point(fa, cuda_device):
    q, k, v = make_inputs(3, 5, 384, 64, seed=6)
    fa.set_option("host_slab_heads", 4)   # 15 heads -> slabs of 4,4,4,3: exercises the double buffer
    try:
        o = fa.attention_host(q.pin_memory(), k.pin_memory(), v.pin_memory(), True, 0.2, 128, 128, device=0)
    finally:
        fa.set_option("host_slab_heads", 0)
    m = error_metrics(o, attention_fp32(q, k, v, True, 0.2))
    assert m["finite"] and m["allclose"], m
    o2 = fa.attention_host(q, k, v, False, 0.2, 128, 128, device=0)   # pageable buffers
    m = error_metrics(o2, attention_fp32(q, k, v, False, 0.2))
    assert m["finite"] and m["allclose"], m


def test_host_buffer_entry_point_with_lse(fa, cuda_device):
    """rsfa_fwd_host through ctypes, with the log-sum-exp copied back as well."""
    from ascend_rsfa import _capi

    lib = _capi.load()
    B, H, S, D = 2, 3, 320, 128
    q, k, v = make_inputs(B, H, S, D, seed=16)
    o = torch.empty_like(q)
    lse = torch.empty(B, H, S, dtype=torch.float32)
    fa.set_option("host_slab_heads", 4)
    try:
        rc = lib.rsfa_fwd_host(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, H, S, D, 1,
                               0.2, 128, 128, _capi.RSFA_DTYPE_F16, 0)
    finally:
        fa.set_option("host_slab_heads", 0)
    assert rc == _capi.RSFA_OK, _capi.strerror(rc)
    ref, lse_ref = attention_fp32(q, k, v, True, 0.2, return_lse=True)
    m = error_metrics(o, ref)
    assert m["finite"] and m["allclose"], m
    assert torch.allclose(lse, lse_ref, atol=2e-3, rtol=2e-3)


def test_device_argument_errors(fa, cuda_device):
    q = torch.zeros(1, 1, 128, 64, dtype=torch.float16, device=cuda_device)
    with pytest.raises(ValueError):
        fa.attention(q, q, q, False, 0.5, 0, 64)
    with pytest.raises(ValueError):
        fa.attention(q, q, q.float(), False, 0.5, 64, 64)
    assert fa.get_num_compute_cores() >= 100


def test_empty_batch_heads_or_sequence_launch_nothing(fa, cuda_device):
    for shape in ((0, 4, 128, 64), (2, 0, 128, 64), (2, 4, 0, 128)):
        q = torch.zeros(shape, dtype=torch.float16, device=cuda_device)
        n0 = fa.launch_count()
        o = fa.attention(q, q, q, True, 0.5, 128, 128)
        o2, lse = fa.attention_with_lse(q, q, q, False, 0.5)
        assert o.shape == q.shape and o2.shape == q.shape and o.dtype == q.dtype
        assert lse.shape == q.shape[:3] and lse.dtype == torch.float32
        assert fa.launch_count() == n0
    h = torch.zeros(0, 2, 64, 64, dtype=torch.float16)
    assert fa.attention_host(h, h, h, False, 0.5).shape == h.shape


def test_launch_counter_counts_kernels(fa, cuda_device):
    q = torch.zeros(1, 1, 256, 128, dtype=torch.float16, device=cuda_device)
    n0 = fa.launch_count()
    fa.attention(q, q, q, False, 0.5, 128, 128)
    fa.attention(q, q, q, True, 0.5, 128, 128)
    torch.cuda.synchronize()
    assert fa.launch_count() - n0 == 2
