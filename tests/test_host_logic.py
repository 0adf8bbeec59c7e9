"""Host-side logic that needs no GPU: tile table, path selection, argument errors, sharding."""
import ctypes

import pytest
import torch

import ascend_rsfa.flash_attention_forward as fa
from ascend_rsfa import _capi, sharding

lib = _capi.load()

CONFIG_SHAPES = [
    (1, 2, 128, 64), (128, 8, 2048, 128), (64, 8, 1024, 256), (16, 16, 4096, 128), (4, 32, 8192, 64),
]


@pytest.mark.parametrize("shape", CONFIG_SHAPES)
@pytest.mark.parametrize("causal", [False, True])
def test_get_tiling_covers_every_baseline_config(shape, causal):
    bm, bn = fa.get_tiling(*shape, causal)
    assert (bm, bn) in {(128, 128), (128, 64), (64, 64), (64, 32)}
    # keyed by (S, D, causal): batch and heads do not matter (the reference raises KeyError)
    assert fa.get_tiling(3, 5, shape[2], shape[3], causal) == (bm, bn)


def test_get_tiling_reference_listed_shapes_do_not_raise():
    # every tuple the reference's dict lists (flash_attention_forward.py:631-663) must resolve
    for z, h, n, d in [(1, 1, 64, 64), (1, 1, 128, 128), (1, 2, 256, 256), (2, 2, 128, 256), (1, 2, 1024, 64),
                       (4, 32, 64, 64), (4, 32, 128, 128), (4, 32, 256, 128), (4, 32, 512, 64),
                       (4, 32, 1024, 64), (4, 32, 1024, 128), (4, 32, 2048, 64), (4, 32, 2048, 128),
                       (4, 32, 4096, 64), (128, 8, 1024, 64), (128, 8, 1024, 128), (128, 8, 1024, 256),
                       (128, 8, 2048, 128), (128, 8, 2048, 256), (128, 8, 4096, 128), (128, 8, 8192, 64)]:
        for causal in (False, True):
            bm, bn = fa.get_tiling(z, h, n, d, causal)
            assert bm > 0 and bn > 0


def test_get_tiling_rejects_impossible_shapes():
    with pytest.raises(ValueError):
        fa.get_tiling(1, 1, 128, 48, False)   # head dim outside {16,32,64,128,256} (:554)
    with pytest.raises(ValueError):
        fa.get_tiling(1, 1, 0, 64, False)


def test_path_selection_follows_the_short_sequence_rule():
    # one key tile (the reference's N_CTX <= 128 rule, :564): the tcgen05 kernel takes it too, except the
    # smallest tiles (D = 16; S <= 64 at D <= 64), which stay on the short-sequence kernel
    assert fa.select_path(128, 64, False, 0.5) == (_capi.RSFA_PATH_TCGEN05, 128, 128)
    assert fa.select_path(64, 64, False, 0.5)[0] == _capi.RSFA_PATH_GENERIC
    assert fa.select_path(128, 16, True, 0.5)[0] == _capi.RSFA_PATH_GENERIC
    assert fa.select_path(64, 128, True, 0.5)[0] == _capi.RSFA_PATH_TCGEN05
    assert fa.select_path(2048, 128, True, 0.5)[0] == _capi.RSFA_PATH_TCGEN05
    assert fa.select_path(8192, 64, False, 0.125)[0] == _capi.RSFA_PATH_TCGEN05
    assert fa.select_path(2048, 32, False, 0.5)[0] == _capi.RSFA_PATH_TCGEN05    # D = 32: the D = 64 kernel
    assert fa.select_path(128, 32, False, 0.5)[0] == _capi.RSFA_PATH_TCGEN05
    assert fa.select_path(64, 32, False, 0.5)[0] == _capi.RSFA_PATH_GENERIC
    assert fa.select_path(2048, 128, False, -0.5)[0] == _capi.RSFA_PATH_GENERIC  # non-positive scale
    assert fa.select_path(2048, 128, False, 0.5) == (1, 128, 128)
    # an instantiated tile is honoured, anything else is replaced by the table's row
    assert fa.select_path(2048, 128, False, 0.5, 128, 64) == (1, 128, 64)
    assert fa.select_path(2048, 128, False, 0.5, 32, 512) == (1,) + fa.get_tiling(1, 1, 2048, 128, False)
    assert fa.select_path(1024, 256, True, 0.0625, 128, 128) == (1, 128, 64)   # D = 256 has one tile


def test_rsfa_fwd_argument_errors_need_no_device():
    st = (ctypes.c_int64 * 16)(*([64 * 128, 128 * 64, 64, 1] * 4))
    ok_ptr = ctypes.c_void_p(4096)
    f = lib.rsfa_fwd
    bad = _capi.RSFA_ERR_INVALID_ARGUMENT
    assert f(None, ok_ptr, ok_ptr, ok_ptr, None, 1, 1, 128, 64, st, 0, 0.5, 64, 64, 0, None) == bad
    assert f(ok_ptr, ok_ptr, ok_ptr, ok_ptr, None, 1, 1, 128, 48, st, 0, 0.5, 64, 64, 0, None) == bad
    assert f(ok_ptr, ok_ptr, ok_ptr, ok_ptr, None, 1, 1, 0, 64, st, 0, 0.5, 64, 64, 0, None) == bad
    assert f(ok_ptr, ok_ptr, ok_ptr, ok_ptr, None, 1, 1, 128, 64, st, 0, 0.5, 0, 64, 0, None) == bad
    assert f(ok_ptr, ok_ptr, ok_ptr, ok_ptr, None, 1, 1, 128, 64, st, 0, 0.5, 64, 64, 7, None) == bad
    assert f(ctypes.c_void_p(4100), ok_ptr, ok_ptr, ok_ptr, None, 1, 1, 128, 64, st, 0, 0.5, 64, 64, 0, None) == bad
    st_bad = (ctypes.c_int64 * 16)(*([64 * 128, 128 * 64, 60, 1] * 4))
    assert f(ok_ptr, ok_ptr, ok_ptr, ok_ptr, None, 1, 1, 128, 64, st_bad, 0, 0.5, 64, 64, 0, None) == bad
    assert f(ok_ptr, ok_ptr, ok_ptr, ok_ptr, None, 1, 1, 128, 64, st, 0, float("nan"), 64, 64, 0, None) == bad


def test_attention_rejects_cpu_tensors_and_bad_shapes():
    q = torch.zeros(1, 1, 64, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fa.attention(q, q, q, False, 0.5, 64, 64)
    with pytest.raises(AssertionError):
        fa.attention(torch.zeros(1, 1, 64, 48, dtype=torch.float16), q, q, False, 0.5, 64, 64)
    with pytest.raises(TypeError):
        fa.attention(q, q, q, causal=False, sm_scale=0.5, BM=64, BN=64)   # positional only, like Function.apply


def test_options_round_trip():
    fa.set_option("wait_limit_ms", 1500)
    assert lib.rsfa_get_option(b"wait_limit_ms") == 1500
    fa.set_option("wait_limit_ms", 2000)
    with pytest.raises(ValueError):
        fa.set_option("no_such_option", 1)
    with pytest.raises(ValueError):
        fa.set_option("force_path", 5)
    # -1 automatic, 0 single-buffered 128-key kernel, 1 double-buffered 64-key kernel, 2 separate-P kernel
    for variant in (0, 1, 2, -1):
        fa.set_option("tcgen05_variant", variant)
        assert lib.rsfa_get_option(b"tcgen05_variant") == variant
    with pytest.raises(ValueError):
        fa.set_option("tcgen05_variant", 3)
    # forcing a variant decides the tile the family runs (2 exists at D = 64 only)
    fa.set_option("tcgen05_variant", 1)
    assert fa.select_path(4096, 64, False, 0.125) == (1, 128, 64)
    fa.set_option("tcgen05_variant", 2)
    assert fa.select_path(512, 64, True, 0.125, 128, 64) == (1, 128, 128)
    assert fa.select_path(512, 128, True, 0.125, 128, 64) == (1, 128, 64)
    fa.set_option("tcgen05_variant", -1)


@pytest.mark.parametrize("heads,world", [(1024, 8), (512, 4), (128, 8), (2, 2), (7, 4), (3, 8)])
def test_head_slabs_partition_exactly(heads, world):
    slabs = [sharding.head_slab(heads, r, world) for r in range(world)]
    assert slabs[0][0] == 0 and slabs[-1][1] == heads
    for a, b in zip(slabs, slabs[1:]):
        assert a[1] == b[0]
    sizes = [hi - lo for lo, hi in slabs]
    assert max(sizes) - min(sizes) <= 1


def test_shard_is_a_view():
    t = torch.arange(2 * 4 * 3 * 8, dtype=torch.float32).reshape(2, 4, 3, 8)
    s = sharding.shard_heads(t, 1, 4)
    assert s.shape == (1, 2, 3, 8) and s.data_ptr() == t.reshape(1, 8, 3, 8)[:, 2:].data_ptr()
    with pytest.raises(ValueError):
        sharding.head_slab(8, 4, 4)


def test_tile_table_is_total_and_consistent():
    """Every (S, D, causal) on the tcgen05 path resolves to an instantiated tile, bucket edges included."""
    for D in (16, 32, 64, 128, 256):
        for causal in (False, True):
            for S in (129, 130, 767, 768, 1535, 1536, 2048, 3071, 3072, 6143, 6144, 8192, 65536, 1 << 20):
                bm, bn = fa.get_tiling(2, 3, S, D, causal)
                assert bm == 128 and bn in ((64,) if D == 256 else (64, 128)), (S, D, causal, bm, bn)
                assert fa.select_path(S, D, causal, 0.1, bm, bn) == (1, bm, bn)
    for D in (16, 32):
        assert fa.get_tiling(1, 1, 4096, D, True) == fa.get_tiling(1, 1, 4096, 64, True)   # the D = 64 kernels' tiles
        assert fa.get_tiling(1, 1, 60, D, True) == (64, 64)                               # short-sequence kernel
    for S in (1, 64, 128):
        assert fa.get_tiling(1, 1, S, 128, False) == (128, 128)    # one key tile on the tcgen05 kernel
        assert fa.get_tiling(1, 1, S, 256, True) == (128, 64)
    assert fa.get_tiling(1, 1, 64, 64, False) == (64, 64)          # short-sequence kernel
    assert fa.get_tiling(1, 1, 128, 16, False) == (64, 64)


def test_work_items_need_no_device_and_count_every_head():
    items = ctypes.c_longlong(0)
    f = lib.rsfa_work_items
    # tcgen05 kernels: blocks of 256 query rows (128 at D = 256) per (batch, head)
    assert f(128, 8, 2048, 128, 0, 0.5, ctypes.byref(items)) == 0 and items.value == 1024 * 8
    assert f(64, 8, 1024, 256, 1, 0.0625, ctypes.byref(items)) == 0 and items.value == 512 * 8
    assert f(4, 32, 8192, 64, 0, 0.125, ctypes.byref(items)) == 0 and items.value == 128 * 32
    # short-sequence kernel: one CTA per 64 rows, all on grid.x - more heads than gridDim.y could hold
    assert f(8192, 16, 64, 64, 0, 0.5, ctypes.byref(items)) == 0 and items.value == 131072
    assert f(70000, 1, 100, 16, 1, 0.5, ctypes.byref(items)) == 0 and items.value == 140000
    assert f(1, 2, 128, 64, 0, 0.5, ctypes.byref(items)) == 0 and items.value == 2      # tcgen05: one item per head
    assert f(1, 2, 64, 64, 0, 0.5, ctypes.byref(items)) == 0 and items.value == 2
    assert f(1, 2, 128, 16, 0, 0.5, ctypes.byref(items)) == 0 and items.value == 4      # short-sequence: 64 rows per CTA
    assert f(1, 1, 0, 64, 0, 0.5, ctypes.byref(items)) == _capi.RSFA_ERR_INVALID_ARGUMENT
    assert f(1, 1, 64, 64, 0, 0.5, None) == _capi.RSFA_ERR_INVALID_ARGUMENT


def test_new_options_round_trip():
    for name, good, bad in (("pdl", (0, 1), 2), ("check_status", (1, 0), -1), ("test_drop_load", (5, -1), -2)):
        for v in good:
            fa.set_option(name, v)
            assert lib.rsfa_get_option(name.encode()) == v
        with pytest.raises(ValueError):
            fa.set_option(name, bad)
    assert lib.rsfa_get_option(b"workspace_devices") == 0      # no device call has been made here
    with pytest.raises(ValueError):
        fa.set_option("workspace_devices", 1)                   # read-only


def test_build_staleness_is_decided_by_content_not_by_file_times(tmp_path):
    import importlib.util
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("rsfa_build", os.path.join(root, "ascend-rsfa_b200", "build.py"))
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    h = b.source_hash(b.FLAGS)
    assert h == b.source_hash(list(b.FLAGS)) and h != b.source_hash(b.FLAGS + ["-DRSFA_TRACE"])
    out = tmp_path / "lib.so"
    assert b.stale(str(out), b.FLAGS)                            # nothing built yet
    out.write_bytes(b"x")
    assert b.stale(str(out), b.FLAGS)                            # a library without a stamp
    (tmp_path / "lib.so.stamp").write_text(h + "\n")
    os.utime(out, (1, 1))                                        # an ancient file time changes nothing
    assert not b.stale(str(out), b.FLAGS)
    (tmp_path / "lib.so.stamp").write_text("0" * 64 + "\n")
    assert b.stale(str(out), b.FLAGS)                            # built from other sources
