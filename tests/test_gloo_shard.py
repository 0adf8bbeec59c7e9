"""The multi-rank host logic on CPU: world_size-2 gloo processes shard the heads, each computes
its slab with the oracle (stand-in for the device kernel, which needs a GPU), and the gathered
result equals the unsharded one."""
import os
import socket
import sys

import torch
import torch.multiprocessing as mp

from conftest import PKG, ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, heads, ok_flags):
    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    from ascend_rsfa import sharding
    from oracle.attention_ref import attention_fp32, make_inputs

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, S, D = heads, 1, 48, 16
        q, k, v = make_inputs(B, H, S, D, seed=11)
        full = attention_fp32(q, k, v, True, 0.3).reshape(1, B * H, S, D)
        mine = [sharding.shard_heads(t, rank, world) for t in (q, k, v)]
        lo, hi = sharding.head_slab(B * H, rank, world)
        assert mine[0].shape[1] == hi - lo
        local = attention_fp32(*mine, True, 0.3) if hi > lo else torch.empty(1, 0, S, D)
        dist.barrier()
        out = sharding.gather_heads(local, B * H)
        ok = torch.equal(out, full)
        # the check bench.py makes on GPUs after its timed region: per-slab checksums of the assembled
        # tensor against the ones every rank computed on its own slab (16-bit data, as on the device)
        half, out_half = local.half(), sharding.gather_heads(local.half(), B * H)
        ok = ok and sharding.gathered_matches_slabs(out_half, half, B * H)
        if hi > lo:   # a single wrong element in this rank's slab of the assembled tensor must be seen
            bad = out_half.clone()
            bad[0, lo, 0, 0] += 1.0
            ok = ok and not torch.equal(sharding.slab_checksums(bad[:, lo:hi]), sharding.slab_checksums(half))
        ok_flags[rank] = int(ok)
    finally:
        dist.destroy_process_group()


def _run(heads):
    world = 2
    ok = mp.get_context("spawn").Array("i", [0] * world)
    mp.spawn(_worker, args=(world, _free_port(), heads, ok), nprocs=world, join=True)
    assert list(ok) == [1] * world


def test_two_ranks_even_split():
    _run(6)


def test_two_ranks_uneven_split():
    _run(5)
