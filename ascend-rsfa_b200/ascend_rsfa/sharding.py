"""(batch x head) sharding across the GPUs of one box.

Every (b, h) pair is an independent attention problem (the reference's task
decode treats the head index as opaque, flash_attention_forward.py:295-299), so
rank r of n takes a contiguous slab of the flattened B*H heads and no data-path
collective exists.  Outputs are gathered only when a caller wants the assembled
tensor (parity checks), outside any timed region.
"""
import torch


def head_slab(total_heads, rank, world_size):
    """[lo, hi) of the flattened heads owned by `rank`; slabs differ by at most one head."""
    if world_size < 1 or not (0 <= rank < world_size) or total_heads < 0:
        raise ValueError("bad rank/world_size/total_heads")
    base, extra = divmod(total_heads, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_heads(t, rank, world_size):
    """View of a contiguous [B, H, S, D] tensor as this rank's [1, n, S, D] slab (zero-copy)."""
    B, H, S, D = t.shape
    lo, hi = head_slab(B * H, rank, world_size)
    return t.reshape(1, B * H, S, D)[:, lo:hi]


def gather_heads(local, total_heads, group=None):
    """All-gather [1, n_r, S, D] slabs into [1, total_heads, S, D] on every rank.  Slabs may
    differ by one head, so they are padded to the largest before the collective."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    _, n, S, D = local.shape
    n_max = -(-total_heads // world)
    padded = local
    if n < n_max:
        pad = torch.zeros((1, n_max - n, S, D), dtype=local.dtype, device=local.device)
        padded = torch.cat([local, pad], dim=1)
    bufs = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(bufs, padded.contiguous(), group=group)
    parts = []
    for r in range(world):
        lo, hi = head_slab(total_heads, r, world)
        parts.append(bufs[r][:, : hi - lo])
    assert head_slab(total_heads, rank, world)[1] - head_slab(total_heads, rank, world)[0] == n
    return torch.cat(parts, dim=1)


def slab_checksums(x):
    """Two 64-bit checksums of a 16-bit tensor that are exact and do not depend on the order of
    summation: the bit patterns as integers, plain and weighted by position (mod 2^64)."""
    bits = x.contiguous().view(torch.int16).reshape(-1).long()
    w = torch.arange(bits.numel(), device=x.device, dtype=torch.int64) % 8191 + 1
    return torch.stack([bits.sum(), (bits * w).sum()])


def gathered_matches_slabs(gathered, local, total_heads, group=None):
    """After gather_heads: does every rank's slab of the assembled [1, total_heads, S, D] tensor carry the
    checksums its owner computed on its own output?  One small all-gather; True on every rank or on none
    only if the caller reduces the answer itself."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    mine = slab_checksums(local)
    sums = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(sums, mine, group=group)
    ok = gathered.shape[1] == total_heads
    for r in range(world):
        lo, hi = head_slab(total_heads, r, world)
        ok = ok and bool(torch.equal(slab_checksums(gathered[:, lo:hi]), sums[r]))
    return ok
