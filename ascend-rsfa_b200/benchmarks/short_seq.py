"""Short sequences (S <= 128): bytes moved per second against the measured HBM copy rate.

    python ascend-rsfa_b200/benchmarks/short_seq.py [--shape B H S D] [--iters N] [--causal 0|1]

A call on S <= 128 is one key tile per query tile: it reads Q, K, V once and writes O once
(4 * B * H * S * D * 2 bytes) and does next to no arithmetic, so HBM bandwidth bounds it - for the
large batches; the small ones (the reference's single-tile kernels _attn_fwd_small /
_attn_fwd_small_causal, ascend_rsfa/flash_attention_forward.py:26-159, serve 2 to 128 heads in its
tests, :673-677) are bound by the latency of one call.  The inputs of successive calls rotate
through a pool larger than the 126 MB L2, so every call reads from DRAM.

bench.py imports measure() for its `short_seq` record; run standalone (one shape, few iterations)
it is the command behind the ncu captures of these kernels.
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
sys.path.insert(0, PKG)
sys.path.insert(0, os.path.dirname(PKG))

import torch

# benchmark configuration cfg1, the two short shapes of the reference's own tests, and a large batch
SHAPES = [(1, 2, 128, 64), (4, 32, 64, 64), (4, 32, 128, 128), (512, 8, 128, 128)]
POOL_BYTES = 300 << 20


def spread(n, k):
    """k indices spread over range(n), first and last included."""
    if n <= k:
        return list(range(n))
    return sorted({int(round(i * (n - 1) / (k - 1))) for i in range(k)})


def measure(fa, dev, hbm_gbs, shape, causal=False, sm_scale=0.5, iters=400, check=True):
    """One record: microseconds per call (CUDA events around `iters` back-to-back calls), GB/s and the
    fraction of `hbm_gbs`, which kernel ran, and parity of 8 heads of one call with the fp32 oracle."""
    B, H, S, D = shape
    nbytes = 4 * B * H * S * D * 2
    sets = int(max(2, min(8192, POOL_BYTES // (3 * nbytes // 4) + 1)))
    g = torch.Generator(device=dev).manual_seed(5)
    pool = torch.randn((sets, 3, B, H, S, D), generator=g, device=dev, dtype=torch.float16)
    views = [(pool[i, 0], pool[i, 1], pool[i, 2]) for i in range(sets)]
    bm, bn = fa.get_tiling(B, H, S, D, causal)
    for i in range(min(10, iters)):
        fa.attention(*views[i % sets], causal, sm_scale, bm, bn)
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(iters):
        fa.attention(*views[i % sets], causal, sm_scale, bm, bn)
    ev1.record()
    torch.cuda.synchronize()
    us = ev0.elapsed_time(ev1) / iters * 1e3
    tc = fa.select_path(S, D, causal, sm_scale, bm, bn)[0] == 1
    rec = {"shape": [B, H, S, D], "causal": bool(causal), "us_per_call": us, "bytes_per_call": nbytes,
           "gb_per_s": nbytes / (us * 1e-6) / 1e9,
           "frac_of_measured_hbm": (nbytes / (us * 1e-6) / 1e9 / hbm_gbs) if hbm_gbs else None,
           "kernel": "tcgen05 (one key tile per work item)" if tc else "short-sequence (mma.sync)",
           "input_sets_rotated": sets}
    if check:
        from oracle.attention_ref import attention_fp32, error_metrics
        o = fa.attention(*views[0], causal, sm_scale, bm, bn)
        torch.cuda.synchronize()
        sel = spread(B * H, 8)
        flat = lambda x: x.reshape(1, B * H, S, D)[:, sel]
        m = error_metrics(flat(o), attention_fp32(flat(views[0][0]).cpu(), flat(views[0][1]).cpu(),
                                                  flat(views[0][2]).cpu(), causal, sm_scale))
        rec["parity"] = {"ok": bool(m["finite"] and m["allclose"]), "heads": len(sel), "max_abs": m["max_abs"]}
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", type=int, nargs=4, default=None, metavar=("B", "H", "S", "D"))
    ap.add_argument("--iters", type=int, default=400)
    ap.add_argument("--causal", type=int, default=0)
    ap.add_argument("--hbm-gbs", type=float, default=0.0, help="measured copy bandwidth to relate to (GB/s)")
    ap.add_argument("--no-check", action="store_true")
    args = ap.parse_args()
    import ascend_rsfa.flash_attention_forward as fa
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    hbm = args.hbm_gbs
    if not hbm:
        try:
            with open(os.path.join(os.path.dirname(PKG), "MEASURED_PEAKS.json")) as f:
                hbm = float(json.load(f)["hbm_gbs"])
        except Exception:
            hbm = 0.0
    for shape in ([tuple(args.shape)] if args.shape else SHAPES):
        print(json.dumps(measure(fa, dev, hbm, shape, bool(args.causal), iters=args.iters, check=not args.no_check)),
              flush=True)
    fa.device_status()


if __name__ == "__main__":
    main()
