"""Offline tile sweep for the tcgen05 kernel family on a B200.

    python ascend-rsfa_b200/tile_sweep.py [--write] [--out FILE] [--iters N]

Counterpart of the reference's tiling/search_optimal_tiling.py: for every (S, D, causal) of the
sweep list it runs each instantiated tile — (128, 128) = single-buffered S, (128, 64) =
double-buffered S — first against the fp32 reference math on two heads (a wrong tile is never
timed, the lesson of the reference's benchmarks/ablation_report_causal.txt), then times it with
CUDA events and keeps the fastest.  `--write` regenerates csrc/tile_table.inc, which
`get_tiling` / `rsfa_get_tiling` serve after the next build.  The Ascend tile sizes of the
reference are not reused: they describe a different machine.
"""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import torch

import ascend_rsfa.flash_attention_forward as fa

# (S, D, heads to time with): heads chosen so every shape holds the same ~0.27 G elements per tensor
SWEEP = [(512, 64, 4096), (1024, 64, 4096), (2048, 64, 2048), (4096, 64, 1024), (8192, 64, 512),
         (512, 128, 2048), (1024, 128, 2048), (2048, 128, 1024), (4096, 128, 512), (8192, 128, 256)]
CANDIDATES = [(128, 128), (128, 64)]
BUCKET_EDGES = [129, 768, 1536, 3072, 6144, 1 << 30]   # S ranges around the measured lengths


def reference(q, k, v, causal, scale):
    s = (q.float() @ k.float().transpose(-1, -2)) * scale
    if causal:
        S = q.shape[-2]
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=q.device).tril_(), float("-inf"))
    return torch.softmax(s, dim=-1) @ v.float()


def time_tile(q, k, v, causal, scale, bm, bn, iters):
    for _ in range(3):
        fa.attention(q, k, v, causal, scale, bm, bn)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fa.attention(q, k, v, causal, scale, bm, bn)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--write", action="store_true")
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--out", default=os.path.join(HERE, "csrc", "tile_table.inc"),
                    help="where --write puts the table (default: the file the build includes)")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(42)
    best = {}
    for S, D, heads in SWEEP:
        # two logit distributions: the usual 1/sqrt(D) and the peaked rows of benchmark configuration cfg2 (sm_scale 0.5)
        # recipe (sm_scale 0.5 on N(0,1) inputs), where O is rescaled much more often
        scales = (1.0 / D ** 0.5, 0.5)
        q, k, v = [torch.randn(1, heads, S, D, generator=g, device=dev).half() for _ in range(3)]
        for causal in (False, True):
            rows = []
            for bm, bn in CANDIDATES:
                ms = 0.0
                good = True
                for scale in scales:
                    path, tm, tn = fa.select_path(S, D, causal, scale, bm, bn)
                    assert (path, tm, tn) == (1, bm, bn), "tile (%d,%d) is not instantiated" % (bm, bn)
                    ref = reference(q[:, :2], k[:, :2], v[:, :2], causal, scale)
                    out = fa.attention(q[:, :2], k[:, :2], v[:, :2], causal, scale, bm, bn).float()
                    fa.device_status()
                    if not (torch.isfinite(out).all() and torch.allclose(out, ref, atol=1e-2, rtol=1e-2)):
                        good = False
                        break
                    ms += time_tile(q, k, v, causal, scale, bm, bn, args.iters)
                if not good:
                    print("S=%d D=%d causal=%d tile (%d,%d): WRONG, not timed" % (S, D, causal, bm, bn))
                    continue
                ms /= len(scales)
                flops = 4.0 * heads * S * S * D / (2 if causal else 1)
                rows.append((ms, bm, bn, flops / ms / 1e9))
            rows.sort()
            best[(S, D, causal)] = rows[0][1:3]
            print("S=%5d D=%3d causal=%d : " % (S, D, causal) +
                  "  ".join("(%d,%d) %.3f ms %.0f TFLOP/s" % (bm, bn, ms, tf) for ms, bm, bn, tf in rows) +
                  "  -> (%d,%d)" % rows[0][1:3])
    if args.write:
        lines = [l for l in open(os.path.join(HERE, "csrc", "tile_table.inc")) if l.startswith("//")]
        for D in (64, 128):
            for causal in (0, 1):
                measured = sorted(S for (S, d, c) in best if d == D and c == bool(causal))
                for lo, hi in zip(BUCKET_EDGES[:-1], BUCKET_EDGES[1:]):
                    inside = [S for S in measured if lo <= S < hi]
                    if not inside:
                        continue
                    bm, bn = best[(inside[0], D, bool(causal))]
                    lines.append("{%d, %d, %d, %d, %d, %d},\n" % (lo, hi - 1, D, causal, bm, bn))
        for causal in (0, 1):
            lines.append("{129, 1 << 30, 256, %d, 128, 64},\n" % causal)
        with open(args.out, "w") as f:
            f.writelines(lines)
        print("wrote %s; rebuild with build.py" % args.out)


if __name__ == "__main__":
    main()
