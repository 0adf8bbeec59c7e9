"""The reference's 12 benchmark shapes on a B200: latency and correctness in one report.

    python ascend-rsfa_b200/benchmarks/run_paper_shapes.py [--json out.json]

Mirrors the methodology of the reference's harness so the rows sit beside its published table
(benchmarks/benchmark_results.txt): B = 128, H = 8, inputs N(0, 0.5) from seed 42, sm_scale = 0.5,
5 warm-ups and 20 timed calls, each timed call bracketed by a device synchronise and a host clock
(benchmarks/run_final_benchmark.py:104-124); the CUDA-event time of the same 20 calls back to back
is given too.  Correctness follows benchmarks/run_correctness_test.py:142-148 — max / mean absolute
error and allclose(atol = rtol = 1e-2) — against the fp32 reference math on sampled heads, with a
separate finiteness check.  Tiles come from get_tiling().
"""
import argparse
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
sys.path.insert(0, PKG)
sys.path.insert(0, os.path.dirname(PKG))

import torch

import ascend_rsfa.flash_attention_forward as fa
from oracle.attention_ref import attention_fp32, error_metrics

SHAPES = [(1024, 128), (1024, 256), (2048, 128), (2048, 256), (4096, 128), (8192, 64)]
B, H = 128, 8
# the reference's published optimised latency on Ascend 910B3, ms (benchmarks/benchmark_results.txt:13-24)
REFERENCE_MS = {(1024, 128, True): 8.95, (1024, 256, True): 25.92, (2048, 128, True): 28.97, (2048, 256, True): 97.26,
                (4096, 128, True): 103.78, (8192, 64, True): 388.51, (1024, 128, False): 6.80, (1024, 256, False): 11.92,
                (2048, 128, False): 26.16, (2048, 256, False): 45.97, (4096, 128, False): 102.08, (8192, 64, False): 302.76}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    rows = []
    for causal in (True, False):
        for S, D in SHAPES:
            torch.manual_seed(42)
            q, k, v = [torch.empty((B, H, S, D), dtype=torch.float16, device=dev).normal_(mean=0.0, std=0.5)
                       for _ in range(3)]
            bm, bn = fa.get_tiling(B, H, S, D, causal)
            for _ in range(args.warmup):
                o = fa.attention(q, k, v, causal, 0.5, bm, bn)
                torch.cuda.synchronize()
            per_call = []
            for _ in range(args.iters):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                o = fa.attention(q, k, v, causal, 0.5, bm, bn)
                torch.cuda.synchronize()
                per_call.append((time.perf_counter() - t0) * 1e3)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.iters):
                o = fa.attention(q, k, v, causal, 0.5, bm, bn)
            e1.record()
            torch.cuda.synchronize()
            fa.device_status()
            ev_ms = e0.elapsed_time(e1) / args.iters
            heads = [(0, 0), (B - 1, H - 1)]
            ref = torch.cat([attention_fp32(q[b:b + 1, h:h + 1].cpu(), k[b:b + 1, h:h + 1].cpu(), v[b:b + 1, h:h + 1].cpu(),
                                            causal, 0.5) for b, h in heads], dim=1)
            got = torch.cat([o[b:b + 1, h:h + 1] for b, h in heads], dim=1)
            m = error_metrics(got, ref)
            flops = 4.0 * B * H * S * S * D / (2 if causal else 1)
            avg = sum(per_call) / len(per_call)
            rows.append({"S": S, "D": D, "causal": causal, "tile": [bm, bn], "avg_ms": avg, "min_ms": min(per_call),
                         "max_ms": max(per_call), "event_ms": ev_ms, "tflops": flops / ev_ms / 1e9,
                         "reference_910b3_ms": REFERENCE_MS[(S, D, causal)], **m})
            del q, k, v, o
    print("| shape (B=128, H=8) | mask | tile | call+sync avg / min / max ms | events ms | TFLOP/s | reference 910B3 ms "
          "| max abs err | mean abs err | allclose 1e-2 | finite |")
    print("|---|---|---|---|---|---|---|---|---|---|---|")
    for r in rows:
        print("| S=%d D=%d | %s | (%d,%d) | %.3f / %.3f / %.3f | %.3f | %.0f | %.2f | %.2e | %.2e | %s | %s |" % (
            r["S"], r["D"], "causal" if r["causal"] else "full", r["tile"][0], r["tile"][1], r["avg_ms"], r["min_ms"],
            r["max_ms"], r["event_ms"], r["tflops"], r["reference_910b3_ms"], r["max_abs"], r["mean_abs"],
            "PASS" if r["allclose"] else "FAIL", r["finite"]))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
