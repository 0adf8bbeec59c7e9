"""Per-role cycle timeline of CTA 0 of the tcgen05 kernels, from the debug build.

    python ascend-rsfa_b200/build.py --trace
    python ascend-rsfa_b200/benchmarks/trace_roles.py B H S D causal [--scale 0.5] [--skip N] [--count N]

The debug library (ascend_rsfa/librsfa_b200_trace.so, built with -DRSFA_TRACE) makes the roles of
CTA 0 - softmax warps, MMA warp, TMA producer - log (clock64, event code) pairs into a buffer handed
over with the "trace_ptr" option.  This script runs one traced launch after a few untraced ones and
prints the merged timeline: absolute cycle, cycles since the same role's previous event, role, event.
The cycle tables under profiles/ were read off such timelines.  The product library has no trace code.
"""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
sys.path.insert(0, PKG)

from ascend_rsfa import _capi

_capi.LIB_PATH = os.path.join(PKG, "ascend_rsfa", "librsfa_b200_trace.so")

import torch

import ascend_rsfa.flash_attention_forward as fa

CAP = 4096          # events per role (kTraceCap in csrc/tcgen05_common.cuh)
ROLES = {0: "SM0", 1: "SM1", 2: "MMA", 3: "TMA", 5: "s0w1", 6: "s0w2", 7: "s0w3", 9: "s1w1", 10: "s1w2", 11: "s1w3"}
SOFTMAX = {1: "S seen", 2: "S in regs", 3: "reference ready", 4: "P half 0 out", 5: "P half 1 out", 6: "O seen",
           7: "epilogue done", 0xb: "half computed", 0xc: "careful path"}
MMA = {1: "P0 seen", 2: "PV0 issued", 3: "P1 seen", 4: "PV1 issued", 5: "QK(j+1) issued", 6: "V present",
       7: "step end", 9: "K ready", 0xa: "item"}


def describe(role, code):
    kind = code >> 12
    if role in (0, 1, 5, 6, 7, 9, 10, 11):
        return "%s j=%d" % (SOFTMAX.get(kind, hex(code)), code & 0xfff)
    if role == 2:
        return "%s t=%d j=%d" % (MMA.get(kind, hex(code)), (code >> 8) & 0xf, code & 0xff)
    return "%s %d" % ({1: "Q load", 2: "K/V load"}.get(code >> 8, hex(code)), code & 0xff)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("shape", type=int, nargs=5, metavar=("B", "H", "S", "D", "causal"))
    ap.add_argument("--scale", type=float, default=0.5)
    ap.add_argument("--skip", type=int, default=0)
    ap.add_argument("--count", type=int, default=400)
    args = ap.parse_args()
    B, H, S, D, causal = args.shape
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(1)
    q, k, v = [torch.randn(B, H, S, D, generator=g, device=dev).half() for _ in range(3)]
    bm, bn = fa.get_tiling(B, H, S, D, bool(causal))
    buf = torch.zeros(12 * 2 * CAP, dtype=torch.int64, device=dev)
    for _ in range(3):
        fa.attention(q, k, v, bool(causal), args.scale, bm, bn)
    torch.cuda.synchronize()
    fa.set_option("trace_ptr", buf.data_ptr())
    fa.attention(q, k, v, bool(causal), args.scale, bm, bn)
    torch.cuda.synchronize()
    fa.set_option("trace_ptr", 0)
    rec = buf.cpu().view(12, CAP, 2)
    events = []
    for role in range(12):
        for i in range(CAP):
            t, code = int(rec[role, i, 0]), int(rec[role, i, 1])
            if t == 0:
                break
            events.append((t, role, code))
    events.sort()
    if not events:
        print("no events: is the library the --trace build?")
        return
    t0, last = events[0][0], {}
    for t, role, code in events[args.skip:args.skip + args.count]:
        print("%9d (+%6d) %-4s %s" % (t - t0, t - last.get(role, t), ROLES.get(role, str(role)), describe(role, code)))
        last[role] = t


if __name__ == "__main__":
    main()
