#!/usr/bin/env python
"""Benchmark of the FlashAttention-2 forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config cfg2] [--causal 0|1] [--e2e-steps E] [--no-extras]

One "step" is one forward pass of `attention()` over the whole configured batch
(default: benchmark configuration cfg2 - B=128, H=8, S=2048, D=128, fp16, sm_scale=0.5,
non-causal; the causal pass of the same shape is timed separately and reported
under "other_mask").  For N > 1 the script is launched with torchrun, one rank per
GPU; the B*H heads of the SAME problem are split across ranks (no collective in
the timed region) and the value is total FLOPs / slowest rank's time.

Prints ONE JSON line on rank 0.  Keys beyond the basic contract:

  value / roofline   device-resident throughput of the K timed steps (inputs already in HBM) against the
                     measured tensor-core peak; a run of 20 steps lasts 35 ms, i.e. it is a burst at full clock
  sustained          the same launch repeated for 3 s with one event pair per launch: median of the last
                     third, the SM clock sampled over that window, and the fraction of the sustained peak
  parity             >= 8 heads spread over every rank's slab (first and last included) of the output of a
                     full launch, against the fp32 oracle on the CPU, AND-ed over ranks; at N > 1 also an
                     NCCL all-gather of the output slabs (outside every timed region) whose per-slab
                     checksums must equal the ones each rank computed locally
  configs            the other benchmark configurations (cfg3, cfg4, cfg5), both masks, 20 steps each
  short_seq          (N = 1) the HBM-bound short-sequence shapes as bytes / time against the measured copy rate
  launch_floor_us    (N = 1) what one launch costs beyond its work items, from CUDA-graph replays of a small problem
  e2e                the same metric through `attention_host()` with pinned host tensors (host->device and
                     device->host copies inside the timed region), with the plain-copy floor of the box beside it
  cpu_baseline       (N = 1) the fp32 reference math on the host cores for a bounded sample

`--impl reference` times the reference math (softmax(QK^T*s)V in fp32 through
PyTorch on the host cores - the reference project has no CPU or CUDA
implementation of its own to run here) on the WHOLE configuration per step.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "ascend-rsfa_b200"))

import torch

METRIC = "attention fwd TFLOP/s (whole job; causal FLOPs counted as half)"
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the 128-key tcgen05 kernel per
# (batch, head) of S=2048, D=128, from the ncu capture summarised in the file below (128 heads of the shape:
# 201.4 MB read + 48.1 MB written); traffic is proportional to the number of heads (Q, K, V read once, O
# written once; the re-reads of K/V are served by L2).
NCU_DRAM_BYTES_PER_HEAD_S2048_D128 = 249.5e6 / 128
NCU_TRAFFIC_SOURCE = "profiles/fwd_tcgen05_d128_s2048_ncu_full.md"
# Peaks used only when MEASURED_PEAKS.json is absent: cuBLAS bf16 burst / sustained TFLOP/s and copy GB/s.
FALLBACK_PEAKS = {"burst": 1590.0, "sustained": 1400.0, "hbm_gbs": 6650.0}
IDLE_BEFORE_TIMING_S = 1.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="cfg2")
    ap.add_argument("--causal", type=int, default=0)
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--sustained-seconds", type=float, default=3.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="leave out the sustained, configs, short_seq and launch_floor records (profiler captures)")
    ap.add_argument("--batch", type=int, default=0,
                    help="override the config's batch size (small cases for profiler captures; the default "
                         "run and every reported number use the config's own)")
    return ap.parse_args()


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"burst": float(d["bf16_tflops"]), "sustained": float(d.get("bf16_tflops_sustained", 0.0)),
                "hbm_gbs": float(d.get("hbm_gbs", 0.0)), "source": "measured"}
    except Exception:
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Polls NVML for SM clock and throttle reasons while the timed region runs."""

    BAD = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20}
    NOTE = {"sw_power_cap": 0x4}

    def __init__(self, index):
        self.samples, self.times, self.reasons, self.max_mhz = [], [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                self.times.append(time.perf_counter())
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for name, bit in list(self.BAD.items()) + list(self.NOTE.items()):
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def median_since(self, t0):
        s = sorted(m for m, t in zip(self.samples, self.times) if t >= t0)
        return s[len(s) // 2] if s else None

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def workload_name(name, cfg, causal):
    B, H, S, D, scale, mult = cfg
    return "%s %s: B=%d H=%d S=%d D=%d sm_scale=%g%s" % (name, "causal" if causal else "non-causal", B, H, S, D,
                                                         scale, "" if mult == 1.0 else " inputs x%g" % mult)


def config_record(name, cfg, causal):
    """The `config` object, the same for both arms."""
    B, H, S, D, _, _ = cfg
    mib = 4.0 * B * H * S * D * 2 / 2 ** 20
    return {"workload": workload_name(name, cfg, causal), "inputs": "fp16 i.i.d. N(0,1) from a seed, [B,H,S,D] contiguous",
            "timing": "CUDA events around the timed steps, after %g s of idle and the warm-up steps" % IDLE_BEFORE_TIMING_S,
            "l2": "inputs+outputs %.0f MiB per step, %s the 126 MB L2" % (mib, "larger than" if mib > 126 else "NOT larger than")}


def cpu_reference_sample(cfg, causal, target_seconds):
    """Time the fp32 reference math on all host cores over whole heads of the config."""
    from oracle.attention_ref import attention_flops, attention_fp32, make_inputs
    B, H, S, D, scale, mult = cfg
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    q, k, v = make_inputs(1, 2, S, D, seed=42, std=mult)
    t0 = time.perf_counter()
    attention_fp32(q, k, v, causal, scale)
    per_head = (time.perf_counter() - t0) / 2.0
    n = int(max(2, min(B * H, 64, target_seconds / max(per_head, 1e-6))))
    q, k, v = make_inputs(1, n, S, D, seed=43, std=mult)
    # chunks of n heads until about target_seconds of CPU work are done, or the whole config is
    done, total = 0, 0.0
    while done < B * H and total < target_seconds:
        t0 = time.perf_counter()
        attention_fp32(q, k, v, causal, scale)
        total += time.perf_counter() - t0
        done += n
    flops = attention_flops(1, done, S, D, causal)
    return {"value": flops / total / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": "%d (batch,head) pairs (the config has %d) of %s, S=%d D=%d, in chunks of %d, fp32 PyTorch on "
                      "the host; full config extrapolates to %.1f s" % (done, B * H, "causal" if causal else "non-causal",
                                                                           S, D, n, total / done * B * H),
            "seconds": total}


def run_reference(args, cfg_name, cfg):
    """The reference arm: the fp32 reference math on the host cores, the WHOLE configuration per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    causal = bool(args.causal)
    B, H, S, D, scale, mult = cfg
    from oracle.attention_ref import attention_flops, attention_fp32, make_inputs
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    heads = B * H
    chunk = min(heads, 128)                      # generated once, reused for every chunk of the step
    q, k, v = make_inputs(1, chunk, S, D, seed=42, std=mult)

    def step():
        done = 0
        while done < heads:
            n = min(chunk, heads - done)
            attention_fp32(q[:, :n], k[:, :n], v[:, :n], causal, scale)
            done += n

    t0 = time.perf_counter()
    step()                                       # warm-up, also tells how long a step takes
    t_step = time.perf_counter() - t0
    warmup = 1
    # as many of the requested steps as fit in about three minutes of host time
    steps = int(max(1, min(args.steps, 180.0 / max(t_step, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    val = attention_flops(B, H, S, D, causal) / dt / 1e12
    sample = ("all %d (batch,head) pairs per step (inputs of %d heads reused), fp32 PyTorch on %d host threads; "
              "%d of the %d requested steps, %d warm-up" % (heads, chunk, cores, steps, args.steps, warmup))
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_record(cfg_name, cfg, causal),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def spread(n, k):
    """k indices spread over range(n), first and last included."""
    if n <= k:
        return list(range(n))
    return sorted({int(round(i * (n - 1) / (k - 1))) for i in range(k)})


def main():
    args = parse_args()
    from oracle.attention_ref import CONFIGS, attention_flops, attention_fp32, error_metrics
    cfg = CONFIGS[args.config]
    if args.impl == "reference":
        run_reference(args, args.config, cfg)
        return

    import ascend_rsfa.flash_attention_forward as fa
    from ascend_rsfa import sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))   # the oracle checks run on the host cores
    peaks = load_peaks()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(x):
        if dist is None:
            return float(x)
        t = torch.tensor([float(x)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_min(x):
        return -reduce_max(-float(x))

    def make_slab(c, seed):
        """This rank's slab of the seeded problem `c`, generated on the device (inputs resident in HBM)."""
        B, H, S, D, _, mult = c
        lo, hi = sharding.head_slab(B * H, rank, world)
        g = torch.Generator(device=dev).manual_seed(seed + rank)

        def mk():
            t = torch.randn((1, hi - lo, S, D), generator=g, device=dev, dtype=torch.float32)
            if mult != 1.0:
                t.mul_(mult)
            return t.to(torch.float16)
        return mk(), mk(), mk()

    def timed(c, tensors, causal, steps, warmup):
        B, H, S, D, scale, _ = c
        q, k, v = tensors
        bm, bn = fa.get_tiling(B, H, S, D, causal)   # the table's tile for this mask
        # every timed region starts from the same state: a second of idle lets the power cap's average
        # settle, so a region that follows another one is not measured at the clocks the first left behind
        time.sleep(IDLE_BEFORE_TIMING_S)
        for _ in range(warmup):
            fa.attention(q, k, v, causal, scale, bm, bn)
        barrier()
        launches0 = fa.launch_count()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(steps):
            fa.attention(q, k, v, causal, scale, bm, bn)
        ev1.record()
        barrier()
        ms = reduce_max(ev0.elapsed_time(ev1) / steps)
        return ms, fa.launch_count() - launches0, (bm, bn)

    def parity(c, tensors, causal, n_heads):
        """Heads spread over this rank's slab (first and last included) of the output of ONE full launch
        against the fp32 oracle on the CPU; AND / MAX over all ranks."""
        B, H, S, D, scale, _ = c
        q, k, v = tensors
        bm, bn = fa.get_tiling(B, H, S, D, causal)
        o = fa.attention(q, k, v, causal, scale, bm, bn)
        torch.cuda.synchronize()
        idx = spread(q.shape[1], n_heads)
        sel = torch.tensor(idx, device=dev)
        ref = attention_fp32(q[:, sel].cpu(), k[:, sel].cpu(), v[:, sel].cpu(), causal, scale)
        m = error_metrics(o[:, sel], ref)
        ok = reduce_min(1.0 if (m["finite"] and m["allclose"]) else 0.0) > 0.5
        return {"ok": ok, "heads": len(idx), "ranks": world, "max_abs": reduce_max(m["max_abs"]),
                "atol": 1e-2, "rtol": 1e-2, "head_index_in_slab": idx if rank == 0 else None}, o

    # ------------------------------------------------------------------ headline: value, other mask, parity
    B, H, S, D, scale, mult = cfg
    if args.batch > 0:
        B = args.batch
        cfg = (B, H, S, D, scale, mult)
    heads = B * H
    main_causal = bool(args.causal)
    slab = make_slab(cfg, 42)
    q, k, v = slab
    n_local = q.shape[1]
    warmup = max(3, args.warmup)
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        ms, launches, (bm, bn) = timed(cfg, slab, main_causal, args.steps, warmup)
    fa.device_status()
    flops = attention_flops(B, H, S, D, main_causal)
    value = flops / (ms * 1e-3) / 1e12
    other_ms, _, _ = timed(cfg, slab, not main_causal, max(5, args.steps // 2), 3)
    other_val = attention_flops(B, H, S, D, not main_causal) / (other_ms * 1e-3) / 1e12
    par, o_local = parity(cfg, slab, main_causal, 8)
    par_other, _ = parity(cfg, slab, not main_causal, 8)
    par["other_mask"] = {"ok": par_other["ok"], "heads": par_other["heads"], "max_abs": par_other["max_abs"]}

    # N > 1: the one allowed use of NCCL - gather the output slabs (outside every timed region) and check
    # that every slab of the assembled tensor has the checksums its owner computed locally
    if dist is not None:
        t0 = time.perf_counter()
        gathered = sharding.gather_heads(o_local, heads)
        torch.cuda.synchronize()
        gather_s = time.perf_counter() - t0
        ok = sharding.gathered_matches_slabs(gathered, o_local, heads)
        par["gather"] = {"ok": reduce_min(1.0 if ok else 0.0) > 0.5, "collective": "ncclAllGather of the O slabs",
                         "bytes": int(gathered.numel() * 2), "seconds": gather_s, "in_timed_region": False}
        par["ok"] = par["ok"] and par["gather"]["ok"]
        del gathered
    del o_local

    extras = not args.no_extras
    sustained = None
    # ------------------------------------------------------------------ operator timing, the reference harness's way
    # One attention() call (output allocation included) followed by a device synchronize, host clock around
    # the pair, as benchmarks/run_final_benchmark.py:111-126 of the reference times its operator (it reports the mean).
    operator = None
    if extras:
        time.sleep(IDLE_BEFORE_TIMING_S)
        for _ in range(3):
            fa.attention(q, k, v, main_causal, scale, bm, bn)
        torch.cuda.synchronize()
        barrier()
        per_call = []
        for _ in range(10):
            t0 = time.perf_counter()
            fa.attention(q, k, v, main_causal, scale, bm, bn)
            torch.cuda.synchronize()
            per_call.append(time.perf_counter() - t0)
        barrier()
        call_s = reduce_max(sorted(per_call)[len(per_call) // 2])
        mean_s = reduce_max(sum(per_call) / len(per_call))
        operator = {"ms_per_call": call_s * 1e3, "tflops": flops / call_s / 1e12, "calls": 10,
                    "mean_ms_per_call": mean_s * 1e3,
                    "note": "median of attention() + torch.cuda.synchronize() per call on the host clock, output "
                            "allocation inside, max over ranks"}
    # ------------------------------------------------------------------ launch floor (N = 1)
    # What one launch costs beyond its work items, on the GPU alone: 100 launches of a small problem are
    # captured in a CUDA graph (the host cannot issue 10 us kernels fast enough through Python) and
    # replayed; with one work item per SM and with two, floor = 2 t(1) - t(2).  The replays last a
    # millisecond, so both run at the same full clock.
    launch_floor = None
    if extras and world == 1:
        try:
            sms = fa.get_num_compute_cores()
            per_graph = 100
            t = {}
            for mult in (1, 2):
                c = (1, (sms // 2) * mult, 512, 128, 0.5, 1.0)      # 2 work items of 256 rows per head
                lq, lk, lv = make_slab(c, 7)
                lbm, lbn = fa.get_tiling(c[0], c[1], c[2], c[3], False)
                for _ in range(3):
                    fa.attention(lq, lk, lv, False, c[4], lbm, lbn)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    for _ in range(per_graph):
                        fa.attention(lq, lk, lv, False, c[4], lbm, lbn)
                graph.replay()
                torch.cuda.synchronize()
                time.sleep(0.5)
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
                for _ in range(3):
                    graph.replay()
                ev1.record()
                torch.cuda.synchronize()
                t[mult] = ev0.elapsed_time(ev1) / (3 * per_graph)
                del graph
            launch_floor = {"us": (2 * t[1] - t[2]) * 1e3, "t_1_item_per_sm_us": t[1] * 1e3,
                            "t_2_items_per_sm_us": t[2] * 1e3,
                            "shape": "S=512 D=128 non-causal, %d and %d heads = 1 and 2 work items per SM; %d launches "
                                     "per CUDA graph, 3 replays; floor = 2 t(1) - t(2)" % (sms // 2, sms, per_graph)}
            fa.device_status()
        except Exception as e:   # a capture problem must not cost the whole benchmark line
            launch_floor = {"us": None, "error": repr(e)[:200]}

    # ------------------------------------------------------------------ the other benchmark configurations
    configs = None
    if extras and args.batch == 0:
        configs = {}
        for name in ("cfg3", "cfg4", "cfg5"):
            if name == args.config:
                continue
            c = CONFIGS[name]
            cB, cH, cS, cD, cscale, _ = c
            if cB * cH < world:
                continue
            tensors = make_slab(c, 42)
            rec = {"workload": workload_name(name, c, False).replace(" non-causal", "")}
            for causal in (False, True):
                # two timed regions of 20 steps, each after its own idle second and warm-up; the faster one is
                # reported and both are listed (a region now and then starts in a lower power state)
                regions = []
                for _ in range(2):
                    r_ms, _, tile = timed(c, tensors, causal, 20, 3)
                    regions.append(r_ms)
                c_ms = min(regions)
                tf = attention_flops(cB, cH, cS, cD, causal) / (c_ms * 1e-3) / 1e12
                p_rec, _ = parity(c, tensors, causal, 8 if world == 1 else 2)
                rec["causal" if causal else "non_causal"] = {
                    "tflops": tf, "ms_per_step": c_ms, "frac_of_measured_burst": tf / world / peaks["burst"],
                    "tile": list(tile), "steps": 20, "ms_per_step_of_each_region": regions,
                    "parity": {"ok": p_rec["ok"], "heads": p_rec["heads"], "ranks": world, "max_abs": p_rec["max_abs"]}}
            configs[name] = rec
            del tensors
        fa.device_status()

    # ------------------------------------------------------------------ short sequences: HBM-bound (N = 1)
    short_seq = None
    if extras and world == 1 and args.batch == 0:
        from benchmarks import short_seq as ss
        short_seq = [ss.measure(fa, dev, peaks["hbm_gbs"], shape) for shape in ss.SHAPES]
        fa.device_status()

    # ------------------------------------------------------------------ sustained clock regime (N = 1)
    if extras and world == 1:
        n_launch = int(max(60, min(6000, args.sustained_seconds / (ms * 1e-3))))
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(n_launch + 1)]
        with ClockSampler(physical_gpu_index(local_rank)) as cs:
            torch.cuda.synchronize()
            t_start = time.perf_counter()
            evs[0].record()
            for i in range(n_launch):
                fa.attention(q, k, v, main_causal, scale, bm, bn)
                evs[i + 1].record()
            torch.cuda.synchronize()
            t_end = time.perf_counter()
        per = [evs[i].elapsed_time(evs[i + 1]) for i in range(n_launch)]
        last = sorted(per[-(n_launch // 3):])
        s_ms = last[len(last) // 2]
        s_mhz = cs.median_since(t_start + (t_end - t_start) * 2.0 / 3.0)
        s_tf = flops / (s_ms * 1e-3) / 1e12
        b_mhz = clocks.summary()["sm_mhz"]
        sustained = {"launches": n_launch, "seconds": t_end - t_start, "ms_per_step": s_ms, "sm_mhz": s_mhz,
                     "tflops": s_tf, "peak": peaks["sustained"],
                     "frac": (s_tf / peaks["sustained"]) if peaks["sustained"] else None,
                     "reasons": sorted(cs.reasons),
                     "ms_x_mhz": {"burst": (ms * b_mhz) if b_mhz else None, "sustained": (s_ms * s_mhz) if s_mhz else None},
                     "note": "median of the last third of back-to-back launches, one CUDA event pair per launch"}
        del evs

    # ------------------------------------------------------------------ end to end: host tensors in and out
    e2e = None
    if not args.no_e2e:
        qh, kh, vh = [t.cpu().pin_memory() for t in (q, k, v)]
        oh = torch.empty_like(qh).pin_memory()
        fa.attention_host(qh, kh, vh, main_causal, scale, bm, bn, device=local_rank, out=oh)
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            fa.attention_host(qh, kh, vh, main_causal, scale, bm, bn, device=local_rank, out=oh)
        barrier()
        e2e_s = reduce_max((time.perf_counter() - t0) / args.e2e_steps)
        m = error_metrics(oh[:, :1], attention_fp32(qh[:, :1], kh[:, :1], vh[:, :1], main_causal, scale))
        # what the copies alone cost on this box with all N ranks copying at once: the same bytes as plain
        # pinned copies, both directions running together on two streams
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        dst = [torch.empty_like(t) for t in (q, k, v)]
        src_o = torch.empty_like(q)

        def copies():
            with torch.cuda.stream(s_in):
                for d_, h_ in zip(dst, (qh, kh, vh)):
                    d_.copy_(h_, non_blocking=True)
            with torch.cuda.stream(s_out):
                oh.copy_(src_o, non_blocking=True)
        copies()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            copies()
        barrier()
        floor_s = reduce_max((time.perf_counter() - t0) / args.e2e_steps)
        nbytes = q.numel() * 2
        e2e = {"value": flops / e2e_s / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_s * 1e3,
               "h2d_bytes_per_step": 3 * nbytes, "d2h_bytes_per_step": nbytes,
               "copy_floor_ms": floor_s * 1e3,
               "copy_floor_note": "the same bytes as plain pinned copies, H2D and D2H together on two streams, all "
                                  "%d rank(s) at once; h2d %.1f GB/s per GPU" % (world, 3 * nbytes / floor_s / 1e9),
               "parity_head0_ok": bool(m["finite"] and m["allclose"]),
               "api": "ascend_rsfa.flash_attention_forward.attention_host -> rsfa_fwd_host"}
        del qh, kh, vh, oh, dst, src_o

    if rank == 0:
        per_gpu = value / world
        record = config_record(args.config, cfg, main_causal)
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": record,
            "sharding": "%d heads over %d GPU(s), %d on rank 0; no collective in the timed region" % (heads, world, n_local),
            "tile": [bm, bn],
            "per_gpu_tflops": per_gpu,
            "pct_of_peak": {"measured_burst": per_gpu / peaks["burst"], "nominal_2250": per_gpu / 2250.0},
            "other_mask": {"causal": (not main_causal), "tflops": other_val, "ms_per_step": other_ms,
                           "pct_of_measured_burst": other_val / world / peaks["burst"]},
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peaks["burst"], "unit": "TFLOP/s",
                         "frac": per_gpu / peaks["burst"],
                         "traffic": (NCU_DRAM_BYTES_PER_HEAD_S2048_D128 * n_local if (S, D) == (2048, 128) else None),
                         "traffic_source": (NCU_TRAFFIC_SOURCE + " (128 heads of this shape, scaled by the number of heads)"
                                            if (S, D) == (2048, 128) else "no ncu capture of this shape"),
                         "algorithmic_bytes": 4.0 * n_local * S * D * 2,
                         "peak_source": peaks["source"] + " cuBLAS bf16 burst (the timed region is a burst at full "
                                        "clock); sustained %.1f, see the `sustained` record" % peaks["sustained"]},
            "clocks": clocks.summary(),
            "gpu_launches": launches,
            "parity": par,
        }
        if operator is not None:
            line["operator"] = operator
        if sustained is not None:
            line["sustained"] = sustained
        if launch_floor is not None:
            line["launch_floor_us"] = launch_floor["us"]
            line["launch_floor"] = launch_floor
        if configs is not None:
            line["configs"] = configs
        if short_seq is not None:
            line["short_seq"] = short_seq
        if e2e is not None:
            line["e2e"] = e2e
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_reference_sample(cfg, main_causal, target_seconds=12.0)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
