#!/usr/bin/env python
"""Benchmark of the FlashAttention-2 forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config cfg2] [--causal 0|1] [--e2e-steps E]

One "step" is one forward pass of `attention()` over the whole configured batch
(default: benchmark configuration cfg2 — B=128, H=8, S=2048, D=128, fp16, sm_scale=0.5,
non-causal; the causal pass of the same shape is timed separately and reported
under "causal").  For N > 1 the script is launched with torchrun, one rank per
GPU; the B*H heads of the SAME problem are split across ranks (no collective in
the timed region) and the value is total FLOPs / slowest rank's time.

Prints ONE JSON line on rank 0.  `value` is device-resident throughput (inputs
already in HBM), `e2e` is the same metric through `attention_host()` with pinned
host tensors (host->device and device->host copies inside the timed region),
`roofline` relates the kernel to the measured tensor-core peak, `cpu_baseline`
is the fp32 reference math on the host cores for a bounded sample.

`--impl reference` times the reference math (softmax(QK^T*s)V in fp32 through
PyTorch on the host cores — the reference project has no CPU or CUDA
implementation of its own to run here) on a bounded sample of the same config.
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
# DRAM bytes (read + write) per (batch, head) of S=2048, D=128: dram__bytes_read.sum + dram__bytes_write.sum
# of one ncu capture of this kernel on 128 heads of the shape (201.4 + 48.0 MB); traffic is proportional
# to the number of heads (Q, K, V read once, O written once; the re-reads of K/V are served by L2).
NCU_DRAM_BYTES_PER_HEAD_S2048_D128 = 249.4e6 / 128
FALLBACK_PEAK_TFLOPS = 1590.0  # earlier measurement on this pool, used only if MEASURED_PEAKS.json is absent


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="cfg2")
    ap.add_argument("--causal", type=int, default=0)
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
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
        return {"burst": FALLBACK_PEAK_TFLOPS, "sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Polls NVML for SM clock and throttle reasons while the timed region runs."""

    BAD = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20}
    NOTE = {"sw_power_cap": 0x4}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
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


def cpu_reference_sample(cfg, causal, target_seconds, repeats=1):
    """Time the fp32 reference math on all host cores over `n` whole heads of the config."""
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
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    causal = bool(args.causal)
    B, H, S, D, scale, mult = cfg
    from oracle.attention_ref import attention_flops, attention_fp32, make_inputs
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n = 8  # heads per step: a bounded sample of the same workload
    q, k, v = make_inputs(1, n, S, D, seed=42, std=mult)
    for _ in range(max(1, min(args.warmup, 2))):
        attention_fp32(q, k, v, causal, scale)
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        attention_fp32(q, k, v, causal, scale)
    dt = (time.perf_counter() - t0) / steps
    val = attention_flops(1, n, S, D, causal) / dt / 1e12
    sample = "%d of %d (batch,head) pairs per step, fp32 PyTorch on %d host threads" % (n, B * H, cores)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "%s %s B=%d H=%d S=%d D=%d" % (cfg_name, "causal" if causal else "non-causal", B, H, S, D),
                   "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    from oracle.attention_ref import CONFIGS, attention_flops
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

    B, H, S, D, scale, mult = cfg
    if args.batch > 0:
        B = args.batch
        cfg = (B, H, S, D, scale, mult)
    heads = B * H
    lo, hi = sharding.head_slab(heads, rank, world)
    n_local = hi - lo
    bm, bn = fa.get_tiling(B, H, S, D, bool(args.causal))

    # This rank's slab of the seeded problem, generated on the device (inputs resident in HBM).
    g = torch.Generator(device=dev).manual_seed(42 + rank)
    def mk():
        t = torch.randn((1, n_local, S, D), generator=g, device=dev, dtype=torch.float32)
        if mult != 1.0:
            t.mul_(mult)
        return t.to(torch.float16)
    q, k, v = mk(), mk(), mk()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(causal, steps, warmup):
        bm, bn = fa.get_tiling(B, H, S, D, causal)   # the table's tile for this mask
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
        ms = ev0.elapsed_time(ev1) / steps
        launches = fa.launch_count() - launches0
        if dist is not None:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, launches

    main_causal = bool(args.causal)
    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        ms, launches = timed(main_causal, args.steps, max(3, args.warmup))
    fa.device_status()
    flops = attention_flops(B, H, S, D, main_causal)
    value = flops / (ms * 1e-3) / 1e12
    other_ms, _ = timed(not main_causal, max(5, args.steps // 2), 3)
    other_val = attention_flops(B, H, S, D, not main_causal) / (other_ms * 1e-3) / 1e12

    # sanity: one head against the fp32 oracle (outside every timed region)
    from oracle.attention_ref import attention_fp32, error_metrics
    o = fa.attention(q[:, :1], k[:, :1], v[:, :1], main_causal, scale, bm, bn)
    err = error_metrics(o, attention_fp32(q[:, :1].cpu(), k[:, :1].cpu(), v[:, :1].cpu(), main_causal, scale))

    # end to end: pinned host tensors in, host tensor out, copies inside the timed region
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
        e2e_s = (time.perf_counter() - t0) / args.e2e_steps
        if dist is not None:
            t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t.item())
        nbytes = q.numel() * 2
        e2e = {"value": flops / e2e_s / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_s * 1e3,
               "h2d_bytes_per_step": 3 * nbytes, "d2h_bytes_per_step": nbytes,
               "api": "ascend_rsfa.flash_attention_forward.attention_host -> rsfa_fwd_host"}
        del qh, kh, vh, oh

    if rank == 0:
        peaks = load_peaks()
        per_gpu = value / world
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": "%s %s: B=%d H=%d S=%d D=%d sm_scale=%g, heads sharded over %d GPU(s)"
                                   % (args.config, "causal" if main_causal else "non-causal", B, H, S, D, scale, world),
                       "tile": [bm, bn], "l2": "inputs+outputs %.0f MiB per GPU, larger than the 126 MB L2"
                                                % (4 * q.numel() * 2 / 2 ** 20)},
            "per_gpu_tflops": per_gpu,
            "pct_of_peak": {"measured_burst": per_gpu / peaks["burst"], "nominal_2250": per_gpu / 2250.0},
            "other_mask": {"causal": (not main_causal), "tflops": other_val, "ms_per_step": other_ms,
                           "pct_of_measured_burst": other_val / world / peaks["burst"]},
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peaks["burst"], "unit": "TFLOP/s",
                         "frac": per_gpu / peaks["burst"],
                         "traffic": (NCU_DRAM_BYTES_PER_HEAD_S2048_D128 * n_local if (S, D) == (2048, 128) else None),
                         "traffic_note": ("scaled from an ncu capture of 128 heads of this shape" if (S, D) == (2048, 128)
                                          else "no ncu capture of this shape") + "; algorithmic bytes %.3e"
                                         % (4.0 * n_local * S * D * 2),
                         "peak_source": peaks["source"] + " cuBLAS bf16 burst; sustained %.1f" % peaks["sustained"],
                         "frac_of_sustained": (per_gpu / peaks["sustained"]) if peaks["sustained"] else None},
            "clocks": clocks.summary(),
            "gpu_launches": launches,
            "parity": err,
        }
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
