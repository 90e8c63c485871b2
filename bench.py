#!/usr/bin/env python
"""Benchmark of the sampling step: one "step" = one pass of the hot path over
one batch of synthetic logits.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4] [--impl reference]

Own arm: `value` is rows/s with the batch resident in HBM (device-pointer
entry point, CUDA events on the launching stream); `e2e` is the same metric
through the host-pointer C-ABI call with pinned host buffers, copies inside
the timed region. `--impl reference` times the CPU restatement of the
reference's routines on the host cores. Under torchrun every rank runs its own
rows (no collective on the data path); rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
METRIC = "sampled_rows_per_s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c4", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--rows", type=int, default=None)
    ap.add_argument("--mode", type=int, default=None, help="0 = mode A, 1 = mode B (default per workload)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU work budget of the cpu_baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--vocab-sharded", action="store_true",
                    help="every rank holds a column slice of the SAME rows (C5): local candidates, one all-gather, "
                         "merge on every rank; total work fixed (strong scaling), no host-pointer leg")
    ap.add_argument("--profile", action="store_true",
                    help="short run for ncu: no e2e leg, no CPU baseline, no clock hold")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def workload_config(w, args, world):
    mode = int(w.cfgs["topp_mode"][0])
    return {
        "workload": w.name, "rows_per_gpu": int(w.B), "vocab": int(w.V), "logits_dtype": w.dtype,
        "topp_mode": "A(model/generate.go)" if mode == 0 else "B(model/qwen/generate.go)",
        "sharding": (f"vocab x{world}, one all-gather of {world}x{int(w.B)} records of 1040 B" if args.vocab_sharded
                     else f"rows x{world}, no collective"),
        "l2": "inputs larger than L2" if w.logits.nbytes > 126 * 2 ** 20 else "L2 flushed between steps",
    }


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while running."""

    def __init__(self, index: int):
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
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.02)

    def start(self):
        if self._nv:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def time_cpu(w, rows, threads, seconds):
    """Rows/s of the CPU restatement on `rows` rows with `threads` threads,
    repeated until about `seconds` of wall time has been spent."""
    from oracle import oracle as orc
    orc.build()
    sub_l, sub_c, sub_u = w.logits[:rows], w.cfgs[:rows], w.uniforms[:rows]
    orc.sample_batch(sub_l[:min(rows, threads)], sub_c[:min(rows, threads)], sub_u[:min(rows, threads)],
                     want_info=False, threads=threads)   # warm
    done, t0, best = 0, time.perf_counter(), None
    while True:
        t1 = time.perf_counter()
        orc.sample_batch(sub_l, sub_c, sub_u, want_info=False, flags=0, threads=threads)
        dt = time.perf_counter() - t1
        best = dt if best is None else min(best, dt)
        done += 1
        if time.perf_counter() - t0 >= seconds or done >= 50:
            break
    return rows / best, done


def reference_arm(args, rank, world):
    """The reference's own CPU implementation of the path (its Go routines restated
    in C++: no Go toolchain exists offline), all host threads, rank 0 only."""
    if rank != 0:
        return
    from gorch_b200 import workloads
    from oracle import oracle as orc
    orc.build()
    threads = orc.hw_threads()
    rows = args.rows or max(threads, 64)
    w = workloads.make(args.workload, rows, args.mode)
    sub = (w.logits, w.cfgs, w.uniforms)
    for _ in range(args.warmup):
        orc.sample_batch(*sub, want_info=False, flags=0, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.sample_batch(*sub, want_info=False, flags=0, threads=threads)
    dt = time.perf_counter() - t0
    value = rows * args.steps / dt
    cfg = workload_config(w, args, 1)
    cfg["rows_per_gpu"] = rows
    cfg["sharding"] = "host threads over rows"
    cfg["l2"] = "n/a (host arm)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": "port",
                         "sample": f"{rows} rows of {w.name} per step, C++ restatement of the Go routines"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    args = parse()
    if args.profile:
        args.no_e2e = args.no_cpu_baseline = True
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from gorch_b200 import build, sampling, workloads
    from gorch_b200.config import CFG_DTYPE, DTYPE_BF16, DTYPE_F32

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    build.build()
    workloads.set_shard(0 if args.vocab_sharded else rank)
    if args.vocab_sharded:
        args.no_e2e = True
    w = workloads.make(args.workload, args.rows, args.mode)
    B, V = w.B, w.V
    dt_code = DTYPE_BF16 if w.dtype == "bf16" else DTYPE_F32
    smp = sampling.CudaSampler(local_rank)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    smp.set_stream(stream.cuda_stream)

    # host (pinned) and device copies of the inputs
    h_logits = torch.from_numpy(w.logits.view(np.int16) if w.dtype == "bf16" else w.logits).pin_memory()
    h_cfgs = torch.from_numpy(w.cfgs.view(np.uint8).reshape(B, 16).copy()).pin_memory()
    h_uni = torch.from_numpy(w.uniforms.copy()).pin_memory()
    h_ids = torch.empty(B, dtype=torch.int32).pin_memory()
    h_flags = torch.empty(B, dtype=torch.int32).pin_memory()
    d_logits = h_logits.cuda(non_blocking=True)
    d_cfgs = h_cfgs.cuda(non_blocking=True)
    d_uni = h_uni.cuda(non_blocking=True)
    d_ids = torch.empty(B, dtype=torch.int32, device="cuda")
    d_flags = torch.empty(B, dtype=torch.int32, device="cuda")
    flush = None
    if w.logits.nbytes <= 126 * 2 ** 20:
        flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()

    def step():
        smp.sample_dev_ptrs(d_logits.data_ptr(), dt_code, B, V, V, d_cfgs.data_ptr(), d_uni.data_ptr(),
                            d_ids.data_ptr(), d_flags.data_ptr())

    if args.vocab_sharded:
        lo, hi = workloads.shard_vocab(V, rank, world)
        d_slice = d_logits[:, lo:hi].contiguous()
        del d_logits
        d_rec = torch.empty((B, sampling.VS_RECORD_BYTES), dtype=torch.uint8, device="cuda")
        d_all = torch.empty((world, B, sampling.VS_RECORD_BYTES), dtype=torch.uint8, device="cuda")
        if flush is None and d_slice.numel() * d_slice.element_size() <= 126 * 2 ** 20:
            flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()

        def step():  # noqa: F811
            smp.vocab_local_ptrs(d_slice.data_ptr(), dt_code, B, hi - lo, hi - lo, lo, d_cfgs.data_ptr(), d_rec.data_ptr())
            if world > 1:
                dist.all_gather_into_tensor(d_all.view(-1), d_rec.view(-1))
            else:
                d_all[0].copy_(d_rec)
            smp.vocab_merge_ptrs(d_all.data_ptr(), world, B, V, d_cfgs.data_ptr(), d_uni.data_ptr(),
                                 d_ids.data_ptr(), d_flags.data_ptr())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        if flush is not None:
            flush.zero_()
        step()
    barrier()
    clocks = ClockSampler(local_rank)
    clocks.start()
    K = args.steps
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    launches0 = smp.counters()["kernel_launches"]
    barrier()
    for a, b in evs:
        if flush is not None:
            flush.zero_()
        a.record(stream)
        step()
        b.record(stream)
    barrier()
    launches = smp.counters()["kernel_launches"] - launches0
    kernel_ms = [a.elapsed_time(b) for a, b in evs]
    total_ms = float(sum(kernel_ms))          # device time of the K steps (flush writes excluded)
    # keep the load on for a moment if the timed region was too short for NVML to see it
    t_end = time.perf_counter() + (0.0 if args.profile else max(0.0, 0.6 - total_ms / 1e3))
    while time.perf_counter() < t_end:
        for _ in range(20):
            step()
        torch.cuda.synchronize()
    clk = clocks.stop()

    # end to end through the host-pointer entry point (pinned host memory both ways)
    e2e_s, ke = 0.0, 1
    if not args.no_e2e:
        smp.set_stream(None)
        ke = max(3, min(K, 20))
        def host_step():
            smp.sample_host_ptrs(h_logits.data_ptr(), dt_code, B, V, V, h_cfgs.data_ptr(), h_uni.data_ptr(),
                                 h_ids.data_ptr(), h_flags.data_ptr())
        host_step(); host_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(ke):
            host_step()
        e2e_s = time.perf_counter() - t0
        if not torch.equal(h_ids.cuda(), d_ids):
            raise SystemExit("host and device entry points disagree")
        smp.set_stream(stream.cuda_stream)
    barrier()

    t = torch.tensor([total_ms, e2e_s * 1e3 / ke * K], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms_max, e2e_ms_max = t.tolist()
    if rank == 0:
        peak, peak_kind = peaks()
        rows_total = B * K if args.vocab_sharded else B * world * K
        value = rows_total / (total_ms_max / 1e3)
        alg_bytes = B * w.bytes_per_row
        if args.vocab_sharded:                 # per GPU: its column slice of every row
            alg_bytes = B * (-(-V // world)) * w.logits.dtype.itemsize
        avg_launch_ms = float(np.mean(kernel_ms))
        achieved = alg_bytes / (avg_launch_ms / 1e3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": world, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": total_ms_max / K, "higher_is_better": True,
            "scaling": "strong" if args.vocab_sharded else "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": workload_config(w, args, world),
            "logits_gbs_per_gpu": achieved,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": measured_traffic(w), "peak_source": peak_kind,
                         "kernel": dominant_kernel(w), "algorithmic_bytes_per_launch": alg_bytes,
                         "timed": "whole step (every kernel of the call), CUDA events on the launching stream"},
            "clocks": clk, "gpu_launches": int(launches),
        }
        if e2e_ms_max > 0:
            line["e2e"] = {"value": rows_total / (e2e_ms_max / 1e3), "unit": "rows/s",
                           "h2d_bytes_per_step": int(w.logits.nbytes + B * 24),
                           "d2h_bytes_per_step": int(B * 8)}
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle as orc
            threads = orc.hw_threads()
            probe, _ = time_cpu(w, min(B, threads), threads, 0.0)
            rows = int(min(B, max(threads, probe * args.cpu_seconds / 3)))
            v, reps = time_cpu(w, rows, threads, args.cpu_seconds)
            line["cpu_baseline"] = {"value": v, "unit": "rows/s", "cores": threads, "kind": "port",
                                    "sample": f"first {rows} rows of {w.name}, best of {reps} passes, "
                                              "C++ restatement of the Go routines"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    smp.release()


def dominant_kernel(w):
    """The kernel that does the streaming for this workload (see profiles/)."""
    row_bytes = w.V * w.logits.dtype.itemsize          # the library's dispatch rule (shim.cu: use_batch_mode)
    if not (w.B >= 384 or (w.B >= 32 and w.B * row_bytes >= 24 << 20)):
        return "sample_cluster_kernel"
    if int(w.cfgs["top_k"][0]) > 0 or float(w.cfgs["temperature"][0]) == 0.0:
        return "narrow_rows_kernel"
    return "wide_rows_kernel"


def measured_traffic(w):
    """DRAM bytes per launch of the dominant kernel from the committed ncu capture
    of this workload (profiles/), or None when no capture covers it."""
    path = os.path.join(ROOT, "gorch_b200", "measured_traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f).get(w.name)
        if rec is None or rec.get("rows") != w.B or rec.get("topp_mode") != int(w.cfgs["topp_mode"][0]):
            return None
        return rec["dram_bytes_per_launch"]
    except Exception:
        return None


if __name__ == "__main__":
    main()
