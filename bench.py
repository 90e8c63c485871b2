#!/usr/bin/env python
"""Benchmark of the sampling step: one "step" = one pass of the hot path over
one batch of synthetic logits.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4] [--impl reference]
                  [--no-configs] [--no-ops] [--op NAME --op-rows R --op-vocab V]

Own arm: `value` is rows/s with the batch resident in HBM (device-pointer
entry point, CUDA events on the launching stream); `e2e` is the same metric
through the host-pointer C-ABI call with pinned host buffers, copies inside
the timed region. After the timed region rank 0 compares the timed call's ids
with the CPU oracle and reports the counts under `parity`. At N=1 the same JSON
line also carries `configs` (every other BASELINE config, 20 timed steps each,
with its own parity counts) and `ops` (TopK, Multinomial, softmax, log-softmax,
cross-entropy forward / backward on 512 x 151,936 f32). `--impl reference`
times the CPU restatement of the reference's routines on the host cores. Under
torchrun every rank runs its own rows (no collective on the data path); rank 0
prints one JSON line.
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
L2_BYTES = 126 * 2 ** 20


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
                    help="short run for ncu: no e2e leg, no CPU baseline, no clock hold, no extra legs")
    ap.add_argument("--no-configs", action="store_true", help="skip the leg that times the other configs")
    ap.add_argument("--no-ops", action="store_true", help="skip the leg that times the row ops")
    ap.add_argument("--op", default=None, choices=["softmax", "log_softmax", "ce_fwd", "ce_bwd", "topk", "multinomial", "lm_head"],
                    help="time one row op only (a small case for a profiler), print its line and exit")
    ap.add_argument("--op-rows", type=int, default=512)
    ap.add_argument("--op-vocab", type=int, default=151936)
    ap.add_argument("--op-dtype", default="f32", choices=["f32", "bf16"])
    ap.add_argument("--op-topk", type=int, default=64)
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
        "sharding": (f"vocab x{world}, one ncclAllGather of {world}x{int(w.B)} records inside the library call" if args.vocab_sharded
                     else f"rows x{world}, no collective"),
        "l2": "inputs larger than L2" if w.logits.nbytes > L2_BYTES else "L2 flushed between steps",
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
    in C++: no Go toolchain exists offline), all host threads, rank 0 only, on the
    workload's own row count."""
    if rank != 0:
        return
    from gorch_b200 import workloads
    from oracle import oracle as orc
    orc.build()
    threads = orc.hw_threads()
    w = workloads.make(args.workload, args.rows, args.mode)
    rows = w.B
    sub = (w.logits, w.cfgs, w.uniforms)
    # a step of the largest configs takes about a second of host time: bound the run to a few minutes
    steps = max(1, min(args.steps, 40))
    warm = max(1, min(args.warmup, 3))
    for _ in range(warm):
        orc.sample_batch(*sub, want_info=False, flags=0, threads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.sample_batch(*sub, want_info=False, flags=0, threads=threads)
    dt = time.perf_counter() - t0
    value = rows * steps / dt
    cfg = workload_config(w, args, 1)
    cfg["sharding"] = "host threads over rows"
    cfg["l2"] = "n/a (host arm)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": 1e3 * dt / steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype, "accum_dtype": "f64",
        "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": "port",
                         "sample": f"{rows} rows of {w.name} per step ({steps} of the {args.steps} steps asked for), "
                                   "C++ restatement of the Go routines"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def parity_counts(w, ids, flags, max_rows=None):
    """The timed call's ids against the CPU oracle (rank 0, after the timed region).
    id_mismatch counts every differing id; of those, `excused` rows are the ones the contract
    leaves open: the uniform within 1e-6 of a CDF edge, or a top-p cut inside a group of equal
    probabilities or inside the kernel's rounding band (flagged by the kernel or seen by the oracle)."""
    from gorch_b200.config import FLAG_BOUNDARY, FLAG_TIE_CUT, FLAG_TOPP_EDGE
    from oracle import oracle as orc
    n = w.B if max_rows is None else min(w.B, max_rows)
    ora = orc.sample_batch(w.logits[:n], w.cfgs[:n], w.uniforms[:n], flags=orc.FAST_KTH, threads=orc.hw_threads())
    ids, flags = np.asarray(ids[:n]).astype(np.int64), np.asarray(flags[:n]).astype(np.uint32)
    info = ora["info"]
    u = w.uniforms[:n]
    near = (np.minimum(np.abs(u - info["edge_lo"]), np.abs(u - info["edge_hi"])) <= 1e-6) | ((flags & FLAG_BOUNDARY) != 0)
    soft = ((flags & (FLAG_TIE_CUT | FLAG_TOPP_EDGE)) != 0) | (info["cut_in_tie"] != 0)
    diff = ids != ora["ids"]
    return {"rows_checked": int(n), "id_mismatch": int(diff.sum()), "excused": int((diff & (near | soft)).sum()),
            "unexcused": int((diff & ~(near | soft)).sum()),
            "boundary_rows": int(((flags & FLAG_BOUNDARY) != 0).sum()),
            "tie_cut_rows": int(((flags & FLAG_TIE_CUT) != 0).sum()),
            "topp_edge_rows": int(((flags & FLAG_TOPP_EDGE) != 0).sum())}


def dominant_kernel(w):
    """The kernel that does the streaming for this workload (see profiles/)."""
    row_bytes = w.V * w.logits.dtype.itemsize          # the library's dispatch rule (shim.cu: use_batch_mode)
    if not (w.B >= 384 or (w.B >= 32 and w.B * row_bytes >= 24 << 20)):
        return "sample_cluster_kernel"
    k = w.cfgs["top_k"]
    t = w.cfgs["temperature"]
    narrow = int(((k > 0) | (t == 0.0)).sum())
    if narrow == w.B:
        return "narrow_rows_kernel"
    if narrow == 0:
        return "wide_rows_kernel"
    return "narrow_rows_kernel || wide_rows_kernel"


def measured_traffic(w):
    """DRAM bytes per launch of the dominant kernel from the committed ncu capture
    of this workload (profiles/), scaled to the rows of this launch, or None when no capture covers it."""
    path = os.path.join(ROOT, "gorch_b200", "measured_traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f).get(w.name)
        if rec is None or rec.get("topp_mode") != int(w.cfgs["topp_mode"][0]):
            return None
        return int(rec["dram_bytes_per_row"] * w.B)
    except Exception:
        return None


class DeviceBatch:
    """One workload resident on the device, with a step() that samples it through the device-pointer entry."""

    def __init__(self, torch, smp, w, pinned=False):
        from gorch_b200.config import DTYPE_BF16, DTYPE_F32
        self.w, self.smp = w, smp
        self.code = DTYPE_BF16 if w.dtype == "bf16" else DTYPE_F32
        B = w.B
        h_logits = torch.from_numpy(w.logits.view(np.int16) if w.dtype == "bf16" else w.logits)
        h_cfgs = torch.from_numpy(w.cfgs.view(np.uint8).reshape(B, 16).copy())
        h_uni = torch.from_numpy(w.uniforms.copy())
        if pinned:
            h_logits, h_cfgs, h_uni = h_logits.pin_memory(), h_cfgs.pin_memory(), h_uni.pin_memory()
        self.h_logits, self.h_cfgs, self.h_uni = h_logits, h_cfgs, h_uni
        self.d_logits = h_logits.cuda(non_blocking=True)
        self.d_cfgs = h_cfgs.cuda(non_blocking=True)
        self.d_uni = h_uni.cuda(non_blocking=True)
        self.d_ids = torch.empty(B, dtype=torch.int32, device="cuda")
        self.d_flags = torch.empty(B, dtype=torch.int32, device="cuda")

    def step(self):
        w = self.w
        self.smp.sample_dev_ptrs(self.d_logits.data_ptr(), self.code, w.B, w.V, w.V, self.d_cfgs.data_ptr(),
                                 self.d_uni.data_ptr(), self.d_ids.data_ptr(), self.d_flags.data_ptr())


def time_steps(torch, stream, fn, steps, warmup, flush):
    """Median and mean device time (ms) of fn() over `steps` launches after `warmup`."""
    ts = []
    for it in range(warmup + steps):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        fn()
        e1.record(stream)
        if it >= warmup:
            ts.append((e0, e1))
    torch.cuda.synchronize()
    ms = [a.elapsed_time(b) for a, b in ts]
    return float(np.median(ms)), float(np.mean(ms))


def configs_leg(torch, smp, stream, flush, peak, skip):
    """Every BASELINE config except the headline: 20 timed steps each after 3 warm-up steps, L2 flushed
    between steps where the batch fits in it; step time, rows/s, algorithmic GB/s, fraction of the HBM
    peak, and the parity counts of the last timed call."""
    from gorch_b200 import workloads
    out = {}
    cases = [("c1", "c1", None), ("c2", "c2", None), ("c2_mode_b", "c2", 1), ("c3", "c3", None),
             ("c4_mode_a", "c4", 0), ("c4", "c4", None), ("c5", "c5", None)]
    for key, name, mode in cases:
        if key == skip:
            continue
        w = workloads.make(name, None, mode)
        db = DeviceBatch(torch, smp, w)
        torch.cuda.synchronize()
        fl = flush if w.logits.nbytes <= L2_BYTES else None
        launches0 = smp.counters()["kernel_launches"]
        med, mean = time_steps(torch, stream, db.step, 20, 3, fl)
        launches = smp.counters()["kernel_launches"] - launches0
        gbs = w.B * w.bytes_per_row / (mean / 1e3) / 1e9
        out[key] = {"workload": w.name, "rows": int(w.B), "vocab": int(w.V), "dtype": w.dtype,
                    "topp_mode": int(w.cfgs["topp_mode"][0]),
                    "us_per_step": round(mean * 1e3, 2), "us_median": round(med * 1e3, 2),
                    "rows_per_s": round(w.B / (mean / 1e3)), "gbs": round(gbs, 1), "frac": round(gbs / peak, 4),
                    "kernel": dominant_kernel(w), "launches_per_step": launches // 23,
                    "l2": "inputs larger than L2" if fl is None else "L2 flushed between steps",
                    "parity": parity_counts(w, db.d_ids.cpu().numpy(), db.d_flags.cpu().numpy())}
        del db
        torch.cuda.empty_cache()
    return out


def ops_leg(torch, smp, stream, flush, peak, only=None, rows=512, vocab=151936, dtype="f32", topk=64,
            iters=20, warmup=3):
    """The row ops beside the sampling step on synthetic normal logits x 2 (the distribution of the
    reference's cross-entropy tests, ce_metal_test.go:44-54). GB/s = algorithmic bytes / time: softmax and
    log-softmax read and write the tensor once, the cross-entropy forward reads it once, the backward reads
    it and writes f32, TopK and Multinomial (over the softmax output, f32) read it once."""
    import ctypes as C

    from gorch_b200 import row_ops, sampling
    B, V = rows, vocab
    tdt = torch.float32 if dtype == "f32" else torch.bfloat16
    code = 0 if dtype == "f32" else 1
    gen = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(B, V, device="cuda", dtype=torch.float32, generator=gen).mul_(2.0).to(tdt)
    out = torch.empty_like(x)
    dx = torch.empty(B, V, device="cuda", dtype=torch.float32)
    tgt = torch.randint(0, V, (B,), device="cuda", dtype=torch.int32, generator=gen)
    row_loss = torch.empty(B, device="cuda")
    row_lse = torch.empty(B, device="cuda")
    mean = torch.empty(1, device="cuda")
    es = x.element_size()
    s = smp
    k = min(topk, V)
    tk_val = torch.empty(B, k, device="cuda", dtype=torch.float32)
    tk_idx = torch.empty(B, k, device="cuda", dtype=torch.int32)
    probs = torch.softmax(x.float(), dim=1)
    uni = torch.rand(B, device="cuda", dtype=torch.float64, generator=gen)
    ids = torch.empty(B, device="cuda", dtype=torch.int32)
    flags = torch.empty(B, device="cuda", dtype=torch.int32)

    def run_topk():
        err = C.c_void_p()
        rc = s._lib.gorch_cuda_topk_dev(s._ctx, x.data_ptr(), code, B, V, V, k, tk_val.data_ptr(), tk_idx.data_ptr(),
                                        flags.data_ptr(), C.byref(err))
        sampling._check(s._lib, rc, err)

    def run_multinomial():
        err = C.c_void_p()
        rc = s._lib.gorch_cuda_multinomial_dev(s._ctx, probs.data_ptr(), B, V, V, uni.data_ptr(), ids.data_ptr(),
                                               flags.data_ptr(), C.byref(err))
        sampling._check(s._lib, rc, err)

    ops = {
        "softmax": (lambda: row_ops.softmax_ptrs(s, x.data_ptr(), code, B, V, V, out.data_ptr(), V, False), 2 * es),
        "log_softmax": (lambda: row_ops.softmax_ptrs(s, x.data_ptr(), code, B, V, V, out.data_ptr(), V, True), 2 * es),
        "ce_fwd": (lambda: row_ops.cross_entropy_fwd_ptrs(s, x.data_ptr(), code, B, V, V, tgt.data_ptr(), row_loss.data_ptr(),
                                                          row_lse.data_ptr(), mean.data_ptr()), es),
        "ce_bwd": (lambda: row_ops.cross_entropy_bwd_ptrs(s, x.data_ptr(), code, B, V, V, tgt.data_ptr(), row_lse.data_ptr(),
                                                          1.0 / B, dx.data_ptr(), V), es + 4),
        "topk": (run_topk, es),
        "multinomial": (run_multinomial, 4),
    }
    ops["ce_fwd"][0]()                      # the backward needs a logsumexp to read
    torch.cuda.synchronize()
    res = {}
    for name, (fn, bytes_per_elem) in ops.items():
        if only not in (None, name):
            continue
        med, _ = time_steps(torch, stream, fn, iters, warmup, flush)
        gbs = B * V * bytes_per_elem / (med / 1e3) / 1e9
        res[name] = {"rows": B, "vocab": V, "dtype": dtype, "us": round(med * 1e3, 1), "gbs": round(gbs, 1),
                     "frac": round(gbs / peak, 4)}
        if name == "topk":
            res[name]["k"] = k
    return res


def lm_head_leg(torch, smp, stream, flush, peak, batches=(64, 512), V=151936, K=1024, iters=20, warmup=3):
    """The projection in front of the sampling step (model/qwen/qwen.go:80-85) under the reference's
    DefaultGenerateConfig (T = 0.8, top_k = 40): random bf16 activations and weights of the Qwen3-0.6B
    LM head's shape. Times the projection alone (logits written), projection + sampling unfused (logits
    through HBM) and fused (no logits written); GB/s = the weight matrix read once / time."""
    from gorch_b200.config import CFG_DTYPE
    gen = torch.Generator(device="cuda").manual_seed(2)
    w = (torch.randn(V, K, device="cuda", generator=gen) * 0.08).to(torch.bfloat16)
    res = {}
    for B in batches:
        x = (torch.randn(B, K, device="cuda", generator=gen) * 0.5).to(torch.bfloat16)
        out = torch.empty(B, V, device="cuda", dtype=torch.float32)
        cfgs = np.zeros(B, dtype=CFG_DTYPE)
        cfgs["temperature"], cfgs["top_k"] = 0.8, 40
        dc = torch.from_numpy(cfgs.view(np.uint8).reshape(B, 16).copy()).cuda()
        du = torch.rand(B, device="cuda", dtype=torch.float64, generator=gen)
        ids = torch.empty(B, device="cuda", dtype=torch.int32)
        fl = torch.empty(B, device="cuda", dtype=torch.int32)
        ids_u = torch.empty(B, device="cuda", dtype=torch.int32)
        proj = lambda: smp.lm_head_logits_ptrs(x.data_ptr(), K, w.data_ptr(), K, B, V, K, out.data_ptr(), V)
        unf = lambda: smp.lm_head_sample_ptrs(x.data_ptr(), K, w.data_ptr(), K, B, V, K, 0, dc.data_ptr(), du.data_ptr(),
                                              ids_u.data_ptr(), fl.data_ptr())
        fus = lambda: smp.lm_head_sample_ptrs(x.data_ptr(), K, w.data_ptr(), K, B, V, K, 40, dc.data_ptr(), du.data_ptr(),
                                              ids.data_ptr(), fl.data_ptr())
        refused0 = smp.counters()["lm_head_refused_rows"]
        t_proj, _ = time_steps(torch, stream, proj, iters, warmup, flush)
        t_unf, _ = time_steps(torch, stream, unf, iters, warmup, flush)
        t_fus, _ = time_steps(torch, stream, fus, iters, warmup, flush)
        wbytes = V * K * 2
        res[f"b{B}"] = {"rows": B, "vocab": V, "hidden": K, "config": "T=0.8 top_k=40",
                        "projection_us": round(t_proj * 1e3, 1), "unfused_us": round(t_unf * 1e3, 1),
                        "fused_us": round(t_fus * 1e3, 1),
                        "fused_weight_gbs": round(wbytes / (t_fus / 1e3) / 1e9, 1),
                        "fused_frac_of_hbm_peak": round(wbytes / (t_fus / 1e3) / 1e9 / peak, 4),
                        "projection_tflops": round(2.0 * B * V * K / (t_proj / 1e3) / 1e12, 1),
                        "fused_equals_unfused_ids": bool(torch.equal(ids, ids_u)),
                        "rows_redone_unfused": int(smp.counters()["lm_head_refused_rows"] - refused0)}
    return res


def main():
    args = parse()
    if args.profile:
        args.no_e2e = args.no_cpu_baseline = args.no_configs = args.no_ops = True
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from gorch_b200 import build, sampling, workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    build.build()
    peak, peak_kind = peaks()
    smp = sampling.CudaSampler(local_rank)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    smp.set_stream(stream.cuda_stream)

    if args.op is not None:                  # one row op, for a profiler
        flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device="cuda")
        if args.op == "lm_head":
            res = lm_head_leg(torch, smp, stream, flush, peak, batches=(args.op_rows,), V=args.op_vocab,
                              iters=max(1, args.steps if args.steps < 200 else 20), warmup=max(1, args.warmup))
            print(json.dumps({"op": "lm_head", **res[f"b{args.op_rows}"]}), flush=True)
            smp.set_stream(None)
            smp.release()
            return
        res = ops_leg(torch, smp, stream, flush, peak, only=args.op, rows=args.op_rows, vocab=args.op_vocab,
                      dtype=args.op_dtype, topk=args.op_topk, iters=max(1, args.steps if args.steps < 200 else 20),
                      warmup=max(1, args.warmup))
        print(json.dumps({"op": args.op, **res[args.op]}), flush=True)
        smp.set_stream(None)
        smp.release()
        return

    workloads.set_shard(0 if args.vocab_sharded else rank)
    if args.vocab_sharded:
        args.no_e2e = True
    w = workloads.make(args.workload, args.rows, args.mode)
    B, V = w.B, w.V
    db = DeviceBatch(torch, smp, w, pinned=True)
    dt_code = db.code
    h_ids = torch.empty(B, dtype=torch.int32).pin_memory()
    h_flags = torch.empty(B, dtype=torch.int32).pin_memory()
    d_ids, d_flags = db.d_ids, db.d_flags
    extra_legs = world == 1 and not args.vocab_sharded and not (args.no_configs and args.no_ops)
    flush = None
    if w.logits.nbytes <= L2_BYTES or extra_legs:
        flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device="cuda")
    main_flush = flush if w.logits.nbytes <= L2_BYTES else None
    torch.cuda.synchronize()
    step = db.step
    phases = None

    if args.vocab_sharded:
        from gorch_b200 import distributed
        lo, hi = workloads.shard_vocab(V, rank, world)
        d_slice = db.d_logits[:, lo:hi].contiguous()
        db.d_logits = None
        distributed.init_vocab_comm(smp, rank, world)       # the library's own NCCL communicator
        max_k = int(w.cfgs["top_k"].max())
        if main_flush is None and d_slice.numel() * d_slice.element_size() <= L2_BYTES:
            main_flush = flush if flush is not None else torch.empty(256 * 2 ** 20, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()

        def step():  # noqa: F811
            distributed.sample_vocab_sharded_device(smp, d_slice, db.d_cfgs, db.d_uni, d_ids, d_flags, V, rank, world, max_k)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        if main_flush is not None:
            main_flush.zero_()
        step()
    barrier()
    clocks = ClockSampler(local_rank)
    clocks.start()
    K = args.steps
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    launches0 = smp.counters()["kernel_launches"]
    barrier()
    for a, b in evs:
        if main_flush is not None:
            main_flush.zero_()
        a.record(stream)
        step()
        b.record(stream)
    barrier()
    launches = smp.counters()["kernel_launches"] - launches0
    kernel_ms = [a.elapsed_time(b) for a, b in evs]
    total_ms = float(sum(kernel_ms))          # device time of the K steps (flush writes excluded)
    if args.vocab_sharded:
        # per-phase device times of one more step (the timing switch adds a sync, so not inside the timed region)
        smp.set_timing(True)
        step()
        torch.cuda.synchronize()
        cn = smp.counters()
        smp.set_timing(False)
        cand = ((max_k + max_k // 4 + 8 + 7) // 8) * 8 if 0 < max_k <= sampling.VS_CAND else sampling.VS_CAND
        cand = min(cand, sampling.VS_CAND)
        phases = {"local_us": round(cn["vs_local_ms"] * 1e3, 1), "all_gather_us": round(cn["vs_gather_ms"] * 1e3, 1),
                  "merge_us": round(cn["vs_merge_ms"] * 1e3, 1), "record_bytes": 16 + 8 * cand,
                  "gathered_bytes_per_rank": int(B * (16 + 8 * cand) * world),
                  "of": "one extra step on rank 0, CUDA events inside the library call"}
    timed_ids, timed_flags = d_ids.cpu().numpy().copy(), d_flags.cpu().numpy().copy()
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
            smp.sample_host_ptrs(db.h_logits.data_ptr(), dt_code, B, V, V, db.h_cfgs.data_ptr(), db.h_uni.data_ptr(),
                                 h_ids.data_ptr(), h_flags.data_ptr())
        host_step(); host_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(ke):
            host_step()
        e2e_s = time.perf_counter() - t0
        if not np.array_equal(h_ids.numpy(), timed_ids):
            raise SystemExit("host and device entry points disagree")
        smp.set_stream(stream.cuda_stream)
    barrier()

    t = torch.tensor([total_ms, e2e_s * 1e3 / ke * K], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms_max, e2e_ms_max = t.tolist()
    if rank == 0:
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
            "scaling": "strong" if args.vocab_sharded else "weak", "vs_baseline": None,
            "dtype": w.dtype, "accum_dtype": "f64", "data": "synthetic",
            "config": workload_config(w, args, world),
            "logits_gbs_per_gpu": achieved,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": None if args.vocab_sharded else measured_traffic(w),
                         "peak_source": peak_kind,
                         "kernel": dominant_kernel(w), "algorithmic_bytes_per_launch": alg_bytes,
                         "timed": "whole step (every kernel of the call), CUDA events on the launching stream"},
            "clocks": clk, "gpu_launches": int(launches),
            "parity": parity_counts(w, timed_ids, timed_flags),
        }
        if phases is not None:
            line["phases"] = phases
        if e2e_ms_max > 0:
            line["e2e"] = {"value": rows_total / (e2e_ms_max / 1e3), "unit": "rows/s",
                           "h2d_bytes_per_step": int(w.logits.nbytes + B * 24),
                           "d2h_bytes_per_step": int(B * 8)}
        if extra_legs:
            # the other configs and the row ops, device-resident, on this same GPU
            db = None
            torch.cuda.empty_cache()
            if not args.no_configs:
                line["configs"] = configs_leg(torch, smp, stream, flush, peak,
                                              skip=args.workload if args.rows is None and args.mode is None else None)
            if not args.no_ops:
                line["ops"] = ops_leg(torch, smp, stream, flush, peak)
                line["lm_head"] = lm_head_leg(torch, smp, stream, flush, peak)
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
    smp.set_stream(None)
    smp.release()


if __name__ == "__main__":
    main()
