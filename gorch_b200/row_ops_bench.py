"""Times the row ops beside the sampling step on one GPU: softmax / log-softmax / cross-entropy
and the tensor-level TopK / Multinomial.

    python -m gorch_b200.row_ops_bench                       # 512 x 151,936 f32, every op
    python -m gorch_b200.row_ops_bench --rows 1500 --vocab 168320 --op ce_fwd
    python -m gorch_b200.row_ops_bench --rows 192 --op softmax --iters 2 --warmup 1   # small case for a profiler

Synthetic normal logits x 2 (the distribution of the reference's cross-entropy tests,
ce_metal_test.go:44-54). Device time by CUDA events on the launching stream, median over the
iterations, a buffer larger than L2 rewritten between launches. GB/s = algorithmic bytes / time:
softmax and log-softmax read and write the tensor once, the cross-entropy forward reads it once,
the backward reads it and writes f32, TopK (k = 64; moe-style k = 8 with --topk 8) and Multinomial
(over the softmax output, f32) read it once. One JSON line per op."""
from __future__ import annotations

import argparse
import json

import numpy as np


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=512)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16"])
    ap.add_argument("--op", default="all", choices=["all", "softmax", "log_softmax", "ce_fwd", "ce_bwd", "topk", "multinomial"])
    ap.add_argument("--topk", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()

    import ctypes as C

    import torch

    from . import row_ops, sampling

    s = sampling.CudaSampler(0)
    st = torch.cuda.Stream()
    torch.cuda.set_stream(st)
    s.set_stream(st.cuda_stream)
    B, V = a.rows, a.vocab
    tdt = torch.float32 if a.dtype == "f32" else torch.bfloat16
    code = 0 if a.dtype == "f32" else 1
    gen = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(B, V, device="cuda", dtype=torch.float32, generator=gen).mul_(2.0).to(tdt)
    out = torch.empty_like(x)
    dx = torch.empty(B, V, device="cuda", dtype=torch.float32)
    tgt = torch.randint(0, V, (B,), device="cuda", dtype=torch.int32, generator=gen)
    row_loss = torch.empty(B, device="cuda")
    row_lse = torch.empty(B, device="cuda")
    mean = torch.empty(1, device="cuda")
    flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device="cuda")
    es = x.element_size()
    ops = {
        "softmax": (lambda: row_ops.softmax_ptrs(s, x.data_ptr(), code, B, V, V, out.data_ptr(), V, False), 2 * es),
        "log_softmax": (lambda: row_ops.softmax_ptrs(s, x.data_ptr(), code, B, V, V, out.data_ptr(), V, True), 2 * es),
        "ce_fwd": (lambda: row_ops.cross_entropy_fwd_ptrs(s, x.data_ptr(), code, B, V, V, tgt.data_ptr(), row_loss.data_ptr(),
                                                          row_lse.data_ptr(), mean.data_ptr()), es),
        "ce_bwd": (lambda: row_ops.cross_entropy_bwd_ptrs(s, x.data_ptr(), code, B, V, V, tgt.data_ptr(), row_lse.data_ptr(),
                                                          1.0 / B, dx.data_ptr(), V), es + 4),
    }
    k = a.topk
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

    ops["topk"] = (run_topk, es)
    ops["multinomial"] = (run_multinomial, 4)
    # the backward needs a logsumexp to read
    ops["ce_fwd"][0]()
    torch.cuda.synchronize()
    for name, (fn, bytes_per_elem) in ops.items():
        if a.op not in ("all", name):
            continue
        ts = []
        for it in range(a.warmup + a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            fn()
            e1.record(st)
            torch.cuda.synchronize()
            if it >= a.warmup:
                ts.append(e0.elapsed_time(e1) * 1e3)
        us = float(np.median(ts))
        print(json.dumps({"op": name, "rows": B, "vocab": V, "dtype": a.dtype, "us": round(us, 1),
                          "algorithmic_gbs": round(B * V * bytes_per_elem / us / 1e3, 1),
                          "rows_per_s": round(B / us * 1e6)}), flush=True)
    s.set_stream(None)
    s.release()


if __name__ == "__main__":
    main()
