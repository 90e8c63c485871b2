"""gorch.Softmax, gorch.LogSoftmax and gorch.CrossEntropyLoss (forward and backward) over [B, V]
logits at vocabulary scale, on the device (ops.go:527-603, loss.go:55-141).

The `*_ptrs` functions take device pointers and are asynchronous on the context's stream; the
array functions upload, run, and download (tests and small jobs). Without the CUDA library every
call raises."""
from __future__ import annotations

import ctypes as C

import numpy as np

from .sampling import CudaSampler, _check, _logits_arg


def softmax_ptrs(s: CudaSampler, x_ptr: int, dtype: int, B: int, V: int, row_stride: int, out_ptr: int,
                 out_stride: int, log: bool = False) -> None:
    err = C.c_void_p()
    rc = s._lib.gorch_cuda_softmax_dev(s._ctx, x_ptr, dtype, B, V, row_stride, out_ptr, out_stride, 1 if log else 0, C.byref(err))
    _check(s._lib, rc, err)


def cross_entropy_fwd_ptrs(s: CudaSampler, logits_ptr: int, dtype: int, B: int, V: int, row_stride: int,
                           targets_ptr: int, row_loss_ptr: int, row_lse_ptr: int, mean_ptr: int | None) -> None:
    err = C.c_void_p()
    rc = s._lib.gorch_cuda_cross_entropy_fwd_dev(s._ctx, logits_ptr, dtype, B, V, row_stride, targets_ptr,
                                                 row_loss_ptr, row_lse_ptr, mean_ptr, C.byref(err))
    _check(s._lib, rc, err)


def cross_entropy_bwd_ptrs(s: CudaSampler, logits_ptr: int, dtype: int, B: int, V: int, row_stride: int,
                           targets_ptr: int, row_lse_ptr: int, scale: float, dx_ptr: int, dx_stride: int) -> None:
    err = C.c_void_p()
    rc = s._lib.gorch_cuda_cross_entropy_bwd_dev(s._ctx, logits_ptr, dtype, B, V, row_stride, targets_ptr,
                                                 row_lse_ptr, float(scale), dx_ptr, dx_stride, C.byref(err))
    _check(s._lib, rc, err)


class _Bufs:
    """Device buffers freed together."""

    def __init__(self, s: CudaSampler):
        self.s, self.held = s, []

    def new(self, arr_or_bytes) -> int:
        if isinstance(arr_or_bytes, np.ndarray):
            b = self.s._buf(max(arr_or_bytes.nbytes, 16))
            self.held.append(b)
            if arr_or_bytes.nbytes:
                self.s._upload(b, np.ascontiguousarray(arr_or_bytes))
        else:
            b = self.s._buf(max(int(arr_or_bytes), 16))
            self.held.append(b)
        return b

    def ptr(self, b: int) -> int:
        return self.s._lib.gorch_cuda_buffer_device_ptr(b)

    def free(self) -> None:
        for b in self.held:
            self.s._lib.gorch_cuda_buffer_free(b)
        self.held = []


def softmax(s: CudaSampler, x, log: bool = False) -> np.ndarray:
    """x [B,V] float32, or uint16 bf16 bit patterns -> same shape and type."""
    a, dtype = _logits_arg(x)
    B, V = a.shape
    out = np.empty_like(a)
    bufs = _Bufs(s)
    try:
        b_x, b_o = bufs.new(a), bufs.new(a.nbytes)
        softmax_ptrs(s, bufs.ptr(b_x), dtype, B, V, V, bufs.ptr(b_o), V, log)
        s.sync()
        if out.nbytes:
            s._download(b_o, out)
    finally:
        bufs.free()
    return out


def cross_entropy(s: CudaSampler, logits, targets):
    """-> (mean loss, row_loss [B] f32, row_lse [B] f32)."""
    a, dtype = _logits_arg(logits)
    B, V = a.shape
    t = np.ascontiguousarray(targets, dtype=np.int32).reshape(B)
    row_loss, row_lse, mean = np.empty(B, np.float32), np.empty(B, np.float32), np.zeros(1, np.float32)
    bufs = _Bufs(s)
    try:
        b_x, b_t = bufs.new(a), bufs.new(t)
        b_l, b_e, b_m = bufs.new(4 * B), bufs.new(4 * B), bufs.new(mean)
        cross_entropy_fwd_ptrs(s, bufs.ptr(b_x), dtype, B, V, V, bufs.ptr(b_t), bufs.ptr(b_l), bufs.ptr(b_e), bufs.ptr(b_m))
        s.sync()
        if B:
            s._download(b_l, row_loss)
            s._download(b_e, row_lse)
            s._download(b_m, mean)
    finally:
        bufs.free()
    return float(mean[0]), row_loss, row_lse


def cross_entropy_backward(s: CudaSampler, logits, targets, row_lse, scale: float) -> np.ndarray:
    """-> dx [B,V] float32."""
    a, dtype = _logits_arg(logits)
    B, V = a.shape
    t = np.ascontiguousarray(targets, dtype=np.int32).reshape(B)
    lse = np.ascontiguousarray(row_lse, dtype=np.float32).reshape(B)
    dx = np.empty((B, V), dtype=np.float32)
    bufs = _Bufs(s)
    try:
        b_x, b_t, b_e, b_d = bufs.new(a), bufs.new(t), bufs.new(lse), bufs.new(dx.nbytes)
        cross_entropy_bwd_ptrs(s, bufs.ptr(b_x), dtype, B, V, V, bufs.ptr(b_t), bufs.ptr(b_e), scale, bufs.ptr(b_d), V)
        s.sync()
        if dx.nbytes:
            s._download(b_d, dx)
    finally:
        bufs.free()
    return dx
