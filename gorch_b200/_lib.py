"""ctypes binding of libgorchcuda.so (the C ABI in include/gorch_cuda_shim.h).

There is no fallback: if the shared library is missing or cannot be loaded,
importing a symbol raises. The library is looked up in-tree only.
"""
from __future__ import annotations

import ctypes as C
import os

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libgorchcuda.so")

# every symbol include/gorch_cuda_shim.h declares
EXPORTS = [
    "gorch_cuda_device_count", "gorch_cuda_create_ctx", "gorch_cuda_release",
    "gorch_cuda_free_string", "gorch_cuda_sync", "gorch_cuda_set_stream",
    "gorch_cuda_set_timing", "gorch_cuda_get_counters", "gorch_cuda_set_kernel_variant",
    "gorch_cuda_buffer_alloc", "gorch_cuda_buffer_free", "gorch_cuda_buffer_length",
    "gorch_cuda_buffer_device_ptr", "gorch_cuda_buffer_upload", "gorch_cuda_buffer_download",
    "gorch_cuda_sample_host", "gorch_cuda_sample_dev", "gorch_cuda_sample_dev_static", "gorch_cuda_sample_row",
    "gorch_cuda_argmax_host", "gorch_cuda_argmax_dev",
    "gorch_cuda_vocab_local_dev", "gorch_cuda_vocab_merge_dev", "gorch_cuda_vocab_merge_owner_dev", "gorch_cuda_vocab_draw_dev",
    "gorch_cuda_sample_vocab_sharded_ex_dev",
    "gorch_cuda_comm_unique_id", "gorch_cuda_comm_init", "gorch_cuda_comm_release", "gorch_cuda_sample_vocab_sharded_dev",
    "gorch_cuda_topk_dev", "gorch_cuda_multinomial_dev",
    "gorch_cuda_lm_head_logits_dev", "gorch_cuda_lm_head_status", "gorch_cuda_lm_head_sample_dev",
    "gorch_cuda_generate_control_dev", "gorch_cuda_generate_step_dev",
    "gorch_cuda_softmax_dev", "gorch_cuda_cross_entropy_fwd_dev", "gorch_cuda_cross_entropy_bwd_dev",
]


GEN_MAX_STOPS = 16   # GORCH_GEN_MAX_STOPS


class GenControl(C.Structure):
    """GorchGenControl of include/gorch_cuda_shim.h."""
    _fields_ = [
        ("tokens", C.c_void_p), ("capacity", C.c_int64), ("lengths", C.c_void_p), ("n_new", C.c_void_p),
        ("cache_len", C.c_void_p), ("done", C.c_void_p), ("next_input", C.c_void_p), ("window_start", C.c_void_p),
        ("live_count", C.c_void_p), ("stop_tokens", C.c_int32 * GEN_MAX_STOPS), ("n_stop", C.c_int32),
        ("max_new", C.c_int32), ("max_seq", C.c_int32), ("cached", C.c_int32),
    ]


class Counters(C.Structure):
    _fields_ = [
        ("sample_launches", C.c_uint64), ("kernel_launches", C.c_uint64), ("argmax_launches", C.c_uint64), ("rows", C.c_uint64),
        ("h2d_bytes", C.c_uint64), ("d2h_bytes", C.c_uint64), ("last_kernel_ms", C.c_float),
        ("vs_local_ms", C.c_float), ("vs_gather_ms", C.c_float), ("vs_merge_ms", C.c_float),
        ("lm_head_refused_rows", C.c_uint64),
    ]


_lib = None


def load() -> C.CDLL:
    """Load libgorchcuda.so; raises RuntimeError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m gorch_b200.build` "
            "(there is no CPU fallback)")
    L = C.CDLL(LIB_PATH)
    p, i32, i64, f32, f64 = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_double
    err = C.POINTER(C.c_void_p)
    sig = {
        "gorch_cuda_device_count": (i32, [C.POINTER(i32), err]),
        "gorch_cuda_create_ctx": (p, [i32, err]),
        "gorch_cuda_release": (None, [p]),
        "gorch_cuda_free_string": (None, [p]),
        "gorch_cuda_sync": (i32, [p, err]),
        "gorch_cuda_set_stream": (i32, [p, p, i32, err]),
        "gorch_cuda_set_timing": (i32, [p, i32]),
        "gorch_cuda_get_counters": (i32, [p, C.POINTER(Counters)]),
        "gorch_cuda_set_kernel_variant": (i32, [p, i32, i32, err]),
        "gorch_cuda_buffer_alloc": (p, [p, C.c_uint64, err]),
        "gorch_cuda_buffer_free": (None, [p]),
        "gorch_cuda_buffer_length": (C.c_uint64, [p]),
        "gorch_cuda_buffer_device_ptr": (p, [p]),
        "gorch_cuda_buffer_upload": (i32, [p, C.c_uint64, p, C.c_uint64, err]),
        "gorch_cuda_buffer_download": (i32, [p, C.c_uint64, p, C.c_uint64, err]),
        "gorch_cuda_sample_host": (i32, [p, p, i32, i64, i64, i64, p, p, p, p, err]),
        "gorch_cuda_sample_dev": (i32, [p, p, i32, i64, i64, i64, p, p, p, p, p, p, err]),
        "gorch_cuda_sample_dev_static": (i32, [p, p, i32, i64, i64, i64, p, p, p, p, err]),
        "gorch_cuda_sample_row": (i64, [p, p, i64, f32, i64, f32, i32, f64, C.POINTER(C.c_uint32), err]),
        "gorch_cuda_argmax_host": (i32, [p, p, i32, i64, i64, i64, p, err]),
        "gorch_cuda_argmax_dev": (i32, [p, p, i32, i64, i64, i64, p, err]),
        "gorch_cuda_vocab_local_dev": (i32, [p, p, i32, i64, i64, i64, i64, p, p, err]),
        "gorch_cuda_vocab_merge_dev": (i32, [p, p, i32, i64, i64, p, p, p, p, err]),
        "gorch_cuda_vocab_merge_owner_dev": (i32, [p, p, i32, i32, i64, i64, p, p, p, p, p, err]),
        "gorch_cuda_vocab_draw_dev": (i32, [p, p, i32, i64, i64, i64, i64, p, p, p, p, err]),
        "gorch_cuda_sample_vocab_sharded_ex_dev": (i32, [p, p, i32, i64, i64, i64, i64, i64, i32, i32, p, p, p, p, err]),
        "gorch_cuda_comm_unique_id": (i32, [p, err]),
        "gorch_cuda_comm_init": (i32, [p, i32, i32, p, err]),
        "gorch_cuda_comm_release": (i32, [p, err]),
        "gorch_cuda_sample_vocab_sharded_dev": (i32, [p, p, i32, i64, i64, i64, i64, i64, i32, p, p, p, p, err]),
        "gorch_cuda_lm_head_logits_dev": (i32, [p, p, i64, p, i64, i64, i64, i64, p, i64, err]),
        "gorch_cuda_lm_head_status": (i32, [p, C.POINTER(C.c_uint32), err]),
        "gorch_cuda_lm_head_sample_dev": (i32, [p, p, i64, p, i64, i64, i64, i64, i32, p, p, p, p, err]),
        "gorch_cuda_topk_dev": (i32, [p, p, i32, i64, i64, i64, i64, p, p, p, err]),
        "gorch_cuda_multinomial_dev": (i32, [p, p, i64, i64, i64, p, p, p, err]),
        "gorch_cuda_softmax_dev": (i32, [p, p, i32, i64, i64, i64, p, i64, i32, err]),
        "gorch_cuda_cross_entropy_fwd_dev": (i32, [p, p, i32, i64, i64, i64, p, p, p, p, err]),
        "gorch_cuda_cross_entropy_bwd_dev": (i32, [p, p, i32, i64, i64, i64, p, p, f32, p, i64, err]),
        "gorch_cuda_generate_control_dev": (i32, [p, p, p, C.POINTER(GenControl), i64, err]),
        "gorch_cuda_generate_step_dev": (i32, [p, p, i32, i64, i64, i64, p, p, p, p, C.POINTER(GenControl), err]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L
