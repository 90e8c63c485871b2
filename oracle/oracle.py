"""ctypes front end for the CPU oracle (libgorch_oracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg. Nothing in the gorch_b200 package imports it.

The library is the C++ restatement in gorch_sampling_oracle.cpp of the
reference's model/generate.go:134-260 and model/qwen/generate.go:77-181.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libgorch_oracle.so")

MODE_A = 0  # model/generate.go:184-228
MODE_B = 1  # model/qwen/generate.go:123-153
FAST_KTH = 1

CFG_DTYPE = np.dtype(
    [("temperature", "<f4"), ("top_k", "<i4"), ("top_p", "<f4"), ("topp_mode", "<i4")]
)

INFO_DTYPE = np.dtype(
    [
        ("kept", "<i8"),
        ("sum_exp", "<f8"),
        ("resum", "<f8"),
        ("edge_lo", "<f8"),
        ("edge_hi", "<f8"),
        ("fallback", "<i4"),
        ("cut_in_tie", "<i4"),
        ("cut_cum", "<f8"),
        ("max_scaled", "<f4"),
        ("threshold", "<f4"),
    ],
    align=True,
)


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it; returns the .so path."""
    src = os.path.join(_HERE, "gorch_sampling_oracle.cpp")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "libgorch_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.gorch_oracle_argmax_f32.restype = C.c_int64
        L.gorch_oracle_argmax_f32.argtypes = [C.c_void_p, C.c_int64]
        L.gorch_oracle_kth_largest_f32.restype = C.c_float
        L.gorch_oracle_kth_largest_f32.argtypes = [C.c_void_p, C.c_int64, C.c_int64]
        L.gorch_oracle_sample_f32.restype = C.c_int64
        L.gorch_oracle_sample_f32.argtypes = [
            C.c_void_p, C.c_int64, C.c_float, C.c_int64, C.c_float, C.c_int32,
            C.c_double, C.c_void_p, C.c_void_p, C.c_int32,
        ]
        L.gorch_oracle_sample_batch.restype = None
        L.gorch_oracle_sample_batch.argtypes = [
            C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
            C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
        ]
        L.gorch_oracle_topk_f32.restype = C.c_int32
        L.gorch_oracle_topk_f32.argtypes = [
            C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
        ]
        L.gorch_oracle_multinomial_f32.restype = None
        L.gorch_oracle_multinomial_f32.argtypes = [
            C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
        ]
        L.gorch_oracle_generate_scripted.restype = C.c_int64
        L.gorch_oracle_generate_scripted.argtypes = [
            C.c_int32, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int64,
            C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
        ]
        L.gorch_oracle_softmax_f32.restype = None
        L.gorch_oracle_softmax_f32.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
        L.gorch_oracle_log_softmax_f32.restype = None
        L.gorch_oracle_log_softmax_f32.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]
        L.gorch_oracle_cross_entropy_fwd_f32.restype = C.c_float
        L.gorch_oracle_cross_entropy_fwd_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
        L.gorch_oracle_cross_entropy_bwd_f32.restype = None
        L.gorch_oracle_cross_entropy_bwd_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_float, C.c_void_p]
        L.gorch_oracle_bf16_to_f32.restype = C.c_float
        L.gorch_oracle_bf16_to_f32.argtypes = [C.c_uint16]
        L.gorch_oracle_f32_to_bf16.restype = C.c_uint16
        L.gorch_oracle_f32_to_bf16.argtypes = [C.c_float]
        L.gorch_oracle_hw_threads.restype = C.c_int32
        L.gorch_oracle_hw_threads.argtypes = []
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def argmax(logits) -> int:
    x = _f32(logits)
    return int(lib().gorch_oracle_argmax_f32(x.ctypes.data, x.size))


def kth_largest(data, k: int) -> float:
    x = _f32(data)
    return float(lib().gorch_oracle_kth_largest_f32(x.ctypes.data, x.size, int(k)))


def sample(logits, temperature, top_k, top_p, u, mode=MODE_A, want_probs=False, flags=0):
    """One row through sample (mode A) / sampleLogits (mode B).

    Returns (id, info) or (id, info, probs)."""
    x = _f32(logits)
    info = np.zeros(1, dtype=INFO_DTYPE)
    probs = np.empty(x.size, dtype=np.float64) if want_probs else None
    tok = lib().gorch_oracle_sample_f32(
        x.ctypes.data, x.size, float(temperature), int(top_k), float(top_p), int(mode),
        float(u), probs.ctypes.data if want_probs else None, info.ctypes.data, int(flags),
    )
    if want_probs:
        return int(tok), info[0], probs
    return int(tok), info[0]


def make_cfgs(B, temperature=1.0, top_k=0, top_p=0.0, mode=MODE_A) -> np.ndarray:
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    cfgs["temperature"] = temperature
    cfgs["top_k"] = top_k
    cfgs["top_p"] = top_p
    cfgs["topp_mode"] = mode
    return cfgs


def sample_batch(logits, cfgs, uniforms, want_probs=False, want_info=True, flags=0, threads=1):
    """A [B,V] batch. logits: float32, or uint16 holding bf16 bit patterns.

    Returns dict(ids, probs|None, info|None)."""
    x = np.ascontiguousarray(logits)
    if x.dtype == np.uint16:
        dtype = 1
    else:
        x = _f32(x)
        dtype = 0
    B, V = x.shape
    cfgs = np.ascontiguousarray(cfgs, dtype=CFG_DTYPE)
    uniforms = np.ascontiguousarray(uniforms, dtype=np.float64)
    assert cfgs.shape == (B,) and uniforms.shape == (B,)
    ids = np.empty(B, dtype=np.int64)
    probs = np.empty((B, V), dtype=np.float64) if want_probs else None
    info = np.zeros(B, dtype=INFO_DTYPE) if want_info else None
    lib().gorch_oracle_sample_batch(
        x.ctypes.data, dtype, B, V, V, cfgs.ctypes.data, uniforms.ctypes.data,
        ids.ctypes.data, probs.ctypes.data if want_probs else None,
        info.ctypes.data if want_info else None, int(flags), int(threads),
    )
    return {"ids": ids, "probs": probs, "info": info}


def topk(x, k: int):
    x = _f32(x)
    B, V = x.shape
    k = int(k)
    values = np.empty((B, max(k, 0)), dtype=np.float32)
    indices = np.empty((B, max(k, 0)), dtype=np.int64)
    rc = lib().gorch_oracle_topk_f32(x.ctypes.data, B, V, k, values.ctypes.data,
                                     indices.ctypes.data)
    if rc != 0:
        raise ValueError(f"TopK k={k} out of range [1, {V}]")  # index_ops.go:158-160
    return values, indices


def multinomial(probs, uniforms) -> np.ndarray:
    p = _f32(probs)
    B, V = p.shape
    u = np.ascontiguousarray(uniforms, dtype=np.float64)
    out = np.empty(B, dtype=np.int64)
    lib().gorch_oracle_multinomial_f32(p.ctypes.data, B, V, u.ctypes.data, out.ctypes.data)
    return out


def generate_scripted(loop: int, prompt, script, max_new: int, max_seq: int, stops=()) -> dict:
    """The reference's generate loop `loop` (0 GenerateWithConfig uncached, 1 generateCached,
    2 qwen.Generate) with the sampler's answers taken from `script`."""
    pr = np.ascontiguousarray(prompt, dtype=np.int64)
    sc = np.full(max(int(max_new), 1), -1, dtype=np.int64)    # a script that ends early reads -1
    sc[: min(len(script), sc.size)] = np.asarray(script, dtype=np.int64)[: sc.size]
    st = np.ascontiguousarray(list(stops), dtype=np.int64)
    out = np.empty(pr.size + max(int(max_new), 0), dtype=np.int64)
    fed = np.empty(max(int(max_new), 1), dtype=np.int64)
    reason = C.c_int32(0)
    calls = C.c_int64(0)
    n_fed = C.c_int64(0)
    n = lib().gorch_oracle_generate_scripted(
        int(loop), pr.ctypes.data, pr.size, sc.ctypes.data, int(max_new), int(max_seq), st.ctypes.data, st.size,
        out.ctypes.data, C.byref(reason), C.byref(calls), fed.ctypes.data, C.byref(n_fed))
    return {"tokens": out[:n].tolist(), "reason": int(reason.value), "sampler_calls": int(calls.value),
            "fed": fed[: n_fed.value].tolist()}


def softmax(x, log: bool = False) -> np.ndarray:
    """gorch.Softmax / gorch.LogSoftmax forward over f32 [B,V] (ops.go:527-551, :566-593)."""
    a = _f32(x)
    B, V = a.shape
    out = np.empty_like(a)
    fn = lib().gorch_oracle_log_softmax_f32 if log else lib().gorch_oracle_softmax_f32
    fn(a.ctypes.data, B, V, out.ctypes.data)
    return out


def cross_entropy_fwd(x, targets):
    """ceForwardCPU + the mean (loss.go:83, :108-124): (mean loss, row_loss [B], row_lse [B])."""
    a = _f32(x)
    B, V = a.shape
    t = np.ascontiguousarray(targets, dtype=np.int32)
    assert t.shape == (B,) and t.min() >= 0 and t.max() < V
    row_loss = np.empty(B, dtype=np.float32)
    row_lse = np.empty(B, dtype=np.float32)
    mean = lib().gorch_oracle_cross_entropy_fwd_f32(a.ctypes.data, t.ctypes.data, B, V, row_loss.ctypes.data, row_lse.ctypes.data)
    return float(mean), row_loss, row_lse


def cross_entropy_bwd(x, targets, row_lse, scale: float) -> np.ndarray:
    """ceBackwardCPU (loss.go:128-141)."""
    a = _f32(x)
    B, V = a.shape
    t = np.ascontiguousarray(targets, dtype=np.int32)
    lse = _f32(row_lse)
    dx = np.empty_like(a)
    lib().gorch_oracle_cross_entropy_bwd_f32(a.ctypes.data, t.ctypes.data, lse.ctypes.data, B, V, float(scale), dx.ctypes.data)
    return dx


def f32_to_bf16_bits(a) -> np.ndarray:
    """tensor.go:85-94 vectorised: float32 -> bf16 bit patterns (uint16), RNE."""
    bits = _f32(a).view(np.uint32)
    is_nan = (((bits >> 23) & 0xFF) == 0xFF) & ((bits & 0x7FFFFF) != 0)
    rounding = np.uint32(0x7FFF) + ((bits >> 16) & np.uint32(1))
    out = ((bits + rounding) >> 16).astype(np.uint16)
    out_nan = ((bits >> 16) | np.uint32(0x40)).astype(np.uint16)
    return np.where(is_nan, out_nan, out)


def bf16_bits_to_f32(a) -> np.ndarray:
    """tensor.go:96-99 vectorised."""
    return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def hw_threads() -> int:
    return int(lib().gorch_oracle_hw_threads())
