"""The reference's generate loops for a batch of sequences with the loop control on the device.

`GenerateWithConfig` / `generateCached` (model/generate.go:52-131) and `qwen.Generate`
(model/qwen/generate.go:35-62) read every sampled id back to the host to test the stop token,
the iteration limit and MaxSeq before the next forward. Here the sampled ids, the growing
results and the per-sequence state live in device memory; each decode step is one call
(`DeviceGenerateState.step`: the sampling kernels plus one control launch), and the host only
looks at a live-row counter every few steps.

The model is the caller's: anything with `forward_dev(state) -> (logits_ptr, dtype, V, row_stride)`
that reads `state.next_input_ptr` (and `state.cache_len_ptr` / `state.window_start_ptr`) on the
context's stream and leaves `[B, V]` logits on the device. Without the CUDA library every call
here raises.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .config import CFG_DTYPE
from .sampling import CudaSampler, _check

LOOP_UNCACHED = 0   # GenerateWithConfig without KV cache (model/generate.go:57-88)
LOOP_CACHED = 1     # generateCached (model/generate.go:93-131)
LOOP_QWEN = 2       # qwen.Generate (model/qwen/generate.go:35-62)

GEN_LIVE, GEN_STOP, GEN_MAX_NEW, GEN_MAX_SEQ, GEN_ERROR = 0, 1, 2, 3, 4


class DeviceGenerateState:
    """Device-resident state of B sequences being generated side by side."""

    def __init__(self, sampler: CudaSampler, prompts, max_new: int, max_seq: int, stop_tokens=(),
                 loop: int = LOOP_CACHED):
        if loop not in (LOOP_UNCACHED, LOOP_CACHED, LOOP_QWEN):
            raise ValueError("loop must be LOOP_UNCACHED, LOOP_CACHED or LOOP_QWEN")
        stops = [int(t) for t in stop_tokens]
        if len(stops) > _lib.GEN_MAX_STOPS:
            raise ValueError(f"at most {_lib.GEN_MAX_STOPS} stop tokens")
        if loop != LOOP_QWEN and len(stops) > 1:
            raise ValueError("GenerateConfig has one StopToken (model/generate.go:19)")
        prompts = [list(map(int, p)) for p in prompts]
        if any(len(p) == 0 for p in prompts):
            # qwen/generate.go:36-38 panics by name; generate.go:70 and :104 slice at (len-1)*V
            raise ValueError("generate: empty prompt")
        if loop == LOOP_CACHED:                                       # generate.go:101-103
            prompts = [p[len(p) - max_seq:] if len(p) > max_seq else p for p in prompts]
        self.s = sampler
        self.B = len(prompts)
        self.loop = loop
        self.max_new = int(max_new)
        self.max_seq = int(max_seq)
        self.capacity = max(max((len(p) for p in prompts), default=0) + max(self.max_new, 0), 1)
        B, cap = self.B, self.capacity
        tokens = np.zeros((B, cap), dtype=np.int32)
        lengths = np.zeros(B, dtype=np.int32)
        for b, p in enumerate(prompts):
            tokens[b, : len(p)] = p
            lengths[b] = len(p)
        start = np.maximum(lengths - self.max_seq, 0).astype(np.int32)
        last = np.array([p[-1] if p else 0 for p in prompts], dtype=np.int32)
        zeros = np.zeros(B, dtype=np.int32)
        self._bufs = {}
        for name, arr in (("tokens", tokens), ("lengths", lengths), ("n_new", zeros), ("cache_len", lengths.copy()),
                          ("done", zeros), ("next_input", last), ("window_start", start),
                          ("live_count", np.array([B], dtype=np.int32)), ("ids", zeros), ("flags", zeros)):
            buf = sampler._buf(max(arr.nbytes, 16))
            self._bufs[name] = buf
            if arr.nbytes:
                sampler._upload(buf, np.ascontiguousarray(arr))
        ptr = sampler._lib.gorch_cuda_buffer_device_ptr
        self.gc = _lib.GenControl()
        self.gc.tokens = ptr(self._bufs["tokens"])
        self.gc.capacity = cap
        self.gc.lengths = ptr(self._bufs["lengths"])
        self.gc.n_new = ptr(self._bufs["n_new"])
        self.gc.cache_len = ptr(self._bufs["cache_len"])
        self.gc.done = ptr(self._bufs["done"])
        self.gc.next_input = ptr(self._bufs["next_input"])
        self.gc.window_start = ptr(self._bufs["window_start"])
        self.gc.live_count = ptr(self._bufs["live_count"])
        for i in range(_lib.GEN_MAX_STOPS):
            self.gc.stop_tokens[i] = stops[i] if i < len(stops) else -1
        self.gc.n_stop = len(stops)
        self.gc.max_new = self.max_new
        self.gc.max_seq = self.max_seq
        self.gc.cached = 0 if loop == LOOP_UNCACHED else 1
        self.ids_ptr = ptr(self._bufs["ids"])
        self.flags_ptr = ptr(self._bufs["flags"])

    # what a model's forward reads
    next_input_ptr = property(lambda self: self.gc.next_input)
    cache_len_ptr = property(lambda self: self.gc.cache_len)
    window_start_ptr = property(lambda self: self.gc.window_start)
    tokens_ptr = property(lambda self: self.gc.tokens)
    lengths_ptr = property(lambda self: self.gc.lengths)

    def release(self) -> None:
        for b in self._bufs.values():
            self.s._lib.gorch_cuda_buffer_free(b)
        self._bufs = {}

    def control(self, ids_ptr: int, flags_ptr: int | None = None) -> None:
        """One loop iteration over ids some sampling call has left on the device."""
        err = C.c_void_p()
        rc = self.s._lib.gorch_cuda_generate_control_dev(self.s._ctx, ids_ptr, flags_ptr, C.byref(self.gc), self.B, C.byref(err))
        _check(self.s._lib, rc, err)

    def step(self, logits_ptr: int, dtype: int, V: int, row_stride: int, cfgs_ptr: int, uniforms_ptr: int) -> None:
        """Sample every row of logits [B,V] and apply one loop iteration; asynchronous."""
        err = C.c_void_p()
        rc = self.s._lib.gorch_cuda_generate_step_dev(self.s._ctx, logits_ptr, dtype, self.B, V, row_stride, cfgs_ptr,
                                                      uniforms_ptr, self.ids_ptr, self.flags_ptr, C.byref(self.gc), C.byref(err))
        _check(self.s._lib, rc, err)

    def _get(self, name: str, shape) -> np.ndarray:
        out = np.empty(shape, dtype=np.int32)
        self.s.sync()
        if out.nbytes:
            self.s._download(self._bufs[name], out)
        return out

    def live(self) -> int:
        """Rows still generating (synchronises the stream)."""
        return int(self._get("live_count", 1)[0])

    def results(self) -> dict:
        tokens = self._get("tokens", (self.B, self.capacity))
        lengths = self._get("lengths", self.B)
        return {"tokens": [tokens[b, : lengths[b]].tolist() for b in range(self.B)],
                "done": self._get("done", self.B), "n_new": self._get("n_new", self.B),
                "cache_len": self._get("cache_len", self.B), "next_input": self._get("next_input", self.B),
                "window_start": self._get("window_start", self.B)}


def generate_on_device(model, prompts, cfgs, uniforms, sampler: CudaSampler, max_new: int, max_seq: int,
                       stop_tokens=(), loop: int = LOOP_CACHED, poll_every: int = 8) -> dict:
    """Runs B sequences to completion. `cfgs` is a CFG_DTYPE array [B] (each row's sampling
    fields), `uniforms` a float64 array [max_new, B]: row b consumes uniforms[i, b] in its i-th
    iteration, as the reference draws one value per sampled token. `model.prefill_dev(state)` and
    `model.forward_dev(state)` each return (logits_ptr, dtype, V, row_stride) for logits [B,V]
    on the device. Returns DeviceGenerateState.results()."""
    cfgs = np.ascontiguousarray(cfgs, dtype=CFG_DTYPE)
    uniforms = np.ascontiguousarray(uniforms, dtype=np.float64).reshape(max(int(max_new), 0), -1)
    st = DeviceGenerateState(sampler, prompts, max_new, max_seq, stop_tokens, loop)
    if uniforms.shape[1] != st.B or cfgs.shape[0] != st.B:
        st.release()
        raise ValueError("cfgs must hold B records and uniforms max_new x B values")
    b_cfg = sampler._buf(max(cfgs.nbytes, 16))
    b_uni = sampler._buf(max(uniforms.nbytes, 16))
    try:
        if cfgs.nbytes:
            sampler._upload(b_cfg, cfgs)
        if uniforms.nbytes:
            sampler._upload(b_uni, uniforms)
        ptr = sampler._lib.gorch_cuda_buffer_device_ptr
        p_cfg, p_uni = ptr(b_cfg), ptr(b_uni)
        steps = 0
        if st.B and max_new > 0:
            logits_ptr, dtype, V, stride = model.prefill_dev(st)
            for i in range(max_new):
                st.step(logits_ptr, dtype, V, stride, p_cfg, p_uni + 8 * st.B * i)
                steps += 1
                if i + 1 == max_new:
                    break
                if (i + 1) % max(int(poll_every), 1) == 0 and st.live() == 0:
                    break
                logits_ptr, dtype, V, stride = model.forward_dev(st)
        out = st.results()
        out["steps"] = steps
        return out
    finally:
        sampler._lib.gorch_cuda_buffer_free(b_cfg)
        sampler._lib.gorch_cuda_buffer_free(b_uni)
        st.release()
