"""Host-side mirror of the reference's sampling interface over libgorchcuda.so.

Names and argument meaning follow the reference:
  argmax(logits)                       model/generate.go:134-144
  sample(logits, T, topK, topP)        model/generate.go:147-240 (mode A)
  sampleLogits(..., rng)               model/qwen/generate.go:92-164 (mode B)
  GenerateWithConfig / generateCached  model/generate.go:52-131
  qwen.Generate                        model/qwen/generate.go:35-65
with one difference the reference cannot express: the uniform is an argument
(the reference calls rand.Float64() inside, generate.go:231).

Everything here calls the CUDA library; there is no CPU path. A missing
library or a machine without a B200-class GPU raises.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .config import (CFG_DTYPE, DTYPE_BF16, DTYPE_F32, MODE_A, MODE_B, GenerateConfig,
                     QwenGenerateConfig)

DEBUG_DTYPE = np.dtype(
    [("sum_exp", "<f8"), ("resum", "<f8"), ("edge_lo", "<f8"), ("edge_hi", "<f8"),
     ("kept", "<i4"), ("max_scaled", "<f4"), ("threshold", "<f4"), ("path", "<i4"),
     ("reserved", "<u4", (8,))]
)


class GorchCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"gorch_cuda error {code}: {message}")
        self.code = code


def _take_err(lib, err: C.c_void_p) -> str:
    if not err.value:
        return ""
    msg = C.string_at(err.value).decode("utf-8", "replace")
    lib.gorch_cuda_free_string(err)
    return msg


def _check(lib, rc: int, err: C.c_void_p) -> None:
    if rc != 0:
        raise GorchCudaError(rc, _take_err(lib, err))


def _logits_arg(logits: np.ndarray):
    x = np.ascontiguousarray(logits)
    if x.dtype == np.uint16:
        return x, DTYPE_BF16
    if x.dtype != np.float32:
        x = x.astype(np.float32)
    return x, DTYPE_F32


VS_CAND = 128                      # GORCH_VS_CAND
VS_RECORD_BYTES = 16 + 8 * VS_CAND  # GORCH_VS_RECORD_BYTES
UNIQUE_ID_BYTES = 128              # GORCH_CUDA_UNIQUE_ID_BYTES


class CudaSampler:
    """One device context (cf. metal.NewDevice, metal/metal.go:228-234): a
    device, a stream and grow-only staging buffers."""

    def __init__(self, device: int = 0):
        self._lib = _lib.load()
        err = C.c_void_p()
        self._ctx = self._lib.gorch_cuda_create_ctx(int(device), C.byref(err))
        if not self._ctx:
            raise GorchCudaError(2, _take_err(self._lib, err))
        self.device = int(device)

    def release(self) -> None:
        if getattr(self, "_ctx", None):
            self._lib.gorch_cuda_release(self._ctx)
            self._ctx = None

    close = release

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()

    # ---- plumbing
    def sync(self) -> None:
        err = C.c_void_p()
        _check(self._lib, self._lib.gorch_cuda_sync(self._ctx, C.byref(err)), err)

    def set_stream(self, stream_handle: int | None) -> None:
        """Run on a caller-owned CUDA stream (its cudaStream_t as an int; 0 is the
        legacy default stream); None goes back to the context's own stream."""
        err = C.c_void_p()
        ext = 0 if stream_handle is None else 1
        _check(self._lib, self._lib.gorch_cuda_set_stream(self._ctx, stream_handle or None, ext, C.byref(err)), err)

    def set_timing(self, on: bool) -> None:
        self._lib.gorch_cuda_set_timing(self._ctx, 1 if on else 0)

    def set_kernel_variant(self, variant: int = 0, cluster_size: int = 0) -> None:
        """Test hook: 0 dispatch by batch shape (default); 1 single-CTA kernel; 2 batch kernels; 3 cluster kernel;
        4 / 5 batch kernels with the wide kernel's 256- / 1024-thread instance; 6 / 7 with the narrow
        kernel's 128- / 256-thread instance. cluster_size 0 = automatic."""
        err = C.c_void_p()
        _check(self._lib, self._lib.gorch_cuda_set_kernel_variant(self._ctx, int(variant), int(cluster_size), C.byref(err)), err)

    def counters(self) -> dict:
        c = _lib.Counters()
        self._lib.gorch_cuda_get_counters(self._ctx, C.byref(c))
        return {name: getattr(c, name) for name, _ in c._fields_}

    # ---- the sampling step, host memory in and out
    def sample_batch(self, logits, cfgs, uniforms, want_flags: bool = True):
        """[B,V] logits (float32, or uint16 bf16 bit patterns), per-row cfgs
        (CFG_DTYPE) and uniforms -> (ids int32[B], flags uint32[B])."""
        x, dtype = _logits_arg(logits)
        if x.ndim != 2:
            raise ValueError("logits must be [B,V]")
        B, V = x.shape
        cfgs = np.ascontiguousarray(cfgs, dtype=CFG_DTYPE)
        uniforms = np.ascontiguousarray(uniforms, dtype=np.float64)
        if cfgs.shape != (B,) or uniforms.shape != (B,):
            raise ValueError("cfgs and uniforms must have one entry per row")
        ids = np.empty(B, dtype=np.int32)
        flags = np.zeros(B, dtype=np.uint32)
        err = C.c_void_p()
        rc = self._lib.gorch_cuda_sample_host(
            self._ctx, x.ctypes.data, dtype, B, V, V, cfgs.ctypes.data, uniforms.ctypes.data,
            ids.ctypes.data, flags.ctypes.data if want_flags else None, C.byref(err))
        _check(self._lib, rc, err)
        return ids, flags

    def sample_host_ptrs(self, logits_ptr: int, dtype: int, B: int, V: int, row_stride: int,
                         cfgs_ptr: int, uniforms_ptr: int, ids_ptr: int, flags_ptr: int | None):
        """Raw-pointer form of sample_batch for callers that manage (pinned) host memory."""
        err = C.c_void_p()
        rc = self._lib.gorch_cuda_sample_host(self._ctx, logits_ptr, dtype, B, V, row_stride,
                                              cfgs_ptr, uniforms_ptr, ids_ptr, flags_ptr,
                                              C.byref(err))
        _check(self._lib, rc, err)

    def sample_dev_ptrs(self, logits_ptr: int, dtype: int, B: int, V: int, row_stride: int,
                        cfgs_ptr: int, uniforms_ptr: int, ids_ptr: int, flags_ptr: int | None = None,
                        probs_ptr: int | None = None, debug_ptr: int | None = None) -> None:
        """Device pointers in and out; asynchronous on the context's stream."""
        err = C.c_void_p()
        rc = self._lib.gorch_cuda_sample_dev(self._ctx, logits_ptr, dtype, B, V, row_stride,
                                             cfgs_ptr, uniforms_ptr, ids_ptr, flags_ptr,
                                             probs_ptr, debug_ptr, C.byref(err))
        _check(self._lib, rc, err)

    # ---- device buffers (cf. metal Buffer, metal/metal.go:357-422)
    def _buf(self, nbytes: int) -> int:
        err = C.c_void_p()
        b = self._lib.gorch_cuda_buffer_alloc(self._ctx, int(nbytes), C.byref(err))
        if not b:
            raise GorchCudaError(2, _take_err(self._lib, err))
        return b

    def _upload(self, buf: int, arr: np.ndarray) -> None:
        err = C.c_void_p()
        _check(self._lib, self._lib.gorch_cuda_buffer_upload(buf, 0, arr.ctypes.data, arr.nbytes, C.byref(err)), err)

    def _download(self, buf: int, arr: np.ndarray) -> None:
        err = C.c_void_p()
        _check(self._lib, self._lib.gorch_cuda_buffer_download(buf, 0, arr.ctypes.data, arr.nbytes, C.byref(err)), err)

    def sample_batch_debug(self, logits, cfgs, uniforms, want_probs: bool = True,
                           pad_elems: int = 0):
        """sample_batch through the device-pointer entry point, also returning the
        dense final probabilities [B,V] (float64) and the per-row debug records.
        `pad_elems` places the logits that many elements into their buffer, to
        exercise rows that do not start on a 16-byte boundary."""
        x, dtype = _logits_arg(logits)
        B, V = x.shape
        cfgs = np.ascontiguousarray(cfgs, dtype=CFG_DTYPE)
        uniforms = np.ascontiguousarray(uniforms, dtype=np.float64)
        ids = np.empty(B, dtype=np.int32)
        flags = np.zeros(B, dtype=np.uint32)
        dbg = np.zeros(B, dtype=DEBUG_DTYPE)
        probs = np.empty((B, V), dtype=np.float64) if want_probs else None
        pad_bytes = pad_elems * x.itemsize
        staged = np.zeros(pad_bytes + x.nbytes, dtype=np.uint8)
        staged[pad_bytes:] = x.view(np.uint8).reshape(-1)
        bufs = []
        try:
            b_log = self._buf(staged.nbytes); bufs.append(b_log)
            b_cfg = self._buf(cfgs.nbytes); bufs.append(b_cfg)
            b_uni = self._buf(uniforms.nbytes); bufs.append(b_uni)
            b_ids = self._buf(ids.nbytes); bufs.append(b_ids)
            b_flg = self._buf(flags.nbytes); bufs.append(b_flg)
            b_dbg = self._buf(dbg.nbytes); bufs.append(b_dbg)
            b_prb = None
            if want_probs:
                b_prb = self._buf(probs.nbytes); bufs.append(b_prb)
            self._upload(b_log, staged)
            self._upload(b_cfg, cfgs)
            self._upload(b_uni, uniforms)
            ptr = self._lib.gorch_cuda_buffer_device_ptr
            self.sample_dev_ptrs(ptr(b_log) + pad_bytes, dtype, B, V, V, ptr(b_cfg), ptr(b_uni),
                                 ptr(b_ids), ptr(b_flg), ptr(b_prb) if want_probs else None,
                                 ptr(b_dbg))
            self.sync()
            self._download(b_ids, ids)
            self._download(b_flg, flags)
            self._download(b_dbg, dbg)
            if want_probs:
                self._download(b_prb, probs)
        finally:
            for b in bufs:
                self._lib.gorch_cuda_buffer_free(b)
        return {"ids": ids, "flags": flags, "debug": dbg, "probs": probs}

    def sample_dev_static_ptrs(self, logits_ptr: int, dtype: int, B: int, V: int, row_stride: int,
                               cfgs_ptr: int, uniforms_ptr: int, ids_ptr: int, flags_ptr: int | None = None) -> None:
        """gorch_cuda_sample_dev_static: device pointers in and out, no device allocation inside
        (row work lists in a fixed array of the library image; at most 4096 rows per call)."""
        err = C.c_void_p()
        rc = self._lib.gorch_cuda_sample_dev_static(self._ctx, logits_ptr, dtype, B, V, row_stride,
                                                    cfgs_ptr, uniforms_ptr, ids_ptr, flags_ptr, C.byref(err))
        _check(self._lib, rc, err)

    # ---- vocab-sharded sampling (every rank holds a column slice of every row)
    def vocab_local_ptrs(self, logits_ptr: int, dtype: int, B: int, Vslice: int, row_stride: int,
                         col_offset: int, cfgs_ptr: int, records_ptr: int) -> None:
        """gorch_cuda_vocab_local_dev: device pointers; fills B records of VS_RECORD_BYTES."""
        err = C.c_void_p()
        rc = self._lib.gorch_cuda_vocab_local_dev(self._ctx, logits_ptr, dtype, B, Vslice, row_stride,
                                                  col_offset, cfgs_ptr, records_ptr, C.byref(err))
        _check(self._lib, rc, err)

    def vocab_merge_ptrs(self, records_ptr: int, nranks: int, B: int, V: int, cfgs_ptr: int,
                         uniforms_ptr: int, ids_ptr: int, flags_ptr: int | None = None) -> None:
        """gorch_cuda_vocab_merge_dev: device pointers; records of all ranks in rank order."""
        err = C.c_void_p()
        rc = self._lib.gorch_cuda_vocab_merge_dev(self._ctx, records_ptr, nranks, B, V, cfgs_ptr,
                                                  uniforms_ptr, ids_ptr, flags_ptr, C.byref(err))
        _check(self._lib, rc, err)

    # ---- the same three steps as one call, the all-gather inside the library (NCCL)
    def comm_unique_id(self) -> bytes:
        """gorch_cuda_comm_unique_id: rank 0 makes the id; every other rank needs the same bytes."""
        buf = C.create_string_buffer(UNIQUE_ID_BYTES)
        err = C.c_void_p()
        _check(self._lib, self._lib.gorch_cuda_comm_unique_id(buf, C.byref(err)), err)
        return buf.raw

    def comm_init(self, rank: int, nranks: int, unique_id: bytes) -> None:
        """gorch_cuda_comm_init (collective): binds a communicator of `nranks` ranks to this context."""
        if len(unique_id) != UNIQUE_ID_BYTES:
            raise ValueError(f"unique id must be {UNIQUE_ID_BYTES} bytes")
        buf = C.create_string_buffer(unique_id, UNIQUE_ID_BYTES)
        err = C.c_void_p()
        _check(self._lib, self._lib.gorch_cuda_comm_init(self._ctx, int(rank), int(nranks), buf, C.byref(err)), err)

    def comm_release(self) -> None:
        err = C.c_void_p()
        _check(self._lib, self._lib.gorch_cuda_comm_release(self._ctx, C.byref(err)), err)

    def sample_vocab_sharded_ptrs(self, logits_ptr: int, dtype: int, B: int, Vslice: int, row_stride: int,
                                  col_offset: int, V: int, max_top_k: int, cfgs_ptr: int, uniforms_ptr: int,
                                  ids_ptr: int, flags_ptr: int | None = None, rows_without_top_k: bool = False,
                                  gather_rows: bool = False) -> None:
        """gorch_cuda_sample_vocab_sharded_dev: device pointers; local pass, all-gather, merge.
        rows_without_top_k: the batch may hold rows with top_k == 0 and no effective top-p cut
        (gorch_cuda_sample_vocab_sharded_ex_dev, bit 0: the owners then draw from their slices and two small
        all-reduces hand the tokens round). gather_rows (bit 1): rows with top_k == 0 that this cannot
        serve (an active top-p cut; every such row when rows_without_top_k is off) are sampled from
        whole rows that an all-reduce brings to every rank: correct, not fast."""
        err = C.c_void_p()
        if rows_without_top_k or gather_rows:
            mode = (1 if rows_without_top_k else 0) | (2 if gather_rows else 0)
            rc = self._lib.gorch_cuda_sample_vocab_sharded_ex_dev(self._ctx, logits_ptr, dtype, B, Vslice, row_stride,
                                                                  col_offset, V, int(max_top_k), mode, cfgs_ptr, uniforms_ptr,
                                                                  ids_ptr, flags_ptr, C.byref(err))
        else:
            rc = self._lib.gorch_cuda_sample_vocab_sharded_dev(self._ctx, logits_ptr, dtype, B, Vslice, row_stride,
                                                               col_offset, V, int(max_top_k), cfgs_ptr, uniforms_ptr,
                                                               ids_ptr, flags_ptr, C.byref(err))
        _check(self._lib, rc, err)

    def vocab_merge_draw(self, all_records, my_rank: int, logits_slice, col_offset: int, cfgs, uniforms, V: int):
        """Steps 2 and 3 of one rank on host arrays, rows without top-k included: records
        [nranks, B, VS_RECORD_BYTES] -> gorch_cuda_vocab_merge_owner_dev -> gorch_cuda_vocab_draw_dev over
        this rank's slice -> (ids, flags) as this rank holds them before the max-reduction over the ranks
        (-1 / 0 in the rows without top-k that another rank owns)."""
        rec = np.ascontiguousarray(all_records, dtype=np.uint8)
        nranks, B = rec.shape[0], rec.shape[1]
        x, dtype = _logits_arg(logits_slice)
        Vs = x.shape[1]
        cfgs = np.ascontiguousarray(cfgs, dtype=CFG_DTYPE)
        uniforms = np.ascontiguousarray(uniforms, dtype=np.float64)
        ids = np.empty(B, dtype=np.int32)
        flags = np.zeros(B, dtype=np.uint32)
        bufs = []
        try:
            b_rec = self._buf(rec.nbytes); bufs.append(b_rec)
            b_log = self._buf(max(x.nbytes, 16)); bufs.append(b_log)
            b_cfg = self._buf(cfgs.nbytes); bufs.append(b_cfg)
            b_uni = self._buf(uniforms.nbytes); bufs.append(b_uni)
            b_ids = self._buf(ids.nbytes); bufs.append(b_ids)
            b_flg = self._buf(flags.nbytes); bufs.append(b_flg)
            b_req = self._buf(B * 24); bufs.append(b_req)
            self._upload(b_rec, rec); self._upload(b_log, x); self._upload(b_cfg, cfgs); self._upload(b_uni, uniforms)
            ptr = self._lib.gorch_cuda_buffer_device_ptr
            err = C.c_void_p()
            rc = self._lib.gorch_cuda_vocab_merge_owner_dev(self._ctx, ptr(b_rec), nranks, int(my_rank), B, int(V), ptr(b_cfg),
                                                            ptr(b_uni), ptr(b_ids), ptr(b_flg), ptr(b_req), C.byref(err))
            _check(self._lib, rc, err)
            rc = self._lib.gorch_cuda_vocab_draw_dev(self._ctx, ptr(b_log), dtype, B, Vs, Vs, int(col_offset), ptr(b_cfg),
                                                     ptr(b_req), ptr(b_ids), ptr(b_flg), C.byref(err))
            _check(self._lib, rc, err)
            self.sync()
            self._download(b_ids, ids)
            self._download(b_flg, flags)
        finally:
            for b in bufs:
                self._lib.gorch_cuda_buffer_free(b)
        return ids, flags

    def vocab_local(self, logits_slice, cfgs, col_offset: int) -> np.ndarray:
        """Step 1 on host arrays: this rank's [B, Vslice] columns -> records [B, VS_RECORD_BYTES] (uint8)."""
        x, dtype = _logits_arg(logits_slice)
        B, Vs = x.shape
        cfgs = np.ascontiguousarray(cfgs, dtype=CFG_DTYPE)
        rec = np.zeros((B, VS_RECORD_BYTES), dtype=np.uint8)
        bufs = []
        try:
            b_log = self._buf(max(x.nbytes, 16)); bufs.append(b_log)
            b_cfg = self._buf(cfgs.nbytes); bufs.append(b_cfg)
            b_rec = self._buf(rec.nbytes); bufs.append(b_rec)
            self._upload(b_log, x)
            self._upload(b_cfg, cfgs)
            ptr = self._lib.gorch_cuda_buffer_device_ptr
            self.vocab_local_ptrs(ptr(b_log), dtype, B, Vs, Vs, int(col_offset), ptr(b_cfg), ptr(b_rec))
            self.sync()
            self._download(b_rec, rec)
        finally:
            for b in bufs:
                self._lib.gorch_cuda_buffer_free(b)
        return rec

    def vocab_merge(self, all_records, cfgs, uniforms, V: int):
        """Step 2 on host arrays: records [nranks, B, VS_RECORD_BYTES] -> (ids, flags) for all B rows."""
        rec = np.ascontiguousarray(all_records, dtype=np.uint8)
        nranks, B = rec.shape[0], rec.shape[1]
        cfgs = np.ascontiguousarray(cfgs, dtype=CFG_DTYPE)
        uniforms = np.ascontiguousarray(uniforms, dtype=np.float64)
        ids = np.empty(B, dtype=np.int32)
        flags = np.zeros(B, dtype=np.uint32)
        bufs = []
        try:
            b_rec = self._buf(rec.nbytes); bufs.append(b_rec)
            b_cfg = self._buf(cfgs.nbytes); bufs.append(b_cfg)
            b_uni = self._buf(uniforms.nbytes); bufs.append(b_uni)
            b_ids = self._buf(ids.nbytes); bufs.append(b_ids)
            b_flg = self._buf(flags.nbytes); bufs.append(b_flg)
            self._upload(b_rec, rec)
            self._upload(b_cfg, cfgs)
            self._upload(b_uni, uniforms)
            ptr = self._lib.gorch_cuda_buffer_device_ptr
            self.vocab_merge_ptrs(ptr(b_rec), nranks, B, int(V), ptr(b_cfg), ptr(b_uni), ptr(b_ids), ptr(b_flg))
            self.sync()
            self._download(b_ids, ids)
            self._download(b_flg, flags)
        finally:
            for b in bufs:
                self._lib.gorch_cuda_buffer_free(b)
        return ids, flags

    # ---- the LM-head projection in front of the sampling step (model/qwen/qwen.go:80-85)
    def lm_head_logits_ptrs(self, x_ptr: int, ldx: int, w_ptr: int, ldw: int, B: int, V: int, K: int,
                            out_ptr: int, ld_out: int) -> None:
        """gorch_cuda_lm_head_logits_dev: logits [B, V] f32 = x [B, K] bf16 @ w [V, K] bf16 ^T; device pointers."""
        err = C.c_void_p()
        rc = self._lib.gorch_cuda_lm_head_logits_dev(self._ctx, x_ptr, ldx, w_ptr, ldw, B, V, K, out_ptr, ld_out, C.byref(err))
        _check(self._lib, rc, err)

    def lm_head_sample_ptrs(self, x_ptr: int, ldx: int, w_ptr: int, ldw: int, B: int, V: int, K: int, fuse_top_k: int,
                            cfgs_ptr: int, uniforms_ptr: int, ids_ptr: int, flags_ptr: int | None = None) -> None:
        """gorch_cuda_lm_head_sample_dev: projection + sampling in one call; device pointers."""
        err = C.c_void_p()
        rc = self._lib.gorch_cuda_lm_head_sample_dev(self._ctx, x_ptr, ldx, w_ptr, ldw, B, V, K, int(fuse_top_k),
                                                     cfgs_ptr, uniforms_ptr, ids_ptr, flags_ptr, C.byref(err))
        _check(self._lib, rc, err)

    def lm_head_status(self) -> int:
        """Status word of the last LM-head call (blocking): 0, or bit 0 when a bounded device wait ran out."""
        st = C.c_uint32(0)
        err = C.c_void_p()
        _check(self._lib, self._lib.gorch_cuda_lm_head_status(self._ctx, C.byref(st), C.byref(err)), err)
        return int(st.value)

    # ---- tensor-level index ops (index_ops.go:153-227)
    def topk(self, x, k: int):
        """gorch.TopK over the last axis of x [B,V] (f32, or uint16 holding bf16): (values [B,k]
        float32 descending, indices [B,k] int32; equal values by ascending index)."""
        a, dtype = _logits_arg(x)
        B, V = a.shape
        vals = np.empty((B, max(int(k), 0)), dtype=np.float32)   # a bad k is refused by the library below
        idx = np.empty((B, max(int(k), 0)), dtype=np.int32)
        bufs = []
        try:
            b_x = self._buf(max(a.nbytes, 16)); bufs.append(b_x)
            b_v = self._buf(max(vals.nbytes, 16)); bufs.append(b_v)
            b_i = self._buf(max(idx.nbytes, 16)); bufs.append(b_i)
            self._upload(b_x, a)
            ptr = self._lib.gorch_cuda_buffer_device_ptr
            err = C.c_void_p()
            rc = self._lib.gorch_cuda_topk_dev(self._ctx, ptr(b_x), dtype, B, V, V, int(k), ptr(b_v), ptr(b_i), None, C.byref(err))
            _check(self._lib, rc, err)
            self.sync()
            if B:
                self._download(b_v, vals)
                self._download(b_i, idx)
        finally:
            for b in bufs:
                self._lib.gorch_cuda_buffer_free(b)
        return vals, idx

    def multinomial(self, probs, uniforms):
        """gorch.Multinomial with the uniforms supplied: probs [B,V] float32 -> (ids [B] int32, flags [B])."""
        p = np.ascontiguousarray(probs, dtype=np.float32)
        B, V = p.shape
        uniforms = np.ascontiguousarray(uniforms, dtype=np.float64)
        ids = np.empty(B, dtype=np.int32)
        flags = np.zeros(B, dtype=np.uint32)
        bufs = []
        try:
            b_p = self._buf(max(p.nbytes, 16)); bufs.append(b_p)
            b_u = self._buf(max(uniforms.nbytes, 16)); bufs.append(b_u)
            b_i = self._buf(max(ids.nbytes, 16)); bufs.append(b_i)
            b_f = self._buf(max(flags.nbytes, 16)); bufs.append(b_f)
            self._upload(b_p, p)
            self._upload(b_u, uniforms)
            ptr = self._lib.gorch_cuda_buffer_device_ptr
            err = C.c_void_p()
            rc = self._lib.gorch_cuda_multinomial_dev(self._ctx, ptr(b_p), B, V, V, ptr(b_u), ptr(b_i), ptr(b_f), C.byref(err))
            _check(self._lib, rc, err)
            self.sync()
            if B:
                self._download(b_i, ids)
                self._download(b_f, flags)
        finally:
            for b in bufs:
                self._lib.gorch_cuda_buffer_free(b)
        return ids, flags

    def argmax_batch(self, logits) -> np.ndarray:
        x, dtype = _logits_arg(logits)
        B, V = x.shape
        ids = np.empty(B, dtype=np.int32)
        err = C.c_void_p()
        rc = self._lib.gorch_cuda_argmax_host(self._ctx, x.ctypes.data, dtype, B, V, V,
                                              ids.ctypes.data, C.byref(err))
        _check(self._lib, rc, err)
        return ids

    def argmax_dev_ptrs(self, logits_ptr: int, dtype: int, B: int, V: int, row_stride: int,
                        ids_ptr: int) -> None:
        err = C.c_void_p()
        rc = self._lib.gorch_cuda_argmax_dev(self._ctx, logits_ptr, dtype, B, V, row_stride,
                                             ids_ptr, C.byref(err))
        _check(self._lib, rc, err)

    # ---- the reference's scalar call shapes
    def argmax(self, logits) -> int:
        """argmax(logits []float32) int  (model/generate.go:134)."""
        x = np.ascontiguousarray(logits, dtype=np.float32).reshape(1, -1)
        return int(self.argmax_batch(x)[0])

    def sample(self, logits, temperature: float, top_k: int, top_p: float, u: float,
               mode: int = MODE_A, return_flag: bool = False):
        """sample(logits, temperature, topK, topP) int  (model/generate.go:147),
        `u` standing in for rand.Float64()."""
        x = np.ascontiguousarray(logits, dtype=np.float32).reshape(-1)
        flag = C.c_uint32(0)
        err = C.c_void_p()
        tok = self._lib.gorch_cuda_sample_row(self._ctx, x.ctypes.data, x.size, float(temperature),
                                              int(top_k), float(top_p), int(mode), float(u),
                                              C.byref(flag), C.byref(err))
        if tok < 0:
            raise GorchCudaError(1, _take_err(self._lib, err))
        return (int(tok), int(flag.value)) if return_flag else int(tok)

    def sample_logits(self, logits, temperature, top_k, top_p, u, return_flag: bool = False):
        """sampleLogits (model/qwen/generate.go:92): the true-nucleus flavour."""
        return self.sample(logits, temperature, top_k, top_p, u, MODE_B, return_flag)

    def next_token(self, last_logits, cfg, u: float) -> int:
        """The branch at model/generate.go:75-79 / qwen/generate.go:49-53."""
        if cfg.temperature == 0:
            return self.argmax(last_logits)
        return self.sample(last_logits, cfg.temperature, cfg.top_k, cfg.top_p, u, cfg.topp_mode)


def generate_with_config(model, token_ids, cfg: GenerateConfig, uniforms, sampler) -> list:
    """GenerateWithConfig (model/generate.go:52-90) and generateCached (:94-131).

    `model` provides max_seq, vocab_size, forward(ids) -> [len, V] logits and,
    for cfg.use_kv_cache, new_cache() / forward_cached(ids, cache) -> logits and
    cache.len(). `uniforms` yields the values the reference would draw from
    math/rand, one per sampled step. `sampler` is a CudaSampler."""
    uni = iter(uniforms)
    result = list(token_ids)
    if cfg.use_kv_cache:
        cache = model.new_cache()
        if len(result) > model.max_seq:
            result = result[len(result) - model.max_seq:]
        logits = np.asarray(model.forward_cached(result, cache), dtype=np.float32)
        last = logits.reshape(-1, model.vocab_size)[len(result) - 1]
        for _ in range(cfg.max_new_tokens):
            nxt = sampler.next_token(last, cfg, 0.0 if cfg.temperature == 0 else next(uni))
            if cfg.stop_token >= 0 and nxt == cfg.stop_token:
                break
            result.append(nxt)
            if cache.len() >= model.max_seq:
                break
            step = np.asarray(model.forward_cached([nxt], cache), dtype=np.float32)
            last = step.reshape(-1)[: model.vocab_size]
        return result
    for _ in range(cfg.max_new_tokens):
        inp = result
        if len(inp) > model.max_seq:
            inp = inp[len(inp) - model.max_seq:]
        logits = np.asarray(model.forward(inp), dtype=np.float32).reshape(-1, model.vocab_size)
        last = logits[len(inp) - 1]
        nxt = sampler.next_token(last, cfg, 0.0 if cfg.temperature == 0 else next(uni))
        if cfg.stop_token >= 0 and nxt == cfg.stop_token:
            break
        result.append(nxt)
    return result


def qwen_generate(model, prompt, cfg: QwenGenerateConfig, sampler, uniforms=None) -> list:
    """qwen.Generate (model/qwen/generate.go:35-65). `model` provides
    new_cache(), forward_cached(ids, cache) -> (1,V) logits, max_seq.
    uniforms default to numpy's default_rng(cfg.seed) stream (the reference
    seeds math/rand with cfg.Seed, :42; that generator is not reproduced)."""
    if len(prompt) == 0:
        raise ValueError("qwen: empty prompt")   # generate.go:36-38 panics
    if uniforms is None:
        rng = np.random.default_rng(cfg.seed)
        uniforms = (float(rng.random()) for _ in iter(int, 1))
    uni = iter(uniforms)
    result = list(prompt)
    cache = model.new_cache()
    last = np.asarray(model.forward_cached(list(prompt), cache), dtype=np.float32).reshape(-1)
    for _ in range(cfg.max_new_tokens):
        nxt = sampler.next_token(last, cfg, 0.0 if cfg.temperature == 0 else next(uni))
        if nxt in cfg.stop_tokens:
            break
        result.append(nxt)
        if cache.len() >= model.max_seq:
            break
        last = np.asarray(model.forward_cached([nxt], cache), dtype=np.float32).reshape(-1)
    return result
