"""gorch_cuda_sample_dev_static: the sampling entry point that never allocates on the device.

It exists for callers that cannot tolerate a cudaMalloc inside the call (a decode loop under
stream capture, a server with a fixed device-memory budget): its row work lists sit in a fixed
array inside the library image instead of a cudaMalloc'd buffer. The test drives it through the
C ABI twice in a row on the same inputs and requires the token ids and flags of both calls to be
identical to what the ordinary device entry point returns (ids are integers: bit-exact), and
checks that a batch beyond its 4096-row limit is refused with a clear error.

Collected last on purpose (file name): a run that stops at the first failure has already run
every other test by the time it gets here.
"""
import numpy as np
import pytest

from gorch_b200 import workloads
from gorch_b200.config import CFG_DTYPE, DTYPE_F32

pytestmark = pytest.mark.gpu


def _device_run(s, entry, logits, cfgs, uniforms, repeats):
    """Upload once, call `entry` `repeats` times, download ids/flags after every call."""
    B, V = logits.shape
    lib = s._lib
    bufs = []
    out = []
    try:
        b_log = s._buf(logits.nbytes); bufs.append(b_log)
        b_cfg = s._buf(cfgs.nbytes); bufs.append(b_cfg)
        b_uni = s._buf(uniforms.nbytes); bufs.append(b_uni)
        b_ids = s._buf(B * 4); bufs.append(b_ids)
        b_flg = s._buf(B * 4); bufs.append(b_flg)
        s._upload(b_log, logits); s._upload(b_cfg, cfgs); s._upload(b_uni, uniforms)
        ptr = lib.gorch_cuda_buffer_device_ptr
        for _ in range(repeats):
            poison = np.full(B, -7, dtype=np.int32)
            s._upload(b_ids, poison)
            entry(ptr(b_log), DTYPE_F32, B, V, V, ptr(b_cfg), ptr(b_uni), ptr(b_ids), ptr(b_flg))
            s.sync()
            ids = np.empty(B, dtype=np.int32); flags = np.empty(B, dtype=np.uint32)
            s._download(b_ids, ids); s._download(b_flg, flags)
            out.append((ids, flags))
    finally:
        for b in bufs:
            lib.gorch_cuda_buffer_free(b)
    return out


def test_static_entry_matches_the_ordinary_one_twice(_sampler_session):
    s = _sampler_session
    s.set_kernel_variant(0, 0)
    w = workloads.mixed_rows(96)                    # greedy, top-k, top-k-off rows; injected ties
    logits = np.ascontiguousarray(w.logits)
    cfgs = np.ascontiguousarray(w.cfgs, dtype=CFG_DTYPE)
    cfgs["top_k"][5] = 5000                         # one row that ends on the single-CTA work list
    uniforms = np.ascontiguousarray(w.uniforms)
    ref = _device_run(s, s.sample_dev_ptrs, logits, cfgs, uniforms, 1)[0]
    got = _device_run(s, s.sample_dev_static_ptrs, logits, cfgs, uniforms, 2)
    for ids, flags in got:
        assert np.array_equal(ids, ref[0])
        assert np.array_equal(flags & ~np.uint32(0x40), ref[1] & ~np.uint32(0x40))   # path bit is informational


def test_static_entry_refuses_oversized_batches(_sampler_session):
    from gorch_b200.sampling import GorchCudaError
    s = _sampler_session
    with pytest.raises(GorchCudaError, match="at most 4096 rows"):
        s.sample_dev_static_ptrs(1, DTYPE_F32, 4097, 16, 16, 1, 1, 1, None)
