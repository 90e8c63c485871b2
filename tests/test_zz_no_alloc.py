"""gorch_cuda_sample_dev_static: the sampling entry point that never allocates on the device.

It exists for callers that cannot tolerate a cudaMalloc inside the call (a decode loop under
stream capture, a server with a fixed device-memory budget): its row work lists sit in a fixed
array inside the library image instead of a cudaMalloc'd buffer. The tests drive it through the
C ABI twice in a row on the same inputs and require the token ids and flags of both calls to be
identical to what the ordinary device entry point returns (ids are integers: bit-exact) and to
match the CPU oracle; run it at its 4096-row limit with every row on the hand-over list, so that
the list reaches the end of the array, and again right after with a small batch, which shows the
counters are cleared between calls; run bf16 rows; check that free device memory is the same
before and after a sequence of calls with growing batches (the ordinary entry would regrow its
work list on that sequence); and check that a batch beyond the limit is refused with a clear error.

Collected last on purpose (file name): a run that stops at the first failure has already run
every other test by the time it gets here.
"""
import numpy as np
import pytest

from gorch_b200 import workloads
from gorch_b200.config import CFG_DTYPE, DTYPE_BF16, DTYPE_F32, MODE_A, MODE_B
from tests.parity import compare

pytestmark = pytest.mark.gpu


def _device_run(s, entry, logits, cfgs, uniforms, repeats):
    """Upload once, call `entry` `repeats` times, download ids/flags after every call."""
    B, V = logits.shape
    code = DTYPE_BF16 if logits.dtype == np.uint16 else DTYPE_F32
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
            entry(ptr(b_log), code, B, V, V, ptr(b_cfg), ptr(b_uni), ptr(b_ids), ptr(b_flg))
            s.sync()
            ids = np.empty(B, dtype=np.int32); flags = np.empty(B, dtype=np.uint32)
            s._download(b_ids, ids); s._download(b_flg, flags)
            out.append((ids, flags))
    finally:
        for b in bufs:
            lib.gorch_cuda_buffer_free(b)
    return out


def _against_oracle(oracle, logits, cfgs, uniforms, ids, flags):
    ora = oracle.sample_batch(logits, cfgs, uniforms, flags=oracle.FAST_KTH, threads=oracle.hw_threads())
    rep = compare({"ids": ids, "flags": flags}, ora, uniforms, check_probs=False, allow_tie_cut=True)
    assert rep["id_mismatch"] == rep["boundary_mismatch"]


def test_static_entry_matches_the_ordinary_one_and_the_oracle_twice(_sampler_session, oracle):
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
        _against_oracle(oracle, logits, cfgs, uniforms, ids, flags)


def test_static_entry_small_batch_and_bf16(_sampler_session, oracle):
    """A batch below the large-batch threshold (the static entry dispatches like the ordinary one:
    the shared-memory cluster kernel serves it) and bf16 rows."""
    s = _sampler_session
    s.set_kernel_variant(0, 0)
    rng = np.random.default_rng(5)
    B, V = 12, 20000
    x = workloads.f32_to_bf16_bits((rng.standard_normal((B, V)) * 3.0).astype(np.float32))
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    for i in range(B):
        cfgs[i] = [(0.7, 64, 0.95, MODE_B), (1.0, 0, 0.9, MODE_B), (0.0, 0, 0.0, MODE_A), (0.9, 600, 0.0, MODE_A)][i % 4]
    u = rng.random(B)
    for ids, flags in _device_run(s, s.sample_dev_static_ptrs, x, cfgs, u, 2):
        _against_oracle(oracle, x, cfgs, u, ids, flags)
    big = workloads.vocab_sharded(400)              # bf16, large-batch kernels
    for ids, flags in _device_run(s, s.sample_dev_static_ptrs, big.logits, big.cfgs, big.uniforms, 2):
        _against_oracle(oracle, big.logits, big.cfgs, big.uniforms, ids, flags)


def test_static_entry_at_its_row_limit(_sampler_session, oracle):
    """4096 rows, every one with top_k > 256: all of them land on the hand-over list, which then
    reaches the last word of the fixed array; the small batch right after must not see stale counts."""
    s = _sampler_session
    s.set_kernel_variant(0, 0)
    rng = np.random.default_rng(6)
    B, V = 4096, 1200
    x = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    cfgs["temperature"], cfgs["top_k"], cfgs["top_p"], cfgs["topp_mode"] = 0.8, 300, 0.9, MODE_B
    u = rng.random(B)
    for ids, flags in _device_run(s, s.sample_dev_static_ptrs, x, cfgs, u, 2):
        _against_oracle(oracle, x, cfgs, u, ids, flags)
    small = workloads.mixed_rows(40)
    ids, flags = _device_run(s, s.sample_dev_static_ptrs, small.logits, small.cfgs, small.uniforms, 1)[0]
    _against_oracle(oracle, small.logits, small.cfgs, small.uniforms, ids, flags)


def test_static_entry_leaves_device_memory_alone(_sampler_session):
    import torch
    s = _sampler_session
    s.set_kernel_variant(0, 0)
    rng = np.random.default_rng(7)
    V = 3000
    sizes = [8, 64, 600, 2000, 4096]
    x = torch.from_numpy((rng.standard_normal((max(sizes), V)) * 2.0).astype(np.float32)).cuda()
    cfgs = np.zeros(max(sizes), dtype=CFG_DTYPE)
    cfgs["temperature"], cfgs["top_k"], cfgs["top_p"], cfgs["topp_mode"] = 0.8, 40, 0.9, MODE_B
    cfgs["top_k"][::3] = 0
    d_cfgs = torch.from_numpy(cfgs.view(np.uint8).reshape(-1, 16).copy()).cuda()
    d_uni = torch.from_numpy(rng.random(max(sizes))).cuda()
    d_ids = torch.empty(max(sizes), dtype=torch.int32, device="cuda")
    d_flags = torch.empty(max(sizes), dtype=torch.int32, device="cuda")
    s.sample_dev_static_ptrs(x.data_ptr(), DTYPE_F32, 8, V, V, d_cfgs.data_ptr(), d_uni.data_ptr(),
                             d_ids.data_ptr(), d_flags.data_ptr())      # first call on the device: symbol lookup
    s.sync()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for B in sizes:
        s.sample_dev_static_ptrs(x.data_ptr(), DTYPE_F32, B, V, V, d_cfgs.data_ptr(), d_uni.data_ptr(),
                                 d_ids.data_ptr(), d_flags.data_ptr())
        s.sync()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"device memory moved by {free0 - free1} bytes across the calls"


def test_static_entry_refuses_oversized_batches(_sampler_session):
    from gorch_b200.sampling import GorchCudaError
    s = _sampler_session
    with pytest.raises(GorchCudaError, match="at most 4096 rows"):
        s.sample_dev_static_ptrs(1, DTYPE_F32, 4097, 16, 16, 1, 1, 1, None)
