"""The LM-head projection in front of the sampling step (model/qwen/qwen.go:80-85: MatMulTransB(last,
Embed.Weight)) and its fusion with sampling, through the C ABI.

Oracle. Logits: a float64 matmul of the same bf16-rounded inputs; gate 1e-3 of the row's largest
magnitude (the tensor cores accumulate bf16 products in f32, in another order than any CPU loop).
Sampling: the CPU oracle's `sample` applied to the logits this library's own projection wrote, so
that the sampling gates stay what they are everywhere else (ids identical except rows whose uniform
lies within 1e-6 of a CDF edge): the fused call never writes those logits, but computes the same
ones (the projection is deterministic)."""
import numpy as np
import pytest

from gorch_b200 import workloads
from gorch_b200.config import CFG_DTYPE, MODE_A, MODE_B
from tests.parity import compare

pytestmark = pytest.mark.gpu


def _inputs(B, V, K, seed, peaks=True):
    rng = np.random.Generator(np.random.Philox(key=seed))
    x = (rng.standard_normal((B, K)) * 0.5).astype(np.float32)
    w = (rng.standard_normal((V, K)) * 0.08).astype(np.float32)
    xb, wb = workloads.f32_to_bf16_bits(x), workloads.f32_to_bf16_bits(w)
    return xb, wb


def _bf16_to_f64(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def _dev(torch, arr):
    if arr.dtype == np.uint16:
        return torch.from_numpy(arr.view(np.int16)).cuda()
    return torch.from_numpy(arr).cuda()


def _project(s, torch, xb, wb):
    B, K = xb.shape
    V = wb.shape[0]
    dx, dw = _dev(torch, xb), _dev(torch, wb)
    out = torch.full((B, V), float("nan"), dtype=torch.float32, device="cuda")
    s.lm_head_logits_ptrs(dx.data_ptr(), K, dw.data_ptr(), K, B, V, K, out.data_ptr(), V)
    s.sync()
    assert s.lm_head_status() == 0
    return out.cpu().numpy()


@pytest.mark.parametrize("B,V,K", [(1, 1000, 64), (7, 4100, 128), (64, 50257, 768), (130, 20000, 1024), (300, 8192, 256)])
def test_projection_against_float64(_sampler_session, B, V, K):
    import torch
    s = _sampler_session
    xb, wb = _inputs(B, V, K, 7000 + B)
    got = _project(s, torch, xb, wb)
    want = _bf16_to_f64(xb) @ _bf16_to_f64(wb).T
    assert not np.isnan(got).any()
    scale = np.abs(want).max(axis=1, keepdims=True)
    assert (np.abs(got - want) <= 1e-3 * scale).all(), float((np.abs(got - want) / scale).max())


def _cfgs(B, kinds):
    c = np.zeros(B, dtype=CFG_DTYPE)
    for b in range(B):
        c[b] = kinds[b % len(kinds)]
    return c


def _sample_call(s, torch, xb, wb, cfgs, uniforms, fuse_top_k):
    B, K = xb.shape
    V = wb.shape[0]
    dx, dw = _dev(torch, xb), _dev(torch, wb)
    dc = torch.from_numpy(cfgs.view(np.uint8).reshape(B, 16).copy()).cuda()
    du = torch.from_numpy(uniforms.copy()).cuda()
    ids = torch.full((B,), -7, dtype=torch.int32, device="cuda")
    flags = torch.zeros(B, dtype=torch.int32, device="cuda")
    s.lm_head_sample_ptrs(dx.data_ptr(), K, dw.data_ptr(), K, B, V, K, fuse_top_k, dc.data_ptr(), du.data_ptr(),
                          ids.data_ptr(), flags.data_ptr())
    s.sync()
    return ids.cpu().numpy(), flags.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("B,V,K", [(64, 50257, 768), (200, 151936, 1024), (5, 8192, 64)])
def test_fused_sampling_matches_the_oracle_on_the_same_logits(_sampler_session, oracle, B, V, K):
    import torch
    s = _sampler_session
    s.set_kernel_variant(0, 0)
    xb, wb = _inputs(B, V, K, 7100 + B)
    logits = _project(s, torch, xb, wb)
    rng = np.random.default_rng(B)
    uniforms = rng.random(B)
    # the reference's DefaultGenerateConfig, greedy, top-k with top-p in both flavours, a large top_k
    cfgs = _cfgs(B, [(0.8, 40, 0.0, MODE_A), (0.0, 0, 0.0, MODE_A), (0.7, 64, 0.95, MODE_B), (1.0, 5, 0.5, MODE_A), (1.3, 200, 0.9, MODE_B)])
    ora = oracle.sample_batch(logits, cfgs, uniforms, flags=oracle.FAST_KTH, threads=oracle.hw_threads())
    refused0 = s.counters()["lm_head_refused_rows"]
    for fuse in (200, 0):                      # fused, then the unfused form of the same call
        ids, flags = _sample_call(s, torch, xb, wb, cfgs, uniforms, fuse)
        rep = compare({"ids": ids, "flags": flags}, ora, uniforms, check_probs=False, allow_tie_cut=True)
        assert rep["id_mismatch"] == rep["boundary_mismatch"]
    assert s.counters()["lm_head_refused_rows"] == refused0, "the fused form should have served every row"


def test_rows_the_fused_form_does_not_serve_fall_back(_sampler_session, oracle):
    import torch
    s = _sampler_session
    s.set_kernel_variant(0, 0)
    B, V, K = 48, 20000, 128
    xb, wb = _inputs(B, V, K, 7200)
    logits = _project(s, torch, xb, wb)
    uniforms = np.random.default_rng(3).random(B)
    cfgs = _cfgs(B, [(0.8, 40, 0.0, MODE_A), (1.0, 0, 0.9, MODE_B), (0.9, 100, 0.0, MODE_A)])   # top-k off; top_k above fuse_top_k
    ora = oracle.sample_batch(logits, cfgs, uniforms, flags=oracle.FAST_KTH, threads=oracle.hw_threads())
    refused0 = s.counters()["lm_head_refused_rows"]
    ids, flags = _sample_call(s, torch, xb, wb, cfgs, uniforms, 40)
    assert s.counters()["lm_head_refused_rows"] - refused0 == 32
    rep = compare({"ids": ids, "flags": flags}, ora, uniforms, check_probs=False, allow_tie_cut=True)
    assert rep["id_mismatch"] == rep["boundary_mismatch"]


def test_bad_shapes_are_refused(_sampler_session):
    from gorch_b200.sampling import GorchCudaError
    s = _sampler_session
    with pytest.raises(GorchCudaError, match="multiple of 64"):
        s.lm_head_logits_ptrs(256, 100, 256, 100, 4, 1000, 100, 256, 1000)
