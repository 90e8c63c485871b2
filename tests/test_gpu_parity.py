"""GPU parity: the CUDA sampling kernels (through the C ABI) against the CPU oracle.

Gates: greedy ids and kept sets bit-exact; final probabilities <= 1e-6
relative; sampled ids identical except where the uniform is within 1e-6 of a
CDF edge (counted). See tests/parity.py.
"""
import numpy as np
import pytest

from gorch_b200 import workloads
from gorch_b200.config import (CFG_DTYPE, FLAG_BOUNDARY, FLAG_FALLBACK, FLAG_NONFINITE, MODE_A,
                               MODE_B)
from tests.parity import compare

pytestmark = pytest.mark.gpu


def cfgs_of(B, T, k, p, mode):
    c = np.zeros(B, dtype=CFG_DTYPE)
    c["temperature"], c["top_k"], c["top_p"], c["topp_mode"] = T, k, p, mode
    return c


def run_both(sampler, oracle, logits, cfgs, uniforms, fast=True, pad=0, want_probs=True,
             allow_tie_cut=False):
    gpu = sampler.sample_batch_debug(logits, cfgs, uniforms, want_probs=want_probs, pad_elems=pad)
    ora = oracle.sample_batch(logits, cfgs, uniforms, want_probs=want_probs,
                              flags=oracle.FAST_KTH if fast else 0, threads=8)
    rep = compare(gpu, ora, uniforms, check_probs=want_probs, allow_tie_cut=allow_tie_cut)
    return gpu, ora, rep


# ---- the reference's own known answers (model/generate_test.go:11-26) ----

def test_reference_known_answers(sampler):
    assert sampler.argmax([1, 5, 3, 2, 4]) == 1
    for u in (0.0, 0.3, 0.999999):
        assert sampler.sample([1, 10, 3, 2], 0.01, 0, 0.0, u) == 1


def test_argmax_ties_and_signed_zero(sampler, oracle):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((64, 5000)).astype(np.float32)
    for b in range(64):
        top = x[b].max()
        cols = rng.choice(5000, size=3, replace=False)
        x[b, cols] = top
    x[0, :] = 0.0
    x[0, 17] = -0.0
    x[1, :] = -np.inf
    x[2, :] = -1.0
    x[2, 7] = -0.0
    x[2, 9] = 0.0
    got = sampler.argmax_batch(x)
    want = np.array([oracle.argmax(x[b]) for b in range(64)])
    assert np.array_equal(got, want)


def test_argmax_nan_rule(sampler, oracle):
    x = np.arange(300, dtype=np.float32).reshape(3, 100).copy()
    x[0, 0] = np.nan          # NaN at index 0: every comparison fails, result 0
    x[1, 50] = np.nan         # NaN elsewhere is never selected
    x[2, 99] = np.nan
    got = sampler.argmax_batch(x)
    want = np.array([oracle.argmax(x[b]) for b in range(3)])
    assert np.array_equal(got, want)
    assert list(got) == [0, 99, 98]


@pytest.mark.parametrize("V", [1, 2, 7, 255, 256, 257, 1000, 1023, 1024, 1025, 2047, 2049, 4097])
@pytest.mark.parametrize("mode", [MODE_A, MODE_B])
def test_small_vocab_sweep(sampler, oracle, V, mode):
    rng = np.random.default_rng(100 + V)
    ks = sorted({0, 1, 5, max(1, V - 1), V, V + 1})
    ps = [0.0, 0.5, 0.66, 0.67, 0.9, 1.0] if V <= 1100 else [0.0, 0.67, 0.9, 1.0]
    if mode == MODE_B:
        ps = [0.0, 0.1, 0.5, 0.9, 0.99, 1.0]
    rows = []
    for k in ks:
        for p in ps:
            for T in (0.7, 1.0):
                rows.append((T, k, p))
    B = len(rows)
    x = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    for i, (T, k, p) in enumerate(rows):
        cfgs[i] = (T, k, p, mode)
    u = rng.random(B)
    run_both(sampler, oracle, x, cfgs, u, fast=False, pad=(V % 4))


@pytest.mark.parametrize("mode", [MODE_A, MODE_B])
def test_mode_a_small_p_and_uniform_edges(sampler, oracle, mode):
    rng = np.random.default_rng(7)
    V = 600
    B = 40
    x = (rng.standard_normal((B, V)) * 1.5).astype(np.float32)
    p = 0.3 if mode == MODE_A else 0.6
    cfgs = cfgs_of(B, 0.9, 0, p, mode)
    u = rng.random(B)
    u[0] = 0.0
    u[1] = 1.0 - 2.0 ** -53
    gpu, ora, _ = run_both(sampler, oracle, x, cfgs, u, fast=False)
    # exact CDF edges as uniforms: any mismatch must be flagged as a boundary case
    edges = ora["info"]["edge_hi"][2:].copy()
    u2 = u.copy()
    u2[2:] = np.minimum(edges, np.nextafter(1.0, 0.0))
    run_both(sampler, oracle, x, cfgs, u2, fast=False)


def test_topk_ties_kept(sampler, oracle):
    """bf16-like coarse values: many ties at the threshold, all must survive
    (model/generate.go:157-164 keeps every value >= the k-th largest)."""
    rng = np.random.default_rng(11)
    B, V = 48, 8192
    x = np.round(rng.standard_normal((B, V)) * 3.0 * 8) / 8
    x = x.astype(np.float32)
    cfgs = cfgs_of(B, 0.7, 64, 0.95, MODE_B)
    cfgs["topp_mode"][::2] = MODE_A
    u = rng.random(B)
    gpu, ora, _ = run_both(sampler, oracle, x, cfgs, u, fast=False, allow_tie_cut=True)
    assert (gpu["debug"]["kept"][::2] >= 64).all()
    assert (ora["info"]["kept"] > 64).any()


def test_bf16_rows(sampler, oracle):
    rng = np.random.default_rng(12)
    B, V = 32, 20000
    x = workloads.f32_to_bf16_bits((rng.standard_normal((B, V)) * 3.0).astype(np.float32))
    cfgs = cfgs_of(B, 0.7, 64, 0.95, MODE_B)
    cfgs["top_k"][8:16] = 0
    cfgs["top_p"][8:16] = 0.0
    cfgs["temperature"][16:24] = 0.0
    u = rng.random(B)
    run_both(sampler, oracle, x, cfgs, u, fast=False, allow_tie_cut=True, pad=3)


def test_nonfinite_rows(sampler, oracle):
    rng = np.random.default_rng(13)
    B, V = 12, 3000
    x = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    x[0, 5] = np.nan
    x[1, 100] = np.inf
    x[2, :] = -np.inf
    x[3, 10:2000] = -np.inf          # legal: zero mass
    x[4, 0] = np.nan
    x[5, 2999] = np.nan
    cfgs = cfgs_of(B, 0.8, 40, 0.0, MODE_A)
    cfgs["top_k"][6:] = 0
    x[6, 7] = np.nan
    x[7, 8] = np.inf
    x[8, 10:2000] = -np.inf
    u = rng.random(B)
    gpu, ora, _ = run_both(sampler, oracle, x, cfgs, u, fast=False)
    for b in (0, 1, 2, 4, 5, 6, 7):
        assert gpu["ids"][b] == V - 1
        assert gpu["flags"][b] & FLAG_NONFINITE and gpu["flags"][b] & FLAG_FALLBACK


def test_all_equal_rows_small(sampler, oracle):
    B, V = 8, 1000
    x = np.full((B, V), 1.25, dtype=np.float32)
    cfgs = cfgs_of(B, 1.0, 0, 0.5, MODE_B)
    cfgs["topp_mode"][4:] = MODE_A
    cfgs["top_p"][4:] = 0.4
    cfgs["top_k"][1] = 10
    cfgs["top_k"][5] = 10
    u = np.linspace(0.01, 0.99, B)
    run_both(sampler, oracle, x, cfgs, u, fast=False)


def test_bad_temperature_rejected(sampler):
    from gorch_b200.sampling import GorchCudaError
    x = np.zeros((1, 16), dtype=np.float32)
    for T in (-1.0, float("nan"), float("inf")):
        with pytest.raises(GorchCudaError):
            sampler.sample_batch(x, cfgs_of(1, T, 0, 0.0, MODE_A), np.array([0.5]))
    out = sampler.sample_batch_debug(x, cfgs_of(1, -1.0, 0, 0.0, MODE_A), np.array([0.5]))
    assert out["ids"][0] == -1


def test_empty_batch(sampler):
    ids, flags = sampler.sample_batch(np.zeros((0, 16), dtype=np.float32),
                                      np.zeros(0, dtype=CFG_DTYPE), np.zeros(0))
    assert ids.size == 0


@pytest.mark.parametrize("mode", [MODE_A, MODE_B])
def test_gpt2_vocab_cycle(sampler, oracle, mode):
    """c3 (mixed rows, injected ties) at full size."""
    w = workloads.mixed_rows(mode=mode)
    gpu, ora, rep = run_both(sampler, oracle, w.logits, w.cfgs, w.uniforms, fast=True)
    for b, want in w.expected_greedy.items():
        if w.cfgs["temperature"][b] == 0:
            assert gpu["ids"][b] == want
    assert rep["id_mismatch"] == rep["boundary_mismatch"]


@pytest.mark.parametrize("mode", [MODE_A, MODE_B])
def test_c1_and_c2(sampler, oracle, mode):
    w1 = workloads.gpt2_step(64, mode=mode)
    run_both(sampler, oracle, w1.logits, w1.cfgs, w1.uniforms, fast=False)
    w2 = workloads.nucleus_batch(mode=mode)
    run_both(sampler, oracle, w2.logits, w2.cfgs, w2.uniforms)


@pytest.mark.parametrize("mode", [MODE_A, MODE_B])
def test_c4_rows(sampler, oracle, mode):
    w = workloads.flat_stress(12, mode=mode)
    run_both(sampler, oracle, w.logits, w.cfgs, w.uniforms)


def test_c5_rows(sampler, oracle):
    w = workloads.vocab_sharded(24)
    run_both(sampler, oracle, w.logits, w.cfgs, w.uniforms, fast=True, allow_tie_cut=True)


def test_host_entry_matches_device_entry(sampler):
    w = workloads.mixed_rows(64)
    ids, flags = sampler.sample_batch(w.logits, w.cfgs, w.uniforms)
    dev = sampler.sample_batch_debug(w.logits, w.cfgs, w.uniforms, want_probs=False)
    assert np.array_equal(ids, dev["ids"])
    assert np.array_equal(flags, dev["flags"])
