"""gorch.TopK and gorch.Multinomial (index_ops.go:153-227) as device ops, through the C ABI:
the reference's own known answers, then seeded cases against the CPU oracle."""
import json
import os

import numpy as np
import pytest

from gorch_b200 import workloads
from gorch_b200.config import FLAG_BOUNDARY, FLAG_FALLBACK
from gorch_b200.sampling import GorchCudaError

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def known():
    with open(os.path.join(HERE, "golden", "reference_known_answers.json")) as f:
        return json.load(f)


def test_reference_topk_cases(sampler, known):
    for c in known["topk"]:
        x = np.array(c["x"], dtype=np.float32)
        vals, idx = sampler.topk(x, c["k"])
        assert vals.tolist() == c["values"]
        assert idx.tolist() == c["indices"]
    bad = known["topk_invalid_k"]
    for k in bad["ks"]:
        with pytest.raises(GorchCudaError):
            sampler.topk(np.zeros(bad["shape"], dtype=np.float32), k)


@pytest.mark.parametrize("B,V,k", [(3, 8, 2), (5, 257, 7), (16, 50257, 40), (4, 4097, 256), (2, 5, 5), (7, 1000, 1)])
def test_topk_matches_oracle(sampler, oracle, B, V, k):
    rng = np.random.Generator(np.random.Philox(key=B * 1000003 + V * 17 + k))
    x = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    x[:, ::3] = np.round(x[:, ::3] * 4) / 4            # ties, also across the k-th value
    vals, idx = sampler.topk(x, k)
    wv, wi = oracle.topk(x, k)
    assert np.array_equal(vals, wv)
    assert np.array_equal(idx.astype(np.int64), wi)    # ascending index among equals, as the oracle


@pytest.mark.parametrize("B,V,k", [(3, 300, 257), (2, 300, 300), (5, 5000, 1000), (6, 50257, 4096), (150, 151936, 300),
                                   (3, 151936, 16384), (4, 20000, 5000)])
def test_topk_large_k_matches_oracle(_sampler_session, oracle, B, V, k):
    """k beyond the one-pass kernel's lists: radix select of the k-th largest, gather, sort. Ties across
    the k-th value (lowest indices win), a row of one value only, -Inf and NaN entries (ordered last)."""
    s = _sampler_session
    rng = np.random.Generator(np.random.Philox(key=B * 1000003 + V * 17 + k))
    x = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    x[:, ::3] = np.round(x[:, ::3] * 2) / 2            # heavy ties, also across the k-th value
    x[0, :] = 1.25                                     # every logit equal: the first k indices
    if B > 1:
        x[1, 5::7] = -np.inf
    vals, idx = s.topk(x, k)
    wv, wi = oracle.topk(x, k)
    assert np.array_equal(vals, wv)
    assert np.array_equal(idx.astype(np.int64), wi)
    bits = oracle.f32_to_bf16_bits(x)
    vals, idx = s.topk(bits, k)
    wv, wi = oracle.topk(oracle.bf16_bits_to_f32(bits), k)
    assert np.array_equal(vals, wv) and np.array_equal(idx.astype(np.int64), wi)


def test_topk_k_limit(_sampler_session):
    with pytest.raises(GorchCudaError, match="k <= 16384"):
        _sampler_session.topk(np.zeros((2, 20000), dtype=np.float32), 16385)


def test_topk_bf16_rows(sampler, oracle):
    w = workloads.vocab_sharded(8)
    vals, idx = sampler.topk(w.logits, 64)
    wv, wi = oracle.topk(oracle.bf16_bits_to_f32(w.logits), 64)
    assert np.array_equal(vals, wv) and np.array_equal(idx.astype(np.int64), wi)


def test_reference_multinomial_one_hot(sampler, known):
    for c in known["multinomial_one_hot"]:
        p = np.array(c["probs"], dtype=np.float32)
        for u in (0.0, 0.25, 0.5, 0.999999):
            ids, _ = sampler.multinomial(p, [u] * p.shape[0])
            assert ids.tolist() == c["want"]


@pytest.mark.parametrize("B,V", [(4, 1), (6, 7), (9, 255), (5, 4096), (32, 50257), (3, 151936)])
def test_multinomial_matches_oracle(sampler, oracle, B, V):
    rng = np.random.Generator(np.random.Philox(key=B * 7919 + V))
    logits = rng.standard_normal((B, V)) * 2.0
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p = (p / p.sum(axis=1, keepdims=True)).astype(np.float32)
    p[:, ::5] = 0.0                                     # zero-probability tokens are never drawn
    u = rng.random(B)
    u[0] = 0.0
    if B > 1:
        u[1] = 0.999999999                              # beyond the (deflated) total: falls through to V-1
    ids, flags = sampler.multinomial(p, u)
    want = oracle.multinomial(p, u)
    excused = (flags & FLAG_BOUNDARY) != 0
    assert np.array_equal(ids[~excused].astype(np.int64), want[~excused])
    assert np.all(p[np.arange(B), ids][(flags & FLAG_FALLBACK) == 0] > 0)


def test_multinomial_nan_row_falls_through(sampler, oracle):
    p = np.full((2, 300), 1.0 / 300, dtype=np.float32)
    p[0, 10] = np.nan                                   # every later comparison fails upstream
    u = np.array([0.5, 0.5])
    ids, flags = sampler.multinomial(p, u)
    assert ids.tolist() == oracle.multinomial(p, u).tolist()


def test_topk_rows_whose_start_is_not_typical(sampler, oracle):
    """The streaming kernel guesses a threshold from the first 4096 logits of a row. Rows whose
    largest values all sit there make the guess too high (fewer than k logits pass it) and are
    done again without it; rows whose start is unusually low make it too generous. Both must
    still return the exact top k."""
    rng = np.random.Generator(np.random.Philox(key=77))
    B, V, k = 12, 151936, 64
    x = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    x[0:4, :20] += 100.0                      # 20 huge logits at the start, k = 64 wanted
    x[4:6, :4096] -= 50.0                     # a start far below the rest
    x[6, :4096] = np.sort(x[6, :4096])[::-1]  # descending start
    x[7] = np.sort(x[7])[::-1]                # whole row descending
    x[8] = np.sort(x[8])                      # whole row ascending
    vals, idx = sampler.topk(x, k)
    wv, wi = oracle.topk(x, k)
    assert np.array_equal(vals, wv) and np.array_equal(idx.astype(np.int64), wi)
    bits = oracle.f32_to_bf16_bits(x)
    vals, idx = sampler.topk(bits, k)
    wv, wi = oracle.topk(oracle.bf16_bits_to_f32(bits), k)
    assert np.array_equal(vals, wv) and np.array_equal(idx.astype(np.int64), wi)


def test_topk_masked_rows(sampler, oracle):
    """-Inf over the start of the row or most of it does not disturb the k largest; a row with
    fewer than k finite logits has its k-th value at -Inf among thousands of ties and is flagged."""
    rng = np.random.Generator(np.random.Philox(key=79))
    B, V, k = 6, 151936, 64
    x = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    x[0:2, :8192] = -np.inf
    x[2:4][:, rng.random(V) < 0.95] = -np.inf
    x[4, 4096:] = -np.inf
    x[5, 30:] = -np.inf                                   # 30 finite logits, k = 64
    vals, idx = sampler.topk(x, k)
    wv, wi = oracle.topk(x, k)
    assert np.array_equal(vals[:5], wv[:5]) and np.array_equal(idx[:5].astype(np.int64), wi[:5])
    assert (idx[5] == -1).all()


@pytest.mark.parametrize("V", [50257, 151936])
def test_multinomial_concentrated_rows(sampler, oracle, V):
    """All the mass at the start, at the end, in one token, in long blocks separated by zeros,
    unnormalised rows (sums of 0.3 and of 40), with uniforms at 0, tiny, mid and next to 1."""
    rng = np.random.Generator(np.random.Philox(key=81 + V))
    shapes, us = 7, [0.0, 1e-12, 0.25, 0.5, 0.75, 1.0 - 1e-9]
    B = shapes * len(us)
    p = np.zeros((B, V), dtype=np.float32)
    u = np.zeros(B)
    for b in range(B):
        shape, u[b] = b % shapes, us[b // shapes]
        if shape == 0:
            p[b, 0] = 1.0
        elif shape == 1:
            p[b, V - 1] = 1.0
        elif shape == 2:
            p[b, :10] = 0.0999
            p[b, 10:] = 0.001 / (V - 10)
        elif shape == 3:
            p[b, -3:] = (0.2, 0.3, 0.5)
        elif shape == 4:
            p[b, 5000:9000] = 1.0 / 8000
            p[b, V - 9000:V - 5000] = 1.0 / 8000
        elif shape == 5:
            p[b] = (rng.random(V) * 0.6 / V).astype(np.float32)         # sums to about 0.3
        else:
            p[b] = (rng.random(V) * 80.0 / V).astype(np.float32)        # sums to about 40
    ids, flags = sampler.multinomial(p, u)
    want = oracle.multinomial(p, u)
    excused = (flags & FLAG_BOUNDARY) != 0
    assert np.array_equal(ids[~excused].astype(np.int64), want[~excused])
    # uniforms at 0 and next to the total sit on an edge of their interval by construction: those
    # rows are flagged, and must still land on a token that has probability, or fall through
    ok = (flags & FLAG_FALLBACK) != 0
    assert np.all((p[np.arange(B), ids] > 0) | ok)
    assert (~excused).sum() >= B // 2
