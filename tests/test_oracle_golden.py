"""Pins the CPU oracle: (1) every known-answer vector the reference's own tests
hold for this path (tests/golden/reference_known_answers.json), (2) the
committed oracle fixtures (drift check), (3) the numpy mirror, written from the
closed forms, on random small rows, (4) the semantics the reference's source
text fixes but its tests do not (ties at the top-k threshold, the inert top-p
of mode A for p >= 2/3, the n-1 fallback)."""
import json
import os

import numpy as np
import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from gorch_b200 import workloads
from gorch_b200.config import CFG_DTYPE, MODE_A, MODE_B
from oracle import oracle_np as onp

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def known():
    with open(os.path.join(GOLD, "reference_known_answers.json")) as f:
        return json.load(f)


def test_reference_argmax(oracle, known):
    for c in known["argmax"]:
        assert oracle.argmax(c["logits"]) == c["want"]
        assert onp.argmax(c["logits"]) == c["want"]


def test_reference_sample_near_greedy(oracle, known):
    for c in known["sample_near_greedy"]:
        for u in (0.0, 0.25, 0.5, 0.999999, 1.0 - 2.0 ** -53):
            for mode in (MODE_A, MODE_B):
                tok, _ = oracle.sample(c["logits"], c["temperature"], c["top_k"], c["top_p"], u, mode)
                assert tok == c["want"]


def test_reference_kth_largest(oracle, known):
    for c in known["kth_largest"]:
        assert oracle.kth_largest(c["data"], c["k"]) == c["want"]
        assert onp.kth_largest(c["data"], c["k"]) == c["want"]


def test_reference_topk(oracle, known):
    for c in known["topk"]:
        v, i = oracle.topk(np.array(c["x"], dtype=np.float32), c["k"])
        assert v.tolist() == c["values"]
        assert i.tolist() == c["indices"]
    bad = known["topk_invalid_k"]
    for k in bad["ks"]:
        with pytest.raises(ValueError):
            oracle.topk(np.zeros(bad["shape"], dtype=np.float32), k)


def test_reference_multinomial_one_hot(oracle, known):
    for c in known["multinomial_one_hot"]:
        for u in (0.0, 0.4, 0.99):
            out = oracle.multinomial(np.array(c["probs"], dtype=np.float32), [u, u])
            assert out.tolist() == c["want"]


def test_reference_bf16_rounding(oracle, known):
    c = known["bf16"][0]
    f = np.array([int(h, 16) for h in c["f32_bits"]], dtype=np.uint32).view(np.float32)
    want = [int(h, 16) for h in c["bf16_bits"]]
    assert oracle.f32_to_bf16_bits(f).tolist() == want
    assert workloads.f32_to_bf16_bits(f).tolist() == want
    for v, w in zip(f, want):
        assert oracle.lib().gorch_oracle_f32_to_bf16(float(v)) == w or np.isnan(v)
    back = oracle.bf16_bits_to_f32(np.array(want, dtype=np.uint16))
    assert back.view(np.uint32).tolist() == [w << 16 for w in want]


def _golden_cases():
    from tests.golden import make_golden
    return make_golden.cases()


def test_committed_fixtures_match_oracle(oracle):
    blob = np.load(os.path.join(GOLD, "oracle_vectors.npz"))
    for key, (x, cfg, u) in _golden_cases().items():
        assert np.array_equal(blob[f"{key}__cfg"], cfg)
        assert np.array_equal(blob[f"{key}__u"], u)
        r = oracle.sample_batch(x, cfg, u, want_probs=True, threads=8)
        assert np.array_equal(r["ids"], blob[f"{key}__ids"]), key
        offs = blob[f"{key}__kept_off"]
        for b in range(x.shape[0]):
            idx = blob[f"{key}__kept_idx"][offs[b]:offs[b + 1]]
            p = blob[f"{key}__kept_p"][offs[b]:offs[b + 1]]
            assert int((r["probs"][b] > 0).sum()) == int(blob[f"{key}__kept_n"][b])
            np.testing.assert_allclose(r["probs"][b][idx], p, rtol=1e-12)


@settings(max_examples=150, deadline=None)
@given(
    n=st.integers(1, 48), seed=st.integers(0, 2 ** 31), T=st.sampled_from([0.25, 0.7, 1.0, 1.3]),
    kfrac=st.floats(0, 1.2), p=st.sampled_from([0.0, 0.1, 0.3, 0.5, 0.66, 0.67, 0.9, 0.99, 1.0]),
    mode=st.sampled_from([MODE_A, MODE_B]), coarse=st.booleans(),
)
def test_oracle_matches_numpy_mirror(oracle, n, seed, T, kfrac, p, mode, coarse):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(n) * 2.0).astype(np.float32)
    if coarse:
        x = np.round(x)          # ties
    k = int(kfrac * n)
    u = float(rng.random())
    tok, info, probs = oracle.sample(x, T, k, p, u, mode, want_probs=True)
    q = onp.final_probs(x, T, k, p, mode)
    np.testing.assert_allclose(probs, q, rtol=1e-12, atol=0, equal_nan=True)
    assert tok == onp.draw(q, u)
    assert info["kept"] == int((q > 0).sum())


def test_topk_keeps_ties(oracle):
    x = np.array([5, 1, 5, 3, 5, 2, 5], dtype=np.float32)
    _, info, probs = oracle.sample(x, 1.0, 2, 0.0, 0.5, MODE_A, want_probs=True)
    assert info["kept"] == 4                      # generate.go:159-163: every value >= threshold stays
    assert np.allclose(probs[[0, 2, 4, 6]], 0.25)


def test_topk_before_softmax(oracle):
    x = np.array([2.0, 1.0, 0.0, -1.0], dtype=np.float32)
    _, info, probs = oracle.sample(x, 1.0, 2, 0.0, 0.5, MODE_A, want_probs=True)
    e = np.exp(np.array([0.0, -1.0]))
    assert np.allclose(probs[:2], e / e.sum())    # denominator over the kept set only
    assert probs[2] == 0 and probs[3] == 0


def test_mode_a_inert_from_two_thirds(oracle):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(200) * 2).astype(np.float32)
    _, _, base = oracle.sample(x, 1.0, 0, 0.0, 0.5, MODE_A, want_probs=True)
    for p in (0.67, 0.8, 0.9, 0.95, 0.99):
        _, info, pr = oracle.sample(x, 1.0, 0, p, 0.5, MODE_A, want_probs=True)
        assert info["kept"] == 200
        np.testing.assert_allclose(pr, base, rtol=1e-14)
    _, info, _ = oracle.sample(x, 1.0, 0, 0.66, 0.5, MODE_A, want_probs=True)
    assert info["kept"] < 200


def test_mode_a_removes_lowest_index_among_equal(oracle):
    x = np.zeros(4, dtype=np.float32)             # probs 0.25 each; 1.5*0.4 = 0.6 -> two removed
    _, info, pr = oracle.sample(x, 1.0, 0, 0.4, 0.5, MODE_A, want_probs=True)
    assert pr.tolist() == [0.0, 0.0, 0.5, 0.5]


def test_mode_a_can_remove_everything(oracle):
    x = np.array([0, 0], dtype=np.float32)        # 0.5 each, 1.5*0.1 = 0.15: both removed -> 0/0
    tok, info, pr = oracle.sample(x, 1.0, 0, 0.1, 0.3, MODE_A, want_probs=True)
    assert np.isnan(pr).all() and tok == 1 and info["fallback"] == 1


def test_mode_b_nucleus(oracle):
    x = np.log(np.array([0.5, 0.3, 0.15, 0.05])).astype(np.float32)
    _, info, pr = oracle.sample(x, 1.0, 0, 0.7, 0.5, MODE_B, want_probs=True)
    assert info["kept"] == 2
    np.testing.assert_allclose(pr[:2], [0.625, 0.375], rtol=1e-6)


def test_fallback_to_last_index(oracle):
    x = np.array([0.0, -np.inf, -np.inf], dtype=np.float32)
    tok, info = oracle.sample(x, 1.0, 0, 0.0, 1.0, MODE_A)    # u = 1.0 is never < cumulative
    assert tok == 2 and info["fallback"] == 1


def test_nan_poisons_to_last_index(oracle):
    x = np.array([1.0, np.nan, 2.0, 0.5], dtype=np.float32)
    for k in (0, 2):
        tok, _ = oracle.sample(x, 1.0, k, 0.0, 0.1, MODE_A)
        assert tok == 3


def test_batch_threads_agree(oracle):
    w = workloads.mixed_rows(32)
    a = oracle.sample_batch(w.logits, w.cfgs, w.uniforms, threads=1)
    b = oracle.sample_batch(w.logits, w.cfgs, w.uniforms, threads=4, flags=oracle.FAST_KTH)
    assert np.array_equal(a["ids"], b["ids"])
