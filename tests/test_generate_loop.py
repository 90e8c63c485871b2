"""Host logic of the generate loops (model/generate.go:52-131, model/qwen/generate.go:35-65)
with a scripted sampler: lengths, stop tokens, MaxSeq truncation, cached == uncached,
the order in which uniforms are consumed. The GPU variant runs the same loops on the library."""
import numpy as np
import pytest

from gorch_b200.config import GenerateConfig, QwenGenerateConfig, greedy_config
from gorch_b200.sampling import generate_with_config, qwen_generate

V = 37


class TinyModel:
    """Deterministic toy LM: logits depend on the last token and the position."""
    max_seq = 12
    vocab_size = V

    def _row(self, tok, pos):
        rng = np.random.default_rng(1000 * pos + tok)
        return rng.standard_normal(V).astype(np.float32)

    def forward(self, ids):
        return np.stack([self._row(t, i) for i, t in enumerate(ids)])

    class Cache:
        def __init__(self):
            self.n = 0

        def len(self):
            return self.n

    def new_cache(self):
        return TinyModel.Cache()

    def forward_cached(self, ids, cache):
        rows = [self._row(t, cache.n + i) for i, t in enumerate(ids)]
        cache.n += len(ids)
        return np.stack(rows)


class ScriptedSampler:
    """argmax / first-token-above-u stand-in with the CudaSampler call shapes."""

    def __init__(self):
        self.uniforms_seen = []

    def next_token(self, last_logits, cfg, u):
        if cfg.temperature == 0:
            return int(np.argmax(last_logits))
        self.uniforms_seen.append(u)
        return int(u * len(last_logits)) % len(last_logits)


def test_lengths_and_greedy_determinism():
    m, s = TinyModel(), ScriptedSampler()
    cfg = greedy_config(5)
    a = generate_with_config(m, [1, 2, 3], cfg, [], s)
    b = generate_with_config(m, [1, 2, 3], cfg, [], s)
    assert len(a) == 8 and a == b and a[:3] == [1, 2, 3]        # generate_test.go:72-90


def test_cached_equals_uncached_greedy():
    m, s = TinyModel(), ScriptedSampler()
    cfg = greedy_config(6)
    cfg2 = GenerateConfig(**{**cfg.__dict__, "use_kv_cache": True})
    assert generate_with_config(m, [4, 5], cfg, [], s) == generate_with_config(m, [4, 5], cfg2, [], s)   # generate_test.go:107-126


def test_sampling_consumes_one_uniform_per_token_in_order():
    m, s = TinyModel(), ScriptedSampler()
    cfg = GenerateConfig(max_new_tokens=4, temperature=0.8, top_k=40)
    us = [0.1, 0.5, 0.9, 0.3, 0.7]
    out = generate_with_config(m, [0], cfg, us, s)
    assert len(out) == 5 and s.uniforms_seen == us[:4]           # generate_test.go:92-103


def test_stop_token_is_not_appended():
    m, s = TinyModel(), ScriptedSampler()
    first = generate_with_config(m, [1], greedy_config(1), [], s)[-1]
    cfg = greedy_config(5)
    cfg.stop_token = first
    assert generate_with_config(m, [1], cfg, [], s) == [1]        # generate.go:82-84


def test_uncached_truncates_to_max_seq_and_cached_stops_there():
    m, s = TinyModel(), ScriptedSampler()
    long_prompt = list(range(20))
    out = generate_with_config(m, long_prompt, greedy_config(2), [], s)
    assert len(out) == 22                                        # generate.go:62-65 truncates the INPUT only
    cfg = greedy_config(50)
    cfg.use_kv_cache = True
    out = generate_with_config(m, [1, 2], cfg, [], s)
    assert len(out) == m.max_seq + 1                             # generate.go:121-123 stops at MaxSeq


def test_qwen_generate_stop_tokens_and_empty_prompt():
    m, s = TinyModel(), ScriptedSampler()
    cfg = QwenGenerateConfig(max_new_tokens=4)
    out = qwen_generate(m, [3], cfg, s)
    assert len(out) == 5
    cfg.stop_tokens = [out[1]]
    assert qwen_generate(m, [3], cfg, s) == [3]                   # qwen/generate.go:54-56
    with pytest.raises(ValueError):
        qwen_generate(m, [], cfg, s)                              # qwen/generate.go:36-38 panics


@pytest.mark.gpu
def test_generate_on_the_library_matches_oracle_steps(_sampler_session, oracle):
    m = TinyModel()
    cfg = GenerateConfig(max_new_tokens=6, temperature=0.8, top_k=10, top_p=0.9)
    us = [0.11, 0.52, 0.93, 0.34, 0.75, 0.26]
    out = generate_with_config(m, [5, 6], cfg, us, _sampler_session)
    ids = [5, 6]
    for u in us:
        logits = m.forward(ids)[-1]
        ids.append(oracle.sample(logits, cfg.temperature, cfg.top_k, cfg.top_p, u, cfg.topp_mode)[0])
    assert out == ids
