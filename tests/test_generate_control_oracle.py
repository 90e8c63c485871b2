"""The scripted generate-loop oracle (oracle.generate_scripted: the control flow of
model/generate.go:57-131 and model/qwen/generate.go:35-62 with the sampler's answers given)
against the behaviour the reference's own tests pin (model/generate_test.go:72-126: result =
prompt + MaxNewTokens ids; the stop token is not appended; cached == uncached) and against the
host loops of gorch_b200.sampling driven by the same script."""
import numpy as np
import pytest

from gorch_b200.config import GenerateConfig, QwenGenerateConfig
from gorch_b200.sampling import generate_with_config, qwen_generate
from oracle import oracle


class ScriptModel:
    """A model whose logits are never looked at: the scripted sampler ignores them."""
    vocab_size = 4

    def __init__(self, max_seq):
        self.max_seq = max_seq
        self.windows = []
        self.fed = []

    def forward(self, ids):
        self.windows.append(len(ids))
        return np.zeros((len(ids), self.vocab_size), dtype=np.float32)

    class Cache:
        n = 0

        def len(self):
            return self.n

    def new_cache(self):
        return ScriptModel.Cache()

    def forward_cached(self, ids, cache):
        if cache.n:
            self.fed.extend(ids)
        cache.n += len(ids)
        return np.zeros((len(ids), self.vocab_size), dtype=np.float32)


class Script:
    def __init__(self, script):
        self.script, self.calls = list(script), 0

    def next_token(self, last_logits, cfg, u):
        self.calls += 1
        return self.script[self.calls - 1]


def test_known_answers_of_the_reference_tests():
    # generate_test.go:72-90: 3 prompt ids + 5 new ones
    r = oracle.generate_scripted(0, [1, 2, 3], [7, 7, 7, 7, 7], 5, 64, [-1])
    assert r["tokens"] == [1, 2, 3, 7, 7, 7, 7, 7] and r["reason"] == 2 and r["sampler_calls"] == 5
    # generate.go:82-84: the stop token ends the loop and is not part of the result
    r = oracle.generate_scripted(0, [1], [9, 8], 5, 64, [9])
    assert r["tokens"] == [1] and r["reason"] == 1 and r["sampler_calls"] == 1
    # generate.go:121-123: the cached loop ends when the cache holds MaxSeq positions, token kept
    r = oracle.generate_scripted(1, [1, 2], [5] * 50, 50, 12, [-1])
    assert len(r["tokens"]) == 13 and r["reason"] == 3 and len(r["fed"]) == 10
    # generate.go:62-65: the uncached loop truncates the input only
    r = oracle.generate_scripted(0, list(range(20)), [5, 5], 2, 12, [-1])
    assert len(r["tokens"]) == 22 and r["fed"] == [8, 9]
    # qwen/generate.go:54-56, 64-71: any of several stop tokens
    r = oracle.generate_scripted(2, [3], [4, 5, 6, 7], 4, 64, [6, 9])
    assert r["tokens"] == [3, 4, 5] and r["reason"] == 1
    # StopToken = -1 never matches (generate.go:82), also if a "token" were negative
    assert oracle.generate_scripted(1, [3], [2, 2], 2, 64, [-1])["reason"] == 2


@pytest.mark.parametrize("loop", [0, 1, 2])
def test_scripted_oracle_equals_the_host_loops(loop):
    rng = np.random.default_rng(100 + loop)
    for case in range(300):
        n_prompt = int(rng.integers(1, 12))      # an empty prompt panics in all three loops
        prompt = rng.integers(0, 6, n_prompt).tolist()
        max_new = int(rng.integers(0, 10))
        max_seq = int(rng.integers(1, 14))
        script = rng.integers(0, 6, max(max_new, 1)).tolist()
        if loop == 2:
            stops = rng.integers(0, 8, int(rng.integers(0, 4))).tolist()
        else:
            stops = [int(rng.integers(-1, 6))]
        want = oracle.generate_scripted(loop, prompt, script, max_new, max_seq, stops)
        m, s = ScriptModel(max_seq), Script(script)
        if loop == 2:
            got = qwen_generate(m, prompt, QwenGenerateConfig(max_new_tokens=max_new, stop_tokens=stops), s, uniforms=[])
        else:
            cfg = GenerateConfig(max_new_tokens=max_new, temperature=0.0, stop_token=stops[0], use_kv_cache=(loop == 1))
            got = generate_with_config(m, prompt, cfg, [], s)
        assert got == want["tokens"], (case, prompt, script, max_new, max_seq, stops)
        assert s.calls == want["sampler_calls"]
        if loop == 0:
            assert m.windows == [n_prompt + i - f for i, f in enumerate(want["fed"])]
        else:
            assert m.fed == want["fed"]
