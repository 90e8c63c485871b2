"""Rows whose largest logits sit at the start of the row (low token ids, as frequent tokens do in
a BPE vocabulary), or whose start is unusually low: the streaming kernels guess a threshold from
the first 4096 logits, and a guess that is too high must be noticed and the row done again.
Checked through the C ABI against the oracle with the usual gates (tests/parity.py), every kernel
variant, f32 and bf16, top-k with and without top-p, greedy, and top-k off (the wide kernel's
sampled anchor and bucket scale meet the same rows)."""
import numpy as np
import pytest

from gorch_b200.config import CFG_DTYPE

from tests.test_gpu_parity import run_both

pytestmark = pytest.mark.gpu


def _rows(V, seed):
    rng = np.random.Generator(np.random.Philox(key=seed))
    B = 36
    x = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    x[0:6, :20] += 30.0                          # 20 dominant logits at the very start
    x[6:10, :300] += 6.0                         # a few hundred raised ones
    x[10:12, :4096] -= 50.0                      # a start far below the rest
    x[12] = np.sort(x[12])[::-1]                 # descending row
    x[13] = np.sort(x[13])                       # ascending row
    x[14, :4096] = np.sort(x[14, :4096])[::-1]
    x[15, 100:164] = 25.0                        # exactly 64 equal dominant logits
    x[16:20, 5000:5020] += 30.0                  # dominant logits where no warp's first step looks
    x[20:22, V // 2: V // 2 + 3] += 45.0         # three far outliers in the middle
    x[22, -40:] += 25.0                          # dominant logits at the very end
    x[23, :] = np.float32(1.5); x[23, 7] = 9.0   # flat row with one peak
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    kinds = [(0.8, 40, 0.0, 0), (1.0, 64, 0.95, 1), (0.7, 64, 0.9, 0), (1.3, 200, 0.0, 0), (0.0, 0, 0.0, 0), (1.0, 5, 0.5, 1),
             (1.0, 0, 0.9, 0), (1.0, 0, 0.99, 1), (0.8, 0, 0.0, 0), (1.2, 0, 0.6, 1)]     # the last four: top-k off
    for b in range(B):
        cfgs[b] = kinds[b % len(kinds)]
    # rows 24..35 repeat the shapes of rows 0..23 that the top-k-off kinds did not meet
    x[24:36] = x[[0, 1, 6, 10, 12, 13, 15, 16, 17, 20, 22, 23]]
    for b in range(24, 36):
        cfgs[b] = kinds[6 + b % 4]
    return x, cfgs, rng.random(B)


@pytest.mark.parametrize("V", [50257, 151936])
def test_front_loaded_rows_f32(sampler, oracle, V):
    x, cfgs, uniforms = _rows(V, 900 + V)
    run_both(sampler, oracle, x, cfgs, uniforms, allow_tie_cut=True)


def test_front_loaded_rows_bf16(sampler, oracle):
    x, cfgs, uniforms = _rows(151936, 901)
    bits = oracle.f32_to_bf16_bits(x)
    run_both(sampler, oracle, bits, cfgs, uniforms, allow_tie_cut=True)


@pytest.mark.parametrize("V", [50257, 151936])
def test_masked_vocabulary_rows(sampler, oracle, V):
    """Large parts of the vocabulary masked with -Inf (constrained decoding): the start of the
    row, most of it at random, all but fewer entries than top_k, all but the last one."""
    rng = np.random.Generator(np.random.Philox(key=950 + V))
    kinds = [(0.8, 40, 0.0, 0), (1.0, 64, 0.95, 1), (0.0, 0, 0.0, 0), (1.0, 0, 0.9, 0), (1.0, 0, 0.99, 1), (0.7, 0, 0.0, 0)]
    shapes = 5
    B = shapes * len(kinds)
    x = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    for b in range(B):
        cfgs[b] = kinds[b // shapes]
        shape = b % shapes
        if shape == 0:
            x[b, :8192] = -np.inf
        elif shape == 1:
            x[b, rng.random(V) < 0.9] = -np.inf
        elif shape == 2:
            keep = rng.choice(V, size=30, replace=False)
            row = np.full(V, -np.inf, dtype=np.float32)
            row[keep] = x[b, keep]
            x[b] = row
        elif shape == 3:
            x[b, :-1] = -np.inf
        else:
            x[b, 4096:] = -np.inf
    run_both(sampler, oracle, x, cfgs, rng.random(B), allow_tie_cut=True)


@pytest.mark.parametrize("V", [50257, 151936])
def test_quantised_peaked_and_wide_range_rows(sampler, oracle, V):
    """Distributions the iid configs never produce: logits quantised to quarters (every value
    shared by hundreds of tokens, so every cut falls inside a run of ties), one dominant token,
    a range of hundreds of units (most exponentials underflow), very small and very large
    temperatures. (No flat row under mode A's top-p: upstream's trimming loop, which the oracle
    restates, is quadratic in the number of tokens it removes and takes minutes there.)"""
    rng = np.random.Generator(np.random.Philox(key=970 + V))
    kinds = [(0.8, 40, 0.0, 0), (1.0, 64, 0.95, 1), (1.0, 0, 0.9, 0), (1.0, 0, 0.99, 1), (0.01, 0, 0.9, 1),
             (100.0, 0, 0.5, 1), (0.05, 50, 0.9, 0), (50.0, 200, 0.99, 1)]
    shapes = 4
    B = shapes * len(kinds)
    x = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    for b in range(B):
        cfgs[b] = kinds[b // shapes]
        shape = b % shapes
        if shape == 0:
            x[b] = np.round(x[b] * 4.0) / 4.0
        elif shape == 1:
            x[b, int(rng.integers(0, V))] += 100.0
        elif shape == 2:
            x[b] *= 40.0
        else:
            x[b] = np.round(x[b]) + np.float32(1e-3) * (np.arange(V) % 3 == 0)
    run_both(sampler, oracle, x, cfgs, rng.random(B), allow_tie_cut=True)
