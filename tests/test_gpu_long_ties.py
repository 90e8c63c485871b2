"""Rows whose top-p cut falls inside a long run of equal logits: thousands of tokens share the
probability at the cut, far more than any kernel's exact list holds. Constant rows are what an
untrained or collapsed model emits, so these are legitimate inputs. Mode A's order among equal
probabilities is pinned upstream (lowest index removed first, generate.go:208-212); mode B's is
not (sort.Slice is unstable), there the oracle's ascending-index order is the convention."""
import numpy as np
import pytest

from gorch_b200.config import CFG_DTYPE, MODE_A, MODE_B
from tests.test_gpu_parity import run_both

pytestmark = pytest.mark.gpu


def cfgs_of(n, T, k, p, mode):
    c = np.zeros(n, dtype=CFG_DTYPE)
    c["temperature"], c["top_k"], c["top_p"], c["topp_mode"] = T, k, p, mode
    return c


@pytest.mark.parametrize("mode,p", [(MODE_B, 0.9), (MODE_B, 0.3), (MODE_A, 0.5), (MODE_A, 0.2)])
def test_constant_rows(sampler, oracle, mode, p):
    B, V = 3, 20011
    x = np.zeros((B, V), np.float32)
    x[1, :] = -3.25
    x[2, :] = 7.0
    u = np.array([0.0, 0.37, 0.999])
    run_both(sampler, oracle, x, cfgs_of(B, 1.0, 0, p, mode), u, allow_tie_cut=(mode == MODE_B))


@pytest.mark.parametrize("mode,p", [(MODE_B, 0.95), (MODE_A, 0.55)])
def test_quantised_flat_rows(sampler, oracle, mode, p):
    rng = np.random.Generator(np.random.Philox(key=4242 + mode))
    B, V = 4, 30000
    x = (np.round(rng.standard_normal((B, V)) * 4.0) / 8.0).astype(np.float32)   # ~30 distinct values
    run_both(sampler, oracle, x, cfgs_of(B, 0.9, 0, p, mode), rng.random(B), allow_tie_cut=(mode == MODE_B))


def test_constant_row_with_top_k_and_top_p(sampler, oracle):
    # every logit ties at the top-k threshold: the kept set is the whole row (generate.go:157-164)
    B, V = 2, 9001
    x = np.full((B, V), 1.5, np.float32)
    run_both(sampler, oracle, x, cfgs_of(B, 0.8, 40, 0.9, MODE_B), np.array([0.2, 0.8]), allow_tie_cut=True)
