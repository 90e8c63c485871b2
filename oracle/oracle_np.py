"""numpy mirror of the CPU oracle, written from the closed forms rather than
loop for loop, so that it cross-checks gorch_sampling_oracle.cpp.

TEST INFRASTRUCTURE ONLY (see oracle.py). Follows model/generate.go:134-260
(mode A) and model/qwen/generate.go:92-164 (mode B). Sequential f64 sums are
kept sequential (python floats) where the reference's result depends on the
order of additions.
"""
from __future__ import annotations

import math

import numpy as np

MODE_A = 0
MODE_B = 1


def argmax(logits) -> int:
    """generate.go:134-144: strict '>' from index 0, so NaN is never selected
    unless it sits at index 0 and the lowest index wins ties."""
    x = np.asarray(logits, dtype=np.float32)
    best = 0
    bv = x[0]
    for i in range(1, x.size):
        if x[i] > bv:
            bv = x[i]
            best = i
    return best


def kth_largest(data, k: int) -> np.float32:
    """generate.go:243-260 as an order statistic (k-th largest with multiplicity)."""
    x = np.sort(np.asarray(data, dtype=np.float32))[::-1]
    return x[k - 1]


def final_probs(logits, temperature, top_k, top_p, mode):
    """Steps generate.go:150-228 / qwen/generate.go:94-153: the filtered,
    renormalised probability vector (float64)."""
    x = np.asarray(logits, dtype=np.float32)
    n = x.size
    with np.errstate(all="ignore"):
        s = (x / np.float32(temperature)).astype(np.float32)
        if 0 < top_k < n:
            th = kth_largest(s, top_k)
            s = np.where(s < th, np.float32(-np.inf), s)
        m = s[0]
        for v in s[1:]:
            if v > m:
                m = v
        d = (s - np.float32(m)).astype(np.float32)
        e = np.array([math.exp(float(v)) if not math.isnan(v) else float("nan") for v in d],
                     dtype=np.float64)
        total = 0.0
        for v in e:
            total += float(v)
        q = e / total
    if 0 < top_p < 1:
        if mode == MODE_A:
            limit = float(np.float32(top_p)) * 1.5
            # ascending (prob, index): the order in which generate.go:206-219 removes
            order = sorted((i for i in range(n) if q[i] > 0), key=lambda i: (q[i], i))
            removed = 0
            while True:
                cum = 0.0
                for i in range(n):
                    if q[i] > 0:
                        cum += float(q[i])
                if cum <= limit or removed >= len(order):
                    break
                q[order[removed]] = 0.0
                removed += 1
            resum = 0.0
            for v in q:
                resum += float(v)
            with np.errstate(all="ignore"):
                q = q / resum
        else:
            p64 = float(np.float32(top_p))
            order = sorted(range(n), key=lambda i: (-q[i], i))
            cum = 0.0
            cut = n
            for r, i in enumerate(order):
                cum += float(q[i])
                if cum >= p64:
                    cut = r + 1
                    break
            resum = 0.0
            for i in order[:cut]:
                resum += float(q[i])
            out = np.zeros(n, dtype=np.float64)
            for i in order[:cut]:
                out[i] = q[i] / resum
            q = out
    return q


def draw(q, u: float) -> int:
    """generate.go:231-239."""
    c = 0.0
    for i, p in enumerate(q):
        c += float(p)
        if u < c:
            return i
    return len(q) - 1


def step(logits, temperature, top_k, top_p, mode, u) -> int:
    """The branch at generate.go:75-79."""
    if temperature == 0:
        return argmax(logits)
    return draw(final_probs(logits, temperature, top_k, top_p, mode), u)
