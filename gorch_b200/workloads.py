"""Seeded synthetic LM-head logits for the five sampling workloads.

No checkpoint or dataset is available offline, so these stand in for real
logits. Everything is drawn on the host with numpy's Philox bit generator so
that every machine sees identical inputs:

  logits stream     key = 0x60C00000 + 16*c
  uniform stream    key + 1
  structure stream  key + 2   (peak columns, tie rows)

for workload index c = 1..5. Values are drawn as float64 standard normals,
scaled by sigma, cast to float32 (and, for c5, rounded to bf16 by
round-to-nearest-even, the rule of the reference's tensor.go:85-94).

Top-p flavour: rows with the GPT-2 vocabulary (V=50257) default to the
reference's model/generate.go semantics (mode A), rows with the Qwen
vocabulary (V=151936) to model/qwen/generate.go (mode B, true nucleus);
`mode=` overrides that for parity runs of the other flavour.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .config import CFG_DTYPE, MODE_A, MODE_B

BASE_KEY = 0x60C00000

GPT2_VOCAB = 50257
QWEN_VOCAB = 151936


@dataclass
class Workload:
    name: str
    logits: np.ndarray      # [B,V] float32, or uint16 holding bf16 bit patterns
    cfgs: np.ndarray        # [B] CFG_DTYPE
    uniforms: np.ndarray    # [B] float64 in [0,1)
    dtype: str              # "f32" | "bf16"
    description: str = ""
    tie_rows: np.ndarray = field(default_factory=lambda: np.zeros(0, dtype=np.int64))
    expected_greedy: dict = field(default_factory=dict)  # row -> id, for injected ties

    @property
    def B(self) -> int:
        return self.logits.shape[0]

    @property
    def V(self) -> int:
        return self.logits.shape[1]

    @property
    def bytes_per_row(self) -> int:
        """Algorithmic bytes per sampled row: one read of the logits row plus
        its config (16), uniform (8) and the id written (4)."""
        return self.V * self.logits.dtype.itemsize + 16 + 8 + 4


_SHARD = 0


def set_shard(shard: int) -> None:
    """Select an independent replica of every stream (key + 4096*shard); shard 0
    is the canonical workload. Used to give each GPU of a weak-scaling run its
    own rows."""
    global _SHARD
    _SHARD = int(shard)


def _rng(c: int, stream: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=BASE_KEY + 16 * c + stream + 4096 * _SHARD))


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round-to-nearest-even, NaN kept quiet."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    is_nan = (((bits >> 23) & 0xFF) == 0xFF) & ((bits & 0x7FFFFF) != 0)
    rounding = np.uint32(0x7FFF) + ((bits >> 16) & np.uint32(1))
    out = ((bits + rounding) >> 16).astype(np.uint16)
    return np.where(is_nan, ((bits >> 16) | np.uint32(0x40)).astype(np.uint16), out)


def _normal_logits(c: int, B: int, V: int, sigma: float) -> np.ndarray:
    rng = _rng(c, 0)
    out = np.empty((B, V), dtype=np.float32)
    step = max(1, (1 << 22) // V)  # ~4M values per draw keeps the f64 scratch small
    for b0 in range(0, B, step):
        b1 = min(B, b0 + step)
        out[b0:b1] = (rng.standard_normal((b1 - b0, V)) * sigma).astype(np.float32)
    return out


def _peak_columns(rng: np.random.Generator, B: int, V: int, npeaks: int) -> np.ndarray:
    """npeaks distinct columns per row: the first distinct values, in order of
    appearance, of 4*npeaks integers drawn per row."""
    draws = rng.integers(0, V, size=(B, 4 * npeaks))
    cols = np.empty((B, npeaks), dtype=np.int64)
    for b in range(B):
        _, first = np.unique(draws[b], return_index=True)
        picked = draws[b][np.sort(first)[:npeaks]]
        if picked.size != npeaks:
            raise RuntimeError("peak draw produced too few distinct columns")
        cols[b] = picked
    return cols


def _add_peaks(logits: np.ndarray, cols: np.ndarray, offset: float) -> None:
    rows = np.arange(logits.shape[0])[:, None]
    logits[rows, cols] = (logits[rows, cols] + np.float32(offset)).astype(np.float32)


def _cfgs(B: int, temperature: float, top_k: int, top_p: float, mode: int) -> np.ndarray:
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    cfgs["temperature"] = temperature
    cfgs["top_k"] = top_k
    cfgs["top_p"] = top_p
    cfgs["topp_mode"] = mode
    return cfgs


def gpt2_step(steps: int = 1000, mode: int | None = None) -> Workload:
    """c1: `steps` independent B=1 GPT-2 sampling steps under the reference's
    DefaultGenerateConfig (T=0.8, k=40, p off), stacked as [steps, 50257]."""
    c, V = 1, GPT2_VOCAB
    logits = _normal_logits(c, steps, V, 2.0)
    _add_peaks(logits, _peak_columns(_rng(c, 2), steps, V, 16), 8.0)
    return Workload("c1_gpt2_step", logits, _cfgs(steps, 0.8, 40, 0.0, MODE_A if mode is None else mode),
                    _rng(c, 1).random(steps), "f32",
                    "GPT-2-small sampling step, T=0.8 k=40, one row per step")


def nucleus_batch(B: int = 64, mode: int | None = None) -> Workload:
    """c2: B=64, V=50257, T=1.0, top-p 0.9, top-k off."""
    c, V = 2, GPT2_VOCAB
    logits = _normal_logits(c, B, V, 2.0)
    _add_peaks(logits, _peak_columns(_rng(c, 2), B, V, 16), 8.0)
    return Workload("c2_nucleus_batch", logits, _cfgs(B, 1.0, 0, 0.9, MODE_A if mode is None else mode),
                    _rng(c, 1).random(B), "f32", "nucleus batch, T=1.0 p=0.9")


MIXED_CYCLE = (
    (0.0, 0, 0.0),     # greedy
    (0.7, 50, 0.95),
    (1.0, 0, 0.8),
    (1.3, 200, 1.0),
)


def mixed_rows(B: int = 256, mode: int | None = None) -> Workload:
    """c3: B=256, V=50257, row i uses MIXED_CYCLE[i % 4]; 5% of the rows get the
    row maximum copied into two other columns (lowest index must win greedy)."""
    c, V = 3, GPT2_VOCAB
    logits = _normal_logits(c, B, V, 2.0)
    srng = _rng(c, 2)
    _add_peaks(logits, _peak_columns(srng, B, V, 16), 8.0)
    n_tie = max(1, round(0.05 * B))
    tie_rows = np.sort(srng.choice(B, size=n_tie, replace=False))
    expected = {}
    for b in tie_rows:
        top = int(np.argmax(logits[b]))
        others = []
        while len(others) < 2:
            j = int(srng.integers(0, V))
            if j != top and j not in others:
                others.append(j)
        logits[b, others] = logits[b, top]
        expected[int(b)] = min([top] + others)
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    for i in range(B):
        t, k, p = MIXED_CYCLE[i % 4]
        cfgs[i] = (t, k, p, MODE_A if mode is None else mode)
    return Workload("c3_mixed_rows", logits, cfgs, _rng(c, 1).random(B), "f32",
                    "mixed per-row configs with injected ties", tie_rows, expected)


def flat_stress(B: int = 512, mode: int | None = None) -> Workload:
    """c4: B=512, V=151936, N(0,0.25^2) with no peaks, T=1.0, top-p 0.99."""
    c, V = 4, QWEN_VOCAB
    logits = _normal_logits(c, B, V, 0.25)
    return Workload("c4_flat_stress", logits, _cfgs(B, 1.0, 0, 0.99, MODE_B if mode is None else mode),
                    _rng(c, 1).random(B), "f32", "flat-distribution stress, T=1.0 p=0.99")


def vocab_sharded(B: int = 1024, mode: int | None = None) -> Workload:
    """c5: B=1024, V=151936 bf16, N(0,3^2) + 32 peaks at +6, T=0.7 k=64 p=0.95."""
    c, V = 5, QWEN_VOCAB
    logits = _normal_logits(c, B, V, 3.0)
    _add_peaks(logits, _peak_columns(_rng(c, 2), B, V, 32), 6.0)
    return Workload("c5_vocab_sharded", f32_to_bf16_bits(logits),
                    _cfgs(B, 0.7, 64, 0.95, MODE_B if mode is None else mode),
                    _rng(c, 1).random(B), "bf16", "large bf16 batch, T=0.7 k=64 p=0.95")


WORKLOADS = {
    "c1": gpt2_step,
    "c2": nucleus_batch,
    "c3": mixed_rows,
    "c4": flat_stress,
    "c5": vocab_sharded,
}


def make(name: str, rows: int | None = None, mode: int | None = None) -> Workload:
    """Build workload `name` ("c1".."c5"); `rows` overrides the row count."""
    fn = WORKLOADS[name]
    if rows is None:
        return fn(mode=mode)
    return fn(rows, mode=mode)


def shard_rows(B: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous block of ceil(B/world) rows owned by `rank`: [lo, hi)."""
    per = -(-B // world)
    lo = min(B, rank * per)
    return lo, min(B, lo + per)


def shard_vocab(V: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous column slice [lo, hi) of a V-wide row owned by `rank`."""
    per = -(-V // world)
    lo = min(V, rank * per)
    return lo, min(V, lo + per)
