"""Regenerates tests/golden/oracle_vectors.npz.

The reference is Go and cannot run offline, so these vectors come from the CPU
oracle (oracle/gorch_sampling_oracle.cpp) after it has been pinned against the
reference's own known answers (reference_known_answers.json). They freeze the
oracle's behaviour on small seeded cases: a change in the oracle, or a GPU
result that differs from them, shows up as a test failure.

Run from the repo root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from gorch_b200 import workloads  # noqa: E402
from gorch_b200.config import CFG_DTYPE, MODE_A, MODE_B  # noqa: E402
from oracle import oracle as orc  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_vectors.npz")


def cases():
    rng = np.random.Generator(np.random.Philox(key=0x601D))
    out = {}
    # a: 48 rows x V=777, every combination class, both modes
    B, V = 48, 777
    x = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    x[:8] = np.round(x[:8] * 2) / 2          # ties
    cfg = np.zeros(B, dtype=CFG_DTYPE)
    combos = [(0.0, 0, 0.0), (0.8, 40, 0.0), (1.0, 0, 0.9), (0.7, 50, 0.95), (1.0, 0, 0.5),
              (1.3, 200, 1.0), (1.0, 5, 0.3), (0.5, 0, 0.0)]
    for i in range(B):
        T, k, p = combos[i % len(combos)]
        cfg[i] = (T, k, p, MODE_A if (i // len(combos)) % 2 == 0 else MODE_B)
    out["a"] = (x, cfg, rng.random(B))
    # b: first rows of the five workloads (the GPT-2 and Qwen vocabularies)
    for name, rows in (("c1", 2), ("c2", 2), ("c3", 8), ("c4", 1), ("c5", 2)):
        for mode in (MODE_A, MODE_B):
            w = workloads.make(name, rows, mode)
            out[f"{name}_m{mode}"] = (w.logits, w.cfgs, w.uniforms)
    return out


def main():
    blob = {}
    for key, (x, cfg, u) in cases().items():
        r = orc.sample_batch(x, cfg, u, want_probs=True, flags=0, threads=8)
        probs = r["probs"]
        # sparse form per row: kept indices and their probabilities; kept sets
        # above 512 tokens are thinned to 256 evenly spaced members (the kept
        # count and the softmax denominator still cover the whole row)
        nz = []
        for b in range(probs.shape[0]):
            z = np.nonzero(probs[b] > 0)[0].astype(np.int32)
            if z.size > 512:
                z = z[np.linspace(0, z.size - 1, 256).astype(np.int64)]
            nz.append(z)
        blob[f"{key}__kept_n"] = np.array([(probs[b] > 0).sum() for b in range(probs.shape[0])], dtype=np.int64)
        offs = np.cumsum([0] + [len(z) for z in nz]).astype(np.int64)
        blob[f"{key}__cfg"] = cfg
        blob[f"{key}__u"] = u
        blob[f"{key}__ids"] = r["ids"]
        blob[f"{key}__kept_off"] = offs
        blob[f"{key}__kept_idx"] = np.concatenate(nz) if nz else np.zeros(0, np.int32)
        blob[f"{key}__kept_p"] = np.concatenate([probs[b][z] for b, z in enumerate(nz)])
        blob[f"{key}__sum_exp"] = r["info"]["sum_exp"]
        if key == "a":
            blob["a__x"] = x       # the workload rows are regenerated from their seeds
    np.savez_compressed(OUT, **blob)
    print(OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
