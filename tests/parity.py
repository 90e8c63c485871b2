"""Shared comparison rules for the GPU-vs-oracle parity tests.

Gates (the contract this repo is measured against):
  * greedy ids and top-k kept sets: bit-exact;
  * filtered probability vectors: <= 1e-6 relative;
  * sampled ids: identical, except rows whose uniform lies within 1e-6 of a CDF
    edge; those are counted, not failed.
"""
from __future__ import annotations

import numpy as np

from gorch_b200.config import (FLAG_BAD_CFG, FLAG_BOUNDARY, FLAG_INTERNAL, FLAG_TIE_CUT,
                               FLAG_TOPP_EDGE)

REL_TOL = 1e-6


def compare(gpu: dict, ora: dict, uniforms, check_probs=True, allow_tie_cut=False):
    """Returns a report dict; raises AssertionError on a gate failure."""
    gids = gpu["ids"].astype(np.int64)
    oids = ora["ids"].astype(np.int64)
    flags = gpu["flags"]
    B = gids.size
    assert not np.any(flags & FLAG_INTERNAL), f"internal-invariant flag on rows {np.nonzero(flags & FLAG_INTERNAL)[0][:8]}"
    assert not np.any(flags & FLAG_BAD_CFG)
    report = {"rows": B, "id_mismatch": 0, "boundary_mismatch": 0, "boundary_rows": 0,
              "max_rel_prob_err": 0.0, "kept_mismatch_rows": 0, "tie_cut_rows": 0}
    info = ora.get("info")
    soft = np.zeros(B, dtype=bool)   # rows where upstream leaves the result unpinned
    if allow_tie_cut:
        soft |= (flags & (FLAG_TIE_CUT | FLAG_TOPP_EDGE)) != 0
        if info is not None:
            soft |= info["cut_in_tie"] != 0
    report["tie_cut_rows"] = int(soft.sum())
    if check_probs and gpu.get("probs") is not None and ora.get("probs") is not None:
        gp, op = gpu["probs"], ora["probs"]
        for b in range(B):
            if soft[b]:
                continue
            g, o = gp[b], op[b]
            if np.isnan(o).any() or np.isnan(g).any():
                assert np.isnan(o).all() and np.isnan(g).all(), f"row {b}: NaN pattern differs"
                continue
            kept_g, kept_o = g > 0, o > 0
            if not np.array_equal(kept_g, kept_o):
                report["kept_mismatch_rows"] += 1
                diff = np.nonzero(kept_g != kept_o)[0]
                raise AssertionError(f"row {b}: kept set differs at {diff[:8]} "
                                     f"(gpu {kept_g.sum()} vs oracle {kept_o.sum()})")
            rel = np.abs(g[kept_o] - o[kept_o]) / o[kept_o]
            m = float(rel.max()) if rel.size else 0.0
            report["max_rel_prob_err"] = max(report["max_rel_prob_err"], m)
            assert m <= REL_TOL, f"row {b}: prob rel err {m:.3e} > {REL_TOL}"
    for b in range(B):
        near = False
        if info is not None:
            u = float(uniforms[b])
            near = min(abs(u - info["edge_lo"][b]), abs(u - info["edge_hi"][b])) <= 1e-6
        near = near or bool(flags[b] & FLAG_BOUNDARY)
        report["boundary_rows"] += int(bool(flags[b] & FLAG_BOUNDARY))
        if gids[b] != oids[b]:
            report["id_mismatch"] += 1
            if near or soft[b]:
                report["boundary_mismatch"] += 1
            else:
                raise AssertionError(
                    f"row {b}: id {gids[b]} != oracle {oids[b]} (u={uniforms[b]!r}, flags={flags[b]:#x})")
    return report
