"""Row sharding across the GPUs of one box: rows are independent (the reference's
sample() touches one row, model/generate.go:147), so each rank samples a contiguous
block and the only communication is the gather of the token ids. One process per GPU
over torch.distributed (NCCL on GPUs; the tests run the same code over gloo).
"""
from __future__ import annotations

import numpy as np

from .workloads import shard_rows


def sample_rows_sharded(sampler, logits, cfgs, uniforms, rank: int, world: int, gather=None):
    """Sample this rank's block of a [B,V] batch and return (ids, flags) for ALL rows.

    `sampler` offers sample_batch(logits, cfgs, uniforms) -> (ids, flags) (a CudaSampler).
    `gather(local_array, counts)` concatenates the ranks' arrays in rank order; by default
    torch.distributed.all_gather_object over the default process group."""
    B = logits.shape[0]
    lo, hi = shard_rows(B, rank, world)
    if hi > lo:
        ids, flags = sampler.sample_batch(logits[lo:hi], cfgs[lo:hi], uniforms[lo:hi])
    else:
        ids, flags = np.zeros(0, np.int32), np.zeros(0, np.uint32)
    if world == 1:
        return ids, flags
    if gather is None:
        gather = _gather_default
    return gather(ids, world), gather(flags, world)


def _gather_default(local: np.ndarray, world: int) -> np.ndarray:
    import torch.distributed as dist
    parts = [None] * world
    dist.all_gather_object(parts, local)
    return np.concatenate(parts)
