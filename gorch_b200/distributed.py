"""Sharding across the GPUs of one box, one process per GPU over torch.distributed
(NCCL on GPUs; the tests run the same code over gloo).

Row sharding: rows are independent (the reference's sample() touches one row,
model/generate.go:147), so each rank samples a contiguous block and the only
communication is the gather of the token ids.

Vocab sharding: every rank holds a contiguous column slice of every row. Each rank
reduces its slice to a fixed-size record per row (local maximum + every local logit at
or above the local top_k-th largest), ONE all-gather brings all records to every rank,
and every rank finishes every row from the joined lists (the global top_k-th largest is
at least every local one, so nothing that survives the global top-k is missing).
"""
from __future__ import annotations

import numpy as np

from .workloads import shard_rows, shard_vocab


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


def sample_vocab_sharded(sampler, logits_slice, cfgs, uniforms, V: int, rank: int, world: int, gather=None):
    """Vocab-sharded sampling of a [B,V] batch of which this rank holds the columns
    shard_vocab(V, rank, world); returns (ids, flags) for all B rows on every rank.

    `sampler` offers vocab_local(logits_slice, cfgs, col_offset) -> records [B, R] (uint8)
    and vocab_merge(all_records [world, B, R], cfgs, uniforms, V) -> (ids, flags)
    (a CudaSampler). `gather(records)` stacks the ranks' arrays in rank order; by default
    torch.distributed.all_gather over the default process group (one collective).
    Rows the kernels cannot take (top_k == 0 or above the record capacity, ties that
    overflow a record) come back with id -1 and FLAG_INTERNAL."""
    lo, hi = shard_vocab(V, rank, world)
    if logits_slice.shape[1] != hi - lo:
        raise ValueError(f"rank {rank} of {world} holds columns [{lo},{hi}) of V={V}, got {logits_slice.shape[1]} columns")
    rec = sampler.vocab_local(logits_slice, cfgs, lo)
    if gather is None:
        gather = _stack_default
    allrec = gather(rec) if world > 1 else rec[None]
    return sampler.vocab_merge(allrec, cfgs, uniforms, V)


def _stack_default(local: np.ndarray) -> np.ndarray:
    import torch
    import torch.distributed as dist
    world = dist.get_world_size()
    t = torch.from_numpy(np.ascontiguousarray(local))
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return np.stack([o.numpy() for o in out])
