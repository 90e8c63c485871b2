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
    one torch.distributed.all_gather over the default process group, with the tensors on
    the device the group's backend moves (NCCL: the GPU; gloo: the host).
    Rows the kernels cannot take (top_k == 0 or above the record capacity, ties that
    overflow a record) come back with id -1 and FLAG_INTERNAL.

    This is the host-array form (the records pass through host memory between the two
    kernels); a GPU job keeps everything on the device with sample_vocab_sharded_device."""
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
    if "nccl" in str(dist.get_backend()):        # NCCL moves device memory only
        t = t.cuda()
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return np.stack([o.cpu().numpy() for o in out])


def init_vocab_comm(sampler, rank: int, world: int) -> None:
    """Binds the library's own NCCL communicator to `sampler` (gorch_cuda_comm_init): rank 0 makes
    the unique id, torch.distributed (any backend) carries its 128 bytes to the other ranks."""
    import torch.distributed as dist
    box = [sampler.comm_unique_id() if rank == 0 else None]
    if world > 1:
        dist.broadcast_object_list(box, src=0)
    sampler.comm_init(rank, world, box[0])


def sample_vocab_sharded_device(sampler, d_slice, d_cfgs, d_uniforms, d_ids, d_flags, V: int, rank: int, world: int,
                                max_top_k: int = 0, rows_without_top_k: bool = False, gather_rows: bool = False) -> None:
    """The device-resident form: `d_slice` [B, hi - lo] (float32, or int16/uint16 holding bf16),
    `d_cfgs` [B, 16] bytes, `d_uniforms` [B] float64, `d_ids` / `d_flags` [B] int32 are torch CUDA
    tensors; local pass, ncclAllGather and merge all run on the sampler's stream inside
    gorch_cuda_sample_vocab_sharded_dev (init_vocab_comm first). Asynchronous. rows_without_top_k: the
    batch may hold rows with top_k == 0 (and no effective top-p cut): their owners draw from their
    slices and two small all-reduces inside the call hand the tokens to every rank. gather_rows: rows with
    top_k == 0 and an active top-p cut (with rows_without_top_k off: every row with top_k == 0) are sampled
    from whole rows that one more all-reduce brings to every rank."""
    import torch
    lo, hi = shard_vocab(V, rank, world)
    B = int(d_slice.shape[0])
    if int(d_slice.shape[1]) != hi - lo or d_slice.stride(1) != 1:
        raise ValueError(f"rank {rank} of {world} holds columns [{lo},{hi}) of V={V}")
    code = 0 if d_slice.dtype == torch.float32 else 1
    sampler.sample_vocab_sharded_ptrs(d_slice.data_ptr(), code, B, hi - lo, int(d_slice.stride(0)), lo, V, max_top_k,
                                      d_cfgs.data_ptr(), d_uniforms.data_ptr(), d_ids.data_ptr(), d_flags.data_ptr(),
                                      rows_without_top_k=rows_without_top_k, gather_rows=gather_rows)
