"""Vocab-sharded sampling over two CPU ranks (gloo). The per-rank sampler is a CPU stand-in
that speaks the kernels' record format, so this covers the host logic: the column slices, the
one all-gather and its rank order, and that every rank ends with every id."""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _case(rows, V):
    from gorch_b200.config import CFG_DTYPE
    rng = np.random.Generator(np.random.Philox(key=0x5EED + rows * 131 + V))
    logits = (rng.standard_normal((rows, V)) * 2.0).astype(np.float32)
    logits[:, ::7] = np.round(logits[:, ::7])          # ties, also at the top-k threshold
    cfgs = np.zeros(rows, dtype=CFG_DTYPE)
    for i in range(rows):
        cfgs[i] = [(0.0, 0, 0.0, 0), (0.7, 5, 0.95, 1), (1.0, 3, 0.0, 0), (1.3, 8, 0.9, 0)][i % 4]
    return logits, cfgs, rng.random(rows)


def _worker(rank, world, port, rows, V, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    from gorch_b200 import workloads
    from gorch_b200.distributed import sample_vocab_sharded
    from vocab_standin import StandInSampler
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    logits, cfgs, uniforms = _case(rows, V)
    lo, hi = workloads.shard_vocab(V, rank, world)
    ids, flags = sample_vocab_sharded(StandInSampler(), logits[:, lo:hi], cfgs, uniforms, V, rank, world)
    np.save(os.path.join(out_dir, f"ids_{rank}.npy"), ids)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("rows,V", [(8, 1000), (5, 37), (3, 257)])
def test_two_ranks_match_the_whole_row(tmp_path, rows, V):
    from oracle import oracle as orc
    port = 31500 + (os.getpid() % 2000) + rows
    mp.spawn(_worker, args=(2, port, rows, V, str(tmp_path)), nprocs=2, join=True)
    logits, cfgs, uniforms = _case(rows, V)
    want = orc.sample_batch(logits, cfgs, uniforms, want_info=False, flags=orc.FAST_KTH)["ids"]
    for rank in range(2):
        got = np.load(tmp_path / f"ids_{rank}.npy")
        assert np.array_equal(got, want)


def test_slice_width_is_checked():
    from gorch_b200.distributed import sample_vocab_sharded
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from vocab_standin import StandInSampler
    logits, cfgs, uniforms = _case(2, 10)
    with pytest.raises(ValueError):
        sample_vocab_sharded(StandInSampler(), logits[:, :4], cfgs, uniforms, 10, 0, 2)
