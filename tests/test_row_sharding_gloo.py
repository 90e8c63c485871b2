"""Row-sharded sampling over two CPU ranks (gloo). The per-rank sampler is a stand-in that
answers from the CPU oracle, so this covers the host logic only: block boundaries, the
gather order, ragged last blocks."""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleSampler:
    def sample_batch(self, logits, cfgs, uniforms):
        from oracle import oracle as orc
        r = orc.sample_batch(logits, cfgs, uniforms, want_info=False, flags=orc.FAST_KTH)
        return r["ids"].astype(np.int32), np.zeros(len(r["ids"]), np.uint32)


def _worker(rank, world, port, rows, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from gorch_b200 import workloads
    from gorch_b200.distributed import sample_rows_sharded
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    w = workloads.mixed_rows(rows)
    ids, flags = sample_rows_sharded(OracleSampler(), w.logits, w.cfgs, w.uniforms, rank, world)
    np.save(os.path.join(out_dir, f"ids_{rank}.npy"), ids)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("rows", [8, 7, 1])
def test_two_ranks_match_single_process(tmp_path, rows):
    from gorch_b200 import workloads
    from oracle import oracle as orc
    port = 29500 + (os.getpid() % 2000) + rows
    mp.spawn(_worker, args=(2, port, rows, str(tmp_path)), nprocs=2, join=True)
    w = workloads.mixed_rows(rows)
    want = orc.sample_batch(w.logits, w.cfgs, w.uniforms, want_info=False, flags=orc.FAST_KTH)["ids"]
    for rank in range(2):
        got = np.load(tmp_path / f"ids_{rank}.npy")
        assert np.array_equal(got, want)


def test_single_rank_is_a_passthrough():
    from gorch_b200 import workloads
    from gorch_b200.distributed import sample_rows_sharded
    w = workloads.mixed_rows(4)
    ids, flags = sample_rows_sharded(OracleSampler(), w.logits, w.cfgs, w.uniforms, 0, 1)
    assert ids.shape == (4,) and flags.shape == (4,)
