"""Vocab-sharded sampling on several GPUs, one process per GPU, through the library's own calls
(gorch_cuda_comm_init, gorch_cuda_sample_vocab_sharded_ex_dev), against the CPU oracle on whole rows.

Opt-in: set GORCH_TEST_RANKS=2 (or 4, 8) on a box that shows that many GPUs:

    GORCH_TEST_RANKS=2 python -m pytest tests/test_gpu_vocab_sharded_ranks.py -q -m gpu

Without the variable every case is skipped (the other vocab-sharding tests need one GPU only: the
ranks' local passes one after another, and the library call on a one-rank communicator). The rows
are short, so that the oracle's quadratic trimming loop for generate.go's top-p rule stays cheap."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RANKS = int(os.environ.get("GORCH_TEST_RANKS", "0") or 0)
JOIN_SECONDS = 300


def _case(bf16, V):
    from gorch_b200 import workloads
    from gorch_b200.config import CFG_DTYPE
    rng = np.random.Generator(np.random.Philox(key=0xBEEF + V + int(bf16)))
    B = 64
    x = (rng.standard_normal((B, V)) * 2.5).astype(np.float32)
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    rows = [(1.0, 0, 0.0, 0), (0.8, 40, 0.0, 0), (0.7, 0, 0.9, 0), (0.0, 0, 0.0, 0),     # no cut, top-k, inert cut, greedy
            (1.0, 0, 0.9, 1), (0.9, 0, 0.6, 0), (1.0, 0, 0.99, 1), (0.7, 64, 0.95, 1)]   # nucleus (B), trimming (A), wide nucleus, top-k + top-p
    for i in range(B):
        cfgs[i] = rows[i % len(rows)]
    logits = workloads.f32_to_bf16_bits(x) if bf16 else x
    return logits, cfgs, rng.random(B)


def _worker(rank, world, port, bf16, V, owner, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from gorch_b200 import distributed, sampling, workloads
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    s = sampling.CudaSampler(rank)
    distributed.init_vocab_comm(s, rank, world)
    logits, cfgs, uniforms = _case(bf16, V)
    B = logits.shape[0]
    lo, hi = workloads.shard_vocab(V, rank, world)
    part = np.ascontiguousarray(logits[:, lo:hi])
    d_x = torch.from_numpy(part.view(np.int16) if bf16 else part).cuda()
    d_cf = torch.from_numpy(cfgs.view(np.uint8).reshape(B, 16).copy()).cuda()
    d_u = torch.from_numpy(uniforms.copy()).cuda()
    d_ids = torch.full((B,), -7, dtype=torch.int32, device="cuda")
    d_fl = torch.zeros(B, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    for _ in range(2):                                 # twice: the second call reuses the scratch of the first
        distributed.sample_vocab_sharded_device(s, d_x, d_cf, d_u, d_ids, d_fl, V, rank, world, max_top_k=64,
                                                rows_without_top_k=owner, gather_rows=True)
    s.sync()
    np.save(os.path.join(out_dir, f"ids_{rank}.npy"), d_ids.cpu().numpy())
    np.save(os.path.join(out_dir, f"flags_{rank}.npy"), d_fl.cpu().numpy().view(np.uint32))
    dist.barrier()
    s.comm_release()
    s.release()
    dist.destroy_process_group()


@pytest.mark.skipif(RANKS < 2, reason="set GORCH_TEST_RANKS=2|4|8 on a box with that many GPUs")
@pytest.mark.parametrize("owner", [True, False])
@pytest.mark.parametrize("bf16,V", [(False, 30011), (True, 30008)])
def test_every_kind_of_row_on_several_gpus(tmp_path, oracle, bf16, V, owner):
    import torch
    import torch.multiprocessing as mp
    from tests.test_gpu_vocab_sharded import check_ids
    if torch.cuda.device_count() < RANKS:
        pytest.skip(f"{RANKS} GPUs asked for, {torch.cuda.device_count()} visible")
    port = 32500 + (os.getpid() % 2000) + int(bf16) * 2 + int(owner)
    ctx = mp.spawn(_worker, args=(RANKS, port, bf16, V, owner, str(tmp_path)), nprocs=RANKS, join=False)
    try:
        import time
        t0 = time.time()
        while not ctx.join(timeout=5):
            assert time.time() - t0 < JOIN_SECONDS, "the ranks did not finish"
    finally:
        for p in ctx.processes:                        # the exact children of this test, if any is left
            if p.is_alive():
                p.terminate()
    logits, cfgs, uniforms = _case(bf16, V)
    first = np.load(tmp_path / "ids_0.npy")
    for rank in range(RANKS):
        ids, flags = np.load(tmp_path / f"ids_{rank}.npy"), np.load(tmp_path / f"flags_{rank}.npy")
        assert np.array_equal(ids, first), "every rank ends with the same ids"
        check_ids(oracle, logits, cfgs, uniforms, ids, flags)
