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


class _RecordingLib:
    """Stands in for libgorchcuda.so in the two vocab-sharded entry points: records the call."""
    def __init__(self):
        self.calls = []

    def gorch_cuda_sample_vocab_sharded_dev(self, ctx, logits, dtype, B, Vslice, stride, off, V, max_k, cfgs, uni, ids, flags, err):
        self.calls.append(("plain", B, Vslice, stride, off, V, max_k, None))
        return 0

    def gorch_cuda_sample_vocab_sharded_ex_dev(self, ctx, logits, dtype, B, Vslice, stride, off, V, max_k, bits, cfgs, uni, ids, flags, err):
        self.calls.append(("ex", B, Vslice, stride, off, V, max_k, bits))
        return 0


def test_device_form_passes_the_slice_and_the_bits_for_rows_without_top_k():
    """The host side of the device-resident call: this rank's column range, and which of the two
    ways of serving rows without top-k the caller asked for (bit 0: the owner's draw, bit 1: whole
    rows gathered), reach the C ABI unchanged."""
    import torch
    from gorch_b200.distributed import sample_vocab_sharded_device
    from gorch_b200.sampling import CudaSampler
    from gorch_b200 import workloads
    s = object.__new__(CudaSampler)                    # no GPU here: only the argument plumbing runs
    s._lib, s._ctx = _RecordingLib(), None
    B, V, world = 3, 1001, 4
    for rank in range(world):
        lo, hi = workloads.shard_vocab(V, rank, world)
        d = torch.zeros(B, hi - lo)
        cf, u = torch.zeros(B, 16, dtype=torch.uint8), torch.zeros(B, dtype=torch.float64)
        ids, fl = torch.zeros(B, dtype=torch.int32), torch.zeros(B, dtype=torch.int32)
        for owner, gather, want in [(False, False, None), (True, False, 1), (False, True, 2), (True, True, 3)]:
            sample_vocab_sharded_device(s, d, cf, u, ids, fl, V, rank, world, max_top_k=40,
                                        rows_without_top_k=owner, gather_rows=gather)
            kind, b, vs, stride, off, v, k, bits = s._lib.calls[-1]
            assert (b, vs, stride, off, v, k) == (B, hi - lo, hi - lo, lo, V, 40)
            assert (kind, bits) == (("plain", None) if want is None else ("ex", want))
    with pytest.raises(ValueError):
        sample_vocab_sharded_device(s, torch.zeros(B, 5), cf, u, ids, fl, V, 0, world)
