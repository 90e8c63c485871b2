"""Vocab-sharded sampling on one GPU: the N ranks' local passes run one after another on column
slices of the same batch (through the C ABI), their records are stacked in rank order as the
all-gather would leave them, and the merge must give what the CPU oracle gives on whole rows."""
import numpy as np
import pytest

from gorch_b200 import workloads
from gorch_b200.config import CFG_DTYPE, FLAG_BOUNDARY, FLAG_INTERNAL, FLAG_TIE_CUT, FLAG_TOPP_EDGE

pytestmark = pytest.mark.gpu


def run_sharded(sampler, logits, cfgs, uniforms, world):
    V = logits.shape[1]
    recs = []
    for r in range(world):
        lo, hi = workloads.shard_vocab(V, r, world)
        recs.append(sampler.vocab_local(np.ascontiguousarray(logits[:, lo:hi]), cfgs, lo))
    return sampler.vocab_merge(np.stack(recs), cfgs, uniforms, V)


def check_ids(oracle, logits, cfgs, uniforms, ids, flags):
    """Ids against the oracle on whole rows. A differing id is excused only where the oracle itself
    shows the row to be open (uniform within 1e-6 of a CDF edge, cut inside a group of equal
    probabilities) or the kernel flagged the cut as decided within rounding: tests/parity.py."""
    from tests.parity import compare
    ora = oracle.sample_batch(logits, cfgs, uniforms, flags=oracle.FAST_KTH, threads=oracle.hw_threads())
    assert not np.any(flags & FLAG_INTERNAL), "rows the kernels could not take"
    rep = compare({"ids": ids, "flags": flags}, ora, uniforms, check_probs=False, allow_tie_cut=True)
    assert rep["id_mismatch"] == rep["boundary_mismatch"]
    assert rep["id_mismatch"] <= max(2, len(ids) // 50), f"{rep['id_mismatch']} of {len(ids)} rows differ (all excused, but too many)"
    return rep


def check(sampler, oracle, logits, cfgs, uniforms, world):
    ids, flags = run_sharded(sampler, logits, cfgs, uniforms, world)
    return check_ids(oracle, logits, cfgs, uniforms, ids, flags)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_c5_rows(sampler, oracle, world):
    w = workloads.vocab_sharded(48)
    check(sampler, oracle, w.logits, w.cfgs, w.uniforms, world)


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("mode", [0, 1])
def test_mixed_small_rows(sampler, oracle, world, mode):
    rng = np.random.Generator(np.random.Philox(key=0xC0FFEE + world + mode))
    B, V = 64, 5003                                    # V not divisible by the rank count
    logits = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    logits[:, ::5] = np.round(logits[:, ::5] * 2) / 2   # many ties, some at the threshold
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    for i in range(B):
        cfgs[i] = [(0.0, 0, 0.0, mode), (0.7, 50, 0.95, mode), (1.0, 1, 0.0, mode), (1.3, 96, 0.9, mode), (0.9, 7, 0.5, mode)][i % 5]
    check(sampler, oracle, logits, cfgs, rng.random(B), world)


def test_bf16_ties_and_tiny_slices(sampler, oracle):
    rng = np.random.Generator(np.random.Philox(key=77))
    B, V = 16, 40                                      # slices of 5 columns: top_k above the slice width
    logits = workloads.f32_to_bf16_bits((rng.standard_normal((B, V)) * 3.0).astype(np.float32))
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    cfgs[:] = (0.7, 8, 0.95, 1)
    check(sampler, oracle, logits, cfgs, rng.random(B), 8)


def test_greedy_lowest_index_across_ranks(sampler):
    B, V = 4, 4096
    logits = np.zeros((B, V), np.float32)
    logits[0, [100, 3000]] = 5.0                       # tie across two ranks: lowest index wins
    logits[1, 4095] = 1.0
    logits[2, 0] = np.nan                              # a NaN at index 0 is never beaten
    logits[2, 77] = 9.0
    logits[3, 2048] = np.nan                           # a NaN elsewhere is never selected
    logits[3, 2049] = 2.0
    cfgs = np.zeros(B, dtype=CFG_DTYPE)                # temperature 0
    ids, flags = run_sharded(sampler, logits, cfgs, np.zeros(B), 4)
    assert ids.tolist() == [100, 4095, 0, 2049]


def test_rows_without_top_k_are_flagged(sampler):
    B, V = 2, 1024
    logits = np.random.default_rng(1).standard_normal((B, V)).astype(np.float32)
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    cfgs[0] = (1.0, 0, 0.9, 1)                         # top-k off: not supported when vocab-sharded
    cfgs[1] = (1.0, 200, 0.9, 1)                       # above the record capacity
    ids, flags = run_sharded(sampler, logits, cfgs, np.full(B, 0.5), 2)
    assert ids.tolist() == [-1, -1] and np.all(flags & FLAG_INTERNAL)


@pytest.mark.parametrize("world", [2, 8])
def test_slices_whose_start_is_not_typical(sampler, oracle, world):
    """A slice whose largest logits all sit in its first 4096 columns defeats the local pass's
    estimated threshold (fewer than top_k logits pass it); the slice is then done again without
    the estimate and the merged result must not change."""
    rng = np.random.Generator(np.random.Philox(key=78 + world))
    B, V = 10, 151936
    logits = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    for r in range(world):
        lo, _ = workloads.shard_vocab(V, r, world)
        logits[0:5, lo:lo + 12] += 60.0 + r     # a dozen huge logits at the start of every slice
    logits[5:7, :4096] -= 40.0
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    for b in range(B):
        cfgs[b] = (0.9, 64, 0.95, 1) if b % 2 else (1.0, 40, 0.0, 0)
    uniforms = rng.random(B)
    check(sampler, oracle, logits, cfgs, uniforms, world)


@pytest.mark.parametrize("world", [2, 8])
def test_masked_slices(sampler, oracle, world):
    """-Inf over a whole slice, over the start of every slice, over most of the row: a masked
    slice is no verdict on the row, and -Inf logits never crowd out the candidates."""
    rng = np.random.Generator(np.random.Philox(key=88 + world))
    B, V = 12, 151936
    logits = (rng.standard_normal((B, V)) * 2.0).astype(np.float32)
    lo1, hi1 = workloads.shard_vocab(V, 1, world)
    logits[0:3, lo1:hi1] = -np.inf                     # slice 1 fully masked
    for r in range(world):
        lo, _ = workloads.shard_vocab(V, r, world)
        logits[3:6, lo:lo + 8192] = -np.inf            # the start of every slice masked
    logits[6:9][:, rng.random(V) < 0.9] = -np.inf      # most of the row masked
    logits[9, 100:] = -np.inf                          # only slice 0 has anything
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    for b in range(B):
        cfgs[b] = [(0.9, 64, 0.95, 1), (1.0, 40, 0.0, 0), (0.0, 0, 0.0, 0)][b % 3]
    check(sampler, oracle, logits, cfgs, rng.random(B), world)


def _fused_call(s, logits, cfgs, uniforms, max_top_k, rows_without_top_k=False, gather_rows=False):
    """gorch_cuda_sample_vocab_sharded_dev on this process's one rank (device buffers of the library)."""
    from gorch_b200.config import DTYPE_BF16, DTYPE_F32
    B, V = logits.shape
    code = DTYPE_BF16 if logits.dtype == np.uint16 else DTYPE_F32
    lib = s._lib
    bufs = []
    try:
        b_log = s._buf(logits.nbytes); bufs.append(b_log)
        b_cfg = s._buf(cfgs.nbytes); bufs.append(b_cfg)
        b_uni = s._buf(uniforms.nbytes); bufs.append(b_uni)
        b_ids = s._buf(B * 4); bufs.append(b_ids)
        b_flg = s._buf(B * 4); bufs.append(b_flg)
        s._upload(b_log, np.ascontiguousarray(logits)); s._upload(b_cfg, cfgs); s._upload(b_uni, uniforms)
        ptr = lib.gorch_cuda_buffer_device_ptr
        s.sample_vocab_sharded_ptrs(ptr(b_log), code, B, V, V, 0, V, max_top_k, ptr(b_cfg), ptr(b_uni), ptr(b_ids), ptr(b_flg),
                                    rows_without_top_k=rows_without_top_k, gather_rows=gather_rows)
        s.sync()
        ids = np.empty(B, dtype=np.int32); flags = np.empty(B, dtype=np.uint32)
        s._download(b_ids, ids); s._download(b_flg, flags)
    finally:
        for b in bufs:
            lib.gorch_cuda_buffer_free(b)
    return ids, flags


def test_collective_inside_the_library_one_rank(_sampler_session, oracle):
    """The fused call (local pass, ncclAllGather, merge) with a communicator of one rank: NCCL is
    loaded and driven by the library itself; records sized by the batch's largest top_k."""
    from gorch_b200.sampling import GorchCudaError
    s = _sampler_session
    s.set_kernel_variant(0, 0)
    w = workloads.vocab_sharded(96)
    with pytest.raises(GorchCudaError, match="comm_init"):
        _fused_call(s, w.logits, w.cfgs, w.uniforms, 64)            # no communicator yet
    s.comm_init(0, 1, s.comm_unique_id())
    try:
        for max_k in (64, 0, 128):
            ids, flags = _fused_call(s, w.logits, w.cfgs, w.uniforms, max_k)
            check_ids(oracle, w.logits, w.cfgs, w.uniforms, ids, flags)
        # a top_k above what the record was sized for is reported, not mis-sampled
        ids, flags = _fused_call(s, w.logits, w.cfgs, w.uniforms, 16)
        assert (ids == -1).all() and (flags & FLAG_INTERNAL).all()
        # rows without top-k through the same call: merge of the sums, the owner's draw, the two all-reduces
        rng = np.random.Generator(np.random.Philox(key=31))
        x = (rng.standard_normal((40, 30011)) * 2.5).astype(np.float32)
        cf = np.zeros(40, dtype=CFG_DTYPE)
        for i in range(40):
            cf[i] = [(1.0, 0, 0.0, 0), (0.8, 40, 0.0, 0), (0.7, 0, 0.9, 0), (0.0, 0, 0.0, 0)][i % 4]
        uu = rng.random(40)
        ids, flags = _fused_call(s, x, cf, uu, 40, rows_without_top_k=True)
        check_ids(oracle, x, cf, uu, ids, flags)
        ids, flags = _fused_call(s, x, cf, uu, 40)               # without the flag such rows are refused, the others served
        assert np.all(ids[0::2] == -1) and np.all(ids[1::2] >= 0)
        # rows without top-k whose top-p cut is active: from whole rows, gathered by an all-reduce
        for i in range(40):
            cf[i] = [(1.0, 0, 0.9, 1), (0.8, 40, 0.0, 0), (0.7, 0, 0.5, 0), (0.0, 0, 0.0, 0), (1.3, 0, 0.0, 0)][i % 5]
        for owner in (True, False):
            ids, flags = _fused_call(s, x, cf, uu, 40, rows_without_top_k=owner, gather_rows=True)
            check_ids(oracle, x, cf, uu, ids, flags)
        xb = workloads.f32_to_bf16_bits(x[:, :30008])            # bf16 rows, a width that is a multiple of 8
        ids, flags = _fused_call(s, xb, cf, uu, 40, rows_without_top_k=True, gather_rows=True)
        check_ids(oracle, xb, cf, uu, ids, flags)
        ids, flags = _fused_call(s, x, cf, uu, 40, rows_without_top_k=True)   # without it the rows with a cut are refused
        assert np.all(ids[0::5] == -1) and np.all(ids[2::5] == -1) and np.all(ids[1::5] >= 0) and np.all(ids[4::5] >= 0)
        # timing of the phases
        s.set_timing(True)
        _fused_call(s, w.logits, w.cfgs, w.uniforms, 64)
        c = s.counters()
        s.set_timing(False)
        assert c["vs_local_ms"] > 0 and c["vs_merge_ms"] > 0 and c["vs_gather_ms"] >= 0
    finally:
        s.comm_release()


def run_sharded_with_owner_draw(sampler, logits, cfgs, uniforms, world):
    """As run_sharded, for batches that hold rows without top-k: every rank merges with its own rank
    number, draws from its own slice for the rows it owns, and the ranks' ids / flags are joined by
    the maximum, as the all-reduce inside gorch_cuda_sample_vocab_sharded_ex_dev does."""
    V = logits.shape[1]
    recs, slices = [], []
    for r in range(world):
        lo, hi = workloads.shard_vocab(V, r, world)
        slices.append((lo, np.ascontiguousarray(logits[:, lo:hi])))
        recs.append(sampler.vocab_local(slices[-1][1], cfgs, lo))
    allrec = np.stack(recs)
    ids = np.full(logits.shape[0], -(2 ** 31), dtype=np.int64)
    flags = np.zeros(logits.shape[0], dtype=np.uint32)
    per_rank = []
    for r in range(world):
        i_r, f_r = sampler.vocab_merge_draw(allrec, r, slices[r][1], slices[r][0], cfgs, uniforms, V)
        per_rank.append(i_r)
        ids = np.maximum(ids, i_r)
        flags = np.maximum(flags, f_r)
    return ids.astype(np.int32), flags, per_rank


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("bf16", [False, True])
def test_rows_without_top_k(sampler, oracle, world, bf16):
    """Plain softmax sampling over a sharded vocabulary (top_k == 0, no effective top-p cut) beside
    top-k and greedy rows: the slices' sums of exponentials are merged, the owner draws."""
    rng = np.random.Generator(np.random.Philox(key=0xABCD + world + (100 if bf16 else 0)))
    B, V = 60, 20011
    x = (rng.standard_normal((B, V)) * 2.5).astype(np.float32)
    x[3, :] = -np.inf; x[3, 17000:17010] = 1.0          # all mass in one late slice
    x[4, 0] = 30.0                                       # nearly all mass at index 0
    logits = workloads.f32_to_bf16_bits(x) if bf16 else x
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    for i in range(B):
        cfgs[i] = [(1.0, 0, 0.0, 0), (0.7, 0, 0.9, 0), (1.3, 0, 1.0, 1), (0.8, 40, 0.0, 0), (0.0, 0, 0.0, 0), (0.9, 0, 0.0, 1)][i % 6]
    u = rng.random(B)
    u[6] = 0.0; u[12] = 1.0 - 2.0 ** -53
    ids, flags, per_rank = run_sharded_with_owner_draw(sampler, logits, cfgs, u, world)
    check_ids(oracle, logits, cfgs, u, ids, flags)
    soft = np.array([i % 6 in (0, 1, 2, 5) for i in range(B)])
    owners = np.stack([p[soft] >= 0 for p in per_rank]).sum(axis=0)
    assert np.all(owners == 1), "every row without top-k has exactly one owner"


def test_rows_without_top_k_but_with_a_cut_are_refused(sampler):
    rng = np.random.Generator(np.random.Philox(key=5))
    x = (rng.standard_normal((4, 4096)) * 2.0).astype(np.float32)
    cfgs = np.zeros(4, dtype=CFG_DTYPE)
    cfgs[:] = (1.0, 0, 0.9, 1)                           # mode B nucleus over the whole vocabulary: not served when sharded
    ids, flags, _ = run_sharded_with_owner_draw(sampler, x, cfgs, rng.random(4), 2)
    assert np.all(ids == -1) and np.all(flags & FLAG_INTERNAL)


def test_nonfinite_rows_without_top_k(sampler):
    B, V = 3, 4096
    x = np.zeros((B, V), np.float32)
    x[0, 3000] = np.nan
    x[1, 10] = np.inf
    x[2, :] = -np.inf
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    cfgs[:] = (1.0, 0, 0.0, 0)
    ids, flags, _ = run_sharded_with_owner_draw(sampler, x, cfgs, np.full(B, 0.5), 4)
    assert ids.tolist() == [V - 1] * 3                   # generate.go:173-181, 239: the walk falls through
