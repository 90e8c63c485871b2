"""Generate-loop control on the device (gorch_cuda_generate_control_dev / _step_dev) against the
scripted loop oracle, row by row and step by step, for the three loops of the reference
(model/generate.go:57-88 uncached, :93-131 cached; model/qwen/generate.go:35-62); then whole
batched generations with a table-lookup model on the device against the per-sequence host loops
driven by the CPU sampling oracle. Token ids, lengths and end reasons are integers: exact."""
import numpy as np
import pytest

from gorch_b200.config import CFG_DTYPE, DTYPE_BF16, DTYPE_F32, MODE_A, MODE_B, GenerateConfig, QwenGenerateConfig
from gorch_b200.generate import (GEN_ERROR, GEN_LIVE, LOOP_CACHED, LOOP_QWEN, LOOP_UNCACHED,
                                 DeviceGenerateState, generate_on_device)
from gorch_b200.sampling import GorchCudaError, generate_with_config, qwen_generate
from tests.parity import compare

pytestmark = pytest.mark.gpu


def _stops_for(loop, rng):
    if loop == LOOP_QWEN:
        return rng.integers(0, 9, int(rng.integers(0, 4))).tolist()
    return [int(rng.integers(-1, 7))]


@pytest.mark.parametrize("loop", [LOOP_UNCACHED, LOOP_CACHED, LOOP_QWEN])
@pytest.mark.parametrize("max_seq", [3, 8, 40])
def test_control_steps_match_the_scripted_loops(_sampler_session, oracle, loop, max_seq):
    s = _sampler_session
    rng = np.random.default_rng(17 * loop + max_seq)
    B, max_new = 300, 9
    prompts = [rng.integers(0, 7, int(rng.integers(1, 12))).tolist() for _ in range(B)]
    scripts = rng.integers(0, 7, (max_new, B)).astype(np.int32)
    stops = _stops_for(loop, rng)
    want = [oracle.generate_scripted(loop, prompts[b], scripts[:, b].tolist(), max_new, max_seq, stops) for b in range(B)]
    st = DeviceGenerateState(s, prompts, max_new, max_seq, stops, loop)
    try:
        fed = [[] for _ in range(B)]
        before = st.results()
        if loop == LOOP_UNCACHED:
            for b in range(B):
                fed[b].append(int(before["window_start"][b]))
        for i in range(max_new):
            s._upload(st._bufs["ids"], np.ascontiguousarray(scripts[i]))
            st.control(st.ids_ptr)
            after = st.results()
            assert st.live() == int(np.count_nonzero(after["done"] == GEN_LIVE))
            for b in range(B):
                if loop == LOOP_UNCACHED:
                    if after["done"][b] == GEN_LIVE:
                        fed[b].append(int(after["window_start"][b]))
                elif after["cache_len"][b] != before["cache_len"][b]:
                    assert after["cache_len"][b] == before["cache_len"][b] + 1
                    fed[b].append(int(after["next_input"][b]))
            before = after
        for b in range(B):
            assert after["tokens"][b] == want[b]["tokens"], (b, prompts[b], scripts[:, b], stops)
            assert after["done"][b] == want[b]["reason"]
            assert after["n_new"][b] == want[b]["sampler_calls"] - (1 if want[b]["reason"] == 1 else 0)
            assert fed[b] == want[b]["fed"], (b, loop)
    finally:
        st.release()


def test_unusable_ids_end_a_row_without_appending(_sampler_session):
    s = _sampler_session
    st = DeviceGenerateState(s, [[1, 2], [3], [4, 5, 6]], 4, 16, [], LOOP_QWEN)
    try:
        flags = s._buf(16)
        s._upload(st._bufs["ids"], np.array([-1, 5, 6], dtype=np.int32))
        s._upload(flags, np.array([0, 0x100, 0, 0], dtype=np.uint32))        # GORCH_FLAG_BAD_CFG on row 1
        st.control(st.ids_ptr, s._lib.gorch_cuda_buffer_device_ptr(flags))
        r = st.results()
        s._lib.gorch_cuda_buffer_free(flags)
        assert r["done"].tolist() == [GEN_ERROR, GEN_ERROR, GEN_LIVE]
        assert r["tokens"] == [[1, 2], [3], [4, 5, 6, 6]] and st.live() == 1
    finally:
        st.release()


def test_bad_control_records_are_refused(_sampler_session):
    s = _sampler_session
    with pytest.raises(ValueError):
        DeviceGenerateState(s, [[1], []], 4, 16, [], LOOP_CACHED)
    with pytest.raises(ValueError):
        DeviceGenerateState(s, [[1]], 4, 16, [1, 2], LOOP_CACHED)
    st = DeviceGenerateState(s, [[1]], 4, 16, [], LOOP_CACHED)
    try:
        st.gc.n_stop = 17
        with pytest.raises(GorchCudaError):
            st.control(st.ids_ptr)
        st.gc.n_stop = 0
        st.gc.done = None
        with pytest.raises(GorchCudaError):
            st.control(st.ids_ptr)
    finally:
        st.release()


# ---- whole generations: a table-lookup model, on the device for the library and on the host for the oracle loops
M_ROWS, V_TAB, MAX_SEQ = 61, 997, 24


def _table():
    rng = np.random.default_rng(5)
    t = (rng.standard_normal((M_ROWS, V_TAB)) * 2.5).astype(np.float32)
    t[:, 3] += 1.5          # token 3 (used as a stop token below) comes up now and then
    return t


class HostTableModel:
    """logits of (token, position) = table[(7 token + 13 position) mod M]."""
    max_seq, vocab_size = MAX_SEQ, V_TAB

    def __init__(self, table):
        self.t = table

    def _row(self, tok, pos):
        return self.t[(7 * tok + 13 * pos) % M_ROWS]

    def forward(self, ids):
        return np.stack([self._row(t, i) for i, t in enumerate(ids)])

    class Cache:
        n = 0

        def len(self):
            return self.n

    def new_cache(self):
        return HostTableModel.Cache()

    def forward_cached(self, ids, cache):
        rows = [self._row(t, cache.n + i) for i, t in enumerate(ids)]
        cache.n += len(ids)
        return np.stack(rows)


class HostQwenTableModel(HostTableModel):
    """qwen's ForwardCached returns the last position's logits only, (1, vocab) (qwen/generate.go:44)."""

    def forward_cached(self, ids, cache):
        return HostTableModel.forward_cached(self, ids, cache)[-1:]


class _DevInts:
    """Lets torch see B int32 values at a raw device pointer."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<i4", "data": (int(ptr), False), "version": 2}


class DeviceTableModel:
    def __init__(self, table, loop):
        """table: float32, or uint16 bf16 bit patterns (given to torch as int16)."""
        import torch
        self.torch = torch
        self.code = DTYPE_BF16 if table.dtype == np.uint16 else DTYPE_F32
        self.t = torch.from_numpy(table.view(np.int16) if table.dtype == np.uint16 else table).cuda()
        self.loop = loop
        self.logits = None

    def _ints(self, ptr, n):
        return self.torch.as_tensor(_DevInts(ptr, n), device="cuda").long()

    def forward_dev(self, st):
        tok = self._ints(st.next_input_ptr, st.B)
        if self.loop == LOOP_UNCACHED:
            # position of the last token inside the window the uncached loop feeds
            pos = self._ints(st.lengths_ptr, st.B) - 1 - self._ints(st.window_start_ptr, st.B)
        else:
            pos = self._ints(st.cache_len_ptr, st.B) - 1
        self.logits = self.t[(7 * tok + 13 * pos) % M_ROWS].contiguous()
        return self.logits.data_ptr(), self.code, V_TAB, V_TAB

    prefill_dev = forward_dev


class OracleSampler:
    def __init__(self, oracle):
        self.o = oracle

    def next_token(self, last_logits, cfg, u):
        if cfg.temperature == 0:
            return self.o.argmax(last_logits)
        return int(self.o.sample(last_logits, cfg.temperature, cfg.top_k, cfg.top_p, u, cfg.topp_mode)[0])


@pytest.mark.parametrize("loop", [LOOP_UNCACHED, LOOP_CACHED, LOOP_QWEN])
@pytest.mark.parametrize("B,bf16", [(48, False), (200, True)])
def test_batched_generation_on_device_matches_the_host_loops(_sampler_session, oracle, loop, B, bf16):
    """48 sequences of f32 logits (the small-batch kernels) and 200 of bf16 logits (the batch
    kernels), every sampling kind, each of the three loops."""
    import torch
    s = _sampler_session
    s.set_kernel_variant(0, 0)
    table = _table()
    if bf16:
        table = oracle.f32_to_bf16_bits(table)
    rng = np.random.default_rng(40 + loop + B)
    max_new = 14
    prompts = [rng.integers(0, V_TAB, int(rng.integers(1, 30 if loop != LOOP_QWEN else 12))).tolist() for _ in range(B)]
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    mode = MODE_B if loop == LOOP_QWEN else MODE_A
    for b in range(B):
        kind = b % 4
        cfgs[b] = (0.0, 0, 0.0, mode) if kind == 0 else (0.8, 40, 0.0, mode) if kind == 1 else \
                  (1.1, 0, 0.9, mode) if kind == 2 else (0.7, 50, 0.95, mode)
    uniforms = rng.random((max_new, B))
    stops = [3, 11] if loop == LOOP_QWEN else [3]
    s.set_stream(torch.cuda.current_stream().cuda_stream)
    try:
        got = generate_on_device(DeviceTableModel(table, loop), prompts, cfgs, uniforms, s, max_new, MAX_SEQ,
                                 stops, loop, poll_every=4)
    finally:
        torch.cuda.synchronize()
        s.set_stream(None)
    host_table = oracle.bf16_bits_to_f32(table) if bf16 else table          # the upcast of tensor.go:96-99
    host = HostQwenTableModel(host_table) if loop == LOOP_QWEN else HostTableModel(host_table)
    smp = OracleSampler(oracle)
    ended = set()
    for b in range(B):
        t, k, p, m = (cfgs[b][f] for f in ("temperature", "top_k", "top_p", "topp_mode"))
        col = uniforms[:, b].tolist()
        if loop == LOOP_QWEN:
            cfg = QwenGenerateConfig(max_new_tokens=max_new, temperature=float(t), top_k=int(k), top_p=float(p), stop_tokens=stops)
            want = qwen_generate(host, prompts[b], cfg, smp, uniforms=col)
        else:
            cfg = GenerateConfig(max_new_tokens=max_new, temperature=float(t), top_k=int(k), top_p=float(p),
                                 stop_token=stops[0], use_kv_cache=(loop == LOOP_CACHED), topp_mode=int(m))
            want = generate_with_config(host, prompts[b], cfg, col, smp)
        assert got["tokens"][b] == want, (loop, b)
        ended.add(int(got["done"][b]))
    assert GEN_LIVE not in ended and len(ended) >= 2       # the batch exercises more than one way to end


@pytest.mark.parametrize("B,bf16", [(6, False), (40, True), (300, False)])
def test_rows_that_have_ended_are_not_sampled(sampler, oracle, B, bf16):
    """gorch_cuda_generate_step_dev hands the loop's own end marks to the sampling kernels: a row
    whose sequence has ended keeps what out_ids / out_flags held, the live rows get exactly the ids
    the oracle draws, and the loop appends to the live rows only. Every dispatch (small-batch
    cluster kernel, batch kernels, single-CTA kernel) and every row kind."""
    from gorch_b200 import workloads
    s = sampler
    rng = np.random.default_rng(900 + B)
    V = 5000
    x = (rng.standard_normal((B, V)) * 2.5).astype(np.float32)
    logits = workloads.f32_to_bf16_bits(x) if bf16 else x
    cfgs = np.zeros(B, dtype=CFG_DTYPE)
    for b in range(B):
        cfgs[b] = [(0.0, 0, 0.0, MODE_A), (0.8, 40, 0.0, MODE_A), (1.1, 0, 0.9, MODE_B), (0.7, 50, 0.95, MODE_B),
                   (0.9, 700, 0.9, MODE_B)][b % 5]
    u = rng.random(B)
    ended = rng.random(B) < 0.4
    ended[0], ended[B - 1] = True, False
    prompts = [[1, 2, 3] for _ in range(B)]
    st = DeviceGenerateState(s, prompts, 4, 64, [], LOOP_QWEN)
    bufs = []
    try:
        done = np.where(ended, 2, GEN_LIVE).astype(np.int32)
        s._upload(st._bufs["done"], done)
        s._upload(st._bufs["ids"], np.full(B, -7, dtype=np.int32))
        s._upload(st._bufs["flags"], np.full(B, 0x7777, dtype=np.int32))
        ptr = s._lib.gorch_cuda_buffer_device_ptr
        for arr in (np.ascontiguousarray(logits), cfgs, np.ascontiguousarray(u)):
            b_ = s._buf(arr.nbytes); bufs.append(b_); s._upload(b_, arr)
        st.step(ptr(bufs[0]), DTYPE_BF16 if bf16 else DTYPE_F32, V, V, ptr(bufs[1]), ptr(bufs[2]))
        ids = st._get("ids", B)
        flags = st._get("flags", B)
        r = st.results()
    finally:
        for b_ in bufs:
            s._lib.gorch_cuda_buffer_free(b_)
        st.release()
    assert np.all(ids[ended] == -7) and np.all(flags[ended] == 0x7777)
    live = np.nonzero(~ended)[0]
    want = oracle.sample_batch(np.ascontiguousarray(logits[live]), np.ascontiguousarray(cfgs[live]),
                               np.ascontiguousarray(u[live]), flags=oracle.FAST_KTH, threads=oracle.hw_threads())
    rep = compare({"ids": ids[live], "flags": flags[live].view(np.uint32)}, want, u[live], check_probs=False,
                  allow_tie_cut=True)
    assert rep["id_mismatch"] == rep["boundary_mismatch"]
    for b in range(B):
        assert r["tokens"][b] == ([1, 2, 3] if ended[b] else [1, 2, 3, int(ids[b])])
        assert r["done"][b] == (2 if ended[b] else GEN_LIVE)
