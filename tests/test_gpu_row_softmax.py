"""gorch_cuda_softmax_dev / gorch_cuda_cross_entropy_{fwd,bwd}_dev against the oracle's
restatement of gorch.Softmax, LogSoftmax and CrossEntropyLoss (ops.go:527-603, loss.go:108-141).

Floating point, so tolerances, each stated where it is used:
  * against a float64 evaluation of the same formula: 2e-6 relative (f32 exp and one rounding);
  * against the oracle, which sums a row sequentially in f32 as upstream does: the oracle's own
    summation error grows with the row length, so the bound is 2e-6 + 2^-24 * sqrt(V) * 4 relative
    on probabilities and the same absolute on log-probabilities / lse;
  * the reference's own Metal-vs-CPU gates (ce_metal_test.go:143-196: lse and loss 1e-3 absolute,
    dLogits 1e-5 absolute) are asserted as well and are far looser.
bf16 outputs may differ from the downcast oracle value by one bf16 step (2^-7 relative)."""
import numpy as np
import pytest

from gorch_b200 import row_ops
from gorch_b200.sampling import GorchCudaError

pytestmark = pytest.mark.gpu

SHAPES = [(7, 300), (16, 64), (3, 20000), (257, 129), (33, 4111), (1, 1), (5, 3), (4, 50257), (3, 151936), (150, 5000)]


def _case(batch, classes, seed=0):
    rng = np.random.default_rng(1000 * seed + classes + batch)
    x = (rng.standard_normal((batch, classes)) * 2.0).astype(np.float32)
    return x, rng.integers(0, classes, batch).astype(np.int32)


def _oracle_tol(V):
    return 2e-6 + 4.0 * np.sqrt(V) * 2.0 ** -24


def _f64_softmax(x):
    z = x.astype(np.float64)
    z = z - z.max(axis=1, keepdims=True)
    e = np.exp(z)
    return e / e.sum(axis=1, keepdims=True), z - np.log(e.sum(axis=1, keepdims=True))


@pytest.mark.parametrize("batch,classes", SHAPES)
def test_softmax_and_log_softmax_f32(_sampler_session, oracle, batch, classes):
    x, _ = _case(batch, classes)
    sm = row_ops.softmax(_sampler_session, x)
    ls = row_ops.softmax(_sampler_session, x, log=True)
    want_sm, want_ls = _f64_softmax(x)
    assert np.allclose(sm, want_sm, rtol=2e-6, atol=1e-37)
    assert np.abs(ls - want_ls).max() <= 2e-6 * max(1.0, np.abs(want_ls).max())
    tol = _oracle_tol(classes)
    assert np.allclose(sm, oracle.softmax(x), rtol=tol, atol=1e-37)
    assert np.abs(ls - oracle.softmax(x, log=True)).max() <= tol * max(1.0, np.abs(want_ls).max())


@pytest.mark.parametrize("batch,classes", SHAPES)
def test_cross_entropy_forward_and_backward_f32(_sampler_session, oracle, batch, classes):
    s = _sampler_session
    x, tgt = _case(batch, classes, 1)
    mean, row_loss, row_lse = row_ops.cross_entropy(s, x, tgt)
    o_mean, o_loss, o_lse = oracle.cross_entropy_fwd(x, tgt)
    tol = _oracle_tol(classes) * max(1.0, float(np.abs(o_lse).max()))
    assert np.abs(row_lse - o_lse).max() <= tol and np.abs(row_loss - o_loss).max() <= tol
    assert abs(mean - o_mean) <= tol + 1e-6 * abs(o_mean)
    assert np.abs(row_lse - o_lse).max() <= 1e-3 and abs(mean - o_mean) <= 1e-3      # ce_metal_test.go:182
    _, want_ls = _f64_softmax(x)
    assert np.abs(row_loss + want_ls[np.arange(batch), tgt]).max() <= 2e-6 * max(1.0, float(np.abs(want_ls).max()))
    scale = 1.0 / batch
    dx = row_ops.cross_entropy_backward(s, x, tgt, o_lse, scale)
    o_dx = oracle.cross_entropy_bwd(x, tgt, o_lse, scale)
    assert np.abs(dx - o_dx).max() <= 1e-5                                                # ce_metal_test.go:193
    assert np.allclose(dx, o_dx, rtol=2e-6, atol=2e-7 * scale)


@pytest.mark.parametrize("batch,classes", [(7, 300), (4, 50257), (3, 151936), (33, 4111)])
def test_bf16_logits(_sampler_session, oracle, batch, classes):
    s = _sampler_session
    x, tgt = _case(batch, classes, 2)
    bits = oracle.f32_to_bf16_bits(x)
    xf = oracle.bf16_bits_to_f32(bits)
    for log in (False, True):
        got = oracle.bf16_bits_to_f32(row_ops.softmax(s, bits, log=log))
        want = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(oracle.softmax(xf, log=log)))
        assert np.allclose(got, want, rtol=2.0 ** -7, atol=1e-37)
        assert np.mean(got != want) < 0.02                      # almost all identical; a few round the other way
    mean, row_loss, row_lse = row_ops.cross_entropy(s, bits, tgt)          # bf16 in, f32 out (loss.go:59-61)
    o_mean, o_loss, o_lse = oracle.cross_entropy_fwd(xf, tgt)
    tol = _oracle_tol(classes) * max(1.0, float(np.abs(o_lse).max()))
    assert np.abs(row_lse - o_lse).max() <= tol and np.abs(row_loss - o_loss).max() <= tol and abs(mean - o_mean) <= 2 * tol
    dx = row_ops.cross_entropy_backward(s, bits, tgt, o_lse, 0.25)
    assert np.allclose(dx, oracle.cross_entropy_bwd(xf, tgt, o_lse, 0.25), rtol=2e-6, atol=1e-7)


def test_special_values_match_the_go_loops(_sampler_session, oracle):
    s = _sampler_session
    rng = np.random.default_rng(3)
    x = rng.standard_normal((9, 5000)).astype(np.float32)
    x[0, 2222] = np.nan
    x[1, 0] = np.nan
    x[2, 4999] = np.inf
    x[3, :] = -np.inf
    x[4, 1000:3000] = -np.inf
    x[5, :] = 7.5
    x[6, :] = -np.inf; x[6, 4098] = np.nan
    x[7, :] = -np.inf; x[7, 17] = 0.0
    x[8, 0] = -np.inf
    tgt = np.arange(9, dtype=np.int32)
    with np.errstate(all="ignore"):
        for log in (False, True):
            got, want = row_ops.softmax(s, x, log=log), oracle.softmax(x, log=log)
            assert (np.isnan(got) == np.isnan(want)).all()
            ok = ~np.isnan(want)
            assert np.array_equal(np.isinf(got[ok]), np.isinf(want[ok]))
            fin = ok & ~np.isinf(want)
            assert np.allclose(got[fin], want[fin], rtol=3e-6, atol=3e-6 if log else 1e-37)
        mean, row_loss, row_lse = row_ops.cross_entropy(s, x, tgt)
        o_mean, o_loss, o_lse = oracle.cross_entropy_fwd(x, tgt)
        assert (np.isnan(row_lse) == np.isnan(o_lse)).all() and np.isnan(mean) == np.isnan(o_mean)
        fin = ~np.isnan(o_lse)
        assert np.allclose(row_lse[fin], o_lse[fin], atol=1e-5) and np.allclose(row_loss[fin], o_loss[fin], atol=1e-5)


def test_strides_misaligned_rows_and_bad_arguments(_sampler_session, oracle):
    s = _sampler_session
    B, V, stride, ostride = 6, 1003, 1009, 1005          # rows start at odd offsets: no 16-byte alignment
    rng = np.random.default_rng(4)
    flat = rng.standard_normal(B * stride + 3).astype(np.float32)
    x = np.stack([flat[3 + b * stride: 3 + b * stride + V] for b in range(B)])
    bufs = row_ops._Bufs(s)
    try:
        b_x, b_o = bufs.new(flat), bufs.new(4 * (B * ostride + 1))
        s._upload(b_o, np.full(B * ostride + 1, -5.0, dtype=np.float32))
        row_ops.softmax_ptrs(s, bufs.ptr(b_x) + 12, 0, B, V, stride, bufs.ptr(b_o) + 4, ostride, False)
        s.sync()
        out = np.empty(B * ostride + 1, dtype=np.float32)
        s._download(b_o, out)
        got = np.stack([out[1 + b * ostride: 1 + b * ostride + V] for b in range(B)])
        assert np.allclose(got, oracle.softmax(x), rtol=3e-6)
        pad = np.concatenate([out[:1]] + [out[1 + b * ostride + V: 1 + (b + 1) * ostride] for b in range(B - 1)])
        assert (pad == -5.0).all()                                       # nothing written between the rows
        with pytest.raises(GorchCudaError):
            row_ops.softmax_ptrs(s, bufs.ptr(b_x), 0, B, V, V - 1, bufs.ptr(b_o), ostride)
        with pytest.raises(GorchCudaError):
            row_ops.softmax_ptrs(s, bufs.ptr(b_x), 0, B, V, stride, bufs.ptr(b_o), V - 1)
        with pytest.raises(GorchCudaError):
            row_ops.softmax_ptrs(s, bufs.ptr(b_x), 0, B, V, stride, None, ostride)
        with pytest.raises(GorchCudaError):
            row_ops.softmax_ptrs(s, bufs.ptr(b_x), 7, B, V, stride, bufs.ptr(b_o), ostride)
    finally:
        bufs.free()
    mean, row_loss, _ = row_ops.cross_entropy(s, x, np.array([0, 1, 2, 3, 4, V], dtype=np.int32))
    assert np.isnan(row_loss[5]) and not np.isnan(row_loss[:5]).any() and np.isnan(mean)


def test_full_vocabulary_batch_properties(_sampler_session):
    """192 x 151,936 (more rows than SMs, 117 MB): rows sum to 1, log-softmax is the log of
    softmax, the cross-entropy gradient of every row sums to 0 and is softmax minus one-hot."""
    s = _sampler_session
    rng = np.random.default_rng(5)
    B, V = 192, 151936
    x = (rng.standard_normal((B, V), dtype=np.float32) * 3.0)
    tgt = rng.integers(0, V, B).astype(np.int32)
    sm = row_ops.softmax(s, x)
    ls = row_ops.softmax(s, x, log=True)
    assert np.abs(sm.astype(np.float64).sum(axis=1) - 1.0).max() <= 2e-6
    assert np.abs(np.log(sm.astype(np.float64)) - ls).max() <= 2e-5        # log of an f32-rounded probability
    mean, row_loss, row_lse = row_ops.cross_entropy(s, x, tgt)
    assert np.allclose(row_loss, -ls[np.arange(B), tgt], atol=2e-5) and abs(mean - float(row_loss.astype(np.float64).mean())) <= 1e-5
    dx = row_ops.cross_entropy_backward(s, x, tgt, row_lse, 1.0)
    assert np.abs(dx.astype(np.float64).sum(axis=1)).max() <= 1e-5
    dx[np.arange(B), tgt] += 1.0
    assert np.allclose(dx, sm, rtol=1e-5, atol=2e-7)                     # the target entry went through p - 1 + 1


def test_sorted_rows(_sampler_session, oracle):
    """Ascending rows make every thread's running maximum grow at each vector (the sums are
    rescaled every time), descending ones never: both must give the same values as a shuffled row."""
    s = _sampler_session
    rng = np.random.default_rng(6)
    base = (rng.standard_normal(151936) * 3.0).astype(np.float32)
    x = np.stack([np.sort(base), np.sort(base)[::-1], base, np.sort(base) * 8.0])
    tgt = np.array([5, 5, 5, 151935], dtype=np.int32)
    want_sm, want_ls = _f64_softmax(x)
    # upstream rounds x - max to f32 before the exponential (ops.go:545), and so does the kernel: a
    # probability whose x - max is d carries up to |d| 2^-24 relative error against exact arithmetic
    d = np.abs(x.astype(np.float64) - x.max(axis=1, keepdims=True))
    got = row_ops.softmax(s, x).astype(np.float64)
    assert (np.abs(got - want_sm) <= (2e-6 + d * 2.0 ** -24) * want_sm + 1e-37).all()
    ls = row_ops.softmax(s, x, log=True)
    assert np.abs(ls - want_ls).max() <= 2e-6 * np.abs(want_ls).max()
    _, row_loss, row_lse = row_ops.cross_entropy(s, x, tgt)
    want_loss = -want_ls[np.arange(4), tgt]
    assert np.abs(row_loss - want_loss).max() <= 2e-6 * np.abs(want_loss).max() + 1e-5
    # the oracle sums sequentially in f32 like upstream: on a descending row most small terms fall
    # below half an ulp of the running sum and are lost, so only upstream's own gate (1e-3) holds there
    _, o_loss, o_lse = oracle.cross_entropy_fwd(x, tgt)
    assert np.abs(row_lse - o_lse).max() <= 1e-3 and np.abs(row_loss - o_loss).max() <= 1e-3
