"""The softmax / log-softmax / cross-entropy restatements in the oracle (ops.go:527-603,
loss.go:108-141) against the properties the reference's own tests pin: rows sum to 1 and keep
their order (tensor_test.go:147-192), LogSoftmax == log(Softmax) (tensor_test.go:165-177), and the
fused cross-entropy equals the composed LogSoftmax / Softmax chain on the shapes of
ce_metal_test.go:72-93 within its gates (loss 1e-4, dLogits 1e-6). The reference holds no golden
numbers for these ops; inputs are seeded normal logits x 2 as in ce_metal_test.go:44-54."""
import numpy as np
import pytest

from oracle import oracle


def test_softmax_known_properties():
    s = oracle.softmax(np.array([[1, 2, 3]], dtype=np.float32))
    assert abs(float(s.sum()) - 1.0) < 1e-5 and s[0, 0] < s[0, 1] < s[0, 2]
    want = np.exp([1.0, 2.0, 3.0]) / np.exp([1.0, 2.0, 3.0]).sum()
    assert np.allclose(s[0], want, rtol=1e-6)
    s2 = oracle.softmax(np.array([[1, 2, 3], [10, 20, 30]], dtype=np.float32))
    assert np.allclose(s2.sum(axis=1), 1.0, atol=1e-5)
    ls = oracle.softmax(np.array([[1, 2, 3]], dtype=np.float32), log=True)
    assert np.allclose(ls, np.log(s.astype(np.float64)), atol=1e-5)


@pytest.mark.parametrize("batch,classes", [(7, 300), (3, 1000), (16, 64), (4, 20000)])
def test_fused_cross_entropy_equals_the_composed_chain(batch, classes):
    rng = np.random.default_rng(17 + classes)
    x = (rng.standard_normal((batch, classes)) * 2.0).astype(np.float32)
    tgt = rng.integers(0, classes, batch)
    ls = oracle.softmax(x, log=True)
    composed_loss = np.float32(-sum(np.float32(ls[i, tgt[i]]) for i in range(batch))) / np.float32(batch)
    sm = oracle.softmax(x)
    scale = np.float32(1.0) / np.float32(batch)
    composed_dx = sm * scale
    composed_dx[np.arange(batch), tgt] -= scale
    mean, row_loss, row_lse = oracle.cross_entropy_fwd(x, tgt)
    dx = oracle.cross_entropy_bwd(x, tgt, row_lse, float(scale))
    assert abs(mean - float(composed_loss)) <= 1e-4
    assert np.abs(dx - composed_dx).max() <= 1e-6
    assert np.allclose(row_loss, row_lse - x[np.arange(batch), tgt], atol=1e-6)


def test_special_values_follow_the_go_loops():
    x = np.zeros((5, 6), dtype=np.float32)
    x[0, 2] = np.nan              # NaN away from index 0: max ignores it, the sum does not
    x[1, 0] = np.nan              # NaN at index 0: rowMax itself is NaN
    x[2, 3] = np.inf              # Inf - Inf
    x[3, :] = -np.inf             # -Inf - -Inf
    x[4, 1] = -np.inf             # a single -Inf is just probability 0
    with np.errstate(all="ignore"):
        s = oracle.softmax(x)
    assert np.isnan(s[:4]).all()
    assert s[4, 1] == 0 and np.allclose(s[4, [0, 2, 3, 4, 5]], 0.2)
