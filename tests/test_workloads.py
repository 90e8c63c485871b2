"""Seeded workloads: determinism, shapes, structure, sharding helpers."""
import numpy as np

from gorch_b200 import workloads
from gorch_b200.config import MODE_A, MODE_B


def test_prefix_stability_and_determinism():
    a = workloads.mixed_rows(16)
    b = workloads.mixed_rows(16)
    c = workloads.mixed_rows(32)
    assert np.array_equal(a.logits, b.logits) and np.array_equal(a.uniforms, b.uniforms)
    assert np.array_equal(a.uniforms, c.uniforms[:16])


def test_shapes_and_configs():
    w1 = workloads.gpt2_step(4)
    assert w1.logits.shape == (4, 50257) and w1.logits.dtype == np.float32
    assert np.allclose(w1.cfgs["temperature"], 0.8) and (w1.cfgs["top_k"] == 40).all()
    assert (w1.cfgs["topp_mode"] == MODE_A).all()
    w4 = workloads.flat_stress(2)
    assert w4.logits.shape == (2, 151936) and (w4.cfgs["topp_mode"] == MODE_B).all()
    assert abs(float(w4.logits.std()) - 0.25) < 0.01
    w5 = workloads.vocab_sharded(2)
    assert w5.logits.dtype == np.uint16 and w5.dtype == "bf16"
    assert w5.bytes_per_row == 151936 * 2 + 28


def test_peaks_and_ties():
    w = workloads.mixed_rows(64)
    assert (np.sort(w.logits, axis=1)[:, -16:].min(axis=1) > 4.0).all()   # 16 peaks at +8
    assert len(w.tie_rows) == 3
    for b, want in w.expected_greedy.items():
        row = w.logits[b]
        assert (row == row.max()).sum() == 3 and int(np.argmax(row)) == want
    cyc = w.cfgs["temperature"][:4].tolist()
    assert cyc[0] == 0.0 and abs(cyc[1] - 0.7) < 1e-6


def test_uniform_range():
    for name in ("c1", "c2", "c3"):
        w = workloads.make(name, 8)
        assert ((w.uniforms >= 0) & (w.uniforms < 1)).all()


def test_shard_helpers_cover_exactly():
    for total in (1, 7, 256, 1000, 151936):
        for world in (1, 2, 4, 8):
            spans = [workloads.shard_rows(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert spans == [workloads.shard_vocab(total, r, world) for r in range(world)]
