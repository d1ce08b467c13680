"""Seeded synthetic inputs: reproducible, right layout, right value sets."""
import numpy as np


def test_streams_are_reproducible_and_counter_based(la):
    s = la.synth
    a = s.splitmix64(42, 1000)
    assert np.array_equal(a, s.splitmix64(42, 1000))
    assert np.array_equal(a[100:200], s.splitmix64(42, 100, offset=100))
    assert not np.array_equal(a, s.splitmix64(43, 1000))


def test_normal_and_uniform_moments(la):
    x = la.synth.normal(7, 200_000)
    assert abs(x.mean()) < 0.01 and abs(x.std() - 1.0) < 0.01
    u = la.synth.uniform(7, 200_000, 0.005, 0.05)
    assert u.min() >= 0.005 and u.max() <= 0.05 and abs(u.mean() - 0.0275) < 3e-4


def test_q4_0_blocks(la, orc):
    rows, cols = 16, 1536
    w = la.synth.q4_0_weights(rows, cols, 3)
    assert w.dtype == np.uint8 and w.size == rows * cols // 32 * 18
    d = w.reshape(-1, 18)[:, :2].copy().view(np.float16).astype(np.float32)
    assert d.min() >= 0.001 * 0.999 and d.max() <= 0.02 * 1.001
    dq = orc.expand_f32(orc.Q4_0, w, rows, cols)
    q = np.rint(dq.reshape(-1, 32) / d).astype(int)
    assert q.min() == -8 and q.max() == 7


def test_tq2_0_blocks_are_ternary(la, orc):
    rows, cols = 8, 1536
    w = la.synth.tq2_0_weights(rows, cols, 5)
    assert w.size == rows * cols // 256 * 66
    d = w.reshape(-1, 66)[:, 64:].copy().view(np.float16).astype(np.float32)
    assert d.min() >= 0.005 * 0.999 and d.max() <= 0.05 * 1.001
    dq = orc.expand_f32(orc.TQ2_0, w, rows, cols).reshape(-1, 256)
    q = np.rint(dq / d).astype(int)
    assert set(np.unique(q)) == {-1, 0, 1}
    counts = np.bincount((q + 1).reshape(-1), minlength=3) / q.size
    assert np.all(np.abs(counts - 1 / 3) < 0.01)
    w4 = la.synth.tq2_0_weights(rows, cols, 5, ncodes=4)
    q4 = np.rint(orc.expand_f32(orc.TQ2_0, w4, rows, cols).reshape(-1, 256) / d).astype(int)
    assert set(np.unique(q4)) == {-1, 0, 1, 2}


def test_lognormal_contexts(la):
    c = la.synth.lognormal_contexts(512, 9)
    assert c.min() >= 16 and c.max() <= 131072
    assert 1500 < np.median(c) < 2800
