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


def test_reference_arm_and_gpu_arm_build_the_same_model(la):
    """oracle/synth_model.py restates the package's seeding rule so that the CPU reference arm of the benchmark does
    not need the CUDA library; both arms must time the same weights, byte for byte."""
    import importlib.util
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    spec = importlib.util.spec_from_file_location("orc_synth_model", root / "oracle" / "synth_model.py")
    sm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sm)
    cfg = la.ModelConfig(hidden=512, n_q_heads=4, n_kv_heads=1, head_dim=128, inter=1024, vocab=640, n_layers=6,
                         kv_bits=2, max_lanes=2, max_context=700, swa_window=512, swa_ring=512, full_every=5,
                         rms_eps=1e-6, rope_theta=1e6, softmax_scale=0.125, embed_scale=1.0)
    layers, emb, fnorm, geo = sm.build(la.synth, cfg, 188, seed=4)
    for i, t in enumerate(layers):
        want = la.model.synth_layer(cfg, i, seed=4)
        assert set(t) == set(want)
        for name in want:
            assert t[name].dtype == want[name].dtype and np.array_equal(t[name], want[name]), (i, name)
    e2, f2 = la.model.synth_embedding(cfg, seed=4)
    assert np.array_equal(emb, e2) and np.array_equal(fnorm, f2)
    assert geo[4] == (cfg.max_context, 0, 0) and geo[0] == (512, 512, 512)
