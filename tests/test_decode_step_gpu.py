"""The composed decode step (lc_model_decode_batch_step_into) vs the oracle's
orc_decode_batch_step on a small model of the same architecture (GQA, TQ2_0
projections, Q4_0 tied embedding, tq2 KV pools, 4 sliding-window layers with a
wrapping ring + 1 full layer).

Why the tolerances differ from the single-kernel tests: activations are f16 between
ops, so a last-bit difference in one op moves later ops by an ulp, and a 2-bit KV code
can flip when its coordinate sits on a level boundary.  The reference's own batched-vs-
single test therefore asks only for argmax equality plus a logit envelope of 0.15 * scale
(local-engine/src/pipeline/batched.rs:471-477,580-588).  Here: with the KV pools forced
identical before each step, logits must agree to 1e-2 * max(1, |logit|_max) and the freshly
written KV rows must match the oracle's byte for byte in >= 99 % of bytes; free-running over
many steps, the reference's envelope and its top-2-gap rule for argmax apply."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def small_cfg(la, max_lanes=3, max_context=64, bits=2):
    return la.ModelConfig(hidden=512, n_q_heads=4, n_kv_heads=1, head_dim=128, inter=1024, vocab=1000, n_layers=5,
                          kv_bits=bits, max_lanes=max_lanes, max_context=max_context, swa_window=16, swa_ring=16,
                          full_every=5, rms_eps=1e-6, rope_theta=1e6, softmax_scale=float(1 / np.sqrt(128)),
                          embed_scale=float(np.sqrt(np.float32(512))))


def build(la, orc, ctx, kernels, cfg):
    layers = [la.model.synth_layer(cfg, i, seed=3) for i in range(cfg.n_layers)]
    emb, fnorm = la.model.synth_embedding(cfg, seed=3)
    gm = la.DecodeModel(ctx, kernels, cfg)
    for i, t in enumerate(layers):
        gm.set_layer(i, t)
    gm.set_embedding(emb, fnorm)
    geo = []
    for i in range(cfg.n_layers):
        kv = gm.kv_buffers(i)
        geo.append((kv["lane_rows"], kv["ring"], kv["window"]))
    assert geo[0] == (16, 16, 16) and geo[4] == (cfg.max_context, 0, 0)
    return gm, orc.OracleModel(cfg, layers, emb, fnorm, geo)


def sync_pools(gm, om):
    for i, pool in enumerate(om.pools):
        kv = gm.kv_buffers(i)
        for name in ("k_codes", "k_norms", "v_codes", "v_norms"):
            kv[name].copy_from_bytes(pool[name].view(np.uint8))


def gpu_step(la, ctx, gm, tokens, positions, n):
    tb, pb = la.CudaBuffer.from_slice(ctx, tokens), la.CudaBuffer.from_slice(ctx, positions)
    nt = la.CudaBuffer.empty(ctx, n * 4)
    b = la.CommandBatch.new(ctx)
    gm.decode_batch_step_into(b, tb, pb, n, True, nt)
    b.commit_and_wait()
    logits = gm.logits_buffer().as_slice(np.float32, n * gm.cfg.vocab).reshape(n, gm.cfg.vocab)
    hidden = gm.hidden_buffer().as_slice(np.float16, n * gm.cfg.hidden).reshape(n, gm.cfg.hidden)
    return logits, hidden, nt.as_slice(np.uint32)


def argmax_consistent(got_tok, want_logits, env):
    """Token flips are legal only at near-ties: top-2 gap <= 2 * envelope (batched.rs:701-725)."""
    for lane, t in enumerate(got_tok):
        row = want_logits[lane]
        best = int(np.argmax(row))
        if int(t) != best:
            top2 = np.partition(row, -2)[-2:]
            assert top2[1] - top2[0] <= 2 * env and row[int(t)] >= top2[1] - 2 * env, f"lane {lane}: {t} vs {best}"


def test_step_by_step_with_identical_kv(la, orc, ctx, kernels):
    """Pools forced identical before every step.  A step whose freshly written KV rows come out
    byte-identical to the oracle's must match it tightly (2e-3 of the logit scale; observed ~4e-4).
    When an f16 last-bit difference upstream flips a 2-bit code (rare: a coordinate sitting on a level
    boundary; about one written coordinate in a thousand), that step is held to the reference's envelope
    instead; the share of differing KV bytes must stay below 0.5 % and at least a fifth of the steps must be exact."""
    cfg = small_cfg(la)
    gm, om = build(la, orc, ctx, kernels, cfg)
    n = cfg.max_lanes
    rng = np.random.default_rng(5)
    exact_steps, flipped_bytes, total_steps = 0, 0, 40
    for step in range(total_steps):  # the ring of 16 wraps twice
        tokens = rng.integers(0, cfg.vocab, n).astype(np.uint32)
        positions = np.full(n, step, np.uint32)
        sync_pools(gm, om)
        want, want_h = om.decode_batch_step(tokens, positions)
        got, got_h, got_tok = gpu_step(la, ctx, gm, tokens, positions, n)
        mism = 0
        for i, pool in enumerate(om.pools):
            kv = gm.kv_buffers(i)
            for name in ("k_codes", "v_codes", "k_norms", "v_norms"):
                mism += int(np.sum(kv[name].as_slice(np.uint8) != pool[name].view(np.uint8)))
        scale = max(1.0, float(np.abs(want).max()))
        err = float(np.abs(got - want).max()) / scale
        tol = 2e-3 if mism == 0 else 0.15
        assert err <= tol, f"step {step}: logits off by {err:.3e} of scale with {mism} differing KV bytes"
        argmax_consistent(got_tok, want, tol * scale)
        if mism == 0:
            exact_steps += 1
            hs = max(1.0, float(np.abs(want_h.astype(np.float32)).max()))
            assert np.abs(got_h.astype(np.float32) - want_h.astype(np.float32)).max() <= 4e-3 * hs
        flipped_bytes += mism
    written = total_steps * cfg.n_layers * 2 * n * (cfg.head_dim * cfg.kv_bits // 8 + 2)
    assert exact_steps >= total_steps // 5, f"only {exact_steps}/{total_steps} steps had byte-identical KV rows"
    assert flipped_bytes <= 0.005 * written, f"{flipped_bytes} of {written} written KV bytes differ"


def test_free_running_many_steps_ragged(la, orc, ctx, kernels):
    """Lanes at different positions, pools never re-synchronised: the reference's envelope applies."""
    cfg = small_cfg(la, max_lanes=4, max_context=96)
    gm, om = build(la, orc, ctx, kernels, cfg)
    rng = np.random.default_rng(6)
    start = np.array([0, 5, 17, 40], np.uint32)
    # bring every lane to its start position by decoding alone (lane isolation: others see position 0 rewritten)
    for lane, s in enumerate(start):
        for p in range(int(s)):
            tok = rng.integers(0, cfg.vocab, cfg.max_lanes).astype(np.uint32)
            pos = np.array([p if l == lane else 0 for l in range(cfg.max_lanes)], np.uint32)
            om.decode_batch_step(tok, pos, want_logits=False)
    sync_pools(gm, om)
    for step in range(30):
        tokens = rng.integers(0, cfg.vocab, cfg.max_lanes).astype(np.uint32)
        positions = start + step
        want, _ = om.decode_batch_step(tokens, positions)
        got, _, got_tok = gpu_step(la, ctx, gm, tokens, positions, cfg.max_lanes)
        scale = max(1.0, float(np.abs(want).max()))
        assert float(np.abs(got - want).max()) <= 0.15 * scale, f"step {step}"
        argmax_consistent(got_tok, want, 0.15 * scale)


def test_lane_isolation_and_graph_replay(la, orc, ctx, kernels):
    """Duplicate tokens/positions in two lanes give bit-identical logits (batched.rs:610-620),
    and a captured graph replays the step."""
    cfg = small_cfg(la, max_lanes=4, max_context=32)
    gm, om = build(la, orc, ctx, kernels, cfg)
    n = 4
    tokens = np.array([7, 7, 9, 7], np.uint32)
    tb = la.CudaBuffer.from_slice(ctx, tokens)
    pb = la.CudaBuffer.from_slice(ctx, np.zeros(n, np.uint32))
    nt = la.CudaBuffer.empty(ctx, n * 4)
    b = la.CommandBatch.new(ctx)
    gm.decode_batch_step_into(b, tb, pb, n, True, nt)   # eager once: sizes the split-K scratch
    b.commit_and_wait()
    eager = gm.logits_buffer().as_slice(np.float32, n * cfg.vocab).reshape(n, cfg.vocab).copy()
    assert np.array_equal(eager[0], eager[1]) and np.array_equal(eager[0], eager[3])
    assert not np.array_equal(eager[0], eager[2])
    b = la.CommandBatch.capture(ctx)
    gm.decode_batch_step_into(b, tb, pb, n, True, nt)
    graph = b.end_capture()
    gm.logits_buffer().zero()
    graph.launch()
    ctx.synchronize()
    replay = gm.logits_buffer().as_slice(np.float32, n * cfg.vocab).reshape(n, cfg.vocab)
    assert np.array_equal(replay, eager)
    graph.destroy()


def test_reset_lane_zeroes_its_rows(la, orc, ctx, kernels):
    cfg = small_cfg(la, max_lanes=2, max_context=32)
    gm, om = build(la, orc, ctx, kernels, cfg)
    gpu_step(la, ctx, gm, np.array([1, 2], np.uint32), np.array([0, 0], np.uint32), 2)
    gm.reset_lane(1)
    ctx.synchronize()
    for i in range(cfg.n_layers):
        kv = gm.kv_buffers(i)
        rows = kv["lane_rows"]
        kn = kv["k_norms"].as_slice(np.float16).reshape(2, rows)
        assert kn[0, 0] != 0 and np.all(kn[1] == 0)


# ---- the kernel routes the batch-64 benchmark takes ----
def bench_route_cfg(la, max_lanes, max_context=1024, vocab=76032):
    """The benchmark model's layer shape (hidden 1536, 8 q / 1 kv heads of 256, GeGLU 6144, tq2 KV, 512-slot ring)
    cut to two layers -- one sliding-window, one full -- and a vocabulary just large enough for the persistent
    512-row projection kernel and the chunked argmax."""
    return la.ModelConfig(hidden=1536, n_q_heads=8, n_kv_heads=1, head_dim=256, inter=6144, vocab=vocab, n_layers=2,
                          kv_bits=2, max_lanes=max_lanes, max_context=max_context, swa_window=512, swa_ring=512,
                          full_every=2, rms_eps=1e-6, rope_theta=1e6, softmax_scale=1.0 / 16.0,
                          embed_scale=float(np.sqrt(np.float32(1536))))


@pytest.fixture(scope="module")
def bench_route_model(la, orc, ctx, kernels):
    cfg = bench_route_cfg(la, 64)
    layers = [la.model.synth_layer(cfg, i, seed=9) for i in range(cfg.n_layers)]
    emb, fnorm = la.model.synth_embedding(cfg, seed=9)
    gm = la.DecodeModel(ctx, kernels, cfg)
    for i, t in enumerate(layers):
        gm.set_layer(i, t)
    gm.set_embedding(emb, fnorm)
    geo = []
    for i in range(cfg.n_layers):
        kv = gm.kv_buffers(i)
        geo.append((kv["lane_rows"], kv["ring"], kv["window"]))
    assert geo == [(512, 512, 512), (cfg.max_context, 0, 0)]
    om = orc.OracleModel(cfg, layers, emb, fnorm, geo)
    # history: every lane's pools hold properly encoded rows for positions 0 .. 899 (the ring has wrapped)
    levels, signs = orc.tq_levels(cfg.head_dim, cfg.kv_bits), orc.tq_signs(cfg.head_dim, la.TQ_SEED)
    hist = 900
    for li, pool in enumerate(om.pools):
        lane_rows, ring, _ = geo[li]
        cb = la.tq_code_bytes(cfg.head_dim, cfg.kv_bits)
        for lane in range(cfg.max_lanes):
            for j, (codes, norms) in enumerate((("k_codes", "k_norms"), ("v_codes", "v_norms"))):
                rows = la.synth.normal_f16((hist, 1, cfg.head_dim), 7000 + 1000 * li + 10 * lane + j)
                c = pool[codes][lane * lane_rows * cb:(lane + 1) * lane_rows * cb]
                n = pool[norms][lane * lane_rows:(lane + 1) * lane_rows]
                orc.encode_kv(rows, levels, signs, c, n, cfg.head_dim, 1, hist, cfg.kv_bits, 0, ring)
    return cfg, gm, om, hist


@pytest.mark.parametrize("lanes", [64, 33, 9])
def test_step_at_the_benchmark_kernel_routes(la, orc, ctx, kernels, bench_route_model, lanes):
    """One teacher-forced step against the oracle on the shapes the batch-64 benchmark runs, so that the kernels
    the benchmark's graph is made of are checked in composition: the tcgen05 decode projections (grouped Q/K/V, O,
    fused GeGLU, down), the fused q/k norm + RoPE + KV write, tensor-core attention over tq2 codes (ragged
    positions, a wrapped 512-slot ring and a full layer), the norm pairs, the persistent 512-row vocabulary
    projection (more than 32 lanes) and the chunked argmax.  Pools are identical before the step; logits must agree
    to 2e-3 of the logit scale when the freshly written KV rows come out byte-identical, else within the
    reference's own envelope (pipeline/batched.rs:471-477, 701-725)."""
    cfg, gm, om, hist = bench_route_model
    sync_pools(gm, om)
    rng = np.random.default_rng(40 + lanes)
    tokens = rng.integers(0, cfg.vocab, lanes).astype(np.uint32)
    positions = (hist - rng.integers(0, 300, lanes)).astype(np.uint32)    # ragged, all past the ring's first wrap
    positions[0] = hist
    want, want_h = om.decode_batch_step(tokens, positions)
    tb, pb = la.CudaBuffer.from_slice(ctx, tokens), la.CudaBuffer.from_slice(ctx, positions)
    nt = la.CudaBuffer.empty(ctx, lanes * 4)
    b = la.CommandBatch.new(ctx)
    gm.decode_batch_step_into(b, tb, pb, lanes, True, nt)
    # embed, first norm, 2 x (Q/K/V, q/k/v post, attention with its in-kernel merge, O, norm pair, GeGLU, down,
    # norm pair), vocabulary, argmax: the grouped and fused forms were taken
    assert b.dispatch_count() == 2 + 2 * 8 + 2
    b.commit_and_wait()
    got = gm.logits_buffer().as_slice(np.float32, lanes * cfg.vocab).reshape(lanes, cfg.vocab)
    got_h = gm.hidden_buffer().as_slice(np.float16, lanes * cfg.hidden).reshape(lanes, cfg.hidden)
    got_tok = nt.as_slice(np.uint32)
    mism = 0
    for i, pool in enumerate(om.pools):
        kv = gm.kv_buffers(i)
        for name in ("k_codes", "v_codes", "k_norms", "v_norms"):
            mism += int(np.sum(kv[name].as_slice(np.uint8) != pool[name].view(np.uint8)))
    assert np.all(np.isfinite(got))
    scale = max(1.0, float(np.abs(want).max()))
    err = float(np.abs(got - want).max()) / scale
    tol = 2e-3 if mism == 0 else 0.15
    assert err <= tol, f"{lanes} lanes: logits off by {err:.3e} of scale with {mism} differing KV bytes"
    argmax_consistent(got_tok, want, tol * scale)
    assert np.array_equal(got_tok, np.argmax(got, axis=1).astype(np.uint32)), "device argmax vs its own logits"
    written = cfg.n_layers * 2 * lanes * (cfg.head_dim * cfg.kv_bits // 8 + 2)
    assert mism <= 0.01 * written, f"{mism} of {written} freshly written KV bytes differ"
    if mism == 0:
        hs = max(1.0, float(np.abs(want_h.astype(np.float32)).max()))
        assert np.abs(got_h.astype(np.float32) - want_h.astype(np.float32)).max() <= 4e-3 * hs


def test_query_fragments_from_the_kv_write_change_nothing(la, ctx, kernels, monkeypatch):
    """At the benchmark's head shape the launch that finishes q also writes the attention kernel's rotated, scaled
    query fragments.  They are the values the attention kernel would derive itself, so a model built with that
    hand-over switched off must produce the same logits bit for bit, over steps that fill and then read the pools."""
    cfg = bench_route_cfg(la, 9, max_context=256, vocab=4096)
    layers = [la.model.synth_layer(cfg, i, seed=21) for i in range(cfg.n_layers)]
    emb, fnorm = la.model.synth_embedding(cfg, seed=21)

    def run():
        gm = la.DecodeModel(ctx, kernels, cfg)
        for i, t in enumerate(layers):
            gm.set_layer(i, t)
        gm.set_embedding(emb, fnorm)
        rng = np.random.default_rng(5)
        outs = []
        for step in range(6):
            tokens = rng.integers(0, cfg.vocab, 9).astype(np.uint32)
            positions = np.full(9, step, np.uint32)
            logits, _, _ = gpu_step(la, ctx, gm, tokens, positions, 9)
            outs.append(logits.copy())
        return np.stack(outs)

    with_frag = run()
    monkeypatch.setenv("LOCAL_CUDA_QFRAG", "0")
    without = run()
    assert np.all(np.isfinite(with_frag))
    assert np.array_equal(with_frag.view(np.uint32), without.view(np.uint32))
