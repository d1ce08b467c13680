"""The single-sequence KV container (lc_kv_cache_*, QuantizedKvCache of local-engine/src/kv_cache/quant_cache.rs), the
prefill / multi-row verify attention over codes, and lane recycling through the scheduler, on the GPU."""
import numpy as np
import pytest

from gpu_util import Guarded, rel_close

pytestmark = pytest.mark.gpu


def seeded_f16(la, n, seed):
    """Values in [-0.5, 0.5) like the reference tests' seeded_f16 (quant_cache.rs:710-721)."""
    return (la.synth.uniform(seed, n) - 0.5).astype(np.float16)


def test_constructor_preconditions(la, ctx):
    """quant_cache.rs:191-209: bits 2..=4, head_dim a power of two <= 512, ring >= window + 255."""
    for args in ((1, 256, 64, 64, 0, 5), (1, 256, 64, 64, 0, 1), (1, 96, 64, 64, 0, 2), (1, 1024, 64, 64, 0, 2),
                 (1, 256, 4096, 600, 512, 2)):
        with pytest.raises(la.Error) as ei:
            la.QuantizedKvCache(ctx, *args)
        assert ei.value.kind == "InvalidArgument"
    c = la.QuantizedKvCache(ctx, 1, 256, 4096, la.swa_ring_capacity(512, 4096), 512, 2)
    assert c.is_ringed() and c.ring_capacity() == 1024 and c.code_bytes() == 64
    full = la.QuantizedKvCache(ctx, 2, 128, 300, bits=4)
    assert not full.is_ringed() and full.ring_capacity() == 0 and full.physical_positions() == 300
    with pytest.raises(la.Error):       # a write past max_positions is refused (quant_cache.rs:400-406)
        b = la.CommandBatch.new(ctx)
        k2 = la.Kernels.new(ctx)
        src = la.CudaBuffer.empty(ctx, 4 * 2 * 128 * 2)
        try:
            full.write_kv_gpu_into(b, k2, src, src, 298, 4)
        finally:
            b.commit_and_wait()
            k2.close()
    c.close()
    full.close()


def test_ring_fused_attention_matches_full_after_wrap(la, orc, ctx, kernels):
    """quant_cache.rs:1042-1107: after the ring has wrapped more than twice, fused attention over the ringed cache is
    bit-identical to the full cache's for the same window; both match the oracle; unwritten rows contribute nothing."""
    hd, n_kv, n_q, window, bits = 128, 1, 2, 64, 4
    cap = la.swa_ring_capacity(window, 4096)     # window + 255 rounded up to a power of two: 512
    total = cap * 2 + 9
    max_pos = total + 1
    full = la.QuantizedKvCache(ctx, n_kv, hd, max_pos, bits=bits)
    ring = la.QuantizedKvCache(ctx, n_kv, hd, max_pos, cap, window, bits)
    assert ring.is_ringed() and ring.physical_positions() == cap
    k_rows = seeded_f16(la, total * n_kv * hd, 5000).reshape(total, n_kv, hd)
    v_rows = seeded_f16(la, total * n_kv * hd, 6000).reshape(total, n_kv, hd)
    d = lambda a: la.CudaBuffer.from_slice(ctx, a)
    for cache in (full, ring):
        cache.reset()
        b = la.CommandBatch.new(ctx)
        for pos in range(0, total, 37):          # multi-row writes of uneven size, crossing the ring's end
            n = min(37, total - pos)
            cache.write_kv_gpu_into(b, kernels, d(k_rows[pos:pos + n]), d(v_rows[pos:pos + n]), pos, n)
        b.commit_and_wait()
    q = seeded_f16(la, n_q * hd, 9999)

    def run(cache):
        out = Guarded(la, ctx, n_q * hd * 2)
        b = la.CommandBatch.new(ctx)
        cache.fused_attention_into(b, kernels, d(q), out.view, total, total - 1, n_q, window, 1.0)
        b.commit_and_wait()
        return out.read(np.uint16)

    got_full, got_ring = run(full), run(ring)
    assert np.array_equal(got_full, got_ring)
    levels, signs = la.tq_levels(hd, bits), la.tq_signs(hd, la.TQ_SEED)
    cb = la.tq_code_bytes(hd, bits)
    kc, kn = np.zeros(max_pos * cb, np.uint8), np.zeros(max_pos, np.float16)
    vc, vn = np.zeros(max_pos * cb, np.uint8), np.zeros(max_pos, np.float16)
    orc.encode_kv(k_rows, levels, signs, kc, kn, hd, n_kv, total, bits, 0, 0)
    orc.encode_kv(v_rows, levels, signs, vc, vn, hd, n_kv, total, bits, 0, 0)
    bufs = full.buffers()
    assert np.array_equal(bufs["keys_q"].as_slice(np.uint8), kc) and np.array_equal(bufs["key_norms"].as_slice(np.float16), kn)
    want = orc.tq_attention_fused(q, kc, kn, vc, vn, levels, signs, None, hd, 0, n_q, n_kv, window, bits, 1, 0, 1.0, total,
                                  total - 1).astype(np.float32)
    rel_close(got_full.view(np.float16), want, 2e-3, "container attention vs oracle")
    # reset: zero norms annihilate every row (quant_cache.rs:364-380, 838-843)
    ring.reset()
    assert not ring.buffers()["key_norms"].as_slice(np.uint16).any() and not ring.buffers()["values_q"].as_slice(np.uint8).any()
    assert not np.any(run(ring).view(np.float16).astype(np.float32))
    # snapshot / restore of a prefix (quant_cache.rs:327-362)
    snap = full.snapshot_prefix(100)
    full.reset()
    full.restore_prefix(snap, 100)
    assert np.array_equal(full.buffers()["keys_q"].as_slice(np.uint8, 100 * cb), kc[:100 * cb])
    assert ring.max_snapshot_positions() == cap and full.max_snapshot_positions() == max_pos
    full.close()
    ring.close()


@pytest.mark.parametrize("hd,n_q,n_kv,bits,n_rows,start,window,ring", [
    (128, 4, 2, 4, 12, 0, 0, 0),         # the reference's prefill test shape (kernels.rs:10126-10285)
    (256, 8, 1, 2, 20, 0, 0, 0),         # its tiled-vs-non-tiled shape (kernels.rs:10295-10448): tensor-core kernel here
    (256, 8, 1, 2, 64, 700, 512, 1024),  # a 64-row chunk deep in a ringed sliding-window layer
    (256, 8, 1, 3, 9, 40, 16, 0),
])
def test_prefill_attention_over_codes(la, orc, ctx, kernels, hd, n_q, n_kv, bits, n_rows, start, window, ring):
    """flash_attention_tq_prefill(_tiled): every row equals the decode kernel at that row's position to 1e-4 (the
    reference's prefill == per-row decode test), meets the oracle at 1e-3, and the tiled entry point meets the
    f16-tile arithmetic of the reference's tiled shader at its own 5e-3; the fused f16 form meets the oracle at 2e-3."""
    kv_len = start + n_rows
    rows = ring if ring else kv_len
    levels, signs = la.tq_levels(hd, bits), la.tq_signs(hd, la.TQ_SEED)
    cb = la.tq_code_bytes(hd, bits)
    kf, vf = la.synth.normal_f16((kv_len, n_kv, hd), 7100 + hd), la.synth.normal_f16((kv_len, n_kv, hd), 7200 + hd)
    kc, kn = np.zeros(rows * n_kv * cb, np.uint8), np.zeros(rows * n_kv, np.float16)
    vc, vn = np.zeros(rows * n_kv * cb, np.uint8), np.zeros(rows * n_kv, np.float16)
    orc.encode_kv(kf, levels, signs, kc, kn, hd, n_kv, kv_len, bits, 0, ring)
    orc.encode_kv(vf, levels, signs, vc, vn, hd, n_kv, kv_len, bits, 0, ring)
    f = lambda a: la.CudaBuffer.from_slice(ctx, a)
    kcb, knb, vcb, vnb, lvb, sgb = f(kc), f(kn), f(vc), f(vn), f(levels), f(signs)
    q16 = la.synth.normal_f16((n_rows, n_q, hd), 7300 + hd)
    rq = orc.hadamard_rotate(q16.astype(np.float32), signs, hd, n_rows * n_q, True, False)
    rqb = f(rq)
    scale = 0.0625
    outs = {}
    for name in ("flash_attention_tq_prefill_into", "flash_attention_tq_prefill_tiled_into"):
        out = Guarded(la, ctx, n_rows * n_q * hd * 4)
        b = la.CommandBatch.new(ctx)
        getattr(kernels, name)(b, rqb, kcb, knb, vcb, vnb, lvb, out.view, hd, kv_len, start, n_rows, n_q, n_kv, window, bits, ring, scale)
        b.commit_and_wait()
        outs[name] = out.read(np.float32).reshape(n_rows, n_q * hd)
    want = orc.flash_attention_tq_prefill(rq, kc, kn, vc, vn, levels, hd, kv_len, start, n_rows, n_q, n_kv, window, bits, ring, scale)
    want_tiled = orc.flash_attention_tq_prefill(rq, kc, kn, vc, vn, levels, hd, kv_len, start, n_rows, n_q, n_kv, window, bits, ring,
                                                scale, tiled=True)
    rel_close(outs["flash_attention_tq_prefill_into"], want, 1e-3, "prefill vs oracle")
    rel_close(outs["flash_attention_tq_prefill_tiled_into"], want_tiled, 5e-3, "tiled entry point vs the tiled shader's arithmetic")
    for r in (0, n_rows // 2, n_rows - 1):       # per-row decode at that row's position
        one = Guarded(la, ctx, n_q * hd * 4)
        b = la.CommandBatch.new(ctx)
        kernels.flash_attention_tq_into(b, f(rq.reshape(n_rows, -1)[r]), kcb, knb, vcb, vnb, lvb, one.view, hd, kv_len, start + r, n_q,
                                        n_kv, window, bits, ring, scale)
        b.commit_and_wait()
        rel_close(outs["flash_attention_tq_prefill_into"][r], one.read(np.float32), 1e-4, f"prefill row {r} vs decode")
    fo = Guarded(la, ctx, n_rows * n_q * hd * 2)
    b = la.CommandBatch.new(ctx)
    kernels.tq_attention_prefill_into(b, f(q16), kcb, knb, vcb, vnb, lvb, sgb, fo.view, hd, kv_len, start, n_rows, n_q, n_kv, window,
                                      bits, ring, scale)
    b.commit_and_wait()
    back = orc.hadamard_rotate(want, signs, hd, n_rows * n_q, False, True)
    rel_close(fo.read(np.float16), back.astype(np.float16).astype(np.float32), 2e-3, "fused prefill vs oracle")


def test_container_prefill_chunk_then_decode(la, orc, ctx, kernels):
    """write_kv_gpu_into + fused_attention_batch_into for a chunk, then single-token decode: the sequence the reference's
    prefill issues per layer (quant_cache.rs:391-444, 620-700), against the oracle."""
    hd, n_kv, n_q, bits, chunk = 256, 1, 8, 2, 48
    cache = la.QuantizedKvCache(ctx, n_kv, hd, 4096, la.swa_ring_capacity(512, 4096), 512, bits)
    levels, signs = la.tq_levels(hd, bits), la.tq_signs(hd, la.TQ_SEED)
    kf, vf = la.synth.normal_f16((chunk + 1, n_kv, hd), 8100), la.synth.normal_f16((chunk + 1, n_kv, hd), 8200)
    q16 = la.synth.normal_f16((chunk + 1, n_q, hd), 8300)
    d = lambda a: la.CudaBuffer.from_slice(ctx, a)
    out = Guarded(la, ctx, chunk * n_q * hd * 2)
    b = la.CommandBatch.new(ctx)
    cache.write_kv_gpu_into(b, kernels, d(kf[:chunk]), d(vf[:chunk]), 0, chunk)
    cache.fused_attention_batch_into(b, kernels, d(q16[:chunk]), out.view, chunk, 0, chunk, n_q, 512, 0.0625)
    b.commit_and_wait()
    ring = cache.ring_capacity()
    cb = la.tq_code_bytes(hd, bits)
    kc, kn = np.zeros(ring * cb, np.uint8), np.zeros(ring, np.float16)
    vc, vn = np.zeros(ring * cb, np.uint8), np.zeros(ring, np.float16)
    orc.encode_kv(kf, levels, signs, kc, kn, hd, n_kv, chunk + 1, bits, 0, ring)
    orc.encode_kv(vf, levels, signs, vc, vn, hd, n_kv, chunk + 1, bits, 0, ring)
    rq = orc.hadamard_rotate(q16[:chunk].astype(np.float32), signs, hd, chunk * n_q, True, False)
    acc = orc.flash_attention_tq_prefill(rq, kc, kn, vc, vn, levels, hd, chunk, 0, chunk, n_q, n_kv, 512, bits, ring, 0.0625)
    want = orc.hadamard_rotate(acc, signs, hd, chunk * n_q, False, True).astype(np.float16).astype(np.float32)
    rel_close(out.read(np.float16), want, 2e-3, "container prefill chunk")
    one = Guarded(la, ctx, n_q * hd * 2)
    b = la.CommandBatch.new(ctx)
    cache.write_kv_gpu_into(b, kernels, d(kf[chunk:]), d(vf[chunk:]), chunk, 1)
    cache.fused_attention_into(b, kernels, d(q16[chunk]), one.view, chunk + 1, chunk, n_q, 512, 0.0625)
    b.commit_and_wait()
    want1 = orc.tq_attention_fused(q16[chunk], kc, kn, vc, vn, levels, signs, None, hd, 0, n_q, n_kv, 512, bits, 1, ring, 0.0625,
                                   chunk + 1, chunk).astype(np.float32)
    rel_close(one.read(np.float16), want1, 2e-3, "container decode after the chunk")
    cache.close()


def test_recycled_lane_equals_a_fresh_lane(la, orc, ctx, kernels):
    """Continuous batching over a model's lanes: a request decoded in a lane that served another request before gives
    bit for bit the logits of the same request in a never-used lane (the scheduler zeroes a lane on admission and on
    completion, kv_cache/quant_unified_pool.rs:333-346, runner.rs:149,174)."""
    cfg = la.ModelConfig(hidden=512, n_q_heads=4, n_kv_heads=1, head_dim=128, inter=1024, vocab=1000, n_layers=3, kv_bits=2,
                         max_lanes=2, max_context=48, swa_window=16, swa_ring=16, full_every=3, rms_eps=1e-6, rope_theta=1e6,
                         softmax_scale=float(1 / np.sqrt(128)), embed_scale=float(np.sqrt(np.float32(512))))
    gm = la.DecodeModel(ctx, kernels, cfg)
    for i in range(cfg.n_layers):
        gm.set_layer(i, la.model.synth_layer(cfg, i, seed=21))
    gm.set_embedding(*la.model.synth_embedding(cfg, seed=21))
    tok_b, pos_b, nxt_b = la.CudaBuffer.empty(ctx, 8), la.CudaBuffer.empty(ctx, 8), la.CudaBuffer.empty(ctx, 8)
    probe = np.array([11, 12, 13, 14, 15], np.uint32)

    def serve(requests):
        """Run the scheduler to completion; returns {id: (tokens, logits of the last step of that request)}."""
        sched = la.LaneScheduler(gm, 2, cfg.max_context, eos_token=cfg.vocab + 1)   # no EOS
        for rid, prompt, max_new in requests:
            sched.submit(rid, prompt, max_new)
        done, last_logits, lane_of = {}, {}, {}
        for _ in range(400):
            if sched.prepare() == 0:
                break
            while (f := sched.pop_finished()) is not None:
                done[f[0]] = f[1]
            tok_b.copy_from_bytes(sched.tokens)
            pos_b.copy_from_bytes(sched.positions)
            b = la.CommandBatch.new(ctx)
            gm.decode_batch_step_into(b, tok_b, pos_b, 2, True, nxt_b)
            b.commit_and_wait()
            logits = gm.logits_buffer().as_slice(np.float32, 2 * cfg.vocab).reshape(2, cfg.vocab).copy()
            for lane in range(2):
                last_logits[(lane, int(sched.positions[lane]), int(sched.tokens[lane]))] = logits[lane]
            sched.consume(nxt_b.as_slice(np.uint32))
        while (f := sched.pop_finished()) is not None:
            done[f[0]] = f[1]
        sched.close()
        return done, last_logits

    # run 1: the probe request alone, in lane 0 of freshly zeroed pools
    for lane in range(2):
        gm.reset_lane(lane)
    fresh, fresh_logits = serve([(1, probe, 6)])
    # run 2: two other requests occupy both lanes first; the probe is admitted into whichever lane frees up
    busy, busy_logits = serve([(7, np.array([3, 4, 5, 6, 7, 8, 9], np.uint32), 9), (8, np.array([20, 21], np.uint32), 4), (1, probe, 6)])
    assert np.array_equal(fresh[1], busy[1]) and len(fresh[1]) == 6
    # the probe's step at (position 4, token 15) -- its last prompt token -- gave identical logits in both runs
    f_key = [k for k in fresh_logits if k[1:] == (4, 15)]
    b_key = [k for k in busy_logits if k[1:] == (4, 15)]
    assert f_key and b_key
    assert np.array_equal(fresh_logits[f_key[0]], busy_logits[b_key[0]])
