"""lc_tq_attention_noalloc_into — the fused code-space attention for callers that
cannot allocate device memory (its split-K partials live in a fixed array inside
the library).  Called through the C ABI twice in a row, on different inputs, and
compared with the regular entry point on the same inputs; the second call runs
over the first call's leftovers in the shared array, so stale partials would show.
Collected last on purpose: a `-x` run has finished every other test before this one."""
import numpy as np
import pytest

from gpu_util import Guarded, rel_close

pytestmark = pytest.mark.gpu


def test_noalloc_attention_matches_regular_entry_point_twice(la, orc, ctx, kernels):
    hd, n_q, n_kv, bits = 256, 8, 1, 2
    levels, signs = la.tq_levels(hd, bits), la.tq_signs(hd, la.TQ_SEED)
    cb = la.tq_code_bytes(hd, bits)
    total = 6000
    kf, vf = la.synth.normal_f16((total, n_kv, hd), 401), la.synth.normal_f16((total, n_kv, hd), 402)
    kc, kn = np.zeros(total * cb, np.uint8), np.zeros(total, np.float16)
    vc, vn = np.zeros(total * cb, np.uint8), np.zeros(total, np.float16)
    orc.encode_kv(kf, levels, signs, kc, kn, hd, n_kv, total, bits, 0, 0)
    orc.encode_kv(vf, levels, signs, vc, vn, hd, n_kv, total, bits, 0, 0)
    dev = lambda a: la.CudaBuffer.from_slice(ctx, a)
    kcb, knb, vcb, vnb, lvb, sgb = dev(kc), dev(kn), dev(vc), dev(vn), dev(levels), dev(signs)

    # (context length, window, query seed): many splits first, then a short windowed call
    for ctxlen, window, seed in ((6000, 0, 403), (700, 512, 404)):
        q = la.synth.normal_f16((n_q, hd), seed)
        qb = dev(q)
        ref, got = Guarded(la, ctx, n_q * hd * 2), Guarded(la, ctx, n_q * hd * 2)
        b = la.CommandBatch.new(ctx)
        kernels.tq_attention_into(b, qb, kcb, knb, vcb, vnb, lvb, sgb, ref.view, hd, ctxlen, ctxlen - 1, n_q, n_kv,
                                  window, bits, 0, 0.0625)
        b.commit_and_wait()
        b = la.CommandBatch.new(ctx)
        la.kernels.tq_attention_noalloc_into(b, qb, kcb, knb, vcb, vnb, lvb, sgb, got.view, hd, ctxlen, ctxlen - 1,
                                             n_q, n_kv, window, bits, 0, 0.0625)
        assert b.dispatch_count() == 2
        b.commit_and_wait()
        want = ref.read(np.float16).astype(np.float32)
        rel_close(got.read(np.float16), want, 2e-3, f"noalloc vs regular, ctx {ctxlen}")
        oracle = orc.tq_attention_fused(q, kc, kn, vc, vn, levels, signs, None, hd, 0, n_q, n_kv, window, bits, 1, 0,
                                        0.0625, ctxlen, ctxlen - 1).astype(np.float32)
        rel_close(got.read(np.float16), oracle, 2e-3, f"noalloc vs oracle, ctx {ctxlen}")


def test_noalloc_attention_rejects_what_does_not_fit(la, ctx):
    """Bad shapes are refused with a status, and a shape whose partials exceed the array names the limit."""
    buf = la.CudaBuffer.empty(ctx, 1 << 12)
    b = la.CommandBatch.new(ctx)
    with pytest.raises(la.Error) as ei:
        la.kernels.tq_attention_noalloc_into(b, buf, buf, buf, buf, buf, buf, buf, buf, 100, 4, 3, 8, 1, 0, 2, 0, 1.0)
    assert ei.value.kind == "InvalidArgument"
    big_q = la.CudaBuffer.empty(ctx, 4096 * 512 * 2)
    with pytest.raises(la.Error) as ei:
        la.kernels.tq_attention_noalloc_into(b, big_q, big_q, big_q, big_q, big_q, big_q, big_q, big_q, 512, 1, 0,
                                             4096, 4096, 0, 2, 0, 1.0)
    assert ei.value.kind == "InvalidArgument" and "built-in scratch holds 4194304 bytes" in str(ei.value)
    b.commit_and_wait()
