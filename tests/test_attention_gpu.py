"""Decode attention over TurboQuant codes (and the FP16-KV variants) vs the CPU
oracle.  Tolerance 1e-3 * max(|want|, 1) for f32 outputs (fp32 online softmax vs
the oracle's f64 softmax); 2e-3 for f16 outputs (one more rounding)."""
import numpy as np
import pytest

import refgen
from gpu_util import Guarded, rel_close

pytestmark = pytest.mark.gpu


class Cache:
    """Oracle-encoded K/V rows in the single-sequence or pool layout."""

    def __init__(self, la, orc, ctx, hd, n_kv, bits, rows, seed):
        self.hd, self.n_kv, self.bits = hd, n_kv, bits
        self.levels, self.signs = la.tq_levels(hd, bits), la.tq_signs(hd, la.TQ_SEED)
        self.cb = la.tq_code_bytes(hd, bits)
        self.kc, self.vc = np.zeros(rows * n_kv * self.cb, np.uint8), np.zeros(rows * n_kv * self.cb, np.uint8)
        self.kn, self.vn = np.zeros(rows * n_kv, np.float16), np.zeros(rows * n_kv, np.float16)
        self.la, self.orc, self.ctx, self.seed = la, orc, ctx, seed

    def fill_single(self, total, ring):
        """Write logical positions 0..total-1 (wrapping when ring != 0)."""
        k = self.la.synth.normal_f16((total, self.n_kv, self.hd), self.seed)
        v = self.la.synth.normal_f16((total, self.n_kv, self.hd), self.seed + 1)
        self.orc.encode_kv(k, self.levels, self.signs, self.kc, self.kn, self.hd, self.n_kv, total, self.bits, 0, ring)
        self.orc.encode_kv(v, self.levels, self.signs, self.vc, self.vn, self.hd, self.n_kv, total, self.bits, 0, ring)

    def fill_pool(self, positions, lane_rows, ring):
        """Every lane gets rows for positions 0..positions[lane]."""
        for lane, pos in enumerate(positions):
            n = int(pos) + 1
            k = self.la.synth.normal_f16((n, self.n_kv, self.hd), self.seed + 10 * lane)
            v = self.la.synth.normal_f16((n, self.n_kv, self.hd), self.seed + 10 * lane + 1)
            off_c, off_n = lane * lane_rows * self.n_kv * self.cb, lane * lane_rows * self.n_kv
            span_c, span_n = lane_rows * self.n_kv * self.cb, lane_rows * self.n_kv
            kc, kn = self.kc[off_c:off_c + span_c], self.kn[off_n:off_n + span_n]
            vc, vn = self.vc[off_c:off_c + span_c], self.vn[off_n:off_n + span_n]
            self.orc.encode_kv(k, self.levels, self.signs, kc, kn, self.hd, self.n_kv, n, self.bits, 0, ring)
            self.orc.encode_kv(v, self.levels, self.signs, vc, vn, self.hd, self.n_kv, n, self.bits, 0, ring)

    def device(self):
        f = lambda a: self.la.CudaBuffer.from_slice(self.ctx, a)
        return f(self.kc), f(self.kn), f(self.vc), f(self.vn), f(self.levels), f(self.signs)


SINGLE_CASES = [
    # hd, n_q, n_kv, bits, total, window, ring, scale
    (256, 8, 1, 2, 300, 0, 0, 1.0),          # the model's shape, full attention, < one split
    (256, 8, 1, 2, 5000, 0, 0, 0.0625),      # long enough for several splits
    (256, 8, 1, 3, 777, 0, 0, 1.0),
    (256, 8, 1, 4, 777, 0, 0, 0.0625),
    (256, 8, 1, 2, 2000, 512, 512, 0.0625),  # SWA layer: 512 window in a 512-slot ring, wrapped
    (256, 8, 1, 2, 2000, 512, 1024, 1.0),    # the reference's 1024-row ring
    (256, 8, 1, 2, 100, 512, 512, 1.0),      # window not yet full
    (128, 4, 2, 4, 333, 0, 0, 1.0),          # 2 kv heads, group of 2
    (64, 6, 2, 3, 200, 50, 64, 1.0),         # group of 3 (padded to 4), odd window
    (512, 8, 8, 2, 150, 0, 0, 1.0),          # MHA: group of 1, head_dim 512
    (512, 16, 1, 4, 90, 0, 0, 1.0),          # group of 16 -> two chunks of 8
    (256, 8, 1, 2, 1, 0, 0, 1.0),            # a single key
]


@pytest.mark.parametrize("hd,n_q,n_kv,bits,total,window,ring,scale", SINGLE_CASES)
def test_flash_attention_tq_matches_oracle(la, orc, ctx, kernels, hd, n_q, n_kv, bits, total, window, ring, scale):
    rows = ring if ring else total
    c = Cache(la, orc, ctx, hd, n_kv, bits, rows, seed=1000 + total)
    c.fill_single(total, ring)
    kc, kn, vc, vn, lv, sg = c.device()
    q = (la.synth.normal(55, n_q * hd) * 1.0).astype(np.float32)
    rq = orc.hadamard_rotate(q, c.signs, hd, n_q, True, False)
    out = Guarded(la, ctx, n_q * hd * 4)
    b = la.CommandBatch.new(ctx)
    kernels.flash_attention_tq_into(b, la.CudaBuffer.from_slice(ctx, rq), kc, kn, vc, vn, lv, out.view, hd, total,
                                    total - 1, n_q, n_kv, window, bits, ring, scale)
    b.commit_and_wait()
    want = orc.flash_attention_tq(rq, c.kc, c.kn, c.vc, c.vn, c.levels, hd, total, total - 1, n_q, n_kv, window, bits, ring, scale)
    rel_close(out.read(np.float32), want, 1e-3, "flash_attention_tq")


def test_kv_len_shorter_than_position(la, orc, ctx, kernels):
    """seq_len = min(kv_len, pos + 1) (attention_flash_tq.metal:178)."""
    hd, n_q, n_kv, bits, total = 256, 8, 1, 2, 64
    c = Cache(la, orc, ctx, hd, n_kv, bits, total, seed=5)
    c.fill_single(total, 0)
    kc, kn, vc, vn, lv, sg = c.device()
    rq = la.synth.normal(56, n_q * hd).astype(np.float32)
    out = Guarded(la, ctx, n_q * hd * 4)
    b = la.CommandBatch.new(ctx)
    kernels.flash_attention_tq_into(b, la.CudaBuffer.from_slice(ctx, rq), kc, kn, vc, vn, lv, out.view, hd, 40, 63, n_q, n_kv, 0, bits, 0, 1.0)
    b.commit_and_wait()
    want = orc.flash_attention_tq(rq, c.kc, c.kn, c.vc, c.vn, c.levels, hd, 40, 63, n_q, n_kv, 0, bits, 0, 1.0)
    rel_close(out.read(np.float32), want, 1e-3, "kv_len < pos + 1")


@pytest.mark.parametrize("bits,window,ring,lane_rows", [(2, 0, 0, 600), (2, 512, 512, 512), (3, 64, 128, 128), (4, 0, 0, 300)])
def test_batched_pool_attention_ragged(la, orc, ctx, kernels, bits, window, ring, lane_rows):
    """Ragged lanes over the unified pool (kernels.rs:10457-10711); also each lane equals a single-sequence call."""
    hd, n_q, n_kv = 256, 8, 1
    cap = lane_rows
    positions = np.array([0, 17, 299, 150, 64, 511 if ring else 299, 1100 if ring else 5], np.uint32)
    n_lanes = positions.size
    c = Cache(la, orc, ctx, hd, n_kv, bits, n_lanes * lane_rows, seed=300 + bits)
    c.fill_pool(positions, lane_rows, ring)
    kc, kn, vc, vn, lv, sg = c.device()
    q16 = la.synth.normal_f16((n_lanes, n_q, hd), 57)
    rq = orc.hadamard_rotate(q16.astype(np.float32), c.signs, hd, n_lanes * n_q, True, False)
    out = Guarded(la, ctx, n_lanes * n_q * hd * 4)
    pos_b = la.CudaBuffer.from_slice(ctx, positions)
    b = la.CommandBatch.new(ctx)
    kernels.flash_attention_tq_batched_into(b, la.CudaBuffer.from_slice(ctx, rq), kc, kn, vc, vn, lv, out.view, pos_b,
                                            hd, cap, n_q, n_kv, window, bits, n_lanes, ring, 0.0625)
    b.commit_and_wait()
    got = out.read(np.float32)
    want = orc.flash_attention_tq_batched(rq, c.kc, c.kn, c.vc, c.vn, c.levels, positions, hd, cap, n_q, n_kv, window,
                                          bits, n_lanes, ring, 0.0625)
    rel_close(got, want, 1e-3, "flash_attention_tq_batched")
    # fused form: f16 q in, f16 attention output out
    fo = Guarded(la, ctx, n_lanes * n_q * hd * 2)
    b = la.CommandBatch.new(ctx)
    kernels.tq_attention_batched_into(b, la.CudaBuffer.from_slice(ctx, q16), kc, kn, vc, vn, lv, sg, fo.view, pos_b, hd,
                                      cap, n_q, n_kv, window, bits, n_lanes, ring, 0.0625)
    b.commit_and_wait()
    wantf = orc.tq_attention_fused(q16, c.kc, c.kn, c.vc, c.vn, c.levels, c.signs, positions, hd, cap, n_q, n_kv,
                                   window, bits, n_lanes, ring, 0.0625)
    rel_close(fo.read(np.float16), wantf.astype(np.float32), 2e-3, "tq_attention_batched")


def test_fused_single_equals_three_call_sequence(la, orc, ctx, kernels):
    """lc_tq_attention_into == rotate_hf -> flash_attention_tq -> rotate_fh (quant_cache.rs:565-596)."""
    hd, n_q, n_kv, bits, total = 256, 8, 1, 2, 3000
    c = Cache(la, orc, ctx, hd, n_kv, bits, total, seed=9)
    c.fill_single(total, 0)
    kc, kn, vc, vn, lv, sg = c.device()
    q16 = la.synth.normal_f16((n_q, hd), 58)
    qb = la.CudaBuffer.from_slice(ctx, q16)
    rq, vacc = la.CudaBuffer.empty(ctx, n_q * hd * 4), la.CudaBuffer.empty(ctx, n_q * hd * 4)
    three, fused = Guarded(la, ctx, n_q * hd * 2), Guarded(la, ctx, n_q * hd * 2)
    b = la.CommandBatch.new(ctx)
    kernels.hadamard_rotate_hf_into(b, qb, sg, rq, hd, n_q, 1, 0)
    kernels.flash_attention_tq_into(b, rq, kc, kn, vc, vn, lv, vacc, hd, total, total - 1, n_q, n_kv, 0, bits, 0, 1.0)
    kernels.hadamard_rotate_fh_into(b, vacc, sg, three.view, hd, n_q, 0, 1)
    kernels.tq_attention_into(b, qb, kc, kn, vc, vn, lv, sg, fused.view, hd, total, total - 1, n_q, n_kv, 0, bits, 0, 1.0)
    b.commit_and_wait()
    want = orc.tq_attention_fused(q16, c.kc, c.kn, c.vc, c.vn, c.levels, c.signs, None, hd, 0, n_q, n_kv, 0, bits, 1, 0,
                                  1.0, total, total - 1).astype(np.float32)
    rel_close(three.read(np.float16), want, 2e-3, "three-call sequence")
    rel_close(fused.read(np.float16), want, 2e-3, "fused call")


def test_fused_attention_close_to_exact_attention_over_decoded_rows(la, orc, ctx, kernels):
    """kernels.rs:9936-10114: code-space attention vs dequantize + plain attention, <= 0.02 * |ref|_inf."""
    hd, n_q, n_kv, bits, total = 256, 8, 1, 4, 512
    c = Cache(la, orc, ctx, hd, n_kv, bits, total, seed=12)
    c.fill_single(total, 0)
    kc, kn, vc, vn, lv, sg = c.device()
    q16 = la.synth.normal_f16((n_q, hd), 59)
    fused = Guarded(la, ctx, n_q * hd * 2)
    b = la.CommandBatch.new(ctx)
    kernels.tq_attention_into(b, la.CudaBuffer.from_slice(ctx, q16), kc, kn, vc, vn, lv, sg, fused.view, hd, total,
                              total - 1, n_q, n_kv, 0, bits, 0, 1.0)
    b.commit_and_wait()
    kd = orc.dequantize_kv(c.kc, c.kn, c.levels, c.signs, hd, n_kv, total, bits, 0, 0)
    vd = orc.dequantize_kv(c.vc, c.vn, c.levels, c.signs, hd, n_kv, total, bits, 0, 0)
    ref = orc.attention_f16(q16, kd, vd, hd, total, total - 1, n_q, n_kv, 0).astype(np.float32)
    assert np.max(np.abs(fused.read(np.float16).astype(np.float32) - ref)) <= 0.02 * np.max(np.abs(ref))


def test_attention_rejects_bad_arguments(la, ctx, kernels):
    buf = la.CudaBuffer.empty(ctx, 1 << 16)
    b = la.CommandBatch.new(ctx)
    for args in ((100, 8, 1, 2), (256, 8, 3, 2), (256, 8, 1, 5)):  # head_dim, n_q, n_kv, bits
        hd, n_q, n_kv, bits = args
        with pytest.raises(la.Error) as ei:
            kernels.flash_attention_tq_into(b, buf, buf, buf, buf, buf, buf, buf, hd, 4, 3, n_q, n_kv, 0, bits, 0, 1.0)
        assert ei.value.kind == "InvalidArgument"
    small = la.CudaBuffer.empty(ctx, 64)
    with pytest.raises(la.Error):
        kernels.flash_attention_tq_into(b, buf, small, buf, buf, buf, buf, buf, 256, 100, 99, 8, 1, 0, 2, 0, 1.0)
    b.commit_and_wait()


# ---- FP16-KV kernels ----
def f16_case(la, hd, n_q, n_kv, total, seed):
    q = (la.synth.normal(seed, n_q * hd) * 0.3).astype(np.float16)
    k = (la.synth.normal(seed + 1, total * n_kv * hd) * 0.3).astype(np.float16)
    v = la.synth.normal_f16((total * n_kv * hd,), seed + 2)
    return q, k, v


@pytest.mark.parametrize("hd,n_q,n_kv,total", [(256, 8, 1, 1500), (128, 4, 2, 100), (256, 8, 1, 256), (512, 2, 2, 700)])
def test_flash_decoding(la, orc, ctx, kernels, hd, n_q, n_kv, total):
    q, k, v = f16_case(la, hd, n_q, n_kv, total, 70)
    out = Guarded(la, ctx, n_q * hd * 2)
    b = la.CommandBatch.new(ctx)
    kernels.flash_decoding_into(ctx, b, la.CudaBuffer.from_slice(ctx, q), la.CudaBuffer.from_slice(ctx, k),
                                la.CudaBuffer.from_slice(ctx, v), out.view, hd, total, total - 1, n_q, n_kv)
    b.commit_and_wait()
    rel_close(out.read(np.float16), orc.attention_f16(q, k, v, hd, total, total - 1, n_q, n_kv, 0).astype(np.float32), 2e-3, "flash_decoding")


@pytest.mark.parametrize("window,total", [(512, 2000), (512, 300), (0, 900), (64, 64)])
def test_flash_attention_windowed_split(la, orc, ctx, kernels, window, total):
    hd, n_q, n_kv = 256, 8, 1
    q, k, v = f16_case(la, hd, n_q, n_kv, total, 80)
    eff = min(total, window) if window else total
    splits = kernels.flash_split_count(eff)
    assert 1 <= splits <= 16 and splits == min(16, max(1, -(-eff // 16)))
    out = Guarded(la, ctx, n_q * hd * 2)
    pm, ps, pa = (la.CudaBuffer.empty(ctx, n_q * splits * 4), la.CudaBuffer.empty(ctx, n_q * splits * 4),
                  la.CudaBuffer.empty(ctx, n_q * splits * hd * 4))
    b = la.CommandBatch.new(ctx)
    kernels.flash_attention_windowed_split_into(b, la.CudaBuffer.from_slice(ctx, q), la.CudaBuffer.from_slice(ctx, k),
                                                la.CudaBuffer.from_slice(ctx, v), out.view, pm, ps, pa, hd, total,
                                                total - 1, n_q, n_kv, window, splits)
    assert b.dispatch_count() == 2
    b.commit_and_wait()
    rel_close(out.read(np.float16), orc.attention_f16(q, k, v, hd, total, total - 1, n_q, n_kv, window).astype(np.float32), 2e-3, "windowed split")


def test_attention_sliding(la, orc, ctx, kernels):
    hd, n_q, n_kv, total, window = 256, 8, 1, 1300, 512
    q, k, v = f16_case(la, hd, n_q, n_kv, total, 90)
    out = Guarded(la, ctx, n_q * hd * 2)
    kernels.attention_sliding(ctx, la.CudaBuffer.from_slice(ctx, q), la.CudaBuffer.from_slice(ctx, k),
                              la.CudaBuffer.from_slice(ctx, v), out.view, hd, total, total - 1, window, n_q, n_kv)
    rel_close(out.read(np.float16), orc.attention_f16(q, k, v, hd, total, total - 1, n_q, n_kv, window).astype(np.float32), 2e-3, "attention_sliding")


def test_attention_is_convex_combination_at_32k(la, orc, ctx, kernels):
    """Size-independent property at the benchmark context (32768 rows, tq2): with every V row equal the output
    equals that row whatever the scores (the oracle comparison at this context is
    test_attention_at_the_benchmark_contexts)."""
    hd, n_q, n_kv, bits, total = 256, 8, 1, 2, 32768
    levels, signs = la.tq_levels(hd, bits), la.tq_signs(hd, la.TQ_SEED)
    cb = la.tq_code_bytes(hd, bits)
    kc = la.synth.splitmix64(1, total * cb // 8).view(np.uint8)
    kn = np.abs(la.synth.normal_f16((total,), 2)) + np.float16(0.5)
    one_c, one_n = orc.tq_encode(la.synth.normal(3, hd).astype(np.float32), bits, signs, levels)
    vc = np.tile(one_c, total)
    vn = np.full(total, one_n, np.float16)
    rq = (la.synth.normal(4, n_q * hd) * 0.5).astype(np.float32)
    out = Guarded(la, ctx, n_q * hd * 4)
    f = lambda a: la.CudaBuffer.from_slice(ctx, a)
    b = la.CommandBatch.new(ctx)
    kernels.flash_attention_tq_into(b, f(rq), f(kc), f(kn), f(vc), f(vn), f(levels), out.view, hd, total, total - 1,
                                    n_q, n_kv, 0, bits, 0, 0.0625)
    b.commit_and_wait()
    got = out.read(np.float32).reshape(n_q, hd)
    row = np.float32(one_n) * levels[(np.unpackbits(one_c, bitorder="little").reshape(hd, bits) * (1 << np.arange(bits))).sum(1)]
    for h in range(n_q):
        rel_close(got[h], row, 1e-3, f"constant-V head {h}")

def random_cache(la, hd, bits, rows, seed):
    """Random code bytes and norms ~ |N(0, I_hd)|: the attention kernels and the oracle consume codes and norms, so a
    parity check at benchmark sizes does not need rows that went through the encoder."""
    cb = la.tq_code_bytes(hd, bits)
    pad = (-rows * cb) % 8
    kc = la.synth.splitmix64(seed, (rows * cb + pad) // 8).view(np.uint8)[:rows * cb].copy()
    vc = la.synth.splitmix64(seed + 1, (rows * cb + pad) // 8).view(np.uint8)[:rows * cb].copy()
    kn = (np.sqrt(hd) * la.synth.uniform(seed + 2, rows, 0.8, 1.2)).astype(np.float16)
    vn = (np.sqrt(hd) * la.synth.uniform(seed + 3, rows, 0.8, 1.2)).astype(np.float16)
    return kc, kn, vc, vn


@pytest.mark.parametrize("bits,total", [(2, 4096), (2, 32768), (2, 131072), (3, 32768), (4, 32768)])
def test_attention_at_the_benchmark_contexts(la, orc, ctx, kernels, bits, total):
    """Batch 1 at the contexts of the attention benchmark configuration (4096, 32768, 131072; tq3 and tq4 at 32768),
    every output element against the oracle: the rotated-space entry point at 1e-3 and the fused f16 entry point at
    2e-3, softmax scale 1/sqrt(256)."""
    hd, n_q, n_kv = 256, 8, 1
    levels, signs = la.tq_levels(hd, bits), la.tq_signs(hd, la.TQ_SEED)
    kc, kn, vc, vn = random_cache(la, hd, bits, total, 9000 + bits)
    f = lambda a: la.CudaBuffer.from_slice(ctx, a)
    kcb, knb, vcb, vnb, lvb, sgb = f(kc), f(kn), f(vc), f(vn), f(levels), f(signs)
    q16 = la.synth.normal_f16((n_q, hd), 9100 + bits)
    rq = orc.hadamard_rotate(q16.astype(np.float32), signs, hd, n_q, True, False)
    out = Guarded(la, ctx, n_q * hd * 4)
    b = la.CommandBatch.new(ctx)
    kernels.flash_attention_tq_into(b, f(rq), kcb, knb, vcb, vnb, lvb, out.view, hd, total, total - 1, n_q, n_kv, 0, bits, 0, 0.0625)
    b.commit_and_wait()
    want = orc.flash_attention_tq(rq, kc, kn, vc, vn, levels, hd, total, total - 1, n_q, n_kv, 0, bits, 0, 0.0625)
    rel_close(out.read(np.float32), want, 1e-3, f"flash_attention_tq tq{bits} at {total}")
    fo = Guarded(la, ctx, n_q * hd * 2)
    b = la.CommandBatch.new(ctx)
    kernels.tq_attention_into(b, f(q16), kcb, knb, vcb, vnb, lvb, sgb, fo.view, hd, total, total - 1, n_q, n_kv, 0, bits, 0, 0.0625)
    b.commit_and_wait()
    wantf = orc.tq_attention_fused(q16, kc, kn, vc, vn, levels, signs, None, hd, 0, n_q, n_kv, 0, bits, 1, 0, 0.0625,
                                   total, total - 1).astype(np.float32)
    rel_close(fo.read(np.float16), wantf, 2e-3, f"tq_attention tq{bits} at {total}")


def test_attention_64_lanes_at_8193_keys_lane_by_lane(la, orc, ctx, kernels):
    """The attention launch of the batch-64 decode benchmark (64 lanes, every lane at position 8192, tq2, the split
    count the launch heuristic picks for it) with five lanes compared against the oracle element by element."""
    hd, n_q, n_kv, bits, lanes, cap, pos = 256, 8, 1, 2, 64, 8192 + 512, 8192
    levels, signs = la.tq_levels(hd, bits), la.tq_signs(hd, la.TQ_SEED)
    cb = la.tq_code_bytes(hd, bits)
    kc, kn, vc, vn = random_cache(la, hd, bits, lanes * cap, 9500)
    f = lambda a: la.CudaBuffer.from_slice(ctx, a)
    q16 = la.synth.normal_f16((lanes, n_q, hd), 9600)
    positions = np.full(lanes, pos, np.uint32)
    fo = Guarded(la, ctx, lanes * n_q * hd * 2)
    b = la.CommandBatch.new(ctx)
    kernels.tq_attention_batched_into(b, f(q16), f(kc), f(kn), f(vc), f(vn), f(levels), f(signs), fo.view, f(positions), hd,
                                      cap, n_q, n_kv, 0, bits, lanes, 0, 0.0625)
    b.commit_and_wait()
    got = fo.read(np.float16).astype(np.float32).reshape(lanes, n_q * hd)
    assert np.all(np.isfinite(got))
    for lane in (0, 1, 21, 42, 63):
        rows = slice(lane * cap, (lane + 1) * cap)
        crows = slice(lane * cap * cb, (lane + 1) * cap * cb)
        want = orc.tq_attention_fused(q16[lane], kc[crows], kn[rows], vc[crows], vn[rows], levels, signs, None, hd, 0, n_q,
                                      n_kv, 0, bits, 1, 0, 0.0625, pos + 1, pos).astype(np.float32)
        rel_close(got[lane], want, 2e-3, f"lane {lane} of 64 at 8193 keys")


@pytest.mark.gpu
def test_cluster_merge_path_equals_split_and_merge_launches(la, orc, ctx, kernels, tmp_path):
    """LOCAL_CUDA_ATTN_CLUSTER=1 (read once per process, hence the child process) lets the tensor-core kernel merge
    its splits through distributed shared memory and rotate back itself: one launch instead of two, and the same
    arithmetic in the same order as the merge kernel, so the outputs must be bit-identical."""
    import os
    import subprocess
    import sys
    script = tmp_path / "cluster_attn.py"
    script.write_text('''
import sys, numpy as np
sys.path.insert(0, %r); sys.path.insert(0, %r)
import __graft_entry__ as entry
la = entry.load_package()
ctx = la.CudaContext.new(0); k = la.Kernels.new(ctx)
hd, n_q, n_kv, bits, lanes, cap = 256, 8, 1, 2, 3, 1536
rows = lanes * cap
d = lambda a: la.CudaBuffer.from_slice(ctx, a)
kc = (la.synth.splitmix64(11, rows * 64 // 8).view(np.uint8)); vc = (la.synth.splitmix64(12, rows * 64 // 8).view(np.uint8))
kn = (16.0 * la.synth.uniform(13, rows, 0.9, 1.1)).astype(np.float16); vn = (16.0 * la.synth.uniform(14, rows, 0.9, 1.1)).astype(np.float16)
q = la.synth.normal_f16((lanes, n_q, hd), 15)
pos = np.array([1400, 700, 40], np.uint32)
out = la.CudaBuffer.empty(ctx, lanes * n_q * hd * 2)
b = la.CommandBatch.new(ctx)
k.tq_attention_batched_into(b, d(q), d(kc), d(kn), d(vc), d(vn), d(la.tq_levels(hd, bits)), d(la.tq_signs(hd, la.TQ_SEED)), out, d(pos),
                            hd, cap, n_q, n_kv, 0, bits, lanes, 0, 0.0625)
n = b.dispatch_count(); b.commit_and_wait()
np.save(sys.argv[1], out.as_slice(np.uint16, lanes * n_q * hd)); print("launches", n)
''' % (str(entry_root()), str(entry_root() / "tests")))
    outs = {}
    for flag in ("0", "1"):
        env = dict(os.environ, LOCAL_CUDA_ATTN_CLUSTER=flag)
        path = tmp_path / f"out{flag}.npy"
        r = subprocess.run([sys.executable, str(script), str(path)], env=env, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        assert f"launches {2 - int(flag)}" in r.stdout
        outs[flag] = np.load(path)
    assert np.array_equal(outs["0"], outs["1"])
    assert np.isfinite(outs["1"].view(np.float16).astype(np.float32)).all()


def entry_root():
    from pathlib import Path
    return Path(__file__).resolve().parent.parent


def test_query_buffer_at_an_odd_offset_takes_the_general_kernel(la, orc, ctx, kernels):
    """The tensor-core kernel loads the query and the signs as 16-byte vectors.  A query wrapped two bytes into an
    allocation must not reach it: the call is served by the CUDA-core kernel and still meets the oracle."""
    hd, n_q, n_kv, bits, total = 256, 8, 1, 2, 700
    c = Cache(la, orc, ctx, hd, n_kv, bits, total, seed=4242)
    c.fill_single(total, 0)
    kc, kn, vc, vn, lv, sg = c.device()
    q16 = la.synth.normal_f16((n_q, hd), 4243)
    raw = la.CudaBuffer.empty(ctx, n_q * hd * 2 + 16)
    raw.copy_from_bytes(q16.view(np.uint8).reshape(-1), offset=2)
    qv = la.CudaBuffer.wrap(ctx, raw.device_ptr + 2, n_q * hd * 2)
    fo = Guarded(la, ctx, n_q * hd * 2)
    b = la.CommandBatch.new(ctx)
    kernels.tq_attention_into(b, qv, kc, kn, vc, vn, lv, sg, fo.view, hd, total, total - 1, n_q, n_kv, 0, bits, 0, 0.0625)
    b.commit_and_wait()
    want = orc.tq_attention_fused(q16, c.kc, c.kn, c.vc, c.vn, c.levels, c.signs, None, hd, 0, n_q, n_kv, 0, bits, 1, 0,
                                  0.0625, total, total - 1).astype(np.float32)
    rel_close(fo.read(np.float16), want, 2e-3, "query at a 2-byte offset")
    # an f32 rotated query that is not even 4-byte aligned is refused with a status
    rqv = la.CudaBuffer.wrap(ctx, raw.device_ptr + 2, 16)
    b = la.CommandBatch.new(ctx)
    with pytest.raises(la.Error) as ei:
        kernels.flash_attention_tq_into(b, rqv, kc, kn, vc, vn, lv, fo.view, 64, 1, 0, 1, 1, 0, bits, 0, 1.0)
    assert ei.value.kind == "InvalidArgument"
    b.commit_and_wait()


def test_captured_graph_survives_later_scratch_growth(la, orc, ctx):
    """A captured graph keeps the split-K scratch address it was recorded with.  A later, larger eager call on the same
    kernels object makes the scratch grow; the old block must stay alive, so replaying the graph afterwards still
    gives the recorded call's result."""
    hd, n_q, n_kv, bits = 128, 4, 1, 3
    k2 = la.Kernels.new(ctx)
    small = Cache(la, orc, ctx, hd, n_kv, bits, 600, seed=611)
    small.fill_single(600, 0)
    kc, kn, vc, vn, lv, sg = small.device()
    q16 = la.synth.normal_f16((n_q, hd), 612)
    qb = la.CudaBuffer.from_slice(ctx, q16)
    out = la.CudaBuffer.empty(ctx, n_q * hd * 2)
    call = lambda b: k2.tq_attention_into(b, qb, kc, kn, vc, vn, lv, sg, out, hd, 600, 599, n_q, n_kv, 0, bits, 0, 0.125)
    b = la.CommandBatch.new(ctx)
    call(b)                      # sizes the scratch for this shape
    b.commit_and_wait()
    first = out.as_slice(np.uint16).copy()
    b = la.CommandBatch.capture(ctx)
    call(b)
    graph = b.end_capture()
    # a much larger call: 64 heads of 512 and a long context need far more partials
    big = Cache(la, orc, ctx, 512, 8, 2, 9000, seed=613)
    bkc, bkn, bvc, bvn, blv, bsg = big.device()
    bq = la.CudaBuffer.from_slice(ctx, la.synth.normal_f16((64, 512), 614))
    bout = la.CudaBuffer.empty(ctx, 64 * 512 * 2)
    b = la.CommandBatch.new(ctx)
    k2.tq_attention_into(b, bq, bkc, bkn, bvc, bvn, blv, bsg, bout, 512, 9000, 8999, 64, 8, 0, 2, 0, 1.0)
    b.commit_and_wait()
    out.zero()
    graph.launch()
    ctx.synchronize()
    assert np.array_equal(out.as_slice(np.uint16), first)
    graph.destroy()
    k2.close()
