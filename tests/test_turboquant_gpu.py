"""TurboQuant KV rows on the GPU vs the CPU oracle.  Packed codes and f16 norms
must be BIT-EXACT with the Rust codec's order (norm mode 0) — stricter than the
reference's own GPU test, which tolerates one-level flips on < 2 % of coordinates
(local-metal/src/kernels.rs:9892-9930).  Mode 1 (Metal summation order) is held
to the oracle's mode 1 the same way."""
import numpy as np
import pytest

import refgen
from gpu_util import Guarded, rel_close

pytestmark = pytest.mark.gpu


def codec(la, orc, hd, bits, seed=None):
    seed = la.TQ_SEED if seed is None else seed
    return la.tq_levels(hd, bits), la.tq_signs(hd, seed)


def gpu_encode(la, ctx, kernels, x, levels, signs, hd, n_kv, ntok, bits, position, ring, rows):
    cb = la.tq_code_bytes(hd, bits)
    packed, norms = Guarded(la, ctx, rows * n_kv * cb), Guarded(la, ctx, rows * n_kv * 2)
    packed.buf.zero(0, rows * n_kv * cb)
    norms.buf.zero(0, rows * n_kv * 2)
    kernels.encode_kv_turboquant(ctx, la.CudaBuffer.from_slice(ctx, x), la.CudaBuffer.from_slice(ctx, levels),
                                 la.CudaBuffer.from_slice(ctx, signs), packed.view, norms.view, hd, n_kv, ntok, bits,
                                 position, ring)
    return packed.read(np.uint8), norms.read(np.uint16)


def test_encode_matches_reference_test_setup(la, orc, ctx, kernels):
    """The inputs of encode_kv_turboquant_matches_cpu_reference (kernels.rs:9823-9890)."""
    hd, n_kv, ntok, bits, position = 128, 4, 3, 4, 2
    i = np.arange(hd)
    signs = np.where(((i * 2654435761) >> 13) & 1 == 0, 1.0, -1.0).astype(np.float32)
    k = 1 << bits
    levels = (((np.arange(k, dtype=np.float32) + 0.5) / np.float32(k) - 0.5) * 6.0 / np.sqrt(np.float32(hd))).astype(np.float32)
    j = np.arange(ntok * n_kv * hd, dtype=np.float32)
    x = ((np.sin(j * np.float32(0.123)) + np.cos(j * np.float32(0.017))) * np.float32(0.7)).astype(np.float16)
    rows = position + ntok
    got_c, got_n = gpu_encode(la, ctx, kernels, x, levels, signs, hd, n_kv, ntok, bits, position, 0, rows)
    cb = la.tq_code_bytes(hd, bits)
    want_c, want_n = np.zeros(rows * n_kv * cb, np.uint8), np.zeros(rows * n_kv, np.float16)
    orc.encode_kv(x, levels, signs, want_c, want_n, hd, n_kv, ntok, bits, position, 0)
    assert np.array_equal(got_c, want_c)
    assert np.array_equal(got_n, want_n.view(np.uint16))
    assert np.all(got_c[: position * n_kv * cb] == 0)  # slots before `position` untouched


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("hd", [64, 128, 256, 512])
def test_encode_bit_exact(la, orc, ctx, kernels, hd, bits, mode):
    n_kv, ntok = 2, 9
    levels, signs = codec(la, orc, hd, bits)
    x = la.synth.normal_f16((ntok, n_kv, hd), seed=hd * 10 + bits)
    x[3] = 0  # a zero row: norm 0, codes of the level nearest 0
    kernels.kernels_set_kv_norm_mode(mode)
    try:
        got_c, got_n = gpu_encode(la, ctx, kernels, x, levels, signs, hd, n_kv, ntok, bits, 0, 0, ntok)
    finally:
        kernels.kernels_set_kv_norm_mode(0)
    cb = la.tq_code_bytes(hd, bits)
    want_c, want_n = np.zeros(ntok * n_kv * cb, np.uint8), np.zeros(ntok * n_kv, np.float16)
    orc.encode_kv(x, levels, signs, want_c, want_n, hd, n_kv, ntok, bits, 0, 0, mode)
    assert np.array_equal(got_n, want_n.view(np.uint16)), "norms"
    assert np.array_equal(got_c, want_c), "codes"


def test_encode_config3_rows_bit_exact(la, orc, ctx, kernels):
    """Benchmark shape: 1 KV head, head_dim 256, tq2, 4096 rows of N(0,1)."""
    hd, n_kv, ntok, bits = 256, 1, 4096, 2
    levels, signs = codec(la, orc, hd, bits)
    x = la.synth.normal_f16((ntok, n_kv, hd), seed=31)
    got_c, got_n = gpu_encode(la, ctx, kernels, x, levels, signs, hd, n_kv, ntok, bits, 0, 0, ntok)
    want_c, want_n = np.zeros(ntok * 64, np.uint8), np.zeros(ntok, np.float16)
    orc.encode_kv(x, levels, signs, want_c, want_n, hd, n_kv, ntok, bits, 0, 0)
    assert np.array_equal(got_c, want_c) and np.array_equal(got_n, want_n.view(np.uint16))


def test_ring_write_wraps_like_full_cache(la, orc, ctx, kernels):
    """Ring rows equal the absolute cache's last `ring` rows after 2-3 wraps (quant_cache.rs:990-1107)."""
    hd, n_kv, bits, ring, total = 256, 1, 2, 16, 45
    levels, signs = codec(la, orc, hd, bits)
    cb = la.tq_code_bytes(hd, bits)
    x = la.synth.normal_f16((total, n_kv, hd), seed=5)
    lv, sg = la.CudaBuffer.from_slice(ctx, levels), la.CudaBuffer.from_slice(ctx, signs)
    full_c, full_n = la.CudaBuffer.empty(ctx, total * cb), la.CudaBuffer.empty(ctx, total * 2)
    ring_c, ring_n = Guarded(la, ctx, ring * cb), Guarded(la, ctx, ring * 2)
    for t0 in range(0, total, 5):  # multi-row writes that straddle the wrap point
        n = min(5, total - t0)
        xb = la.CudaBuffer.from_slice(ctx, x[t0:t0 + n])
        kernels.encode_kv_turboquant(ctx, xb, lv, sg, full_c, full_n, hd, n_kv, n, bits, t0, 0)
        kernels.encode_kv_turboquant(ctx, xb, lv, sg, ring_c.view, ring_n.view, hd, n_kv, n, bits, t0, ring)
    fc, rc = full_c.as_slice(np.uint8).reshape(total, cb), ring_c.read(np.uint8).reshape(ring, cb)
    fn, rn = full_n.as_slice(np.uint16), ring_n.read(np.uint16)
    for t in range(total - ring, total):
        assert np.array_equal(fc[t], rc[t % ring]) and fn[t] == rn[t % ring]


@pytest.mark.parametrize("ring", [0, 8])
def test_batched_encode_equals_single_sequence_bytewise(la, orc, ctx, kernels, ring):
    """kernels.rs:10645-10653: the per-lane pool rows are byte-identical to single-sequence encodes."""
    hd, n_kv, bits, n_lanes, cap = 256, 2, 3, 5, 32
    levels, signs = codec(la, orc, hd, bits)
    cb = la.tq_code_bytes(hd, bits)
    positions = np.array([0, 7, 13, 31, 20], np.uint32)
    x = la.synth.normal_f16((n_lanes, n_kv, hd), seed=77)
    lane_rows = cap
    pool_c, pool_n = Guarded(la, ctx, n_lanes * lane_rows * n_kv * cb), Guarded(la, ctx, n_lanes * lane_rows * n_kv * 2)
    pool_c.buf.zero(0, pool_c.nbytes)
    pool_n.buf.zero(0, pool_n.nbytes)
    b = la.CommandBatch.new(ctx)
    kernels.encode_kv_turboquant_batched_into(b, la.CudaBuffer.from_slice(ctx, x), la.CudaBuffer.from_slice(ctx, levels),
                                              la.CudaBuffer.from_slice(ctx, signs), pool_c.view, pool_n.view,
                                              la.CudaBuffer.from_slice(ctx, positions), hd, n_kv, lane_rows, bits,
                                              n_lanes, ring)
    b.commit_and_wait()
    got_c, got_n = pool_c.read(np.uint8), pool_n.read(np.uint16)
    want_c, want_n = np.zeros_like(got_c), np.zeros(got_n.size, np.float16)
    orc.encode_kv_batched(x, levels, signs, want_c, want_n, positions, hd, n_kv, lane_rows, bits, n_lanes, ring)
    assert np.array_equal(got_c, want_c) and np.array_equal(got_n, want_n.view(np.uint16))
    # each lane's row equals the single-sequence encode of the same vector
    for lane in range(n_lanes):
        one_c, one_n = np.zeros(n_kv * cb, np.uint8), np.zeros(n_kv, np.float16)
        orc.encode_kv(x[lane], levels, signs, one_c, one_n, hd, n_kv, 1, bits, 0, 0)
        ppos = int(positions[lane]) % ring if ring else int(positions[lane])
        s = (lane * lane_rows + ppos) * n_kv
        assert np.array_equal(got_c[s * cb:(s + n_kv) * cb], one_c)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_dequantize_matches_cpu_decode(la, orc, ctx, kernels, bits):
    """quant_cache.rs:789-844: GPU dequant vs CPU decode, stale (zero-norm) rows decode to exact 0."""
    hd, n_kv, ntok = 256, 2, 11
    levels, signs = codec(la, orc, hd, bits)
    cb = la.tq_code_bytes(hd, bits)
    x = la.synth.normal_f16((ntok, n_kv, hd), seed=3)
    pc, pn = np.zeros((ntok + 2) * n_kv * cb, np.uint8), np.zeros((ntok + 2) * n_kv, np.float16)
    orc.encode_kv(x, levels, signs, pc, pn, hd, n_kv, ntok, bits, 0, 0)
    total = ntok + 2  # two never-written rows at the end
    out = Guarded(la, ctx, total * n_kv * hd * 2)
    kernels.dequantize_kv_turboquant(ctx, la.CudaBuffer.from_slice(ctx, pc), la.CudaBuffer.from_slice(ctx, pn),
                                     la.CudaBuffer.from_slice(ctx, levels), la.CudaBuffer.from_slice(ctx, signs),
                                     out.view, hd, n_kv, total, bits, 0, 0)
    got = out.read(np.float16).astype(np.float32)
    want = orc.dequantize_kv(pc, pn, levels, signs, hd, n_kv, total, bits, 0, 0).astype(np.float32)
    rel_close(got, want, 1e-3, "dequantize_kv")
    assert np.all(got[ntok * n_kv * hd:] == 0.0)
    rel = np.linalg.norm(got[: ntok * n_kv * hd] - x.astype(np.float32).reshape(-1)) / np.linalg.norm(x.astype(np.float32))
    assert rel < {2: 0.40, 3: 0.22, 4: 0.12}[bits]


def test_dequantize_window_from_ring(la, orc, ctx, kernels):
    """quant_cache.rs:905-952: token_start skips rows; ring slots are read, logical slots written."""
    hd, n_kv, bits, ring, total, start = 128, 1, 4, 8, 19, 13
    levels, signs = codec(la, orc, hd, bits)
    cb = la.tq_code_bytes(hd, bits)
    x = la.synth.normal_f16((total, n_kv, hd), seed=4)
    rc, rn = np.zeros(ring * cb, np.uint8), np.zeros(ring, np.float16)
    for t in range(total):
        orc.encode_kv(x[t], levels, signs, rc, rn, hd, n_kv, 1, bits, t, ring)
    out = Guarded(la, ctx, total * hd * 2)
    out.buf.zero(0, total * hd * 2)
    b = la.CommandBatch.new(ctx)
    kernels.dequantize_kv_turboquant_into(b, la.CudaBuffer.from_slice(ctx, rc), la.CudaBuffer.from_slice(ctx, rn),
                                          la.CudaBuffer.from_slice(ctx, levels), la.CudaBuffer.from_slice(ctx, signs),
                                          out.view, hd, n_kv, total, bits, start, ring)
    b.commit_and_wait()
    got = out.read(np.float16).astype(np.float32).reshape(total, hd)
    want = orc.dequantize_kv(rc, rn, levels, signs, hd, n_kv, total, bits, start, ring).astype(np.float32).reshape(total, hd)
    assert np.all(got[:start] == 0.0)
    rel_close(got[start:], want[start:], 1e-3, "windowed dequant")


@pytest.mark.parametrize("variant", ["ff", "hf", "fh"])
@pytest.mark.parametrize("hd", [64, 256, 512])
def test_hadamard_rotate(la, orc, ctx, kernels, hd, variant):
    heads = 5
    signs = la.tq_signs(hd, 11)
    x32 = (refgen.seeded_vec(heads * hd, 13) * 4).astype(np.float32)
    if variant == "hf":
        x_in = x32.astype(np.float16)
        x32 = x_in.astype(np.float32)
    else:
        x_in = x32
    for pre, post in ((1, 0), (0, 1), (1, 1)):
        out = Guarded(la, ctx, heads * hd * (2 if variant == "fh" else 4))
        b = la.CommandBatch.new(ctx)
        fn = {"ff": kernels.hadamard_rotate_into, "hf": kernels.hadamard_rotate_hf_into, "fh": kernels.hadamard_rotate_fh_into}[variant]
        fn(b, la.CudaBuffer.from_slice(ctx, x_in), la.CudaBuffer.from_slice(ctx, signs), out.view, hd, heads, pre, post)
        b.commit_and_wait()
        got = out.read(np.float16 if variant == "fh" else np.float32).astype(np.float32)
        want = orc.hadamard_rotate(x32, signs, hd, heads, bool(pre), bool(post))
        rel_close(got, want, 1e-3 if variant == "fh" else 1e-5, f"hadamard_rotate_{variant} pre={pre} post={post}")


def test_encode_decode_round_trip_at_scale(la, orc, ctx, kernels):
    """Size-independent property at pool scale: encode -> dequantize recovers each row's norm and direction."""
    hd, n_kv, ntok, bits = 256, 1, 8192, 2
    levels, signs = codec(la, orc, hd, bits)
    x = la.synth.normal_f16((ntok, n_kv, hd), seed=99)
    lv, sg = la.CudaBuffer.from_slice(ctx, levels), la.CudaBuffer.from_slice(ctx, signs)
    pc, pn = la.CudaBuffer.empty(ctx, ntok * 64), la.CudaBuffer.empty(ctx, ntok * 2)
    out = la.CudaBuffer.empty(ctx, ntok * hd * 2)
    kernels.encode_kv_turboquant(ctx, la.CudaBuffer.from_slice(ctx, x), lv, sg, pc, pn, hd, n_kv, ntok, bits, 0, 0)
    kernels.dequantize_kv_turboquant(ctx, pc, pn, lv, sg, out, hd, n_kv, ntok, bits, 0, 0)
    xh = out.as_slice(np.float16).astype(np.float32).reshape(ntok, hd)
    xf = x.astype(np.float32).reshape(ntok, hd)
    norms = pn.as_slice(np.float16).astype(np.float32)
    assert np.allclose(norms, np.linalg.norm(xf, axis=1), rtol=2e-3)
    cos = np.sum(xh * xf, axis=1) / (np.linalg.norm(xh, axis=1) * np.linalg.norm(xf, axis=1))
    assert cos.min() > 0.90 and cos.mean() > 0.93


def test_device_position_past_the_lane_rows_is_skipped_and_reported(la, orc, ctx):
    """Positions of the per-lane entry points live in a device buffer the host cannot check.  A lane whose position lies
    past its pool rows (no ring) must not be written -- its neighbours' rows and the guard band stay untouched -- the
    other lanes are encoded as usual, attention over that lane is clamped to the rows that exist, and the kernels
    object's status word reports it as InvalidArgument."""
    import ctypes as C
    hd, n_kv, bits, cap, n_lanes = 256, 1, 2, 8, 3
    k2 = la.Kernels.new(ctx)
    levels, signs = codec(la, orc, hd, bits)
    cb = la.tq_code_bytes(hd, bits)
    x = la.synth.normal_f16((n_lanes, n_kv, hd), seed=77)
    positions = np.array([3, 8 + 5, 7], np.uint32)          # lane 1 points 6 rows past its 8
    rows = n_lanes * cap
    packed, norms = Guarded(la, ctx, rows * cb), Guarded(la, ctx, rows * 2)
    packed.buf.zero(0, rows * cb)
    norms.buf.zero(0, rows * 2)
    d = lambda a: la.CudaBuffer.from_slice(ctx, a)
    lv, sg, pb = d(levels), d(signs), d(positions)
    b = la.CommandBatch.new(ctx)
    k2.encode_kv_turboquant_batched_into(b, d(x), lv, sg, packed.view, norms.view, pb, hd, n_kv, cap, bits, n_lanes, 0)
    b.commit_and_wait()
    got_c, got_n = packed.read(np.uint8).reshape(rows, cb), norms.read(np.uint16)
    want_c, want_n = np.zeros(rows * cb, np.uint8), np.zeros(rows, np.float16)
    ok = np.array([3, 0, 7], np.uint32)                       # the oracle encodes lanes 0 and 2 only
    orc.encode_kv_batched(x, levels, signs, want_c, want_n, ok, hd, n_kv, cap, bits, n_lanes, 0)
    want_c = want_c.reshape(rows, cb)
    want_c[cap + 0] = 0
    want_n[cap + 0] = 0
    assert np.array_equal(got_c, want_c) and np.array_equal(got_n, want_n.view(np.uint16))
    # attention with the same positions: finite output, lane 1 clamped to its 8 rows (all zero norms here)
    q = la.synth.normal_f16((n_lanes, 8, hd), seed=78)
    out = Guarded(la, ctx, n_lanes * 8 * hd * 2)
    b = la.CommandBatch.new(ctx)
    k2.tq_attention_batched_into(b, d(q), packed.view, norms.view, packed.view, norms.view, lv, sg, out.view, pb, hd, cap,
                                 8, n_kv, 0, bits, n_lanes, 0, 0.0625)
    b.commit_and_wait()
    assert np.all(np.isfinite(out.read(np.float16).astype(np.float32)))
    st = C.c_int(0)
    with pytest.raises(la.Error) as ei:
        k2.kernels_device_status(C.addressof(st))
    assert ei.value.kind == "InvalidArgument" and st.value == 3
    k2.close()
