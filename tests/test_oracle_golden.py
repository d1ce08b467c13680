"""Pin the CPU oracle against every known-answer test the reference holds for
the hot path, and cross-check its C block decoding against an independent
numpy restatement of the reference's test payload builders.  No GPU needed."""
import numpy as np
import pytest

import refgen


def f16_bytes(v):
    return np.array([v], dtype=np.float16).view(np.uint8)


# ---- block layouts: local-engine/src/qat_recover.rs:199-313 ----
def test_dequant_tq2_0_matches_ggml_layout(orc):
    qs = np.zeros(64, dtype=np.uint8)
    qs[0] = 0b0001_1011  # l0=3, l1=2, l2=1, l3=0
    buf = np.concatenate([qs, f16_bytes(2.0)])
    out = orc.dequant(orc.TQ2_0, buf, 256).astype(np.float32)
    assert out.size == 256
    assert out[0] == 4.0 and out[32] == 2.0 and out[64] == 0.0 and out[96] == -2.0
    assert out[1] == -2.0  # qs[1] = 0 -> q = 0 everywhere -> d * (0 - 1)


def test_dequant_tq2_0_truncates_to_num_elements(orc):
    buf = np.concatenate([np.zeros(64, np.uint8), f16_bytes(1.0)])
    assert orc.dequant(orc.TQ2_0, buf, 10).size == 10


def test_dequant_q4_0_split_nibble_layout(orc):
    # local-engine/src/pipeline/init_gemma4_qat.rs:241-265
    def block(d, nibbles):
        b = np.empty(18, np.uint8)
        b[:2] = f16_bytes(d)
        n = np.asarray(nibbles, dtype=np.uint8)
        b[2:] = (n[:16] & 15) | (n[16:] << 4)
        return b

    nib1 = np.full(32, 8, np.uint8)
    nib1[0], nib1[1] = 15, 0
    raw = np.concatenate([block(2.0, np.full(32, 8)), block(0.5, nib1)])
    out = orc.dequant(orc.Q4_0, raw, 64).astype(np.float32)
    assert np.all(out[:32] == 0.0)
    assert out[32] == 3.5 and out[33] == -4.0
    # high nibble goes to the second half of the block
    nib2 = np.full(32, 8, np.uint8)
    nib2[16] = 15
    assert orc.dequant(orc.Q4_0, block(1.0, nib2), 32).astype(np.float32)[16] == 7.0


def test_block_byte_sizes(orc):
    # local-engine/src/gguf.rs:516-530: 66 bytes / 256 weights, 18 bytes / 32 weights
    assert orc.row_bytes(orc.TQ2_0, 256) == 66 and orc.row_bytes(orc.TQ2_0, 1536) == 396
    assert orc.row_bytes(orc.Q4_0, 32) == 18 and orc.row_bytes(orc.Q4_0, 1536) == 864


@pytest.mark.parametrize("fmt,rows,cols,seed", [("q4", 5, 96, 0xBEEF), ("tq2", 5, 512, 0xC0DE), ("tq2", 7, 768, 0xFACE)])
def test_c_expansion_matches_reference_payload_builders(orc, fmt, rows, cols, seed):
    """The C block decode and the numpy restatement of kernels.rs:8790-8840 agree bit for bit."""
    if fmt == "q4":
        raw, dq = refgen.q4_0_payload(rows, cols, seed)
        got = orc.expand_f32(orc.Q4_0, raw, rows, cols)
    else:
        raw, dq = refgen.tq2_0_payload(rows, cols, seed)
        got = orc.expand_f32(orc.TQ2_0, raw, rows, cols)
    assert np.array_equal(got, dq)
    v = refgen.test_vector(cols)
    want = refgen.cpu_matvec(dq, v.astype(np.float32))
    mv = orc.matvec(orc.Q4_0 if fmt == "q4" else orc.TQ2_0, raw, v, rows, cols)
    refgen.assert_close(mv, want, 1e-6, "oracle matvec vs cpu_matvec")


def test_baseline_matmul_follows_qat_recover_rounding(orc):
    raw, dq = refgen.q4_0_payload(9, 64, 0x51A7)
    a = refgen.sin_matrix(3, 64, 0.013, 0.7)
    base = orc.baseline_matmul_nt(orc.Q4_0, a, raw, 3, 64, 9, threads=2)
    w16 = orc.dequant(orc.Q4_0, raw, 9 * 64).astype(np.float32).reshape(9, 64)
    want = a.astype(np.float32) @ w16.T
    refgen.assert_close(base, want, 1e-5, "baseline matmul")


def test_tq2_dequant_utility(orc):
    # shaders/tq2_dequant.metal:4-16: no zero point, one scale per byte
    packed = np.array([0b11100100, 0b00011011], np.uint8)
    scales = np.array([0.5, 2.0], np.float16)
    out = orc.tq2_dequant(packed, scales, 8).astype(np.float32)
    assert out.tolist() == [0.0, 0.5, 1.0, 1.5, 6.0, 4.0, 2.0, 0.0]


# ---- codec: local-engine/src/turboquant.rs:357-472 ----
def test_fwht_is_orthonormal_involution(orc):
    v = np.array([1.0, -2.0, 3.0, 0.5, -1.0, 2.0, -0.5, 4.0], np.float32)
    w = orc.fwht_normalized(v)
    assert abs(np.linalg.norm(v) - np.linalg.norm(w)) < 1e-4
    assert np.all(np.abs(orc.fwht_normalized(w) - v) < 1e-4)


def test_rotation_inverse_recovers_input(orc):
    signs = orc.tq_signs(256, 42)
    x = refgen.seeded_vec(256, 7)
    y = orc.hadamard_rotate(x, signs, 256, 1, True, False)
    z = orc.hadamard_rotate(y, signs, 256, 1, False, True)
    assert np.all(np.abs(z - x) < 1e-3)


def test_signs_follow_splitmix64(orc):
    # turboquant.rs:66-80, restated in Python integers
    M = 0xFFFFFFFFFFFFFFFF
    for seed in (0, 7, 0x7459C0DE):
        state = seed | 1
        want = []
        for _ in range(64):
            state = (state + 0x9E3779B97F4A7C15) & M
            z = state
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
            z ^= z >> 31
            want.append(1.0 if z & 1 == 0 else -1.0)
        assert orc.tq_signs(64, seed).tolist() == want


def test_lloyd_max_levels_symmetric_increasing(orc):
    for bits in (2, 3, 4):
        l = orc.lloyd_max_gaussian(bits)
        assert l.size == 1 << bits
        assert np.all(np.diff(l) > 0)
        assert np.all(np.abs(l + l[::-1]) < 0.05)
    # the 2-bit Lloyd-Max quantiser of N(0,1) is the textbook (+-0.4528, +-1.510)
    l2 = orc.lloyd_max_gaussian(2)
    assert np.allclose(l2, [-1.510, -0.4528, 0.4528, 1.510], atol=2e-3)


def test_encode_decode_low_relative_error_at_4bit(orc):
    dim = 256
    signs, levels = orc.tq_signs(dim, 123), orc.tq_levels(dim, 4)
    x = refgen.seeded_vec(dim, 99)
    codes, norm = orc.tq_encode(x, 4, signs, levels)
    assert codes.size == orc.tq_code_bytes(dim, 4)
    xh = orc.tq_decode(codes, norm, dim, 4, signs, levels)
    assert np.sqrt(np.sum((x - xh) ** 2) / np.sum(x * x)) < 0.10


def test_encode_zero_vector(orc):
    dim = 128
    signs, levels = orc.tq_signs(dim, 3), orc.tq_levels(dim, 4)
    codes, norm = orc.tq_encode(np.zeros(dim, np.float32), 4, signs, levels)
    assert float(norm) == 0.0
    # every coordinate is 0 -> the level nearest 0 (lowest index on a tie), in both nibbles
    c = int(np.argmin(np.abs(levels)))
    assert c in (7, 8) and np.all(codes == (c | (c << 4)))
    assert np.all(orc.tq_decode(codes, norm, dim, 4, signs, levels) == 0.0)


def test_inner_product_preserved(orc):
    dim = 256
    signs, levels = orc.tq_signs(dim, 5), orc.tq_levels(dim, 4)
    k, q = refgen.seeded_vec(dim, 1), refgen.seeded_vec(dim, 2)
    codes, norm = orc.tq_encode(k, 4, signs, levels)
    kh = orc.tq_decode(codes, norm, dim, 4, signs, levels)
    exact, approx = float(q @ k), float(q @ kh)
    assert abs(exact - approx) / max(abs(exact), 1e-3) < 0.15


def test_code_bytes_match_bitwidth(orc):
    assert [orc.tq_code_bytes(256, b) for b in (4, 3, 2)] == [128, 96, 64]


def test_swa_ring_capacity(orc):
    # local-engine/src/kv_cache/quant_cache.rs:965-974
    assert orc.swa_ring_capacity(512, 131072) == 1024
    assert orc.swa_ring_capacity(512, 600) == 600


def np_cpu_tq_encode(x, signs, levels, bits):
    """local-metal/src/kernels.rs:9784-9822 in numpy f32 (sequential norm sum)."""
    x = x.astype(np.float32)
    s = np.float32(0.0)
    for v in x:
        s = np.float32(s + np.float32(v * v))
    norm = np.float32(np.sqrt(s))
    inv = np.float32(1.0) / norm if norm > 0 else np.float32(0.0)
    rot = ((x * inv).astype(np.float32) * signs).astype(np.float32)
    n, ln = rot.size, 1
    while ln < n:
        r = rot.reshape(-1, 2, ln)
        a, b = r[:, 0, :].copy(), r[:, 1, :].copy()
        r[:, 0, :], r[:, 1, :] = a + b, a - b
        ln <<= 1
    y = (rot * (np.float32(1.0) / np.sqrt(np.float32(n)))).astype(np.float32)
    d = np.abs(y[:, None] - levels[None, :].astype(np.float32))
    codes = np.argmin(d, axis=1).astype(np.uint32)  # first minimum == strict '<' scan
    bitstream = ((codes[:, None] >> np.arange(bits, dtype=np.uint32)[None, :]) & 1).astype(np.uint8).reshape(-1)
    return np.packbits(bitstream, bitorder="little"), norm


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_oracle_encode_matches_kernel_test_checker(orc, bits):
    """oracle (C) == numpy restatement of the reference's cpu_tq_encode, on that test's inputs."""
    hd, rows = 128, 12
    i = np.arange(hd)
    signs = np.where(((i * 2654435761) >> 13) & 1 == 0, 1.0, -1.0).astype(np.float32)
    k = 1 << bits
    levels = (((np.arange(k, dtype=np.float32) + 0.5) / np.float32(k) - 0.5) * 6.0 / np.sqrt(np.float32(hd))).astype(np.float32)
    j = np.arange(rows * hd, dtype=np.float32)
    inp = ((np.sin(j * np.float32(0.123)) + np.cos(j * np.float32(0.017))) * np.float32(0.7)).astype(np.float16)
    for r in range(rows):
        x = inp[r * hd:(r + 1) * hd].astype(np.float32)
        want_codes, want_norm = np_cpu_tq_encode(x, signs, levels, bits)
        codes, norm = orc.tq_encode(x, bits, signs, levels, 0)
        assert np.array_equal(codes, want_codes)
        assert norm == np.float16(want_norm)


def test_ring_encode_equals_full_cache_rows(orc):
    """Ring vs absolute storage hold identical rows after wraps (quant_cache.rs:990-1107)."""
    hd, n_kv, bits, ring, total = 64, 2, 3, 8, 21
    signs, levels = orc.tq_signs(hd, 9), orc.tq_levels(hd, bits)
    cb = orc.tq_code_bytes(hd, bits)
    x = refgen.seeded_vec(total * n_kv * hd, 5).astype(np.float16).reshape(total, n_kv, hd)
    full_c, full_n = np.zeros(total * n_kv * cb, np.uint8), np.zeros(total * n_kv, np.float16)
    ring_c, ring_n = np.zeros(ring * n_kv * cb, np.uint8), np.zeros(ring * n_kv, np.float16)
    for t in range(total):
        orc.encode_kv(x[t], levels, signs, full_c, full_n, hd, n_kv, 1, bits, t, 0)
        orc.encode_kv(x[t], levels, signs, ring_c, ring_n, hd, n_kv, 1, bits, t, ring)
    fc, rc = full_c.reshape(total, n_kv * cb), ring_c.reshape(ring, n_kv * cb)
    for t in range(total - ring, total):
        assert np.array_equal(fc[t], rc[t % ring])
    # and windowed attention over either store is identical
    q = refgen.seeded_vec(4 * hd, 77)
    a = orc.flash_attention_tq(q, full_c, full_n, full_c, full_n, levels, hd, total, total - 1, 4, n_kv, ring, bits, 0)
    b = orc.flash_attention_tq(q, ring_c, ring_n, ring_c, ring_n, levels, hd, total, total - 1, 4, n_kv, ring, bits, ring)
    assert np.array_equal(a, b)


def test_attention_over_codes_equals_dequant_then_softmax(orc):
    """fused code-space attention == decode rows + plain softmax attention (kernels.rs:9936-10114)."""
    hd, n_q, n_kv, bits, ctx = 64, 4, 2, 4, 37
    signs, levels = orc.tq_signs(hd, 1), orc.tq_levels(hd, bits)
    cb = orc.tq_code_bytes(hd, bits)
    kf = refgen.seeded_vec(ctx * n_kv * hd, 3).astype(np.float16)
    vf = refgen.seeded_vec(ctx * n_kv * hd, 4).astype(np.float16)
    kc, kn = np.zeros(ctx * n_kv * cb, np.uint8), np.zeros(ctx * n_kv, np.float16)
    vc, vn = kc.copy(), kn.copy()
    orc.encode_kv(kf, levels, signs, kc, kn, hd, n_kv, ctx, bits, 0, 0)
    orc.encode_kv(vf, levels, signs, vc, vn, hd, n_kv, ctx, bits, 0, 0)
    q = (refgen.seeded_vec(n_q * hd, 8) * 4).astype(np.float16)
    fused = orc.tq_attention_fused(q, kc, kn, vc, vn, levels, signs, None, hd, 0, n_q, n_kv, 0, bits, 1, 0, 1.0, ctx, ctx - 1)
    kd = orc.dequantize_kv(kc, kn, levels, signs, hd, n_kv, ctx, bits, 0, 0)
    vd = orc.dequantize_kv(vc, vn, levels, signs, hd, n_kv, ctx, bits, 0, 0)
    plain = orc.attention_f16(q, kd, vd, hd, ctx, ctx - 1, n_q, n_kv, 0)
    ref = plain.astype(np.float32)
    assert np.max(np.abs(fused.astype(np.float32) - ref)) <= 0.02 * max(np.max(np.abs(ref)), 1e-3)
