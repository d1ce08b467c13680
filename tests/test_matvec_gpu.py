"""Fused-dequant matvec / small-M matmul parity: CUDA path through the C ABI vs
the CPU oracle, on the reference tests' own generators and shapes
(local-metal/src/kernels.rs:9233-9760) and on the benchmark configurations.
Tolerance: 1e-3 * max(|want|, 1) — fp32 accumulate, one f16 rounding on store."""
import numpy as np
import pytest

import refgen
from gpu_util import Guarded, rel_close

pytestmark = pytest.mark.gpu
TOL = 1e-3


def run_matvec(la, ctx, kernels, name, raw, v, rows, cols, f32out, into):
    m, x = la.CudaBuffer.from_slice(ctx, raw), la.CudaBuffer.from_slice(ctx, v)
    out = Guarded(la, ctx, rows * (4 if f32out else 2))
    if into:
        b = la.CommandBatch.new(ctx)
        getattr(kernels, name + "_into")(b, m, x, out.view, rows, cols)
        assert b.dispatch_count() == 1
        b.commit_and_wait()
    else:
        getattr(kernels, name)(ctx, m, x, out.view, rows, cols)
    return out.read(np.float32 if f32out else np.float16).astype(np.float32)


@pytest.mark.parametrize("into", [False, True])
@pytest.mark.parametrize("f32out", [False, True])
@pytest.mark.parametrize("rows,cols", [(5, 96), (33, 1536), (100, 6144), (1, 32)])
def test_matvec_q4_0_matches_cpu_reference(la, orc, ctx, kernels, rows, cols, f32out, into):
    raw, dq = refgen.q4_0_payload(rows, cols, 0xBEEF)
    v = refgen.test_vector(cols)
    got = run_matvec(la, ctx, kernels, "matvec_q4_0" + ("_f32out" if f32out else ""), raw, v, rows, cols, f32out, into)
    rel_close(got, orc.matvec(orc.Q4_0, raw, v, rows, cols), TOL, "matvec_q4_0")
    refgen.assert_close(got, refgen.cpu_matvec(dq, v.astype(np.float32)), 0.01 if f32out else 0.02, "vs kernels.rs tolerance")


@pytest.mark.parametrize("into", [False, True])
@pytest.mark.parametrize("f32out", [False, True])
@pytest.mark.parametrize("rows,cols", [(5, 512), (7, 256), (37, 1536), (100, 6144), (13, 2048)])
def test_matvec_tq2_0_matches_cpu_reference(la, orc, ctx, kernels, rows, cols, f32out, into):
    raw, dq = refgen.tq2_0_payload(rows, cols, 0xC0DE)
    v = refgen.test_vector(cols)
    got = run_matvec(la, ctx, kernels, "matvec_tq2_0" + ("_f32out" if f32out else ""), raw, v, rows, cols, f32out, into)
    rel_close(got, orc.matvec(orc.TQ2_0, raw, v, rows, cols), TOL, "matvec_tq2_0")
    refgen.assert_close(got, refgen.cpu_matvec(dq, v.astype(np.float32)), 0.01 if f32out else 0.02, "vs kernels.rs tolerance")


def test_matvec_tq2_0_soa_matches_cpu_reference(la, orc, ctx, kernels):
    rows, cols = 37, 1536
    raw, _ = refgen.tq2_0_payload(rows, cols, 0x50A)
    qs, scales = refgen.tq2_0_repack_soa(raw, rows, cols)
    v = refgen.test_vector(cols)
    out = Guarded(la, ctx, rows * 2)
    b = la.CommandBatch.new(ctx)
    kernels.matvec_tq2_0_soa_into(b, la.CudaBuffer.from_slice(ctx, qs), la.CudaBuffer.from_slice(ctx, scales),
                                  la.CudaBuffer.from_slice(ctx, v), out.view, rows, cols)
    b.commit_and_wait()
    rel_close(out.read(np.float16), orc.matvec(orc.TQ2_0, raw, v, rows, cols), TOL, "matvec_tq2_0_soa")


def test_config1_q4_0_6144x1536(la, orc, ctx, kernels):
    rows, cols = 6144, 1536
    w = la.synth.q4_0_weights(rows, cols, seed=101)
    x = la.synth.normal_f16((cols,), seed=102)
    got = run_matvec(la, ctx, kernels, "matvec_q4_0", w, x, rows, cols, False, True)
    rel_close(got, orc.matvec(orc.Q4_0, w, x, rows, cols), TOL, "config 1")


def test_config2_tq2_0_8192x1536_m1(la, orc, ctx, kernels):
    rows, cols = 8192, 1536
    w = la.synth.tq2_0_weights(rows, cols, seed=201)
    x = la.synth.normal_f16((cols,), seed=202)
    got = run_matvec(la, ctx, kernels, "matvec_tq2_0", w, x, rows, cols, False, True)
    rel_close(got, orc.matvec(orc.TQ2_0, w, x, rows, cols), TOL, "config 2, M=1")


def run_matmul(la, ctx, kernels, name, a, raw, m, k, n, f32out=False):
    out = Guarded(la, ctx, m * n * (4 if f32out else 2))
    b = la.CommandBatch.new(ctx)
    getattr(kernels, name)(b, la.CudaBuffer.from_slice(ctx, a), la.CudaBuffer.from_slice(ctx, raw), out.view, m, k, n)
    b.commit_and_wait()
    return out.read(np.float32 if f32out else np.float16).astype(np.float32).reshape(m, n)


@pytest.mark.parametrize("k,n", [(1536, 6144), (6144, 1536), (1536, 100)])
def test_matmul_nt_q4_0_small_m(la, orc, ctx, kernels, k, n):
    """kernels.rs:9429-9461: M = 1..8, gate/up-like, down-like and ragged N."""
    raw, _ = refgen.q4_0_payload(n, k, (0x5A1D + n) & 0xFFFFFFFF)
    for m in range(1, 9):
        a = refgen.sin_matrix(m, k, 0.011, 0.6)
        got = run_matmul(la, ctx, kernels, "matmul_nt_q4_0_into", a, raw, m, k, n)
        rel_close(got, orc.matmul_nt(orc.Q4_0, a, raw, m, k, n), TOL, f"matmul_nt_q4_0 m={m}")


@pytest.mark.parametrize("k,n", [(1536, 6144), (6144, 1536), (1536, 100), (256, 37)])
def test_matmul_nt_tq2_0_small_m(la, orc, ctx, kernels, k, n):
    """kernels.rs:9468-9533."""
    raw, _ = refgen.tq2_0_payload(n, k, (0x2B19 + n) & 0xFFFFFFFF)
    for m in range(1, 9):
        a = refgen.sin_matrix(m, k, 0.017, 0.6, np.cos)
        got = run_matmul(la, ctx, kernels, "matmul_nt_tq2_0_into", a, raw, m, k, n)
        rel_close(got, orc.matmul_nt(orc.TQ2_0, a, raw, m, k, n), TOL, f"matmul_nt_tq2_0 m={m}")


@pytest.mark.parametrize("m", [1, 3, 16])
def test_multivec_nt(la, orc, ctx, kernels, m):
    """kernels.rs:9652-9698: M <= 16, N = 33 (not a multiple of any tile)."""
    k, n = 512, 33
    a = refgen.sin_matrix(m, k, 0.013, 0.7)
    raw, _ = refgen.q4_0_payload(n, k, 0x77)
    rel_close(run_matmul(la, ctx, kernels, "multivec_nt_q4_0_into", a, raw, m, k, n),
              orc.matmul_nt(orc.Q4_0, a, raw, m, k, n), TOL, "multivec_nt_q4_0")
    raw, _ = refgen.tq2_0_payload(n, k, 0x78)
    rel_close(run_matmul(la, ctx, kernels, "multivec_nt_tq2_0_into", a, raw, m, k, n),
              orc.matmul_nt(orc.TQ2_0, a, raw, m, k, n), TOL, "multivec_nt_tq2_0")


def test_multivec_rejects_m_out_of_range(la, ctx, kernels):
    k, n = 256, 8
    raw, _ = refgen.tq2_0_payload(n, k, 1)
    a = la.CudaBuffer.from_slice(ctx, np.zeros((17, k), np.float16))
    out = la.CudaBuffer.empty(ctx, 17 * n * 2)
    b = la.CommandBatch.new(ctx)
    with pytest.raises(la.Error) as ei:
        kernels.multivec_nt_tq2_0_into(b, a, la.CudaBuffer.from_slice(ctx, raw), out, 17, k, n)
    assert ei.value.kind == "InvalidArgument"
    b.commit_and_wait()


def test_quant_kernels_reject_misaligned_cols(la, ctx, kernels):
    """kernels.rs:9752-9760."""
    buf = la.CudaBuffer.empty(ctx, 4096)
    with pytest.raises(la.Error) as ei:
        kernels.matvec_q4_0(ctx, buf, buf, buf, 4, 33)
    assert ei.value.kind == "InvalidArgument" and "not /32" in str(ei.value)
    with pytest.raises(la.Error) as ei:
        kernels.matvec_tq2_0(ctx, buf, buf, buf, 4, 128)
    assert ei.value.kind == "InvalidArgument" and "not /256" in str(ei.value)


def test_short_buffers_are_rejected(la, ctx, kernels):
    small, big = la.CudaBuffer.empty(ctx, 64), la.CudaBuffer.empty(ctx, 1 << 16)
    with pytest.raises(la.Error):
        kernels.matvec_q4_0(ctx, small, big, big, 64, 1536)   # weights too small
    with pytest.raises(la.Error):
        kernels.matvec_q4_0(ctx, big, big, small, 64, 32)     # output too small


def test_tq2_dequant(la, orc, ctx, kernels):
    n = 4 * 1000 + 2
    packed = refgen.xorshift_bytes(5, (n + 3) // 4)
    scales = (refgen.seeded_vec((n + 3) // 4, 3) + 1.0).astype(np.float16)
    out = Guarded(la, ctx, n * 2)
    kernels.tq2_dequant(ctx, la.CudaBuffer.from_slice(ctx, packed), la.CudaBuffer.from_slice(ctx, scales), out.view, n)
    assert np.array_equal(out.read(np.uint16), orc.tq2_dequant(packed, scales, n).view(np.uint16))


def test_matvec_is_linear_at_full_size(la, ctx, kernels):
    """Size-independent property at the benchmark shape: W(a + b) = Wa + Wb up to rounding."""
    rows, cols = 8192, 1536
    w = la.synth.tq2_0_weights(rows, cols, seed=7)
    a = la.synth.normal_f16((cols,), 8, 0.25)
    b = la.synth.normal_f16((cols,), 9, 0.25)
    ab = (a.astype(np.float32) + b.astype(np.float32)).astype(np.float16)
    exact = np.flatnonzero(ab.astype(np.float32) == a.astype(np.float32) + b.astype(np.float32))
    a, b, ab = [np.where(np.isin(np.arange(cols), exact), v, 0).astype(np.float16) for v in (a, b, ab)]
    ya = run_matvec(la, ctx, kernels, "matvec_tq2_0_f32out", w, a, rows, cols, True, True)
    yb = run_matvec(la, ctx, kernels, "matvec_tq2_0_f32out", w, b, rows, cols, True, True)
    yab = run_matvec(la, ctx, kernels, "matvec_tq2_0_f32out", w, ab, rows, cols, True, True)
    rel_close(yab, ya + yb, 1e-4, "linearity")


# ---- tensor-core paths: m > 8.  Up to m = 64: the lean tcgen05 decode kernel (TQ2_0, f16 out) or the register-direct
# mma.sync kernel; above, or with both switched off, the large-tile tcgen05 kernel ----
@pytest.fixture(params=["default", "mma_sync", "tcgen05_large"])
def tc_kernels(request, la, ctx, kernels, monkeypatch):
    """The session's kernels object, one created with LOCAL_CUDA_DECODE_TC=0 (mma.sync kernel for 8 < m <= 64), or
    one with LOCAL_CUDA_DECODE_MMA=0 as well (large-tile tcgen05 kernel for every m > 8)."""
    if request.param == "default":
        kernels.decode_mma = True
        yield kernels
        return
    monkeypatch.setenv("LOCAL_CUDA_DECODE_TC", "0")
    if request.param == "tcgen05_large":
        monkeypatch.setenv("LOCAL_CUDA_DECODE_MMA", "0")
    k2 = la.Kernels.new(ctx)
    k2.decode_mma = request.param == "mma_sync"
    yield k2
    k2.close()


TC_TOL_TQ2 = 1e-3   # TQ2_0 operands are exact in f16
TC_TOL_Q4 = 1e-3    # vs the f32-weight oracle: Q4_0 keeps exact weights on every tensor-core path (integer operands with
                    # a per-block f32 scale, or rounded weights plus the rounding remainder)


def device_status_ok(kernels):
    import ctypes as C
    st = C.c_int(0)
    kernels.kernels_device_status(C.addressof(st))
    assert st.value == 0


@pytest.mark.parametrize("m,k,n", [(70, 256, 96), (70, 512, 128), (16, 1536, 8192), (64, 1536, 8192), (64, 6144, 1536),
                                   (200, 512, 64), (9, 256, 1), (33, 2048, 1536), (17, 768, 130), (64, 1536, 2560),
                                   (40, 1536, 12288), (64, 256, 31)])
def test_matmul_nt_tq2_0_tensor_core(la, orc, ctx, tc_kernels, m, k, n):
    kernels = tc_kernels
    """kernels.rs:9551-9600 (m = 70 spans tiles) plus the benchmark shapes (config 2 at M = 16 and 64)."""
    raw, _ = refgen.tq2_0_payload(n, k, 0x2B19) if n * k <= 1 << 20 else (la.synth.tq2_0_weights(n, k, 5, ncodes=4), None)
    a = refgen.sin_matrix(m, k, 0.017, 0.6, np.cos) if n * k <= 1 << 20 else la.synth.normal_f16((m, k), 6)
    got = run_matmul(la, ctx, kernels, "matmul_nt_tq2_0_into", a, raw, m, k, n)
    rel_close(got, orc.matmul_nt(orc.TQ2_0, a, raw, m, k, n), TC_TOL_TQ2, f"tcgen05 tq2_0 m={m} k={k} n={n}")
    device_status_ok(kernels)


@pytest.mark.parametrize("m,k,n", [(70, 256, 128), (70, 64, 96), (16, 1536, 300), (64, 1536, 6144), (64, 768, 129),
                                   (130, 128, 256), (33, 96, 40), (9, 32, 7)])
def test_matmul_nt_q4_0_tensor_core(la, orc, ctx, tc_kernels, m, k, n):
    kernels = tc_kernels
    raw, _ = refgen.q4_0_payload(n, k, 0x51A7) if n * k <= 1 << 20 else (la.synth.q4_0_weights(n, k, 7), None)
    a = refgen.sin_matrix(m, k, 0.013, 0.7) if n * k <= 1 << 20 else la.synth.normal_f16((m, k), 8)
    """The reference's M > 8 kernel multiplies with f32 weights d (q - 8) (matvec_quant.metal:477-506), and so does its
    per-lane vocabulary projection (pipeline/batched.rs:427-447): every path must meet the f32-weight oracle at 1e-3."""
    want32 = orc.matmul_nt(orc.Q4_0, a, raw, m, k, n)
    got = run_matmul(la, ctx, kernels, "matmul_nt_q4_0_into", a, raw, m, k, n)
    rel_close(got, want32, TC_TOL_Q4, f"tensor-core q4_0 m={m} k={k} n={n}")
    got32 = run_matmul(la, ctx, kernels, "matmul_nt_q4_0_f32out_into", a, raw, m, k, n, f32out=True)
    rel_close(got32, want32, 2e-4, "tensor-core q4_0 f32 out")
    device_status_ok(kernels)


def test_expired_barrier_wait_reports_timeout(la, orc, ctx, monkeypatch):
    """Every barrier wait of the tcgen05 matmul is bounded.  LOCAL_CUDA_TEST_WAIT_EXPIRY=1 gives a kernels object
    whose launches wait (with a short limit) for an arrival nobody makes: the launch must come back by itself, leave
    the status word set so that lc_kernels_device_status returns Timeout, and leave the context usable."""
    import ctypes as C
    monkeypatch.setenv("LOCAL_CUDA_TEST_WAIT_EXPIRY", "1")
    k2 = la.Kernels.new(ctx)
    monkeypatch.delenv("LOCAL_CUDA_TEST_WAIT_EXPIRY")
    m, k, n = 128, 512, 256          # m > 64: the large-tile tcgen05 kernel
    raw = la.synth.tq2_0_weights(n, k, 81)
    a = la.synth.normal_f16((m, k), 82)
    run_matmul(la, ctx, k2, "matmul_nt_tq2_0_into", a, raw, m, k, n)   # returns: no wait is endless
    st = C.c_int(0)
    with pytest.raises(la.Error) as ei:
        k2.kernels_device_status(C.addressof(st))
    assert ei.value.kind == "Timeout" and st.value != 0
    k2.close()
    # the context and a regular kernels object still work
    k3 = la.Kernels.new(ctx)
    got = run_matmul(la, ctx, k3, "matmul_nt_tq2_0_into", a, raw, m, k, n)
    k3.close()
    rel_close(got, orc.matmul_nt(orc.TQ2_0, a, raw, m, k, n), TC_TOL_TQ2, "after an expired wait")


@pytest.mark.parametrize("which", ["decode_matmul", "vocabulary"])
def test_expired_wait_in_the_decode_kernels_reports_timeout(la, orc, ctx, monkeypatch, which):
    """The same self-test for the two tcgen05 kernels of the decode step: with LOCAL_CUDA_TEST_WAIT_EXPIRY=1 their
    readiness barriers expect an arrival nobody makes and every wait has a short limit.  The launch must return, the
    status word must read Timeout, and a regular kernels object must work afterwards on the same context."""
    import ctypes as C
    if which == "decode_matmul":
        m, k, n, fmt, entry, f32 = 64, 1536, 512, orc.TQ2_0, "matmul_nt_tq2_0_into", False
        raw = la.synth.tq2_0_weights(n, k, 83)
    else:
        m, k, n, fmt, entry, f32 = 64, 256, 19200, orc.Q4_0, "matmul_nt_q4_0_f32out_into", True
        raw = la.synth.q4_0_weights(n, k, 83)
    a = la.synth.normal_f16((m, k), 84)
    monkeypatch.setenv("LOCAL_CUDA_TEST_WAIT_EXPIRY", "1")
    k2 = la.Kernels.new(ctx)
    monkeypatch.delenv("LOCAL_CUDA_TEST_WAIT_EXPIRY")
    run_matmul(la, ctx, k2, entry, a, raw, m, k, n, f32out=f32)   # returns: no wait is endless
    st = C.c_int(0)
    with pytest.raises(la.Error) as ei:
        k2.kernels_device_status(C.addressof(st))
    assert ei.value.kind == "Timeout" and st.value != 0
    k2.close()
    k3 = la.Kernels.new(ctx)
    got = run_matmul(la, ctx, k3, entry, a, raw, m, k, n, f32out=f32)
    k3.close()
    rel_close(got, orc.matmul_nt(fmt, a, raw, m, k, n), TC_TOL_TQ2 if fmt == orc.TQ2_0 else 2e-4, "after an expired wait")


def test_tensor_core_and_cuda_core_paths_agree(la, orc, ctx, kernels, monkeypatch):
    """LOCAL_AI_MMA=0 forces the CUDA-core path (kernels.rs:6290-6298); both must give the same TQ2_0 result
    up to summation order."""
    m, k, n = 64, 1536, 512
    raw = la.synth.tq2_0_weights(n, k, 11)
    a = la.synth.normal_f16((m, k), 12)
    tc = run_matmul(la, ctx, kernels, "matmul_nt_tq2_0_into", a, raw, m, k, n)
    monkeypatch.setenv("LOCAL_AI_MMA", "0")
    k2 = la.Kernels.new(ctx)
    cc = run_matmul(la, ctx, k2, "matmul_nt_tq2_0_into", a, raw, m, k, n)
    k2.close()
    assert np.max(np.abs(tc - cc)) <= 2e-3 * max(1.0, float(np.abs(cc).max()))


def test_split_k_is_deterministic_and_lane_isolated(la, orc, ctx, tc_kernels):
    kernels = tc_kernels
    """Small-n projections run split-K on the tensor-core path (deterministic last-arriver reduction):
    repeated launches and duplicate batch rows must agree bit for bit."""
    m, k, n = 64, 6144, 1536   # the down projection: 12 row tiles x 12 splits
    raw = la.synth.tq2_0_weights(n, k, 21)
    a = la.synth.normal_f16((m, k), 22)
    a[5] = a[3]
    r1 = run_matmul(la, ctx, kernels, "matmul_nt_tq2_0_into", a, raw, m, k, n)
    r2 = run_matmul(la, ctx, kernels, "matmul_nt_tq2_0_into", a, raw, m, k, n)
    assert np.array_equal(r1, r2)
    assert np.array_equal(r1[5], r1[3])
    rel_close(r1, orc.matmul_nt(orc.TQ2_0, a, raw, m, k, n), TC_TOL_TQ2, "split-K down projection")
    device_status_ok(kernels)


@pytest.mark.parametrize("m,k,n", [(64, 256, 76000), (40, 384, 75800), (64, 1536, 20000), (33, 512, 19001), (9, 768, 40000), (130, 256, 19200)])
def test_matmul_nt_q4_0_wide_matrix(la, orc, ctx, kernels, m, k, n):
    """Vocabulary-sized Q4_0 projections at decode batch sizes take a persistent kernel: with f32 out and K a multiple
    of 256 the tcgen05 one (128-row tiles, weights as two f16 operands in tensor memory), else the 512-row mma.sync one
    (ragged last tile, several tiles per CTA, steps that outnumber the barrier ring; more than 64 batch rows go
    through the tcgen05 kernel in chunks of 64); results must meet the f32-weight oracle."""
    raw = la.synth.q4_0_weights(n, k, 31)
    a = la.synth.normal_f16((m, k), 32)
    want32 = orc.matmul_nt(orc.Q4_0, a, raw, m, k, n)
    got32 = run_matmul(la, ctx, kernels, "matmul_nt_q4_0_f32out_into", a, raw, m, k, n, f32out=True)
    rel_close(got32, want32, 2e-4, "wide q4_0 f32 out")
    got = run_matmul(la, ctx, kernels, "matmul_nt_q4_0_into", a, raw, m, k, n)
    rel_close(got, want32, TC_TOL_Q4, "wide q4_0 f16 out")


@pytest.mark.parametrize("m,k,n", [(64, 1536, 6144), (33, 512, 200), (16, 256, 64), (64, 2048, 1000), (4, 512, 256), (70, 512, 256)])
def test_geglu_fused_equals_separate_launches(la, orc, ctx, kernels, m, k, n):
    """gelu_tanh(x Wg^T) * (x Wu^T): one launch for decode batches, the three separate dispatches otherwise; both
    must give what matmul, matmul, gelu_mul give (up to the f32 summation order of the K splits: gate and up are
    rounded to f16 in between, as the separate projections store them) and meet the oracle."""
    wg, wu = la.synth.tq2_0_weights(n, k, 51), la.synth.tq2_0_weights(n, k, 52)
    a = la.synth.normal_f16((m, k), 53, 0.5)
    d = lambda arr: la.CudaBuffer.from_slice(ctx, arr)
    da, dg, du = d(a), d(wg), d(wu)
    out = Guarded(la, ctx, m * n * 2)
    gt, ut = la.CudaBuffer.empty(ctx, m * n * 2), la.CudaBuffer.empty(ctx, m * n * 2)
    b = la.CommandBatch.new(ctx)
    kernels.matmul_nt_tq2_0_geglu_into(b, da, dg, du, gt, ut, out.view, m, k, n)
    assert b.dispatch_count() == (1 if m <= 64 else 2)   # fused (also at m <= 8: the tcgen05 kernel) | grouped + gelu
    b.commit_and_wait()
    fused = out.read(np.float16)
    g2, u2, o2 = la.CudaBuffer.empty(ctx, m * n * 2), la.CudaBuffer.empty(ctx, m * n * 2), la.CudaBuffer.empty(ctx, m * n * 2)
    b = la.CommandBatch.new(ctx)
    kernels.matmul_nt_tq2_0_into(b, da, dg, g2, m, k, n)
    kernels.matmul_nt_tq2_0_into(b, da, du, u2, m, k, n)
    kernels.gelu_mul_into(b, g2, u2, o2, m * n)
    b.commit_and_wait()
    rel_close(fused.astype(np.float32), o2.as_slice(np.float16, m * n).astype(np.float32), 2e-3, "geglu fused vs separate")
    want_g = orc.matmul_nt(orc.TQ2_0, a, wg, m, k, n).astype(np.float16)
    want_u = orc.matmul_nt(orc.TQ2_0, a, wu, m, k, n).astype(np.float16)
    rel_close(fused.astype(np.float32), orc.gelu_mul(want_g.ravel(), want_u.ravel()).astype(np.float32), 4e-3, "geglu vs oracle")


@pytest.mark.parametrize("m,k,n", [(1, 256, 76000), (8, 384, 75800), (3, 1536, 80000)])
def test_q4_0_wide_matrix_small_batch_keeps_exact_weights(la, orc, ctx, kernels, m, k, n):
    """Batch <= 8 against a vocabulary-sized Q4_0 table: tensor-core kernel with integer operands and per-block f32
    scaling, so the result must meet the f32-weight oracle at the matvec tolerance (not only the f16-weight one)."""
    raw = la.synth.q4_0_weights(n, k, 61)
    a = la.synth.normal_f16((m, k), 62)
    want = orc.matmul_nt(orc.Q4_0, a, raw, m, k, n)
    got32 = run_matmul(la, ctx, kernels, "matmul_nt_q4_0_f32out_into", a, raw, m, k, n, f32out=True)
    rel_close(got32, want, 2e-4, "wide q4_0 small batch, f32 out")
    got = run_matmul(la, ctx, kernels, "matmul_nt_q4_0_into", a, raw, m, k, n)
    rel_close(got, want, TOL, "wide q4_0 small batch, f16 out")
    if m == 1:
        y = run_matvec(la, ctx, kernels, "matvec_q4_0_f32out", raw, a[0], n, k, True, True)
        rel_close(y, want[0], 2e-4, "matvec_q4_0_f32out on a wide table")


@pytest.mark.parametrize("m,k,n", [(1, 256, 19000), (8, 512, 20001), (2, 1536, 19100)])
def test_tq2_0_streaming_small_batch(la, orc, ctx, kernels, m, k, n):
    """Batch <= 8 over a TQ2_0 matrix with enough rows for the streaming tensor-core kernel (ragged last group)."""
    raw = la.synth.tq2_0_weights(n, k, 71, ncodes=4)
    a = la.synth.normal_f16((m, k), 72)
    want = orc.matmul_nt(orc.TQ2_0, a, raw, m, k, n)
    got = run_matmul(la, ctx, kernels, "matmul_nt_tq2_0_into", a, raw, m, k, n)
    rel_close(got, want, TOL, "streaming tq2_0 small batch")
    if m == 1:
        y = run_matvec(la, ctx, kernels, "matvec_tq2_0_f32out", raw, a[0], n, k, True, True)
        rel_close(y, want[0], 2e-4, "matvec_tq2_0_f32out, streaming")


@pytest.mark.parametrize("fmt,rows,cols,count", [("tq2_0", 8192, 1536, 6), ("q4_0", 6144, 1536, 5), ("tq2_0", 200, 512, 3),
                                                 ("q4_0", 4100, 256, 7)])
def test_matvec_group_equals_single_launches(la, orc, ctx, kernels, fmt, rows, cols, count):
    """Several matrices of one shape against one vector in one launch (the streaming kernel walks them as one run of
    64-row groups; small sets fall back to one launch each): every output equals the single-matrix entry point's bit
    for bit and meets the oracle."""
    gen = la.synth.q4_0_weights if fmt == "q4_0" else la.synth.tq2_0_weights
    ws = [gen(rows, cols, 70 + i) for i in range(count)]
    x = la.synth.normal_f16((1, cols), 69)
    dx = la.CudaBuffer.from_slice(ctx, x)
    dws = [la.CudaBuffer.from_slice(ctx, w) for w in ws]
    outs = [Guarded(la, ctx, rows * 2) for _ in range(count)]
    b = la.CommandBatch.new(ctx)
    getattr(kernels, f"matvec_{fmt}_group_into")(b, dws, count, dx, [o.view for o in outs], rows, cols)
    streamed = rows >= 64 and ((rows + 63) // 64) * count >= 2 * ctx.caps()["sm_count"]
    assert b.dispatch_count() == (1 if streamed else count)
    b.commit_and_wait()
    f = orc.Q4_0 if fmt == "q4_0" else orc.TQ2_0
    for i in range(count):
        got = outs[i].read(np.float16)
        single = la.CudaBuffer.empty(ctx, rows * 2)
        b = la.CommandBatch.new(ctx)
        getattr(kernels, f"matvec_{fmt}_into")(b, dws[i], dx, single, rows, cols)
        b.commit_and_wait()
        if not streamed:
            assert np.array_equal(got.view(np.uint16), single.as_slice(np.uint16))
        rel_close(got, orc.matmul_nt(f, x, ws[i], 1, cols, rows).reshape(-1), 2e-3, f"group matvec {i}")
