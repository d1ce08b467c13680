// Routing of the quantized batched matmul C[m, n] = A[m, k] x W[n, k]^T, the
// stand-in for Kernels::matmul_nt_q4_0_into / matmul_nt_tq2_0_into
// (local-metal/src/kernels.rs:6459-6563).  The reference picks between four
// Metal kernels by m (batchm <= 4, smallm <= 8, simdgroup MMA, scalar tile);
// here: for TQ2_0 with f16 output and m <= 64 the lean tcgen05 kernel
// (qmatmul_tcd.cu; it is also the faster launch at m <= 8, LOCAL_CUDA_SMALL_M=8
// keeps those on the CUDA-core kernel); otherwise the register-resident CUDA-core
// path that streams the weights once for up to 16 rows (qmatvec.cu, m <= 8), the
// register-direct mma.sync kernel for decode batches 8 < m <= 64 (qmatmul_mma.cu:
// Q4_0, f32 out, shapes the tcgen05 kernel declines), and the large-tile tcgen05
// kernel for larger m (qmatmul_tc.cu).  The matvec entry points (lc_matvec_*) stay
// on the CUDA-core kernels.
// LOCAL_AI_MMA=0 forces the CUDA-core path for every m, as it forces the non-MMA
// kernels in the reference; LOCAL_CUDA_DECODE_TC=0 / LOCAL_CUDA_DECODE_MMA=0
// switch the two decode kernels off (with both off, 8 < m <= 64 runs on
// qmatmul_tc.cu as well).
#include <stdlib.h>
#include "lc_internal.h"

int lc_qgemm_cuda_core(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input,
                       const lc_buf *weight, lc_buf *output, uint32_t m, uint32_t kk, uint32_t n);
int lc_check_qargs(int fmt, const char *name, lc_kernels *k, lc_batch *b, const lc_buf *w, const lc_buf *x,
                   const lc_buf *out, uint32_t m, uint32_t kk, uint32_t n, size_t out_elem);
// qmatmul_tc.cu: returns LC_OK when it launched, or a negative value when the
// shape is outside what the tensor-core kernel covers (caller falls through).
int lc_qgemm_tcgen05(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input,
                     const lc_buf *weight, lc_buf *output, uint32_t m, uint32_t kk, uint32_t n);

// qmatmul_mma.cu: same contract as lc_qgemm_tcgen05_grouped, for 8 < m <= 64.
int lc_qgemm_mma_grouped(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input, int ng,
                         const lc_buf *const *weights, lc_buf *const *outputs, const uint32_t *ns, uint32_t m,
                         uint32_t kk);

// qmatmul_tcd.cu: tcgen05 decode matmul (TQ2_0, f16 out, 8 < m <= 64); same return contract.
int lc_qgemm_tcd_launch(lc_kernels *k, lc_batch *b, const lc_buf *input, int ng, const lc_buf *const *weights,
                        lc_buf *const *outputs, const uint32_t *ns, uint32_t m, uint32_t kk, bool geglu);

// qmatmul_tcv.cu: persistent tcgen05 kernel for very tall Q4_0 matrices (the vocabulary projection), f32 out, m <= 64;
// same return contract.
int lc_qgemm_tcv_launch(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight, lc_buf *output, uint32_t m,
                        uint32_t kk, uint32_t n);

static int route(int fmt, bool f32out, const char *name, lc_kernels *k, lc_batch *b, const lc_buf *input,
                 const lc_buf *weight, lc_buf *output, uint32_t m, uint32_t kk, uint32_t n) {
    int st = lc_check_qargs(fmt, name, k, b, weight, input, output, m, kk, n, f32out ? 4 : 2);
    if (st != LC_OK) return st;
    if (n == 0) return LC_OK;
    const lc_buf *ws[1] = {weight};
    lc_buf *os[1] = {output};
    const uint32_t ns[1] = {n};
    if (k->mma && k->decode_tc && fmt == 1 && !f32out && m > k->small_m && m <= 64) {
        st = lc_qgemm_tcd_launch(k, b, input, 1, ws, os, ns, m, kk, false);
        if (st >= 0) return st;
    }
    if (k->mma && k->vocab_tc && fmt == 0 && f32out && m > 8) {
        // The persistent vocabulary kernel takes 64 batch rows per launch; larger batches go through it in chunks.
        // Each chunk streams the table once, and still 262144 x 1536 at 128 / 256 / 512 rows takes 238 / 474 / 970 us
        // against 762 / 1510 / 2999 us for the large-tile kernel, which runs every Q4_0 tile twice.
        bool covered = m <= 4096;
        for (uint32_t m0 = 0; m0 < m && covered; m0 += 64) {
            const uint32_t mc = m - m0 < 64 ? m - m0 : 64;
            lc_buf in_v = *input, out_v = *output;
            in_v.dptr = (char *)input->dptr + (size_t)m0 * kk * 2;
            in_v.bytes = input->bytes - (size_t)m0 * kk * 2;
            in_v.owned = false;
            out_v.dptr = (char *)output->dptr + (size_t)m0 * n * 4;
            out_v.bytes = output->bytes - (size_t)m0 * n * 4;
            out_v.owned = false;
            st = lc_qgemm_tcv_launch(k, b, &in_v, weight, &out_v, mc, kk, n);
            if (st > 0) return st;
            if (st < 0) {
                if (m0 != 0) return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: vocabulary kernel declined chunk %u after accepting the first", name, m0 / 64);
                covered = false;
            }
        }
        if (covered) return LC_OK;
    }
    if (k->mma && m > 8) {
        if (m <= 64) {
            if (k->decode_mma) {
                st = lc_qgemm_mma_grouped(fmt, f32out, k, b, input, 1, ws, os, ns, m, kk);
                if (st >= 0) return st;
            }
        }
        st = lc_qgemm_tcgen05(fmt, f32out, k, b, input, weight, output, m, kk, n);
        if (st >= 0) return st;
    }
    return lc_qgemm_cuda_core(fmt, f32out, k, b, input, weight, output, m, kk, n);
}

int lc_qgemm_tcgen05_grouped(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input, int ng,
                             const lc_buf *const *weights, lc_buf *const *outputs, const uint32_t *ns, uint32_t m,
                             uint32_t kk);

// Several TQ2_0 projections of the same activations (Q/K/V; gate/up) as one launch when the tensor-core
// path applies, else one after the other.
int lc_matmul_nt_tq2_0_grouped(lc_kernels *k, lc_batch *b, const lc_buf *input, int ng, const lc_buf *const *weights,
                               lc_buf *const *outputs, const uint32_t *ns, uint32_t m, uint32_t kk) {
    for (int g = 0; g < ng; g++) {
        int st = lc_check_qargs(1, "matmul_nt_tq2_0", k, b, weights[g], input, outputs[g], m, kk, ns[g], 2);
        if (st != LC_OK) return st;
    }
    if (k->mma && k->decode_tc && m > k->small_m && m <= 64) {
        const int st = lc_qgemm_tcd_launch(k, b, input, ng, weights, outputs, ns, m, kk, false);
        if (st >= 0) return st;
    }
    if (k->mma && m > 8) {
        int st = -1;
        if (k->decode_mma && m <= 64) st = lc_qgemm_mma_grouped(1, false, k, b, input, ng, weights, outputs, ns, m, kk);
        if (st < 0) st = lc_qgemm_tcgen05_grouped(1, false, k, b, input, ng, weights, outputs, ns, m, kk);
        if (st >= 0) return st;
    }
    for (int g = 0; g < ng; g++) {
        int st = lc_qgemm_cuda_core(1, false, k, b, input, weights[g], outputs[g], m, kk, ns[g]);
        if (st != LC_OK) return st;
    }
    return LC_OK;
}

int lc_qgemm_mma_geglu(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *w_gate, const lc_buf *w_up,
                       lc_buf *output, uint32_t m, uint32_t kk, uint32_t n);

extern "C" {

// The GeGLU half of the feed-forward block, gelu_tanh(x W_gate^T) * (x W_up^T) (local-engine/src/layer.rs:825-838):
// one launch on the decode path (8 < m <= 64), else the two projections into `gate_tmp` / `up_tmp` followed by
// gelu_mul.  `output` may alias `gate_tmp`.
int lc_matmul_nt_tq2_0_geglu_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *w_gate,
                                  const lc_buf *w_up, lc_buf *gate_tmp, lc_buf *up_tmp, lc_buf *output, uint32_t m,
                                  uint32_t kk, uint32_t n) {
    if (!gate_tmp || !up_tmp) return lc_fail(LC_ERR_INVALID_ARGUMENT, "matmul_nt_tq2_0_geglu: NULL argument");
    int st = lc_check_qargs(1, "matmul_nt_tq2_0_geglu", k, b, w_gate, input, output, m, kk, n, 2);
    if (st == LC_OK) st = lc_check_qargs(1, "matmul_nt_tq2_0_geglu", k, b, w_up, input, up_tmp, m, kk, n, 2);
    if (st == LC_OK) st = lc_check_qargs(1, "matmul_nt_tq2_0_geglu", k, b, w_gate, input, gate_tmp, m, kk, n, 2);
    if (st != LC_OK) return st;
    if (n == 0 || m == 0) return LC_OK;
    static const bool fused_ok = []() { const char *e = getenv("LOCAL_CUDA_GEGLU_FUSED"); return !(e && e[0] == '0'); }();
    if (fused_ok && k->mma && m > k->small_m && m <= 64) {
        if (k->decode_tc) {
            const lc_buf *ws[2] = {w_gate, w_up};
            lc_buf *os[2] = {output, output};
            const uint32_t ns[2] = {n, n};
            st = lc_qgemm_tcd_launch(k, b, input, 2, ws, os, ns, m, kk, true);
            if (st >= 0) return st;
        }
        if (k->decode_mma && m > 8) {
            st = lc_qgemm_mma_geglu(k, b, input, w_gate, w_up, output, m, kk, n);
            if (st >= 0) return st;
        }
    }
    const lc_buf *ws[2] = {w_gate, w_up};
    lc_buf *os[2] = {gate_tmp, up_tmp};
    const uint32_t ns[2] = {n, n};
    st = lc_matmul_nt_tq2_0_grouped(k, b, input, 2, ws, os, ns, m, kk);
    if (st != LC_OK) return st;
    return lc_gelu_mul_into(k, b, gate_tmp, up_tmp, output, m * n);
}

int lc_matmul_nt_q4_0_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                           lc_buf *output, uint32_t m, uint32_t kk, uint32_t n) {
    return route(0, false, "matmul_nt_q4_0", k, b, input, weight, output, m, kk, n);
}

int lc_matmul_nt_tq2_0_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                            lc_buf *output, uint32_t m, uint32_t kk, uint32_t n) {
    return route(1, false, "matmul_nt_tq2_0", k, b, input, weight, output, m, kk, n);
}

int lc_matmul_nt_q4_0_f32out_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                                  lc_buf *output, uint32_t m, uint32_t kk, uint32_t n) {
    return route(0, true, "matmul_nt_q4_0_f32out", k, b, input, weight, output, m, kk, n);
}

}  // extern "C"
