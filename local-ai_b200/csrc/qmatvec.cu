// Fused-dequant matvec and register-resident small-M matmul over GGUF Q4_0 /
// TQ2_0 blocks.  Stands in for shaders/matvec_quant.metal (matvec_q4_0 :64-155,
// matvec_tq2_0 :172-312, matvec_tq2_0_soa :322-387, matmul_nt_tq2_0_batchm
// :813-916, multivec_nt_* :936-1038) and shaders/tq2_dequant.metal.
//
// Design (not the Metal one): a CTA streams a contiguous run of weight rows
// from HBM into shared memory with 16-byte coalesced loads — GGUF rows are only
// 2-byte aligned (18 B / 66 B blocks), so the run is copied as the enclosing
// 16-byte-aligned byte range and indexed from the remainder — then each warp
// owns one staged row: lanes unpack 2-byte pieces of the block in registers,
// multiply with the activations held in shared memory and finish with one
// shuffle reduction per output.  All MT activation rows reuse the unpacked
// weights, so the weight bytes are read from HBM once per MT rows.
#include "lc_internal.h"

namespace {

constexpr int FMT_Q4_0 = 0;
constexpr int FMT_TQ2_0 = 1;
constexpr int NTHREADS = 256;
constexpr int NWARPS = NTHREADS / 32;

template <int FMT> struct Fmt;
template <> struct Fmt<FMT_Q4_0> { static constexpr int bytes = 18, elems = 32; };
template <> struct Fmt<FMT_TQ2_0> { static constexpr int bytes = 66, elems = 256; };

__device__ __forceinline__ void store_out(__half *p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void store_out(float *p, float v) { *p = v; }

// Copy global bytes [start, start+len) of `w` into `stage`, as the enclosing
// 16-byte-aligned range.  Returns nothing; the data begins at stage + (start & 15).
// Never reads at or beyond w_bytes.
__device__ __forceinline__ void stage_rows(const uint8_t *__restrict__ w, size_t w_bytes, size_t start,
                                           size_t len, uint8_t *stage) {
    const size_t pad = start & 15;
    const size_t a0 = start - pad;
    const int n16 = (int)((pad + len + 15) >> 4);
    for (int i = threadIdx.x; i < n16; i += NTHREADS) {
        const size_t g = a0 + ((size_t)i << 4);
        if (g + 16 <= w_bytes) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(w + g));
            *reinterpret_cast<uint4 *>(stage + ((size_t)i << 4)) = v;
        } else {
            for (int b = 0; b < 16; b++)
                if (g + b < w_bytes) stage[((size_t)i << 4) + b] = w[g + b];
        }
    }
}

// out[mi*n + row] = sum_k X[mi*K + k] * W[row, k], mi in [m0, m0+MT).
template <int FMT, int MT, typename OutT, bool XSMEM>
__global__ void __launch_bounds__(NTHREADS)
qgemv_kernel(const uint8_t *__restrict__ w, size_t w_bytes, const __half *__restrict__ x,
             OutT *__restrict__ out, int n, int K, int m, int rows_per_chunk, int nchunks) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    extern __shared__ __align__(16) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m0 = blockIdx.y * MT;
    const int mvalid = min(MT, m - m0);
    const int nb = K / Fmt<FMT>::elems;
    const size_t rb = (size_t)nb * Fmt<FMT>::bytes;

    __half *xs = reinterpret_cast<__half *>(smem);
    uint8_t *stage = smem + (XSMEM ? (((size_t)MT * K * 2 + 15) & ~(size_t)15) : 0);
    if (XSMEM) {
        // K is a multiple of 32, so each activation row is a whole number of 16-byte pieces.
        const int per_row = K >> 3;
        for (int i = threadIdx.x; i < MT * per_row; i += NTHREADS) {
            const int mi = i / per_row, c = i - mi * per_row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (mi < mvalid) v = __ldg(reinterpret_cast<const uint4 *>(x + (size_t)(m0 + mi) * K) + c);
            reinterpret_cast<uint4 *>(xs)[i] = v;
        }
    }
    const __half *xg = x + (size_t)m0 * K;

    for (int chunk = blockIdx.x; chunk < nchunks; chunk += gridDim.x) {
        const int row0 = chunk * rows_per_chunk;
        const int nrows = min(rows_per_chunk, n - row0);
        const size_t start = (size_t)row0 * rb;
        __syncthreads();  // previous chunk fully consumed (and xs visible on the first pass)
        stage_rows(w, w_bytes, start, (size_t)nrows * rb, stage);
        __syncthreads();
        const uint8_t *base = stage + (start & 15);

        for (int r = warp; r < nrows; r += NWARPS) {
            const uint8_t *rowp = base + (size_t)r * rb;
            float acc[MT];
#pragma unroll
            for (int i = 0; i < MT; i++) acc[i] = 0.f;

            if (FMT == FMT_TQ2_0) {
                // Lane l owns qs bytes 2l and 2l+1 of every block: elements
                // (l>>4)*128 + lp*32 + 2(l&15) + {0,1}, lp = 0..3.
                const int xoff = (lane >> 4) * 128 + 2 * (lane & 15);
                for (int b = 0; b < nb; b++) {
                    const uint8_t *blk = rowp + b * 66;
                    const unsigned w16 = *reinterpret_cast<const uint16_t *>(blk + 2 * lane);
                    const float d = __half2float(*reinterpret_cast<const __half *>(blk + 64));
                    float wv[8];
#pragma unroll
                    for (int lp = 0; lp < 4; lp++) {
                        wv[2 * lp] = (float)((int)((w16 >> (2 * lp)) & 3u) - 1);
                        wv[2 * lp + 1] = (float)((int)((w16 >> (8 + 2 * lp)) & 3u) - 1);
                    }
                    const int xb = b * 256 + xoff;
#pragma unroll
                    for (int mi = 0; mi < MT; mi++) {
                        if (mi < mvalid) {
                            float s = 0.f;
#pragma unroll
                            for (int lp = 0; lp < 4; lp++) {
                                const __half2 xv =
                                    XSMEM ? *reinterpret_cast<const __half2 *>(xs + (size_t)mi * K + xb + lp * 32)
                                          : __ldg(reinterpret_cast<const __half2 *>(xg + (size_t)mi * K + xb + lp * 32));
                                const float2 xf = __half22float2(xv);
                                s = fmaf(wv[2 * lp], xf.x, s);
                                s = fmaf(wv[2 * lp + 1], xf.y, s);
                            }
                            acc[mi] = fmaf(d, s, acc[mi]);
                        }
                    }
                }
            } else {
                // Unit u = (block b, 2-byte piece h): bytes 2h, 2h+1 of the block's
                // 16 code bytes -> elements 2h, 2h+1 (low nibbles), 16+2h, 17+2h (high).
                const int units = nb * 8;
                for (int u = lane; u < units; u += 32) {
                    const int b = u >> 3, h = u & 7;
                    const uint8_t *blk = rowp + b * 18;
                    const float d = __half2float(*reinterpret_cast<const __half *>(blk));
                    const unsigned w16 = *reinterpret_cast<const uint16_t *>(blk + 2 + 2 * h);
                    const float q0 = (float)((int)(w16 & 15u) - 8);
                    const float q1 = (float)((int)((w16 >> 8) & 15u) - 8);
                    const float q2 = (float)((int)((w16 >> 4) & 15u) - 8);
                    const float q3 = (float)((int)((w16 >> 12) & 15u) - 8);
                    const int xb = b * 32 + 2 * h;
#pragma unroll
                    for (int mi = 0; mi < MT; mi++) {
                        if (mi < mvalid) {
                            const __half2 lo =
                                XSMEM ? *reinterpret_cast<const __half2 *>(xs + (size_t)mi * K + xb)
                                      : __ldg(reinterpret_cast<const __half2 *>(xg + (size_t)mi * K + xb));
                            const __half2 hi =
                                XSMEM ? *reinterpret_cast<const __half2 *>(xs + (size_t)mi * K + xb + 16)
                                      : __ldg(reinterpret_cast<const __half2 *>(xg + (size_t)mi * K + xb + 16));
                            const float2 lf = __half22float2(lo), hf = __half22float2(hi);
                            float s = q0 * lf.x;
                            s = fmaf(q1, lf.y, s);
                            s = fmaf(q2, hf.x, s);
                            s = fmaf(q3, hf.y, s);
                            acc[mi] = fmaf(d, s, acc[mi]);
                        }
                    }
                }
            }
#pragma unroll
            for (int mi = 0; mi < MT; mi++) {
                float v = acc[mi];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0 && mi < mvalid) store_out(out + (size_t)(m0 + mi) * n + row0 + r, v);
            }
        }
    }
}

// SoA TQ2_0 (matvec_quant.metal:322-387): qs[(row*nb+b)*64 ..], scales[row*nb+b].
// One warp per row, lane owns 2 adjacent qs bytes; read straight from global.
__global__ void __launch_bounds__(NTHREADS)
matvec_tq2_0_soa_kernel(const uint8_t *__restrict__ qs, const __half *__restrict__ scales,
                        const __half *__restrict__ x, __half *__restrict__ out, int rows, int K) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * NWARPS + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int nb = K / 256;
    const int xoff = (lane >> 4) * 128 + 2 * (lane & 15);
    float acc = 0.f;
    for (int b = 0; b < nb; b++) {
        const size_t blk = (size_t)row * nb + b;
        const unsigned w16 = __ldg(reinterpret_cast<const uint16_t *>(qs + blk * 64) + lane);
        const float d = __half2float(__ldg(scales + blk));
        float s = 0.f;
#pragma unroll
        for (int lp = 0; lp < 4; lp++) {
            const float2 xf = __half22float2(__ldg(reinterpret_cast<const __half2 *>(x + b * 256 + xoff + lp * 32)));
            s = fmaf((float)((int)((w16 >> (2 * lp)) & 3u) - 1), xf.x, s);
            s = fmaf((float)((int)((w16 >> (8 + 2 * lp)) & 3u) - 1), xf.y, s);
        }
        acc = fmaf(d, s, acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[row] = __float2half_rn(acc);
}

// shaders/tq2_dequant.metal:4-16, over all elements.
__global__ void tq2_dequant_kernel(const uint8_t *__restrict__ packed, const __half *__restrict__ scales,
                                   __half *__restrict__ out, uint32_t n) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t bi = i >> 2;
    const unsigned q = (packed[bi] >> (2 * (i & 3))) & 3u;
    out[i] = __float2half_rn(__half2float(scales[bi]) * (float)q);
}

template <int FMT, int MT, typename OutT, bool XSMEM>
int launch_qgemv(lc_kernels *k, lc_batch *b, const uint8_t *w, size_t w_bytes, const __half *x, OutT *out,
                 int n, int K, int m) {
    const size_t rb = (size_t)(K / Fmt<FMT>::elems) * Fmt<FMT>::bytes;
    int rpc = (int)(12288 / rb);
    rpc = rpc < NWARPS ? NWARPS : (rpc > 64 ? 64 : rpc);
    rpc = (rpc / NWARPS) * NWARPS;
    const int nchunks = (n + rpc - 1) / rpc;
    const size_t xbytes = XSMEM ? (((size_t)MT * K * 2 + 15) & ~(size_t)15) : 0;
    const size_t smem = xbytes + (size_t)rpc * rb + 32;
    auto kern = qgemv_kernel<FMT, MT, OutT, XSMEM>;
    static lc_smem_optin optin;  // per instantiation
    LC_CUDA_TRY(lc_ensure_smem(kern, optin, b->ctx, smem));
    int gx = k->ctx->sm_count * 4;
    if (gx > nchunks) gx = nchunks;
    dim3 grid(gx, (m + MT - 1) / MT);
    LC_LAUNCH_CHECKED(lc_launch(kern, dim3(grid), dim3(NTHREADS), smem, b, w, w_bytes, x, out, n, K, m, rpc, nchunks));
    LC_CHECK_LAUNCH("qgemv");
    b->dispatch_count++;
    return LC_OK;
}

template <int FMT, int MT, typename OutT>
int launch_qgemv_x(lc_kernels *k, lc_batch *b, const uint8_t *w, size_t w_bytes, const __half *x, OutT *out,
                   int n, int K, int m) {
    // Activations live in shared memory when MT rows of K halfs fit comfortably.
    if ((size_t)MT * K * 2 <= 96 * 1024)
        return launch_qgemv<FMT, MT, OutT, true>(k, b, w, w_bytes, x, out, n, K, m);
    return launch_qgemv<FMT, MT, OutT, false>(k, b, w, w_bytes, x, out, n, K, m);
}

template <int FMT, typename OutT>
int dispatch_qgemv(lc_kernels *k, lc_batch *b, const uint8_t *w, size_t w_bytes, const __half *x, OutT *out,
                   int n, int K, int m) {
    if (m <= 1) return launch_qgemv_x<FMT, 1, OutT>(k, b, w, w_bytes, x, out, n, K, m);
    if (m <= 2) return launch_qgemv_x<FMT, 2, OutT>(k, b, w, w_bytes, x, out, n, K, m);
    if (m <= 4) return launch_qgemv_x<FMT, 4, OutT>(k, b, w, w_bytes, x, out, n, K, m);
    if (m <= 8) return launch_qgemv_x<FMT, 8, OutT>(k, b, w, w_bytes, x, out, n, K, m);
    return launch_qgemv_x<FMT, 16, OutT>(k, b, w, w_bytes, x, out, n, K, m);
}

}  // namespace

// Shared argument validation for every quantized contraction
// (the reference checks only block alignment: kernels.rs:5720-5724, 5857-5861).
template <int FMT>
static int check_qargs(const char *name, lc_kernels *k, lc_batch *b, const lc_buf *w, const lc_buf *x,
                       const lc_buf *out, uint32_t m, uint32_t kk, uint32_t n, size_t out_elem) {
    if (!k || !b || !w || !x || !out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    const uint32_t be = Fmt<FMT>::elems;
    if (kk == 0 || kk % be != 0) return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: cols %u not /%u", name, kk, be);
    LC_REQUIRE(kk <= (1u << 20), "%s: cols %u too large", name, kk);
    LC_REQUIRE(m >= 1, "%s: m must be >= 1", name);
    const size_t rb = (size_t)(kk / be) * Fmt<FMT>::bytes;
    LC_REQUIRE(w->bytes >= rb * n, "%s: weight buffer %zu B < %zu B", name, w->bytes, rb * n);
    LC_REQUIRE(x->bytes >= (size_t)m * kk * 2, "%s: input buffer %zu B < %zu B", name, x->bytes,
               (size_t)m * kk * 2);
    LC_REQUIRE(out->bytes >= (size_t)m * n * out_elem, "%s: output buffer %zu B < %zu B", name, out->bytes,
               (size_t)m * n * out_elem);
    LC_REQUIRE(lc_aligned(w->dptr, 16) && lc_aligned(x->dptr, 16) && lc_aligned(out->dptr, 4),
               "%s: weight and input buffers must be 16-byte aligned", name);
    return LC_OK;
}

// Entry used by the other translation units (matmul routing, decode step).
// qmatvec_mma.cu: streaming tensor-core kernel for m <= 8 and matrices large enough for bandwidth to matter;
// returns -1 for everything else.
int lc_qgemv_mma_stream(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                        lc_buf *output, uint32_t m, uint32_t kk, uint32_t n);
int lc_qgemv_mma_stream_group(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input, int count,
                              const lc_buf *const *weights, lc_buf *const *outputs, uint32_t m, uint32_t kk, uint32_t n);

int lc_qgemm_cuda_core(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input,
                       const lc_buf *weight, lc_buf *output, uint32_t m, uint32_t kk, uint32_t n) {
    if (n == 0) return LC_OK;
    if (k->mma && k->decode_mma && m <= 8) {
        const int st = lc_qgemv_mma_stream(fmt, f32out, k, b, input, weight, output, m, kk, n);
        if (st >= 0) return st;
    }
    const uint8_t *w = (const uint8_t *)weight->dptr;
    const __half *x = (const __half *)input->dptr;
    if (fmt == FMT_Q4_0) {
        const size_t wb = (size_t)(kk / 32) * 18 * n;
        if (f32out) return dispatch_qgemv<FMT_Q4_0, float>(k, b, w, wb, x, (float *)output->dptr, n, kk, m);
        return dispatch_qgemv<FMT_Q4_0, __half>(k, b, w, wb, x, (__half *)output->dptr, n, kk, m);
    }
    const size_t wb = (size_t)(kk / 256) * 66 * n;
    if (f32out) return dispatch_qgemv<FMT_TQ2_0, float>(k, b, w, wb, x, (float *)output->dptr, n, kk, m);
    return dispatch_qgemv<FMT_TQ2_0, __half>(k, b, w, wb, x, (__half *)output->dptr, n, kk, m);
}

extern "C" {

#define LC_MATVEC_PAIR(NAME, FMT, F32OUT)                                                                  \
    int NAME##_into(lc_kernels *k, lc_batch *b, const lc_buf *matrix, const lc_buf *vector, lc_buf *output, \
                    uint32_t rows, uint32_t cols) {                                                        \
        int st = check_qargs<FMT>(#NAME, k, b, matrix, vector, output, 1, cols, rows, F32OUT ? 4 : 2);     \
        if (st != LC_OK) return st;                                                                        \
        return lc_qgemm_cuda_core(FMT, F32OUT, k, b, vector, matrix, output, 1, cols, rows);               \
    }                                                                                                      \
    int NAME(lc_kernels *k, lc_ctx *ctx, const lc_buf *matrix, const lc_buf *vector, lc_buf *output,       \
             uint32_t rows, uint32_t cols) {                                                               \
        if (!ctx) return lc_fail(LC_ERR_INVALID_ARGUMENT, #NAME ": ctx is NULL");                          \
        return lc_run_and_wait(ctx, [&](lc_batch *b) {                                                     \
            return NAME##_into(k, b, matrix, vector, output, rows, cols);                                  \
        });                                                                                                \
    }

// Several matrices of one shape against the same vector, one output each, in one launch when the streaming
// tensor-core kernel applies (it treats them as one long run of 64-row groups), else one launch per matrix.
#define LC_MATVEC_GROUP(NAME, FMT)                                                                                \
    int NAME(lc_kernels *k, lc_batch *b, const lc_buf *const *matrices, uint32_t count, const lc_buf *vector,        \
             lc_buf *const *outputs, uint32_t rows, uint32_t cols) {                                                 \
        if (!matrices || !outputs) return lc_fail(LC_ERR_INVALID_ARGUMENT, #NAME ": NULL argument");                 \
        LC_REQUIRE(count >= 1 && count <= 96, #NAME ": count %u not in 1..=96", count);                             \
        for (uint32_t i = 0; i < count; i++) {                                                                       \
            int st = check_qargs<FMT>(#NAME, k, b, matrices[i], vector, outputs[i], 1, cols, rows, 2);              \
            if (st != LC_OK) return st;                                                                              \
        }                                                                                                            \
        if (rows == 0) return LC_OK;                                                                                 \
        if (k->mma && k->decode_mma) {                                                                               \
            const int st = lc_qgemv_mma_stream_group(FMT, false, k, b, vector, (int)count, matrices, outputs, 1, cols, rows); \
            if (st >= 0) return st;                                                                                  \
        }                                                                                                            \
        for (uint32_t i = 0; i < count; i++) {                                                                       \
            int st = lc_qgemm_cuda_core(FMT, false, k, b, vector, matrices[i], outputs[i], 1, cols, rows);          \
            if (st != LC_OK) return st;                                                                              \
        }                                                                                                            \
        return LC_OK;                                                                                                \
    }
LC_MATVEC_GROUP(lc_matvec_q4_0_group_into, FMT_Q4_0)
LC_MATVEC_GROUP(lc_matvec_tq2_0_group_into, FMT_TQ2_0)

LC_MATVEC_PAIR(lc_matvec_q4_0, FMT_Q4_0, false)
LC_MATVEC_PAIR(lc_matvec_q4_0_f32out, FMT_Q4_0, true)
LC_MATVEC_PAIR(lc_matvec_tq2_0, FMT_TQ2_0, false)
LC_MATVEC_PAIR(lc_matvec_tq2_0_f32out, FMT_TQ2_0, true)

int lc_matvec_tq2_0_soa_into(lc_kernels *k, lc_batch *b, const lc_buf *qs, const lc_buf *scales,
                             const lc_buf *vector, lc_buf *output, uint32_t rows, uint32_t cols) {
    if (!k || !b || !qs || !scales || !vector || !output)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_matvec_tq2_0_soa_into: NULL argument");
    if (cols == 0 || cols % 256 != 0)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "matvec_tq2_0_soa: cols %u not /256", cols);
    const size_t blocks = (size_t)rows * (cols / 256);
    LC_REQUIRE(qs->bytes >= blocks * 64 && scales->bytes >= blocks * 2, "matvec_tq2_0_soa: weight buffers too small");
    LC_REQUIRE(vector->bytes >= (size_t)cols * 2 && output->bytes >= (size_t)rows * 2,
               "matvec_tq2_0_soa: vector/output buffers too small");
    LC_REQUIRE(lc_aligned(qs->dptr, 4) && lc_aligned(vector->dptr, 4), "matvec_tq2_0_soa: buffers must be 4-byte aligned");
    if (rows == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(matvec_tq2_0_soa_kernel, dim3((rows + NWARPS - 1) / NWARPS), dim3(NTHREADS), 0, b, (const uint8_t *)qs->dptr, (const __half *)scales->dptr, (const __half *)vector->dptr,
        (__half *)output->dptr, (int)rows, (int)cols));
    LC_CHECK_LAUNCH("matvec_tq2_0_soa");
    b->dispatch_count++;
    return LC_OK;
}

int lc_multivec_nt_q4_0_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                             lc_buf *output, uint32_t m, uint32_t kk, uint32_t n) {
    int st = check_qargs<FMT_Q4_0>("multivec_nt_q4_0", k, b, weight, input, output, m, kk, n, 2);
    if (st != LC_OK) return st;
    // kernels.rs:6393-6398
    if (m < 1 || m > 16) return lc_fail(LC_ERR_INVALID_ARGUMENT, "multivec_nt_q4_0: m %u not in 1..=16", m);
    return lc_qgemm_cuda_core(FMT_Q4_0, false, k, b, input, weight, output, m, kk, n);
}

int lc_multivec_nt_tq2_0_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                              lc_buf *output, uint32_t m, uint32_t kk, uint32_t n) {
    int st = check_qargs<FMT_TQ2_0>("multivec_nt_tq2_0", k, b, weight, input, output, m, kk, n, 2);
    if (st != LC_OK) return st;
    if (m < 1 || m > 16) return lc_fail(LC_ERR_INVALID_ARGUMENT, "multivec_nt_tq2_0: m %u not in 1..=16", m);
    return lc_qgemm_cuda_core(FMT_TQ2_0, false, k, b, input, weight, output, m, kk, n);
}

int lc_tq2_dequant(lc_kernels *k, lc_ctx *ctx, const lc_buf *packed, const lc_buf *scales, lc_buf *output,
                   uint32_t num_elements) {
    if (!k || !ctx || !packed || !scales || !output)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_tq2_dequant: NULL argument");
    const size_t nbytes = ((size_t)num_elements + 3) / 4;
    LC_REQUIRE(packed->bytes >= nbytes && scales->bytes >= nbytes * 2 && output->bytes >= (size_t)num_elements * 2,
               "tq2_dequant: buffers too small for %u elements", num_elements);
    if (num_elements == 0) return LC_OK;
    return lc_run_and_wait(ctx, [&](lc_batch *b) {
        LC_LAUNCH_CHECKED(lc_launch(tq2_dequant_kernel, dim3((num_elements + 255) / 256), dim3(256), 0, b, (const uint8_t *)packed->dptr, (const __half *)scales->dptr, (__half *)output->dptr, num_elements));
        LC_CHECK_LAUNCH("tq2_dequant");
        b->dispatch_count++;
        return (int)LC_OK;
    });
}

}  // extern "C"

// Exposed for matmul routing.
int lc_check_qargs(int fmt, const char *name, lc_kernels *k, lc_batch *b, const lc_buf *w, const lc_buf *x,
                   const lc_buf *out, uint32_t m, uint32_t kk, uint32_t n, size_t out_elem) {
    return fmt == FMT_Q4_0 ? check_qargs<FMT_Q4_0>(name, k, b, w, x, out, m, kk, n, out_elem)
                           : check_qargs<FMT_TQ2_0>(name, k, b, w, x, out, m, kk, n, out_elem);
}
