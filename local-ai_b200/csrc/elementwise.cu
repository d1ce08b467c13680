// The small per-layer ops of a decode step.  Stand in for shaders/rms_norm.metal
// (:4-88), qk_norm.metal (:6-55), rope.metal (:14-53, :157-196), gelu.metal
// (:23-37), residual_add.metal, scale_in_place.metal (scale, gather_strided_f16,
// logit_softcap_f32), plus two device-side replacements for work the reference
// does on the CPU through unified memory: the embedding-row gather
// (local-engine/src/layer.rs:255-281) and greedy argmax (sampler.rs:148-158).
// All activations are f16 with f32 internals; every kernel rounds once on store.
#include <math.h>

#include "lc_internal.h"

namespace {

__device__ __forceinline__ float block_sum(float v, float *sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = (threadIdx.x < (unsigned)nw) ? sh[threadIdx.x] : 0.f;
    if (warp == 0) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) sh[0] = t;
    }
    __syncthreads();
    const float r = sh[0];
    __syncthreads();
    return r;
}

// out[row] = x * rsqrt(mean(x^2) + eps) * w (+ residual). One CTA per row.
// In-place (out == in) is allowed: each thread reads its elements before writing them.
__global__ void rms_norm_kernel(const __half *in, const __half *__restrict__ weight,
                                const __half *__restrict__ residual, __half *out, unsigned dim, float eps) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    __shared__ float sh[32];
    const size_t base = (size_t)blockIdx.x * dim;
    float s = 0.f;
    for (unsigned i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = __half2float(in[base + i]);
        s = fmaf(v, v, s);
    }
    s = block_sum(s, sh);
    const float rms = rsqrtf(s / (float)dim + eps);
    for (unsigned i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = __half2float(in[base + i]) * rms * __half2float(weight[i]);
        if (residual) v += __half2float(residual[base + i]);
        out[base + i] = __float2half_rn(v);
    }
}

// NEOX half-split RoPE; rows of [heads, hd]; position from positions[row] or the scalar.
__global__ void rope_kernel(const __half *in, __half *out, const uint32_t *__restrict__ positions,
                            unsigned position, float theta, unsigned hd, unsigned heads, unsigned rows, float factor,
                            int copy_tail) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    const unsigned half = hd / 2;
    const unsigned idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * heads * half) return;
    const unsigned i = idx % half, rh = idx / half;  // rh = row*heads + head
    const unsigned row = rh / heads;
    const size_t i0 = (size_t)rh * hd + i, i1 = i0 + half;
    const unsigned angles = (unsigned)((float)hd * factor) / 2;
    if (i >= angles) {
        if (copy_tail) {
            out[i0] = in[i0];
            out[i1] = in[i1];
        }
        return;
    }
    const float x0 = __half2float(in[i0]), x1 = __half2float(in[i1]);
    const float freq = 1.0f / powf(theta, (float)(2 * i) / (float)hd);
    const float ang = (float)(positions ? positions[row] : position) * freq;
    const float c = cosf(ang), s = sinf(ang);
    out[i0] = __float2half_rn(x0 * c - x1 * s);
    out[i1] = __float2half_rn(x0 * s + x1 * c);
}

__global__ void gelu_mul_kernel(const __half *a, const __half *b, __half *out, unsigned n) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x = __half2float(a[i]);
    const float x3 = x * x * x;
    float inner = 0.7978845608f * (x + 0.044715f * x3);
    inner = fminf(fmaxf(inner, -10.0f), 10.0f);
    const float g = 0.5f * x * (1.0f + tanhf(inner));
    out[i] = __float2half_rn(g * __half2float(b[i]));
}

__global__ void residual_add_kernel(const __half *a, const __half *b, __half *out, unsigned n) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2half_rn(__half2float(a[i]) + __half2float(b[i]));
}

__global__ void scale_in_place_kernel(__half *data, float scalar, unsigned n) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) data[i] = __float2half_rn(__half2float(data[i]) * scalar);
}

__global__ void logit_softcap_kernel(float *data, float cap, unsigned n) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) data[i] = cap * tanhf(data[i] / cap);
}

__global__ void gather_strided_kernel(const __half *__restrict__ src, __half *__restrict__ dst, unsigned row_stride,
                                      unsigned base_off, unsigned pld, unsigned n_rows) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    const unsigned gid = blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= n_rows * pld) return;
    const unsigned i = gid / pld, p = gid - i * pld;
    dst[gid] = src[(size_t)i * row_stride + base_off + p];
}

// out[r, :] = f16(f16((q-8)*d) * scale) for row tokens[r] of a Q4_0 table.
// Two roundings, like dequant-to-f16 followed by scale_in_place.
__global__ void embed_rows_q4_0_kernel(const uint8_t *__restrict__ table, const uint32_t *__restrict__ tokens,
                                       __half *__restrict__ out, unsigned cols, float scale, int apply_scale) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    const unsigned r = blockIdx.x;
    const size_t rb = (size_t)cols / 32 * 18;
    const uint8_t *row = table + (size_t)tokens[r] * rb;
    for (unsigned e = threadIdx.x; e < cols; e += blockDim.x) {
        const unsigned blk = e >> 5, j = e & 31;
        const uint8_t *p = row + (size_t)blk * 18;
        const float d = __half2float(*reinterpret_cast<const __half *>(p));
        const unsigned byte = p[2 + (j & 15)];
        const unsigned qv = j < 16 ? (byte & 15u) : (byte >> 4);
        __half h = __float2half_rn(((float)qv - 8.0f) * d);
        if (apply_scale) h = __float2half_rn(__half2float(h) * scale);
        out[(size_t)r * cols + e] = h;
    }
}

// First maximum of each row (strict '>' scan order => lowest index wins ties).
__global__ void argmax_rows_kernel(const float *__restrict__ v, uint32_t *__restrict__ out, unsigned cols) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    __shared__ float bv_s[32];
    __shared__ unsigned bi_s[32];
    const float *row = v + (size_t)blockIdx.x * cols;
    float bv = -INFINITY;
    unsigned bi = 0xffffffffu;
    for (unsigned i = threadIdx.x; i < cols; i += blockDim.x) {
        const float x = row[i];
        if (x > bv) { bv = x; bi = i; }
    }
    auto better = [](float a, unsigned ai, float b, unsigned bi2) { return a > b || (a == b && ai < bi2); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const unsigned oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { bv_s[warp] = bv; bi_s[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < nw ? bv_s[lane] : -INFINITY;
        bi = lane < nw ? bi_s[lane] : 0xffffffffu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const unsigned oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        // All -inf / NaN rows: the scalar scan returns index 0.
        if (lane == 0) out[blockIdx.x] = bi == 0xffffffffu ? 0u : bi;
    }
}

// The same for long rows (a vocabulary of logits): grid = (chunks, rows).  Every CTA scans one chunk of one row and
// stores its (value, index) candidate; the last CTA of a row to arrive (a counter that it resets) merges the
// candidates in chunk order, so ties still go to the lowest index.
__global__ void argmax_rows_chunked_kernel(const float *__restrict__ v, uint32_t *__restrict__ out, unsigned cols,
                                           unsigned chunk, float2 *__restrict__ cand, unsigned int *__restrict__ counters) {
    lc_pdl_trigger();
    lc_pdl_wait();
    __shared__ float bv_s[32];
    __shared__ unsigned bi_s[32];
    __shared__ unsigned int is_last;
    const unsigned r = blockIdx.y, c0 = blockIdx.x * chunk, c1 = min(cols, c0 + chunk);
    const float *row = v + (size_t)r * cols;
    float bv = -INFINITY;
    unsigned bi = 0xffffffffu;
    auto better = [](float a, unsigned ai, float b, unsigned bi2) { return a > b || (a == b && ai < bi2); };
    if ((((size_t)row & 15) == 0) && (c0 & 3) == 0) {
        const unsigned n4 = (c1 - c0) / 4;
        const float4 *p4 = reinterpret_cast<const float4 *>(row + c0);
        for (unsigned i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 x = __ldcs(p4 + i);
            const unsigned base = c0 + 4 * i;
            if (x.x > bv) { bv = x.x; bi = base; }
            if (x.y > bv) { bv = x.y; bi = base + 1; }
            if (x.z > bv) { bv = x.z; bi = base + 2; }
            if (x.w > bv) { bv = x.w; bi = base + 3; }
        }
        for (unsigned i = c0 + 4 * n4 + threadIdx.x; i < c1; i += blockDim.x) {
            const float x = row[i];
            if (better(x, i, bv, bi)) { bv = x; bi = i; }
        }
    } else {
        for (unsigned i = c0 + threadIdx.x; i < c1; i += blockDim.x) {
            const float x = row[i];
            if (x > bv) { bv = x; bi = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const unsigned oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { bv_s[warp] = bv; bi_s[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < nw ? bv_s[lane] : -INFINITY;
        bi = lane < nw ? bi_s[lane] : 0xffffffffu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const unsigned oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            cand[(size_t)r * gridDim.x + blockIdx.x] = make_float2(bv, __uint_as_float(bi));
            __threadfence();
            const unsigned int prev = atomicAdd(&counters[r], 1u);
            is_last = prev == gridDim.x - 1 ? 1u : 0u;
            if (is_last) counters[r] = 0u;
        }
    }
    __syncthreads();
    if (!is_last || warp != 0) return;
    __threadfence();
    bv = -INFINITY;
    bi = 0xffffffffu;
    for (unsigned c = lane; c < gridDim.x; c += 32) {
        const float2 q = __ldcg(cand + (size_t)r * gridDim.x + c);
        const unsigned qi = __float_as_uint(q.y);
        if (better(q.x, qi, bv, bi)) { bv = q.x; bi = qi; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const unsigned oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[r] = bi == 0xffffffffu ? 0u : bi;
}

// Fused per-head RMSNorm + NEOX RoPE in place (shaders/qk_norm.metal:70-144 qk_norm_rope): identical to
// qk_norm followed by rope_batch_decode, including the f16 rounding between the two.
// grid = rows * heads, block = head_dim / 2; thread i owns the pair (i, i + head_dim/2).
__global__ void qk_norm_rope_kernel(__half *qk, const __half *__restrict__ weight, const uint32_t *__restrict__ positions,
                                    float theta, unsigned hd, unsigned heads, float eps, float factor) {
    lc_pdl_trigger();
    lc_pdl_wait();
    __shared__ float sh[32];
    const unsigned half = hd / 2, i = threadIdx.x;
    const unsigned rh = blockIdx.x, row = rh / heads;
    __half *p = qk + (size_t)rh * hd;
    const float a = __half2float(p[i]), c = __half2float(p[i + half]);
    const float ss = block_sum(fmaf(a, a, c * c), sh);
    const float rms = rsqrtf(ss / (float)hd + eps);
    const float n0 = __half2float(__float2half_rn(a * rms * __half2float(weight[i])));
    const float n1 = __half2float(__float2half_rn(c * rms * __half2float(weight[i + half])));
    const unsigned angles = (unsigned)((float)hd * factor) / 2;
    if (i >= angles) {
        p[i] = __float2half_rn(n0);
        p[i + half] = __float2half_rn(n1);
        return;
    }
    const float freq = 1.0f / powf(theta, (float)(2 * i) / (float)hd);
    const float ang = (float)positions[row] * freq;
    const float cs = cosf(ang), sn = sinf(ang);
    p[i] = __float2half_rn(n0 * cs - n1 * sn);
    p[i + half] = __float2half_rn(n0 * sn + n1 * cs);
}

// Two dependent norms in one pass over a row (the pair every decoder layer issues back to back,
// local-engine/src/layer.rs:808-822, 843-853 + the next layer's attention norm):
//   resid  = f16(rms_norm(in, w1) + residual)           (rms_norm_add)
//   normed = f16(rms_norm(resid, w2))                   (rms_norm)
// The f16 `resid` row is kept in shared memory between the two.  grid = rows, dynamic smem = dim * 2 bytes.
__global__ void rms_norm_add_norm_kernel(const __half *in, const __half *__restrict__ w1, const __half *residual,
                                         __half *out_resid, const __half *__restrict__ w2, __half *out_normed,
                                         unsigned dim, float eps) {
    lc_pdl_trigger();
    lc_pdl_wait();
    extern __shared__ __align__(16) __half row_s[];
    __shared__ float sh[32];
    const size_t base = (size_t)blockIdx.x * dim;
    float s = 0.f;
    for (unsigned i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = __half2float(in[base + i]);
        s = fmaf(v, v, s);
    }
    s = block_sum(s, sh);
    const float rms1 = rsqrtf(s / (float)dim + eps);
    float s2 = 0.f;
    for (unsigned i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = __half2float(in[base + i]) * rms1 * __half2float(w1[i]) + __half2float(residual[base + i]);
        const __half h = __float2half_rn(v);
        row_s[i] = h;
        out_resid[base + i] = h;
        const float hv = __half2float(h);
        s2 = fmaf(hv, hv, s2);
    }
    s2 = block_sum(s2, sh);
    const float rms2 = rsqrtf(s2 / (float)dim + eps);
    for (unsigned i = threadIdx.x; i < dim; i += blockDim.x)
        out_normed[base + i] = __float2half_rn(__half2float(row_s[i]) * rms2 * __half2float(w2[i]));
}

// The same two norms for rows whose length is a multiple of 8 (at most 8192): one thread per 8 elements, every
// global load issued up front as a 16-byte access (the norm weights before the dependency wait), the row held in
// registers between the two norms.
__device__ __forceinline__ float block_sum_once(float v, float *sh) {   // `sh` must not be reused without a barrier
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < nw; w++) t += sh[w];
    return t;
}
__device__ __forceinline__ void unpack8(const uint4 &q, float (&f)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&q);
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const float2 v = __half22float2(h[e]);
        f[2 * e] = v.x;
        f[2 * e + 1] = v.y;
    }
}
__global__ void rms_norm_add_norm_vec_kernel(const __half *in, const __half *__restrict__ w1, const __half *residual,
                                             __half *out_resid, const __half *__restrict__ w2, __half *out_normed,
                                             unsigned dim, float eps) {
    lc_pdl_trigger();
    __shared__ float sh1[32], sh2[32];
    const unsigned i = threadIdx.x * 8;
    const bool live = i < dim;
    uint4 qw1 = make_uint4(0, 0, 0, 0), qw2 = qw1, qin = qw1, qres = qw1;
    if (live) {
        qw1 = *reinterpret_cast<const uint4 *>(w1 + i);
        qw2 = *reinterpret_cast<const uint4 *>(w2 + i);
    }
    lc_pdl_wait();
    const size_t base = (size_t)blockIdx.x * dim + i;
    if (live) {
        qin = *reinterpret_cast<const uint4 *>(in + base);
        qres = *reinterpret_cast<const uint4 *>(residual + base);
    }
    float x[8], r[8], a[8], c[8];
    unpack8(qin, x);
    unpack8(qres, r);
    unpack8(qw1, a);
    unpack8(qw2, c);
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < 8; e++) s = fmaf(x[e], x[e], s);
    const float rms1 = rsqrtf(block_sum_once(s, sh1) / (float)dim + eps);
    float s2 = 0.f;
    uint4 qo;
    __half2 *ho = reinterpret_cast<__half2 *>(&qo);
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
        ho[e / 2] = __floats2half2_rn(x[e] * rms1 * a[e] + r[e], x[e + 1] * rms1 * a[e + 1] + r[e + 1]);
        const float2 hv = __half22float2(ho[e / 2]);
        x[e] = hv.x;
        x[e + 1] = hv.y;
        s2 = fmaf(hv.x, hv.x, s2);
        s2 = fmaf(hv.y, hv.y, s2);
    }
    if (live) *reinterpret_cast<uint4 *>(out_resid + base) = qo;
    const float rms2 = rsqrtf(block_sum_once(live ? s2 : 0.f, sh2) / (float)dim + eps);
#pragma unroll
    for (int e = 0; e < 8; e += 2) ho[e / 2] = __floats2half2_rn(x[e] * rms2 * c[e], x[e + 1] * rms2 * c[e + 1]);
    if (live) *reinterpret_cast<uint4 *>(out_normed + base) = qo;
}

inline unsigned cdiv(unsigned a, unsigned b) { return (a + b - 1) / b; }

int rms_norm_common(const char *name, lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                    const lc_buf *residual, lc_buf *output, uint32_t dim, uint32_t rows, float eps) {
    if (!k || !b || !input || !weight || !output) return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    LC_REQUIRE(dim >= 1, "%s: dim must be >= 1", name);
    const size_t n = (size_t)dim * rows * 2;
    LC_REQUIRE(input->bytes >= n && output->bytes >= n && weight->bytes >= (size_t)dim * 2 &&
                   (!residual || residual->bytes >= n),
               "%s: buffers too small for %u rows of %u", name, rows, dim);
    if (rows == 0) return LC_OK;
    const unsigned threads = dim >= 1024 ? 512 : (dim >= 256 ? 256 : 64);
    LC_LAUNCH_CHECKED(lc_launch(rms_norm_kernel, dim3(rows), dim3(threads), 0, b, (const __half *)input->dptr, (const __half *)weight->dptr,
                                                     residual ? (const __half *)residual->dptr : nullptr,
                                                     (__half *)output->dptr, dim, eps));
    LC_CHECK_LAUNCH(name);
    b->dispatch_count++;
    return LC_OK;
}

}  // namespace

extern "C" {

int lc_rms_norm_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight, lc_buf *output,
                     uint32_t dim, uint32_t rows, float eps) {
    return rms_norm_common("rms_norm", k, b, input, weight, nullptr, output, dim, rows, eps);
}

int lc_rms_norm_add_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                         const lc_buf *residual, lc_buf *output, uint32_t dim, uint32_t rows, float eps) {
    if (!residual) return lc_fail(LC_ERR_INVALID_ARGUMENT, "rms_norm_add: residual is NULL");
    return rms_norm_common("rms_norm_add", k, b, input, weight, residual, output, dim, rows, eps);
}

int lc_qk_norm_gpu_into(lc_kernels *k, lc_batch *b, lc_buf *qk_data, const lc_buf *weight, uint32_t head_dim,
                        uint32_t num_heads, float eps) {
    return rms_norm_common("qk_norm", k, b, qk_data, weight, nullptr, qk_data, head_dim, num_heads, eps);
}

int lc_rope_into(lc_kernels *k, lc_batch *b, const lc_buf *input, lc_buf *output, uint32_t head_dim,
                 uint32_t position, float theta, float partial_rotary_factor, uint32_t num_heads) {
    if (!k || !b || !input || !output) return lc_fail(LC_ERR_INVALID_ARGUMENT, "rope: NULL argument");
    LC_REQUIRE(head_dim >= 2 && head_dim % 2 == 0, "rope: head_dim %u must be even", head_dim);
    const size_t n = (size_t)head_dim * num_heads * 2;
    LC_REQUIRE(input->bytes >= n && output->bytes >= n, "rope: buffers too small");
    const unsigned total = num_heads * (head_dim / 2);
    if (total == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(rope_kernel, dim3(cdiv(total, 256)), dim3(256), 0, b, (const __half *)input->dptr, (__half *)output->dptr, nullptr,
                                                         position, theta, head_dim, num_heads, 1,
                                                         partial_rotary_factor, 1));
    LC_CHECK_LAUNCH("rope");
    b->dispatch_count++;
    return LC_OK;
}

int lc_rope_batch_decode_into(lc_kernels *k, lc_batch *b, lc_buf *qk, const lc_buf *positions, float theta,
                              uint32_t head_dim, uint32_t num_heads, uint32_t seq_len, float partial_rotary_factor) {
    if (!k || !b || !qk || !positions) return lc_fail(LC_ERR_INVALID_ARGUMENT, "rope_batch_decode: NULL argument");
    LC_REQUIRE(head_dim >= 2 && head_dim % 2 == 0, "rope_batch_decode: head_dim %u must be even", head_dim);
    LC_REQUIRE(qk->bytes >= (size_t)seq_len * num_heads * head_dim * 2 && positions->bytes >= (size_t)seq_len * 4,
               "rope_batch_decode: buffers too small");
    const unsigned total = seq_len * num_heads * (head_dim / 2);
    if (total == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(rope_kernel, dim3(cdiv(total, 256)), dim3(256), 0, b, (const __half *)qk->dptr, (__half *)qk->dptr,
                                                         (const uint32_t *)positions->dptr, 0, theta, head_dim,
                                                         num_heads, seq_len, partial_rotary_factor, 0));
    LC_CHECK_LAUNCH("rope_batch_decode");
    b->dispatch_count++;
    return LC_OK;
}

int lc_gelu_mul_into(lc_kernels *k, lc_batch *b, const lc_buf *a, const lc_buf *bb, lc_buf *out, uint32_t count) {
    if (!k || !b || !a || !bb || !out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "gelu_mul: NULL argument");
    const size_t n = (size_t)count * 2;
    LC_REQUIRE(a->bytes >= n && bb->bytes >= n && out->bytes >= n, "gelu_mul: buffers too small for %u", count);
    if (count == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(gelu_mul_kernel, dim3(cdiv(count, 256)), dim3(256), 0, b, (const __half *)a->dptr, (const __half *)bb->dptr,
                                                             (__half *)out->dptr, count));
    LC_CHECK_LAUNCH("gelu_mul");
    b->dispatch_count++;
    return LC_OK;
}

int lc_residual_add_into(lc_kernels *k, lc_batch *b, const lc_buf *a, const lc_buf *bb, lc_buf *output,
                         uint32_t count) {
    if (!k || !b || !a || !bb || !output) return lc_fail(LC_ERR_INVALID_ARGUMENT, "residual_add: NULL argument");
    const size_t n = (size_t)count * 2;
    LC_REQUIRE(a->bytes >= n && bb->bytes >= n && output->bytes >= n, "residual_add: buffers too small for %u", count);
    if (count == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(residual_add_kernel, dim3(cdiv(count, 256)), dim3(256), 0, b, (const __half *)a->dptr, (const __half *)bb->dptr,
                                                                 (__half *)output->dptr, count));
    LC_CHECK_LAUNCH("residual_add");
    b->dispatch_count++;
    return LC_OK;
}

int lc_scale_in_place_gpu_into(lc_kernels *k, lc_batch *b, lc_buf *data, float scalar, uint32_t count) {
    if (!k || !b || !data) return lc_fail(LC_ERR_INVALID_ARGUMENT, "scale_in_place: NULL argument");
    LC_REQUIRE(data->bytes >= (size_t)count * 2, "scale_in_place: buffer too small for %u", count);
    if (count == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(scale_in_place_kernel, dim3(cdiv(count, 256)), dim3(256), 0, b, (__half *)data->dptr, scalar, count));
    LC_CHECK_LAUNCH("scale_in_place");
    b->dispatch_count++;
    return LC_OK;
}

int lc_logit_softcap_gpu_into(lc_kernels *k, lc_batch *b, lc_buf *data, float cap, uint32_t count) {
    if (!k || !b || !data) return lc_fail(LC_ERR_INVALID_ARGUMENT, "logit_softcap: NULL argument");
    LC_REQUIRE(data->bytes >= (size_t)count * 4, "logit_softcap: buffer too small for %u", count);
    if (count == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(logit_softcap_kernel, dim3(cdiv(count, 256)), dim3(256), 0, b, (float *)data->dptr, cap, count));
    LC_CHECK_LAUNCH("logit_softcap");
    b->dispatch_count++;
    return LC_OK;
}

int lc_gather_strided_f16_into(lc_kernels *k, lc_batch *b, const lc_buf *src, lc_buf *dst, uint32_t row_stride,
                               uint32_t base_off, uint32_t pld, uint32_t n_rows) {
    if (!k || !b || !src || !dst) return lc_fail(LC_ERR_INVALID_ARGUMENT, "gather_strided_f16: NULL argument");
    if (n_rows == 0 || pld == 0) return LC_OK;
    LC_REQUIRE(src->bytes >= ((size_t)(n_rows - 1) * row_stride + base_off + pld) * 2 &&
                   dst->bytes >= (size_t)n_rows * pld * 2,
               "gather_strided_f16: buffers too small");
    LC_LAUNCH_CHECKED(lc_launch(gather_strided_kernel, dim3(cdiv(n_rows * pld, 256)), dim3(256), 0, b, (const __half *)src->dptr, (__half *)dst->dptr, row_stride, base_off, pld, n_rows));
    LC_CHECK_LAUNCH("gather_strided_f16");
    b->dispatch_count++;
    return LC_OK;
}

int lc_embed_rows_q4_0_into(lc_kernels *k, lc_batch *b, const lc_buf *table, const lc_buf *tokens, lc_buf *output,
                            uint32_t n_rows, uint32_t cols, uint32_t vocab, float scale) {
    if (!k || !b || !table || !tokens || !output) return lc_fail(LC_ERR_INVALID_ARGUMENT, "embed_rows_q4_0: NULL argument");
    if (cols == 0 || cols % 32 != 0) return lc_fail(LC_ERR_INVALID_ARGUMENT, "embed_rows_q4_0: cols %u not /32", cols);
    LC_REQUIRE(table->bytes >= (size_t)vocab * (cols / 32) * 18 && tokens->bytes >= (size_t)n_rows * 4 &&
                   output->bytes >= (size_t)n_rows * cols * 2,
               "embed_rows_q4_0: buffers too small");
    if (n_rows == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(embed_rows_q4_0_kernel, dim3(n_rows), dim3(256), 0, b, (const uint8_t *)table->dptr, (const uint32_t *)tokens->dptr,
                                                          (__half *)output->dptr, cols, scale, scale != 1.0f));
    LC_CHECK_LAUNCH("embed_rows_q4_0");
    b->dispatch_count++;
    return LC_OK;
}

int lc_argmax_rows_f32_into(lc_kernels *k, lc_batch *b, const lc_buf *values, lc_buf *out_index, uint32_t rows,
                            uint32_t cols) {
    if (!k || !b || !values || !out_index) return lc_fail(LC_ERR_INVALID_ARGUMENT, "argmax_rows_f32: NULL argument");
    LC_REQUIRE(cols >= 1, "argmax_rows_f32: cols must be >= 1");
    LC_REQUIRE(values->bytes >= (size_t)rows * cols * 4 && out_index->bytes >= (size_t)rows * 4,
               "argmax_rows_f32: buffers too small");
    if (rows == 0) return LC_OK;
    if (cols >= 32768 && rows <= 65535) {
        // long rows: enough chunks that every SM streams a share of the logits
        unsigned chunks = (4u * (unsigned)k->ctx->sm_count + rows - 1) / rows;
        if (chunks > 64) chunks = 64;
        unsigned chunk = ((cols + chunks - 1) / chunks + 1023u) & ~1023u;
        chunks = (cols + chunk - 1) / chunk;
        int st = lc_reserve_scratch(k, b, (size_t)rows * chunks * sizeof(float2), rows);
        if (st != LC_OK) return st;
        LC_LAUNCH_CHECKED(lc_launch(argmax_rows_chunked_kernel, dim3(chunks, rows), dim3(256), 0, b, (const float *)values->dptr,
                                    (uint32_t *)out_index->dptr, cols, chunk, (float2 *)k->scratch, k->counters));
        b->dispatch_count++;
        return LC_OK;
    }
    LC_LAUNCH_CHECKED(lc_launch(argmax_rows_kernel, dim3(rows), dim3(1024), 0, b, (const float *)values->dptr, (uint32_t *)out_index->dptr, cols));
    LC_CHECK_LAUNCH("argmax_rows_f32");
    b->dispatch_count++;
    return LC_OK;
}


int lc_qk_norm_rope_batch_decode_into(lc_kernels *k, lc_batch *b, lc_buf *qk, const lc_buf *weight, const lc_buf *positions,
                                      float theta, uint32_t head_dim, uint32_t num_heads, uint32_t seq_len, float eps,
                                      float partial_rotary_factor) {
    if (!k || !b || !qk || !weight || !positions) return lc_fail(LC_ERR_INVALID_ARGUMENT, "qk_norm_rope: NULL argument");
    LC_REQUIRE(head_dim >= 2 && head_dim % 2 == 0 && head_dim <= 2048, "qk_norm_rope: head_dim %u must be even and <= 2048", head_dim);
    LC_REQUIRE(qk->bytes >= (size_t)seq_len * num_heads * head_dim * 2 && positions->bytes >= (size_t)seq_len * 4 &&
                   weight->bytes >= head_dim * 2u,
               "qk_norm_rope: buffers too small");
    if (seq_len * num_heads == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(qk_norm_rope_kernel, dim3(seq_len * num_heads), dim3(head_dim / 2), 0, b, (__half *)qk->dptr,
                                (const __half *)weight->dptr, (const uint32_t *)positions->dptr, theta, head_dim, num_heads,
                                eps, partial_rotary_factor));
    b->dispatch_count++;
    return LC_OK;
}

int lc_rms_norm_add_norm_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight, const lc_buf *residual,
                              lc_buf *out_residual, const lc_buf *weight2, lc_buf *out_normed, uint32_t dim, uint32_t rows,
                              float eps) {
    if (!k || !b || !input || !weight || !residual || !out_residual || !weight2 || !out_normed)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "rms_norm_add_norm: NULL argument");
    LC_REQUIRE(dim >= 1 && dim <= 32768, "rms_norm_add_norm: dim %u out of range", dim);
    const size_t n = (size_t)dim * rows * 2;
    LC_REQUIRE(input->bytes >= n && residual->bytes >= n && out_residual->bytes >= n && out_normed->bytes >= n &&
                   weight->bytes >= (size_t)dim * 2 && weight2->bytes >= (size_t)dim * 2,
               "rms_norm_add_norm: buffers too small for %u rows of %u", rows, dim);
    if (rows == 0) return LC_OK;
    if (dim % 8 == 0 && dim <= 8192 && lc_aligned(input->dptr, 16) && lc_aligned(residual->dptr, 16) &&
        lc_aligned(out_residual->dptr, 16) && lc_aligned(out_normed->dptr, 16) && lc_aligned(weight->dptr, 16) &&
        lc_aligned(weight2->dptr, 16)) {
        const unsigned vthreads = ((dim / 8 + 31) / 32) * 32;
        LC_LAUNCH_CHECKED(lc_launch(rms_norm_add_norm_vec_kernel, dim3(rows), dim3(vthreads), 0, b, (const __half *)input->dptr,
                                    (const __half *)weight->dptr, (const __half *)residual->dptr, (__half *)out_residual->dptr,
                                    (const __half *)weight2->dptr, (__half *)out_normed->dptr, dim, eps));
        b->dispatch_count++;
        return LC_OK;
    }
    const unsigned threads = dim >= 1024 ? 512 : (dim >= 256 ? 256 : 64);
    const size_t smem = (size_t)dim * 2;
    static lc_smem_optin optin;
    LC_CUDA_TRY(lc_ensure_smem(rms_norm_add_norm_kernel, optin, b->ctx, smem));
    LC_LAUNCH_CHECKED(lc_launch(rms_norm_add_norm_kernel, dim3(rows), dim3(threads), smem, b, (const __half *)input->dptr,
                                (const __half *)weight->dptr, (const __half *)residual->dptr, (__half *)out_residual->dptr,
                                (const __half *)weight2->dptr, (__half *)out_normed->dptr, dim, eps));
    b->dispatch_count++;
    return LC_OK;
}

}  // extern "C"
