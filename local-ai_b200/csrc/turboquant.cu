// TurboQuant KV rows on the GPU: encode (single + per-lane batched), dequantize,
// and the randomized-Hadamard rotation.  Stands in for
// shaders/dequantize_kv.metal:119-407 and shaders/attention_flash_tq.metal:50-139;
// the host-side codec set-up mirrors local-engine/src/turboquant.rs:66-80,114-199.
//
// Bit-exactness contract: with kv_norm_mode 0 the encode kernel reproduces
// TurboQuant::encode_into (turboquant.rs:241-276) bit for bit on identical
// inputs — the sum of squares is accumulated sequentially in index order with
// separately rounded multiply and add, the reciprocal, square root and 1/sqrt(d)
// are IEEE-rounded, and no multiply-add is fused.  Mode 1 sums in the Metal
// kernel's pairwise order (dequantize_kv.metal:247-257) instead.  The
// butterflies compute the same a+b / a-b pairs as the CPU loop, in any order.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "lc_internal.h"
#include "attention_tq.h"

namespace {

constexpr int MAX_HD = 512;

__device__ __forceinline__ unsigned tq_unpack(const uint8_t *codes, unsigned d, unsigned bits) {
    const unsigned bit_off = d * bits;
    const unsigned byte = bit_off >> 3, shift = bit_off & 7u;
    unsigned v = codes[byte];
    if (shift + bits > 8u) v |= (unsigned)codes[byte + 1] << 8;
    return (v >> shift) & ((1u << bits) - 1u);
}

// One CTA of `hd` threads per (token|lane, kv head) row.
//   slot rule, single sequence (BATCHED == false), dequantize_kv.metal:236-244:
//     ring ? ((position + tok) % ring) * n_kv + head : (position + tok) * n_kv + head
//   slot rule, per lane (BATCHED == true), dequantize_kv.metal:349-351:
//     (lane * lane_capacity + (ring ? pos % ring : pos)) * n_kv + head
// Encode one row held one element per thread (xv) into `packed_row` / `*norm_out`.
// sh/red/code_sh are MAX_HD-sized shared arrays, norm_sh one shared float.  Block = hd threads.
__device__ __forceinline__ void encode_row(float xv, unsigned t, unsigned hd, unsigned bits,
                                           const float *__restrict__ levels, const float *__restrict__ signs,
                                           int norm_mode, uint8_t *__restrict__ packed_row, __half *__restrict__ norm_out,
                                           float *sh, float *red, unsigned *code_sh, float *norm_sh) {
    const unsigned code_bytes = (hd * bits + 7) >> 3;
    red[t] = __fmul_rn(xv, xv);
    __syncthreads();
    if (norm_mode == 0) {
        if (t == 0) {
            // the reference's sequential f32 sum, in index order: the additions are a dependent chain, the loads
            // are not (16 values per round as four 16-byte loads; hd is a multiple of 32)
            const float4 *r4 = reinterpret_cast<const float4 *>(red);
            float s = 0.f;
            for (unsigned i = 0; i < hd / 4; i += 4) {
                const float4 a = r4[i], b = r4[i + 1], c = r4[i + 2], e = r4[i + 3];
                s = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(s, a.x), a.y), a.z), a.w);
                s = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(s, b.x), b.y), b.z), b.w);
                s = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(s, c.x), c.y), c.z), c.w);
                s = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(s, e.x), e.y), e.z), e.w);
            }
            *norm_sh = __fsqrt_rn(s);
        }
    } else {
        for (unsigned stride = hd >> 1; stride > 0; stride >>= 1) {
            if (t < stride) red[t] = __fadd_rn(red[t], red[t + stride]);
            __syncthreads();
        }
        if (t == 0) *norm_sh = __fsqrt_rn(red[0]);
    }
    __syncthreads();
    const float norm = *norm_sh;
    float v = xv;
    if (norm > 0.f) v = __fmul_rn(xv, __fdiv_rn(1.0f, norm));
    else if (norm_mode == 1) v = __fmul_rn(xv, 0.f);
    const float rotated = lc_fwht_value(__fmul_rn(v, signs[t]), sh, hd, t);
    const float inv_sqrt_d = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));
    const float y = __fmul_rn(rotated, inv_sqrt_d);

    const unsigned k = 1u << bits;
    unsigned best = 0;
    float bd = INFINITY;
    for (unsigned i = 0; i < k; i++) {
        const float dd = fabsf(__fsub_rn(y, levels[i]));
        if (dd < bd) { bd = dd; best = i; }
    }
    if (t == 0) *norm_out = __float2half_rn(norm);
    // LSB-first packing: code i of the row sits at bit i * bits
    if (bits != 3) {
        // 2- and 4-bit codes never straddle a byte: the 8 / bits neighbouring lanes of a warp OR their codes together
        const unsigned per = 8 / bits;
        unsigned byte_val = best << (bits * (t & (per - 1)));
        for (unsigned o = 1; o < per; o <<= 1) byte_val |= __shfl_xor_sync(0xffffffffu, byte_val, o);
        if ((t & (per - 1)) == 0) packed_row[t / per] = (uint8_t)byte_val;
        return;
    }
    code_sh[t] = best;
    __syncthreads();
    // one thread per output byte
    if (t < code_bytes) {
        unsigned byte_val = 0;
        for (unsigned bp = 0; bp < 8; bp++) {
            const unsigned gb = t * 8 + bp;
            const unsigned ci = gb / bits;
            if (ci >= hd) break;
            byte_val |= ((code_sh[ci] >> (gb - ci * bits)) & 1u) << bp;
        }
        packed_row[t] = (uint8_t)byte_val;
    }
}

template <bool BATCHED>
__global__ void encode_kv_kernel(const __half *__restrict__ input, const float *__restrict__ levels,
                                 const float *__restrict__ signs, uint8_t *__restrict__ packed,
                                 __half *__restrict__ norms, const uint32_t *__restrict__ positions,
                                 unsigned hd, unsigned n_kv, unsigned lane_capacity, unsigned bits,
                                 unsigned position, unsigned ring, int norm_mode, int *status) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    __shared__ float sh[MAX_HD];
    __shared__ __align__(16) float red[MAX_HD];
    __shared__ unsigned code_sh[MAX_HD];
    __shared__ float norm_sh;
    const unsigned t = threadIdx.x, g_in = blockIdx.x;
    const unsigned row = g_in / n_kv, head = g_in - row * n_kv;
    size_t slot;
    if (BATCHED) {
        const unsigned pos = positions[row];
        const unsigned ppos = ring ? pos % ring : pos;
        if (ppos >= lane_capacity) {   // a device-resident position past the lane's rows: write nothing, report
            if (t == 0) atomicExch(status, LC_DEV_STATUS_POSITION);
            return;
        }
        slot = ((size_t)row * lane_capacity + ppos) * n_kv + head;
    } else {
        const unsigned logical = position + row;
        slot = (size_t)(ring ? logical % ring : logical) * n_kv + head;
    }
    const unsigned code_bytes = (hd * bits + 7) >> 3;
    const float xv = __half2float(input[(size_t)g_in * hd + t]);
    encode_row(xv, t, hd, bits, levels, signs, norm_mode, packed + slot * code_bytes, norms + slot, sh, red, code_sh,
               &norm_sh);
}

// Everything between the Q/K/V projections and attention for one decode step, in one launch: per-head RMSNorm
// (learned weights for Q and K, unit weights for V), NEOX RoPE on Q and K, TurboQuant encode of the K and V rows
// into the per-lane pools.  Same arithmetic and the same f16 rounding points as the separate dispatches of
// layer.rs:773-790 + quant_unified_pool.rs:138-181.  One CTA per (lane, head, role): grid = (n_lanes,
// n_q + 2 n_kv), block = head_dim; n_q = 0 leaves the queries alone.
__global__ void kv_write_kernel(__half *q, const __half *__restrict__ q_norm_w, unsigned n_q,
                                const __half *__restrict__ kin, const __half *__restrict__ vin,
                                const __half *__restrict__ k_norm_w, const uint32_t *__restrict__ positions,
                                const float *__restrict__ levels, const float *__restrict__ signs,
                                uint8_t *__restrict__ k_packed, __half *__restrict__ k_norms,
                                uint8_t *__restrict__ v_packed, __half *__restrict__ v_norms, unsigned hd, unsigned n_kv,
                                unsigned lane_capacity, unsigned bits, unsigned ring, float eps, float theta,
                                float rotary_factor, int norm_mode, int *status, uint4 *qfrag, float q_scale) {
    lc_pdl_trigger();
    __shared__ float sh[MAX_HD];
    __shared__ __align__(16) float red[MAX_HD];
    __shared__ unsigned code_sh[MAX_HD];
    __shared__ float norm_sh;
    __shared__ float red2[32];
    const unsigned t = threadIdx.x, row = blockIdx.x, r = blockIdx.y;
    const int role = r < n_q ? 0 : (r < n_q + n_kv ? 1 : 2);   // Q, K, V
    const unsigned head = role == 0 ? r : (role == 1 ? r - n_q : r - n_q - n_kv);
    // norm weight and rotation frequency do not depend on the predecessor
    float w = 1.0f;
    if (role == 0) w = __half2float(q_norm_w[t]);
    else if (role == 1) w = __half2float(k_norm_w[t]);
    const unsigned half = hd / 2, i = t < half ? t : t - half;
    const unsigned angles = (unsigned)((float)hd * rotary_factor) / 2;
    const bool rotate = role != 2 && i < angles;
    const float freq = rotate ? 1.0f / powf(theta, (float)(2 * i) / (float)hd) : 0.f;
    lc_pdl_wait();
    const unsigned pos = positions[row];
    __half *qrow = q + ((size_t)row * n_q + head) * hd;
    const size_t g_in = (size_t)row * n_kv + head;
    const float x = __half2float(role == 0 ? qrow[t] : (role == 1 ? kin[g_in * hd + t] : vin[g_in * hd + t]));
    float ss = x * x;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((t & 31) == 0) red2[t >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (unsigned wi = 0; wi < (hd + 31) / 32; wi++) tot += red2[wi];
    const float rms = rsqrtf(tot / (float)hd + eps);
    const float xn = __half2float(__float2half_rn(x * rms * w));
    float xr = xn;
    if (role != 2) {
        sh[t] = xn;
        __syncthreads();
        if (rotate) {
            const float x0 = sh[i], x1 = sh[i + half];
            const float ang = (float)pos * freq;
            const float c = cosf(ang), sn = sinf(ang);
            xr = __half2float(__float2half_rn(t < half ? x0 * c - x1 * sn : x0 * sn + x1 * c));
        }
        // `sh` is next written two barriers further on (encode_row); the query path below uses `red` instead
    }
    if (role == 0) {
        qrow[t] = __float2half_rn(xr);
        if (qfrag) {
            // The tensor-core attention kernel's first steps, done here where the row is already in registers: signs,
            // 256-point Walsh-Hadamard transform, softmax scale / sqrt(hd), split into an f16 and the f16 of the
            // remainder, stored in that kernel's fragment order (hd == 256 and heads in groups of 8: host-checked).
            // Same operations in the same order as the kernel's own prologue, so attention results do not change.
            const float rotated = lc_fwht_value(__fmul_rn(xr, signs[t]), red, hd, t);
            const float v = __fmul_rn(rotated, __fdiv_rn(q_scale, __fsqrt_rn((float)hd)));
            const __half hi = __float2half_rn(v), lo = __float2half_rn(__fsub_rn(v, __half2float(hi)));
            const uint32_t own = (uint32_t)__half_as_ushort(hi) | ((uint32_t)__half_as_ushort(lo) << 16);
            const uint32_t p1 = __shfl_down_sync(0xffffffffu, own, 1), p2 = __shfl_down_sync(0xffffffffu, own, 2),
                           p3 = __shfl_down_sync(0xffffffffu, own, 3);
            if ((t & 3) == 0) {
                uint4 e;
                e.x = (own & 0xFFFFu) | (p1 << 16);
                e.y = (p2 & 0xFFFFu) | (p3 << 16);
                e.z = (own >> 16) | (p1 & 0xFFFF0000u);
                e.w = (p2 >> 16) | (p3 & 0xFFFF0000u);
                qfrag[((size_t)row * (n_q >> 3) + (head >> 3)) * 512 + ((t & 63) >> 2) * 32 + 4 * (head & 7) + (t >> 6)] = e;
            }
        }
        return;
    }
    const unsigned ppos = ring ? pos % ring : pos;
    if (ppos >= lane_capacity) {   // a device-resident position past the lane's rows: write nothing, report
        if (t == 0) atomicExch(status, LC_DEV_STATUS_POSITION);
        return;
    }
    const size_t slot = ((size_t)row * lane_capacity + ppos) * n_kv + head;
    const unsigned code_bytes = (hd * bits + 7) >> 3;
    encode_row(xr, t, hd, bits, levels, signs, norm_mode, (role == 1 ? k_packed : v_packed) + slot * code_bytes,
               (role == 1 ? k_norms : v_norms) + slot, sh, red, code_sh, &norm_sh);
}

// dequantize_kv.metal:132-189. grid = n_kv * (num_tokens - token_start).
__global__ void dequantize_kv_kernel(const uint8_t *__restrict__ packed, const __half *__restrict__ norms,
                                     const float *__restrict__ levels, const float *__restrict__ signs,
                                     __half *__restrict__ output, unsigned hd, unsigned n_kv, unsigned bits,
                                     unsigned group_offset, unsigned ring) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    __shared__ float sh[MAX_HD];
    const unsigned t = threadIdx.x;
    const size_t g = (size_t)blockIdx.x + group_offset;
    size_t src = g;
    if (ring) {
        const size_t token = g / n_kv, head = g - token * n_kv;
        src = (token % ring) * n_kv + head;
    }
    const unsigned code_bytes = (hd * bits + 7) >> 3;
    const float rotated = lc_fwht_value(levels[tq_unpack(packed + src * code_bytes, t, bits)], sh, hd, t);
    const float inv_sqrt_d = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));
    const float norm = __half2float(norms[src]);
    output[g * hd + t] = __float2half_rn(rotated * inv_sqrt_d * signs[t] * norm);
}

__device__ __forceinline__ float ld_as_float(const float *p) { return *p; }
__device__ __forceinline__ float ld_as_float(const __half *p) { return __half2float(*p); }
__device__ __forceinline__ void st_from_float(float *p, float v) { *p = v; }
__device__ __forceinline__ void st_from_float(__half *p, float v) { *p = __float2half_rn(v); }

// attention_flash_tq.metal:58-89. grid = num_heads, block = head_dim.
template <typename TIn, typename TOut>
__global__ void hadamard_rotate_kernel(const TIn *__restrict__ input, const float *__restrict__ signs,
                                       TOut *__restrict__ output, unsigned hd, unsigned pre, unsigned post) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    __shared__ float sh[MAX_HD];
    const unsigned t = threadIdx.x;
    const size_t base = (size_t)blockIdx.x * hd;
    const float x = ld_as_float(input + base + t);
    float y = lc_fwht_value(pre ? x * signs[t] : x, sh, hd, t) * __fdiv_rn(1.0f, __fsqrt_rn((float)hd));
    if (post) y *= signs[t];
    st_from_float(output + base + t, y);
}

bool pow2(unsigned v) { return v && !(v & (v - 1)); }

int check_codec(const char *name, unsigned hd, unsigned bits) {
    // kv_cache/quant_cache.rs:191-200: bits in 2..=4, head_dim a power of two <= 512.
    if (bits < 2 || bits > 4) return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: bits %u not in 2..=4", name, bits);
    if (!pow2(hd) || hd > MAX_HD || hd < 32)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: head_dim %u must be a power of two in 32..=512", name, hd);
    return LC_OK;
}

template <typename TIn, typename TOut>
int rotate_into(const char *name, lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *signs,
                lc_buf *output, uint32_t hd, uint32_t heads, uint32_t pre, uint32_t post) {
    if (!k || !b || !input || !signs || !output) return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    int st = check_codec(name, hd, 2);
    if (st != LC_OK) return st;
    const size_t n = (size_t)hd * heads;
    LC_REQUIRE(input->bytes >= n * sizeof(TIn) && output->bytes >= n * sizeof(TOut) && signs->bytes >= hd * 4,
               "%s: buffers too small for %u heads of %u", name, heads, hd);
    if (heads == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(hadamard_rotate_kernel<TIn, TOut>, dim3(heads), dim3(hd), 0, b, (const TIn *)input->dptr, (const float *)signs->dptr, (TOut *)output->dptr, hd, pre, post));
    LC_CHECK_LAUNCH(name);
    b->dispatch_count++;
    return LC_OK;
}

}  // namespace

extern "C" {

// ---- host-side codec set-up (what TurboQuant::new computes on the CPU) ----
size_t lc_tq_code_bytes(uint32_t head_dim, uint32_t bits) { return ((size_t)head_dim * bits + 7) / 8; }

int lc_tq_signs(uint32_t dim, uint64_t seed, float *signs) {
    if (!signs) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_tq_signs: signs is NULL");
    uint64_t state = seed | 1ull;
    for (uint32_t i = 0; i < dim; i++) {
        state += 0x9E3779B97F4A7C15ull;
        uint64_t z = state;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        signs[i] = (z & 1ull) ? -1.0f : 1.0f;
    }
    return LC_OK;
}

int lc_tq_levels(uint32_t dim, uint32_t bits, float *levels) {
    if (!levels) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_tq_levels: levels is NULL");
    if (bits < 1 || bits > 4) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_tq_levels: bits %u not in 1..=4", bits);
    // Lloyd-Max centroids of N(0,1): 8192-cell midpoint grid on [-6, 6], 100
    // sweeps, all in f32 with the two fused multiply-adds the Rust code asks for.
    const int N = 8192;
    const uint32_t k = 1u << bits;
    const float lo = -6.0f, hi = 6.0f;
    const float dx = (hi - lo) / (float)N;
    float *xs = new float[N], *pdf = new float[N];
    for (int i = 0; i < N; i++) {
        xs[i] = fmaf((float)i + 0.5f, dx, lo);
        const float x = xs[i];
        pdf[i] = expf(-0.5f * x * x) * 0.70710678118654752440f * 1.12837916709551257390f / 2.0f;
    }
    for (uint32_t i = 0; i < k; i++) levels[i] = 6.0f * ((((float)i + 0.5f) / (float)k) - 0.5f);
    float sum[16], wsum[16];
    for (int it = 0; it < 100; it++) {
        for (uint32_t j = 0; j < k; j++) sum[j] = wsum[j] = 0.f;
        for (int i = 0; i < N; i++) {
            uint32_t best = 0;
            float bd = INFINITY;
            for (uint32_t j = 0; j < k; j++) {
                const float d = fabsf(xs[i] - levels[j]);
                if (d < bd) { bd = d; best = j; }
            }
            sum[best] = fmaf(pdf[i], xs[i], sum[best]);
            wsum[best] += pdf[i];
        }
        for (uint32_t j = 0; j < k; j++)
            if (wsum[j] > 1e-12f) levels[j] = sum[j] / wsum[j];
    }
    for (uint32_t i = 1; i < k; i++) {  // insertion sort, k <= 16
        const float v = levels[i];
        int j = (int)i - 1;
        while (j >= 0 && levels[j] > v) { levels[j + 1] = levels[j]; j--; }
        levels[j + 1] = v;
    }
    const float scale = 1.0f / sqrtf((float)dim);
    for (uint32_t i = 0; i < k; i++) levels[i] *= scale;
    delete[] xs;
    delete[] pdf;
    return LC_OK;
}

size_t lc_swa_ring_capacity(size_t window, size_t max_positions) {
    const size_t min_safe = window + 256 - 1;  // MAX_PREFILL_CHUNK = 256
    size_t v = window * 2 > min_safe ? window * 2 : min_safe, p = 1;
    while (p < v) p <<= 1;
    return p < max_positions ? p : max_positions;
}

uint32_t lc_kv_bits_from_env(void) {
    const char *v = getenv("LOCAL_AI_KV_QUANT");
    if (v && strcmp(v, "tq3") == 0) return 3;
    if (v && strcmp(v, "tq4") == 0) return 4;
    return 2;
}

int lc_kernels_set_kv_norm_mode(lc_kernels *k, int mode) {
    if (!k || (mode != 0 && mode != 1)) return lc_fail(LC_ERR_INVALID_ARGUMENT, "kv norm mode must be 0 or 1");
    k->kv_norm_mode = mode;
    return LC_OK;
}

// ---- device entry points ----
int lc_encode_kv_turboquant_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *levels,
                                 const lc_buf *signs, lc_buf *packed, lc_buf *norms, uint32_t head_dim,
                                 uint32_t n_kv_heads, uint32_t num_tokens, uint32_t bits, uint32_t position,
                                 uint32_t ring_capacity) {
    if (!k || !b || !input || !levels || !signs || !packed || !norms)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "encode_kv_turboquant: NULL argument");
    int st = check_codec("encode_kv_turboquant", head_dim, bits);
    if (st != LC_OK) return st;
    LC_REQUIRE(n_kv_heads >= 1, "encode_kv_turboquant: n_kv_heads must be >= 1");
    const size_t groups = (size_t)n_kv_heads * num_tokens, cb = lc_tq_code_bytes(head_dim, bits);
    LC_REQUIRE(input->bytes >= groups * head_dim * 2, "encode_kv_turboquant: input too small");
    LC_REQUIRE(levels->bytes >= (4u << bits) && signs->bytes >= head_dim * 4u, "encode_kv_turboquant: codec buffers too small");
    const size_t rows = ring_capacity ? ring_capacity : (size_t)position + num_tokens;
    LC_REQUIRE(packed->bytes >= rows * n_kv_heads * cb && norms->bytes >= rows * n_kv_heads * 2,
               "encode_kv_turboquant: cache buffers hold fewer than %zu rows", rows);
    if (groups == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(encode_kv_kernel<false>, dim3((unsigned)groups), dim3(head_dim), 0, b, (const __half *)input->dptr, (const float *)levels->dptr, (const float *)signs->dptr,
        (uint8_t *)packed->dptr, (__half *)norms->dptr, nullptr, head_dim, n_kv_heads, 0, bits, position,
        ring_capacity, k->kv_norm_mode, k->dev_status));
    LC_CHECK_LAUNCH("encode_kv_turboquant");
    b->dispatch_count++;
    return LC_OK;
}

int lc_encode_kv_turboquant(lc_kernels *k, lc_ctx *ctx, const lc_buf *input, const lc_buf *levels,
                            const lc_buf *signs, lc_buf *packed, lc_buf *norms, uint32_t head_dim,
                            uint32_t n_kv_heads, uint32_t num_tokens, uint32_t bits, uint32_t position,
                            uint32_t ring_capacity) {
    if (!ctx) return lc_fail(LC_ERR_INVALID_ARGUMENT, "encode_kv_turboquant: ctx is NULL");
    return lc_run_and_wait(ctx, [&](lc_batch *b) {
        return lc_encode_kv_turboquant_into(k, b, input, levels, signs, packed, norms, head_dim, n_kv_heads,
                                            num_tokens, bits, position, ring_capacity);
    });
}

int lc_encode_kv_turboquant_batched_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *levels,
                                         const lc_buf *signs, lc_buf *packed, lc_buf *norms,
                                         const lc_buf *positions, uint32_t head_dim, uint32_t n_kv_heads,
                                         uint32_t lane_capacity, uint32_t bits, uint32_t n_lanes,
                                         uint32_t ring_capacity) {
    if (!k || !b || !input || !levels || !signs || !packed || !norms || !positions)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "encode_kv_turboquant_batched: NULL argument");
    int st = check_codec("encode_kv_turboquant_batched", head_dim, bits);
    if (st != LC_OK) return st;
    LC_REQUIRE(n_kv_heads >= 1, "encode_kv_turboquant_batched: n_kv_heads must be >= 1");
    const size_t groups = (size_t)n_kv_heads * n_lanes, cb = lc_tq_code_bytes(head_dim, bits);
    LC_REQUIRE(input->bytes >= groups * head_dim * 2 && positions->bytes >= (size_t)n_lanes * 4,
               "encode_kv_turboquant_batched: input/positions too small");
    LC_REQUIRE(levels->bytes >= (4u << bits) && signs->bytes >= head_dim * 4u,
               "encode_kv_turboquant_batched: codec buffers too small");
    LC_REQUIRE(ring_capacity <= lane_capacity, "encode_kv_turboquant_batched: ring %u exceeds lane capacity %u",
               ring_capacity, lane_capacity);
    const size_t rows = (size_t)n_lanes * lane_capacity;
    LC_REQUIRE(packed->bytes >= rows * n_kv_heads * cb && norms->bytes >= rows * n_kv_heads * 2,
               "encode_kv_turboquant_batched: pool buffers hold fewer than %zu rows", rows);
    if (groups == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(encode_kv_kernel<true>, dim3((unsigned)groups), dim3(head_dim), 0, b, (const __half *)input->dptr, (const float *)levels->dptr, (const float *)signs->dptr,
        (uint8_t *)packed->dptr, (__half *)norms->dptr, (const uint32_t *)positions->dptr, head_dim, n_kv_heads,
        lane_capacity, bits, 0, ring_capacity, k->kv_norm_mode, k->dev_status));
    LC_CHECK_LAUNCH("encode_kv_turboquant_batched");
    b->dispatch_count++;
    return LC_OK;
}

int lc_dequantize_kv_turboquant_into(lc_kernels *k, lc_batch *b, const lc_buf *packed, const lc_buf *norms,
                                     const lc_buf *levels, const lc_buf *signs, lc_buf *output,
                                     uint32_t head_dim, uint32_t n_kv_heads, uint32_t num_tokens, uint32_t bits,
                                     uint32_t token_start, uint32_t ring_capacity) {
    if (!k || !b || !packed || !norms || !levels || !signs || !output)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "dequantize_kv_turboquant: NULL argument");
    int st = check_codec("dequantize_kv_turboquant", head_dim, bits);
    if (st != LC_OK) return st;
    LC_REQUIRE(n_kv_heads >= 1, "dequantize_kv_turboquant: n_kv_heads must be >= 1");
    if (token_start >= num_tokens) return LC_OK;
    const size_t cb = lc_tq_code_bytes(head_dim, bits);
    const size_t rows = ring_capacity ? (ring_capacity < num_tokens ? ring_capacity : num_tokens) : num_tokens;
    LC_REQUIRE(packed->bytes >= rows * n_kv_heads * cb && norms->bytes >= rows * n_kv_heads * 2,
               "dequantize_kv_turboquant: cache buffers too small");
    LC_REQUIRE(output->bytes >= (size_t)num_tokens * n_kv_heads * head_dim * 2,
               "dequantize_kv_turboquant: output too small");
    LC_REQUIRE(levels->bytes >= (4u << bits) && signs->bytes >= head_dim * 4u,
               "dequantize_kv_turboquant: codec buffers too small");
    const unsigned groups = n_kv_heads * (num_tokens - token_start);
    LC_LAUNCH_CHECKED(lc_launch(dequantize_kv_kernel, dim3(groups), dim3(head_dim), 0, b, (const uint8_t *)packed->dptr, (const __half *)norms->dptr, (const float *)levels->dptr,
        (const float *)signs->dptr, (__half *)output->dptr, head_dim, n_kv_heads, bits,
        token_start * n_kv_heads, ring_capacity));
    LC_CHECK_LAUNCH("dequantize_kv_turboquant");
    b->dispatch_count++;
    return LC_OK;
}

int lc_dequantize_kv_turboquant(lc_kernels *k, lc_ctx *ctx, const lc_buf *packed, const lc_buf *norms,
                                const lc_buf *levels, const lc_buf *signs, lc_buf *output, uint32_t head_dim,
                                uint32_t n_kv_heads, uint32_t num_tokens, uint32_t bits, uint32_t token_start,
                                uint32_t ring_capacity) {
    if (!ctx) return lc_fail(LC_ERR_INVALID_ARGUMENT, "dequantize_kv_turboquant: ctx is NULL");
    return lc_run_and_wait(ctx, [&](lc_batch *b) {
        return lc_dequantize_kv_turboquant_into(k, b, packed, norms, levels, signs, output, head_dim, n_kv_heads,
                                                num_tokens, bits, token_start, ring_capacity);
    });
}

int lc_hadamard_rotate_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *signs,
                            lc_buf *output, uint32_t head_dim, uint32_t num_heads, uint32_t pre_sign,
                            uint32_t post_sign) {
    return rotate_into<float, float>("hadamard_rotate", k, b, input, signs, output, head_dim, num_heads, pre_sign, post_sign);
}
int lc_hadamard_rotate_hf_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *signs,
                               lc_buf *output, uint32_t head_dim, uint32_t num_heads, uint32_t pre_sign,
                               uint32_t post_sign) {
    return rotate_into<__half, float>("hadamard_rotate_hf", k, b, input, signs, output, head_dim, num_heads, pre_sign, post_sign);
}
int lc_hadamard_rotate_fh_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *signs,
                               lc_buf *output, uint32_t head_dim, uint32_t num_heads, uint32_t pre_sign,
                               uint32_t post_sign) {
    return rotate_into<float, __half>("hadamard_rotate_fh", k, b, input, signs, output, head_dim, num_heads, pre_sign, post_sign);
}


static int kv_write_common(const char *name, lc_kernels *k, lc_batch *b, lc_buf *q, const lc_buf *q_norm_weight,
                           uint32_t n_q_heads, const lc_buf *k_in, const lc_buf *v_in, const lc_buf *k_norm_weight,
                           const lc_buf *positions, const lc_buf *levels, const lc_buf *signs, lc_buf *k_packed,
                           lc_buf *k_norms, lc_buf *v_packed, lc_buf *v_norms, uint32_t head_dim, uint32_t n_kv_heads,
                           uint32_t lane_capacity, uint32_t bits, uint32_t n_lanes, uint32_t ring_capacity, float eps,
                           float rope_theta, float partial_rotary_factor, lc_buf *qfrag = nullptr,
                           float softmax_scale = 0.f) {
    if (!k || !b || !k_in || !v_in || !k_norm_weight || !positions || !levels || !signs || !k_packed || !k_norms ||
        !v_packed || !v_norms || (n_q_heads && (!q || !q_norm_weight)))
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    int st = check_codec(name, head_dim, bits);
    if (st != LC_OK) return st;
    LC_REQUIRE(n_kv_heads >= 1, "%s: n_kv_heads must be >= 1", name);
    LC_REQUIRE(n_q_heads + 2 * n_kv_heads <= 65535, "%s: too many heads", name);
    const size_t groups = (size_t)n_kv_heads * n_lanes, cb = lc_tq_code_bytes(head_dim, bits);
    LC_REQUIRE(k_in->bytes >= groups * head_dim * 2 && v_in->bytes >= groups * head_dim * 2 &&
                   positions->bytes >= (size_t)n_lanes * 4 && k_norm_weight->bytes >= head_dim * 2u,
               "%s: input buffers too small", name);
    if (n_q_heads)
        LC_REQUIRE(q->bytes >= (size_t)n_lanes * n_q_heads * head_dim * 2 && q_norm_weight->bytes >= head_dim * 2u,
                   "%s: query buffers too small", name);
    LC_REQUIRE(levels->bytes >= (4u << bits) && signs->bytes >= head_dim * 4u, "%s: codec buffers too small", name);
    if (qfrag) {
        LC_REQUIRE(n_q_heads && lc_qfrag_supported(head_dim, bits, n_q_heads, n_kv_heads),
                   "%s: query fragments need head_dim 256, 2-bit codes and q heads in groups of 8 per kv head", name);
        LC_REQUIRE(qfrag->bytes >= (size_t)n_lanes * n_q_heads * head_dim * 4 && lc_aligned(qfrag->dptr, 16),
                   "%s: query fragment buffer too small or misaligned", name);
    }
    LC_REQUIRE(ring_capacity <= lane_capacity, "%s: ring %u exceeds lane capacity %u", name, ring_capacity, lane_capacity);
    const size_t rows = (size_t)n_lanes * lane_capacity * n_kv_heads;
    LC_REQUIRE(k_packed->bytes >= rows * cb && v_packed->bytes >= rows * cb && k_norms->bytes >= rows * 2 &&
                   v_norms->bytes >= rows * 2,
               "%s: pool buffers hold fewer than %zu rows", name, rows);
    if (groups == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(kv_write_kernel, dim3(n_lanes, n_q_heads + 2 * n_kv_heads), dim3(head_dim), 0, b,
                                q ? (__half *)q->dptr : nullptr, q_norm_weight ? (const __half *)q_norm_weight->dptr : nullptr,
                                n_q_heads, (const __half *)k_in->dptr, (const __half *)v_in->dptr,
                                (const __half *)k_norm_weight->dptr, (const uint32_t *)positions->dptr,
                                (const float *)levels->dptr, (const float *)signs->dptr, (uint8_t *)k_packed->dptr,
                                (__half *)k_norms->dptr, (uint8_t *)v_packed->dptr, (__half *)v_norms->dptr, head_dim,
                                n_kv_heads, lane_capacity, bits, ring_capacity, eps, rope_theta, partial_rotary_factor,
                                k->kv_norm_mode, k->dev_status, qfrag ? (uint4 *)qfrag->dptr : (uint4 *)nullptr,
                                softmax_scale));
    b->dispatch_count++;
    return LC_OK;
}

int lc_kv_write_batched_into(lc_kernels *k, lc_batch *b, const lc_buf *k_in, const lc_buf *v_in, const lc_buf *k_norm_weight,
                             const lc_buf *positions, const lc_buf *levels, const lc_buf *signs, lc_buf *k_packed,
                             lc_buf *k_norms, lc_buf *v_packed, lc_buf *v_norms, uint32_t head_dim, uint32_t n_kv_heads,
                             uint32_t lane_capacity, uint32_t bits, uint32_t n_lanes, uint32_t ring_capacity, float eps,
                             float rope_theta, float partial_rotary_factor) {
    return kv_write_common("kv_write_batched", k, b, nullptr, nullptr, 0, k_in, v_in, k_norm_weight, positions, levels, signs,
                           k_packed, k_norms, v_packed, v_norms, head_dim, n_kv_heads, lane_capacity, bits, n_lanes,
                           ring_capacity, eps, rope_theta, partial_rotary_factor);
}

int lc_qkv_post_batched_into(lc_kernels *k, lc_batch *b, lc_buf *q, const lc_buf *q_norm_weight, uint32_t n_q_heads,
                             const lc_buf *k_in, const lc_buf *v_in, const lc_buf *k_norm_weight, const lc_buf *positions,
                             const lc_buf *levels, const lc_buf *signs, lc_buf *k_packed, lc_buf *k_norms,
                             lc_buf *v_packed, lc_buf *v_norms, uint32_t head_dim, uint32_t n_kv_heads,
                             uint32_t lane_capacity, uint32_t bits, uint32_t n_lanes, uint32_t ring_capacity, float eps,
                             float rope_theta, float partial_rotary_factor) {
    if (!q || !q_norm_weight || n_q_heads == 0)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "qkv_post_batched: the query buffer, its norm weight and n_q_heads are required");
    return kv_write_common("qkv_post_batched", k, b, q, q_norm_weight, n_q_heads, k_in, v_in, k_norm_weight, positions, levels,
                           signs, k_packed, k_norms, v_packed, v_norms, head_dim, n_kv_heads, lane_capacity, bits, n_lanes,
                           ring_capacity, eps, rope_theta, partial_rotary_factor);
}

}  // extern "C"

int lc_qkv_post_frag(lc_kernels *k, lc_batch *b, lc_buf *q, const lc_buf *q_norm_weight, uint32_t n_q_heads,
                     const lc_buf *k_in, const lc_buf *v_in, const lc_buf *k_norm_weight, const lc_buf *positions,
                     const lc_buf *levels, const lc_buf *signs, lc_buf *k_packed, lc_buf *k_norms, lc_buf *v_packed,
                     lc_buf *v_norms, uint32_t head_dim, uint32_t n_kv_heads, uint32_t lane_capacity, uint32_t bits,
                     uint32_t n_lanes, uint32_t ring_capacity, float eps, float rope_theta, float partial_rotary_factor,
                     lc_buf *qfrag, float softmax_scale) {
    if (!q || !q_norm_weight || n_q_heads == 0)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "qkv_post_batched: the query buffer, its norm weight and n_q_heads are required");
    return kv_write_common("qkv_post_batched", k, b, q, q_norm_weight, n_q_heads, k_in, v_in, k_norm_weight, positions, levels,
                           signs, k_packed, k_norms, v_packed, v_norms, head_dim, n_kv_heads, lane_capacity, bits, n_lanes,
                           ring_capacity, eps, rope_theta, partial_rotary_factor, qfrag, softmax_scale);
}
