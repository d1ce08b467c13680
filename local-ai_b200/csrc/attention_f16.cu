// FP16-KV decode attention: the three kernels the reference keeps beside the
// code-space path.  Stands in for shaders/flash_decoding.metal:10-189
// (flash_decoding_split / _reduce), shaders/attention_flash.metal:398-503
// (flash_attention_windowed_split) and shaders/attention_sliding.metal:18-78.
// All three are the same computation — softmax(q.K^T * scale) V over the keys
// t in [max(0, pos+1-window), min(kv_len, pos+1)) of one query position — so
// they share one split-K kernel and one merge kernel here; they differ only in
// who owns the partial buffers and how the split count is chosen.
// K/V are f16 [kv_len, n_kv, hd]; q and output are f16 [n_q, hd].
#include <math.h>

#include "lc_internal.h"

namespace {

constexpr int NT = 256;
constexpr int NW = NT / 32;
constexpr int MAX_DPL2 = 8;  // half2 pairs per lane: head_dim <= 512

// grid = (num_splits, n_q). Split s owns a contiguous run of keys; the 8 warps
// stripe it; lane owns dims {2*lane + 64*i, +1}.
__global__ void __launch_bounds__(NT)
f16_attn_split_kernel(const __half *__restrict__ q, const __half *__restrict__ k, const __half *__restrict__ v,
                      float *__restrict__ pmax, float *__restrict__ psum, float *__restrict__ pacc, unsigned hd,
                      unsigned kv_len, unsigned current_pos, unsigned n_q, unsigned n_kv, unsigned window,
                      unsigned num_splits, float scale) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    __shared__ float m_s[NW], l_s[NW];
    __shared__ float acc_s[NW][512];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned split = blockIdx.x, qh = blockIdx.y;
    const unsigned kvh = qh / (n_q / n_kv);
    const unsigned seq_len = min(kv_len, current_pos + 1u);
    const unsigned win_start = (window > 0u && current_pos + 1u > window) ? current_pos + 1u - window : 0u;
    const unsigned n_keys = seq_len > win_start ? seq_len - win_start : 0u;
    const unsigned per = (n_keys + num_splits - 1) / num_splits;
    const unsigned begin = win_start + split * per;
    const unsigned end = min(seq_len, begin + per);
    const int dpl2 = (int)hd / 64;  // hd is a multiple of 64

    float2 qr[MAX_DPL2], acc[MAX_DPL2];
#pragma unroll
    for (int i = 0; i < MAX_DPL2; i++) {
        acc[i] = make_float2(0.f, 0.f);
        qr[i] = make_float2(0.f, 0.f);
        if (i < dpl2) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(q + (size_t)qh * hd + 2 * lane + 64 * i));
            qr[i] = make_float2(f.x * scale, f.y * scale);
        }
    }
    float m_run = -INFINITY, l_run = 0.f;
    for (unsigned t = begin + warp; t < end; t += NW) {
        const __half *kr = k + ((size_t)t * n_kv + kvh) * hd;
        const __half *vr = v + ((size_t)t * n_kv + kvh) * hd;
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_DPL2; i++)
            if (i < dpl2) {
                const float2 kf = __half22float2(__ldg(reinterpret_cast<const __half2 *>(kr + 2 * lane + 64 * i)));
                dot = fmaf(qr[i].x, kf.x, dot);
                dot = fmaf(qr[i].y, kf.y, dot);
            }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float m_new = fmaxf(m_run, dot);
        const float rescale = expf(m_run - m_new);
        const float w = expf(dot - m_new);
        l_run = l_run * rescale + w;
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < MAX_DPL2; i++)
            if (i < dpl2) {
                const float2 vf = __half22float2(__ldg(reinterpret_cast<const __half2 *>(vr + 2 * lane + 64 * i)));
                acc[i].x = fmaf(w, vf.x, acc[i].x * rescale);
                acc[i].y = fmaf(w, vf.y, acc[i].y * rescale);
            }
    }
    if (lane == 0) {
        m_s[warp] = m_run;
        l_s[warp] = l_run;
    }
#pragma unroll
    for (int i = 0; i < MAX_DPL2; i++)
        if (i < dpl2) {
            acc_s[warp][2 * lane + 64 * i] = acc[i].x;
            acc_s[warp][2 * lane + 64 * i + 1] = acc[i].y;
        }
    __syncthreads();
    float gmax = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; w++) gmax = fmaxf(gmax, m_s[w]);
    const size_t pi = (size_t)qh * num_splits + split;
    for (unsigned d = threadIdx.x; d < hd; d += NT) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) {
            const float f = (m_s[w] == -INFINITY) ? 0.f : expf(m_s[w] - gmax);
            o += f * acc_s[w][d];
        }
        pacc[pi * hd + d] = o;
    }
    if (threadIdx.x == 0) {
        float gsum = 0.f;
        for (int w = 0; w < NW; w++) {
            const float f = (m_s[w] == -INFINITY) ? 0.f : expf(m_s[w] - gmax);
            gsum += f * l_s[w];
        }
        pmax[pi] = gmax;
        psum[pi] = gsum;
    }
}

// flash_decoding.metal:120-189: LSE merge of the partials, f16 store. grid = n_q.
__global__ void f16_attn_reduce_kernel(const float *__restrict__ pmax, const float *__restrict__ psum,
                                       const float *__restrict__ pacc, __half *__restrict__ out, unsigned hd,
                                       unsigned num_splits) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    const unsigned qh = blockIdx.x;
    float gmax = -INFINITY;
    for (unsigned s = 0; s < num_splits; s++) gmax = fmaxf(gmax, pmax[(size_t)qh * num_splits + s]);
    float gsum = 0.f;
    for (unsigned s = 0; s < num_splits; s++) {
        const float m = pmax[(size_t)qh * num_splits + s];
        gsum += (m == -INFINITY ? 0.f : expf(m - gmax)) * psum[(size_t)qh * num_splits + s];
    }
    const float inv = gsum > 0.f ? 1.f / gsum : 0.f;
    for (unsigned d = threadIdx.x; d < hd; d += blockDim.x) {
        float o = 0.f;
        for (unsigned s = 0; s < num_splits; s++) {
            const float m = pmax[(size_t)qh * num_splits + s];
            o += (m == -INFINITY ? 0.f : expf(m - gmax)) * pacc[((size_t)qh * num_splits + s) * hd + d];
        }
        out[(size_t)qh * hd + d] = __float2half_rn(o * inv);
    }
}

int f16_attention(const char *name, lc_batch *b, const lc_buf *q, const lc_buf *k, const lc_buf *v, lc_buf *output,
                  float *pmax, float *psum, float *pacc, uint32_t hd, uint32_t kv_len, uint32_t current_pos,
                  uint32_t n_q, uint32_t n_kv, uint32_t window, uint32_t num_splits, float scale) {
    if (!b || !q || !k || !v || !output) return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    LC_REQUIRE(hd >= 64 && hd <= 512 && hd % 64 == 0, "%s: head_dim %u must be a multiple of 64 up to 512", name, hd);
    LC_REQUIRE(n_kv >= 1 && n_q >= 1 && n_q % n_kv == 0, "%s: num_q_heads %u must be a multiple of num_kv_heads %u",
               name, n_q, n_kv);
    LC_REQUIRE(num_splits >= 1, "%s: num_splits must be >= 1", name);
    const uint32_t seq_len = kv_len < current_pos + 1 ? kv_len : current_pos + 1;
    LC_REQUIRE(q->bytes >= (size_t)n_q * hd * 2 && output->bytes >= (size_t)n_q * hd * 2, "%s: q/output too small", name);
    LC_REQUIRE(k->bytes >= (size_t)seq_len * n_kv * hd * 2 && v->bytes >= (size_t)seq_len * n_kv * hd * 2,
               "%s: K/V hold fewer than %u rows", name, seq_len);
    LC_REQUIRE(lc_aligned(q->dptr, 4) && lc_aligned(k->dptr, 4) && lc_aligned(v->dptr, 4), "%s: buffers must be 4-byte aligned", name);
    LC_LAUNCH_CHECKED(lc_launch(f16_attn_split_kernel, dim3(dim3(num_splits, n_q)), dim3(NT), 0, b, (const __half *)q->dptr, (const __half *)k->dptr, (const __half *)v->dptr, pmax, psum, pacc, hd, kv_len,
        current_pos, n_q, n_kv, window, num_splits, scale));
    LC_CHECK_LAUNCH(name);
    b->dispatch_count++;
    LC_LAUNCH_CHECKED(lc_launch(f16_attn_reduce_kernel, dim3(n_q), dim3(hd < 256 ? hd : 256), 0, b, pmax, psum, pacc, (__half *)output->dptr, hd,
                                                                        num_splits));
    LC_CHECK_LAUNCH(name);
    b->dispatch_count++;
    return LC_OK;
}

// Library-owned partials for the entry points whose reference signature has none.
int f16_attention_scratch(const char *name, lc_kernels *kn, lc_batch *b, const lc_buf *q, const lc_buf *k,
                          const lc_buf *v, lc_buf *output, uint32_t hd, uint32_t kv_len, uint32_t current_pos,
                          uint32_t n_q, uint32_t n_kv, uint32_t window, uint32_t num_splits, float scale) {
    if (!kn) return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: kernels is NULL", name);
    const size_t parts = (size_t)n_q * num_splits;
    int st = lc_reserve_scratch(kn, b, parts * (hd + 2) * sizeof(float), 0);
    if (st != LC_OK) return st;
    float *pmax = (float *)kn->scratch, *psum = pmax + parts, *pacc = psum + parts;
    return f16_attention(name, b, q, k, v, output, pmax, psum, pacc, hd, kv_len, current_pos, n_q, n_kv, window,
                         num_splits, scale);
}

}  // namespace

extern "C" {

uint32_t lc_flash_split_count(const lc_kernels *k, uint32_t eff_seq_len) {
    (void)k;
    const uint32_t c = (eff_seq_len + 15) / 16;  // kernels.rs:1265-1278
    return c < 1 ? 1 : (c > 16 ? 16 : c);
}

int lc_flash_attention_windowed_split_into(lc_kernels *k, lc_batch *b, const lc_buf *q, const lc_buf *kk,
                                           const lc_buf *v, lc_buf *output, lc_buf *partial_max,
                                           lc_buf *partial_sum, lc_buf *partial_acc, uint32_t head_dim,
                                           uint32_t kv_len, uint32_t current_pos, uint32_t num_q_heads,
                                           uint32_t num_kv_heads, uint32_t window, uint32_t num_splits) {
    if (!k || !partial_max || !partial_sum || !partial_acc)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "flash_attention_windowed_split: NULL argument");
    const size_t parts = (size_t)num_q_heads * num_splits;
    LC_REQUIRE(partial_max->bytes >= parts * 4 && partial_sum->bytes >= parts * 4 &&
                   partial_acc->bytes >= parts * head_dim * 4,
               "flash_attention_windowed_split: partial buffers too small for %u heads x %u splits", num_q_heads,
               num_splits);
    return f16_attention("flash_attention_windowed_split", b, q, kk, v, output, (float *)partial_max->dptr,
                         (float *)partial_sum->dptr, (float *)partial_acc->dptr, head_dim, kv_len, current_pos,
                         num_q_heads, num_kv_heads, window, num_splits, 1.0f);
}

int lc_flash_decoding_into(lc_kernels *k, lc_ctx *ctx, lc_batch *b, const lc_buf *q, const lc_buf *kk,
                           const lc_buf *v, lc_buf *output, uint32_t head_dim, uint32_t kv_len, uint32_t current_pos,
                           uint32_t num_q_heads, uint32_t num_kv_heads) {
    (void)ctx;  // the reference needs it to renew the encoder between split and reduce
    const uint32_t seq_len = kv_len < current_pos + 1 ? kv_len : current_pos + 1;
    // 256-key splits (FD_SPLIT_SIZE, flash_decoding.metal:12); one split when seq_len <= 256,
    // where the reference falls back to its single-pass kernel (kernels.rs:1411-1428).
    uint32_t splits = (seq_len + 255) / 256;
    if (splits < 1) splits = 1;
    return f16_attention_scratch("flash_decoding", k, b, q, kk, v, output, head_dim, kv_len, current_pos,
                                 num_q_heads, num_kv_heads, 0, splits, 1.0f);
}

int lc_attention_sliding(lc_kernels *k, lc_ctx *ctx, const lc_buf *q, const lc_buf *kk, const lc_buf *v,
                         lc_buf *output, uint32_t head_dim, uint32_t kv_len, uint32_t current_pos, uint32_t window,
                         uint32_t num_q_heads, uint32_t num_kv_heads) {
    if (!ctx) return lc_fail(LC_ERR_INVALID_ARGUMENT, "attention_sliding: ctx is NULL");
    const uint32_t seq_len = kv_len < current_pos + 1 ? kv_len : current_pos + 1;
    const uint32_t ws = (window > 0 && current_pos + 1 > window) ? current_pos + 1 - window : 0;
    const uint32_t eff = seq_len > ws ? seq_len - ws : 0;
    // The reference caps the window at its 2048-entry score array
    // (attention_sliding.metal:33); this kernel has no such cap.
    return lc_run_and_wait(ctx, [&](lc_batch *b) {
        return f16_attention_scratch("attention_sliding", k, b, q, kk, v, output, head_dim, kv_len, current_pos,
                                     num_q_heads, num_kv_heads, window, lc_flash_split_count(k, eff), 1.0f);
    });
}

}  // extern "C"
