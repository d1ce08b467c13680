// Decode attention straight over TurboQuant codes, split-K across CTAs.
// Stands in for shaders/attention_flash_tq.metal:154-274 (flash_attention_tq)
// and :569-690 (flash_attention_tq_batched), plus the rotate -> attend ->
// inverse-rotate sequence the KV containers wrap around them
// (kv_cache/quant_cache.rs:565-596, kv_cache/quant_unified_pool.rs:218-256).
//
// Differences from the Metal design, all behaviour-preserving:
//  * one CTA serves every q-head that shares a kv-head, so a key/value row is
//    read from HBM once per group instead of once per q-head;
//  * the context is split across CTAs (grid.x) so one long sequence fills the
//    GPU; partial (max, sum, acc) triples are merged by a second kernel;
//  * in the fused form the query rotation runs in the prologue and the inverse
//    rotation + f16 store in the merge kernel, removing two launches and the
//    f32 round trips through rq / vacc.
#include <math.h>
#include <stdlib.h>

#include "lc_internal.h"
#include "attention_tq.h"

namespace {

constexpr int NT = 256;
constexpr int NW = NT / 32;
constexpr int TILE = 32;  // keys per warp step: one key per lane in the QK phase


// In-place unnormalised FWHT on `rows` rows of HD floats in shared memory,
// cooperatively by the whole CTA.  Ends with a barrier.
template <int HD>
__device__ __forceinline__ void fwht_rows(float *sh, int rows) {
    const int pairs = rows * (HD / 2);
    for (int len = 1; len < HD; len <<= 1) {
        __syncthreads();
        for (int p = threadIdx.x; p < pairs; p += NT) {
            const int i = p & (len - 1);
            const int idx = ((p - i) << 1) + i;
            const float a = sh[idx], b = sh[idx + len];
            sh[idx] = a + b;
            sh[idx + len] = a - b;
        }
    }
    __syncthreads();
}

template <int HD, int BITS, int G>
__global__ void __launch_bounds__(NT) tq_attn_split_kernel(const TqAttnParams p) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    constexpr int DPL = HD / 32;
    constexpr int CB = HD * BITS / 8;
    constexpr int NLEV = 1 << BITS;
    constexpr unsigned MASK = NLEV - 1;
    extern __shared__ __align__(16) float smem_f[];
    float *rq_s = smem_f;                   // [HD][G]
    float *lev_s = rq_s + HD * G;           // [16]
    float *pw_s = lev_s + 16;               // [NW][TILE][G]
    float *comb = pw_s + NW * TILE * G;     // [NW][G][HD] + m[NW][G] + l[NW][G]; also the rotation scratch

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t split = blockIdx.x;
    const uint32_t gchunks = (p.group + G - 1) / G;
    const uint32_t kv_head = blockIdx.y / gchunks, gchunk = blockIdx.y - kv_head * gchunks;
    const uint32_t lane_idx = blockIdx.z;
    const int gvalid = min((int)G, (int)(p.group - gchunk * G));
    const uint32_t qh0 = kv_head * p.group + gchunk * G;

    uint32_t pos, seq_len;
    if (p.positions) {
        pos = p.positions[lane_idx];
        seq_len = pos + 1u;
        if (p.ring == 0u && seq_len > p.lane_capacity) {   // never read past the lane's rows
            seq_len = p.lane_capacity;
            if (p.status && threadIdx.x == 0) atomicExch(p.status, LC_DEV_STATUS_POSITION);
        }
    } else {
        pos = p.current_pos + (p.row_positions ? lane_idx : 0u);
        seq_len = min(p.kv_len, pos + 1u);
    }
    const uint32_t win_start = (p.window > 0u && pos + 1u > p.window) ? (pos + 1u - p.window) : 0u;
    const uint32_t n_keys = seq_len > win_start ? seq_len - win_start : 0u;
    uint32_t per = (n_keys + p.n_splits - 1) / p.n_splits;
    per = (per + TILE - 1) & ~(uint32_t)(TILE - 1);
    const uint32_t k_begin = win_start + split * per;
    const uint32_t k_end = min(seq_len, k_begin + per);
    const size_t lane_base = (size_t)lane_idx * p.lane_capacity;

    // ---- prologue: query into shared memory as rq_s[d][g] (scaled) ----
    if (threadIdx.x < 16) lev_s[threadIdx.x] = threadIdx.x < NLEV ? p.levels[threadIdx.x] : 0.f;
    if (p.fused_q) {
        float *tmp = comb;  // [G][HD]
        for (int i = threadIdx.x; i < G * HD; i += NT) {
            const int g = i / HD, d = i - g * HD;
            float v = 0.f;
            if (g < gvalid) v = __half2float(p.q[((size_t)lane_idx * p.n_q + qh0 + g) * HD + d]) * p.signs[d];
            tmp[i] = v;
        }
        fwht_rows<HD>(tmp, G);
        const float f = p.scale / sqrtf((float)HD);
        for (int i = threadIdx.x; i < G * HD; i += NT) {
            const int g = i / HD, d = i - g * HD;
            rq_s[d * G + g] = tmp[i] * f;
        }
    } else {
        for (int i = threadIdx.x; i < G * HD; i += NT) {
            const int g = i / HD, d = i - g * HD;
            float v = 0.f;
            if (g < gvalid) v = p.rq[((size_t)lane_idx * p.n_q + qh0 + g) * HD + d] * p.scale;
            rq_s[d * G + g] = v;
        }
    }
    __syncthreads();

    float m_run[G], l_run[G], acc[G][DPL];
#pragma unroll
    for (int g = 0; g < G; g++) {
        m_run[g] = -INFINITY;
        l_run[g] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; i++) acc[g][i] = 0.f;
    }
    float *pw = pw_s + warp * TILE * G;

    for (uint32_t t0 = k_begin + warp * TILE; t0 < k_end; t0 += NW * TILE) {
        // ---- QK: lane owns key t0 + lane, walks all HD codes ----
        const uint32_t t = t0 + lane;
        const bool valid = t < k_end;
        float s[G];
#pragma unroll
        for (int g = 0; g < G; g++) s[g] = 0.f;
        float vnorm = 0.f;
        if (valid) {
            const size_t slot = (lane_base + (p.ring ? t % p.ring : t)) * p.n_kv + kv_head;
            const uint32_t *kw = reinterpret_cast<const uint32_t *>(p.kc + slot * CB);
            constexpr int GW = (BITS == 3) ? 3 : 1;       // words per group
            constexpr int GC = GW * 32 / BITS;            // codes per group
#pragma unroll 2
            for (int grp = 0; grp < CB / 4 / GW; grp++) {
                uint32_t w[GW];
#pragma unroll
                for (int i = 0; i < GW; i++) w[i] = __ldg(kw + grp * GW + i);
#pragma unroll
                for (int c = 0; c < GC; c++) {
                    const int bo = c * BITS, wi = bo >> 5, sh = bo & 31;
                    unsigned code = w[wi] >> sh;
                    if (sh + BITS > 32) code |= w[wi + 1 < GW ? wi + 1 : wi] << (32 - sh);
                    code &= MASK;
                    const float lv = lev_s[code];
                    const float *rqd = rq_s + (grp * GC + c) * G;
#pragma unroll
                    for (int g = 0; g < G; g++) s[g] = fmaf(rqd[g], lv, s[g]);
                }
            }
            const float knorm = __half2float(p.kn[slot]);
            vnorm = __half2float(p.vn[slot]);
#pragma unroll
            for (int g = 0; g < G; g++) s[g] *= knorm;
        }
        // ---- online softmax for the tile ----
#pragma unroll
        for (int g = 0; g < G; g++) {
            float tm = valid ? s[g] : -INFINITY;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
            const float m_new = fmaxf(m_run[g], tm);  // finite: lane 0 of every tile is valid
            const float rescale = expf(m_run[g] - m_new);
            const float w = valid ? expf(s[g] - m_new) : 0.f;
            float ws = w;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ws += __shfl_xor_sync(0xffffffffu, ws, o);
            l_run[g] = l_run[g] * rescale + ws;
            m_run[g] = m_new;
#pragma unroll
            for (int i = 0; i < DPL; i++) acc[g][i] *= rescale;
            pw[lane * G + g] = w * vnorm;
        }
        __syncwarp();
        // ---- PV: lane owns dims [lane*DPL, lane*DPL + DPL) ----
        const int nk = (int)min((uint32_t)TILE, k_end - t0);
        constexpr int BO = DPL * BITS;  // bits of codes owned by one lane
#pragma unroll 4
        for (int j = 0; j < nk; j++) {
            const uint32_t tj = t0 + j;
            const size_t slot = (lane_base + (p.ring ? tj % p.ring : tj)) * p.n_kv + kv_head;
            const uint8_t *vrow = p.vc + slot * CB;
            const unsigned bitoff = lane * BO, byte0 = bitoff >> 3, shb = bitoff & 7u;
            constexpr int NBYTES = (BO + 7 + 7) / 8 > 8 ? 8 : (BO + 7 + 7) / 8;
            unsigned long long bits = 0;
#pragma unroll
            for (int b = 0; b < NBYTES; b++)
                if (byte0 + b < (unsigned)CB) bits |= (unsigned long long)__ldg(vrow + byte0 + b) << (8 * b);
            bits >>= shb;
            float pj[G];
#pragma unroll
            for (int g = 0; g < G; g++) pj[g] = pw[j * G + g];
#pragma unroll
            for (int i = 0; i < DPL; i++) {
                const float lv = lev_s[(unsigned)(bits >> (i * BITS)) & MASK];
#pragma unroll
                for (int g = 0; g < G; g++) acc[g][i] = fmaf(pj[g], lv, acc[g][i]);
            }
        }
        __syncwarp();
    }

    // ---- merge the 8 warps of this CTA ----
    float *acc_s = comb;                       // [NW][G][HD]
    float *m_s = comb + NW * G * HD;           // [NW][G]
    float *l_s = m_s + NW * G;                 // [NW][G]
    __syncthreads();                           // comb may still hold the rotation scratch
#pragma unroll
    for (int g = 0; g < G; g++) {
        if (lane == 0) {
            m_s[warp * G + g] = m_run[g];
            l_s[warp * G + g] = l_run[g];
        }
#pragma unroll
        for (int i = 0; i < DPL; i++) acc_s[(warp * G + g) * HD + lane * DPL + i] = acc[g][i];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < gvalid * HD; i += NT) {
        const int g = i / HD, d = i - g * HD;
        float gmax = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; w++) gmax = fmaxf(gmax, m_s[w * G + g]);
        float gsum = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) {
            const float mw = m_s[w * G + g];
            const float f = (mw == -INFINITY) ? 0.f : expf(mw - gmax);
            gsum += f * l_s[w * G + g];
            o += f * acc_s[(w * G + g) * HD + d];
        }
        const size_t qh = (size_t)lane_idx * p.n_q + qh0 + g;
        if (p.direct_out) {
            p.out[qh * HD + d] = gsum > 0.f ? o / gsum : 0.f;
        } else {
            float *pp = p.partial + (qh * p.n_splits + split) * (size_t)(HD + 2);
            if (d == 0) {
                pp[0] = gmax;
                pp[1] = gsum;
            }
            pp[2 + d] = o;
        }
    }
}

// Merge n_splits partials of one (lane, q-head); optionally inverse-rotate and
// store f16 (fused form).  grid = lanes * n_q, block = HD.
template <bool FUSED>
__global__ void tq_attn_merge_kernel(const float *__restrict__ partial, const float *__restrict__ signs,
                                     float *__restrict__ out_f32, __half *__restrict__ out_f16, unsigned hd,
                                     unsigned n_splits) {
    lc_pdl_trigger();  // successors may be scheduled; they wait for this grid before reading its output
    lc_pdl_wait();     // everything below may read what the predecessor wrote
    __shared__ float sh[512];
    const unsigned t = threadIdx.x;
    const size_t qh = blockIdx.x;
    const float *pp = partial + qh * n_splits * (size_t)(hd + 2);
    float gmax = -INFINITY;
    for (unsigned s = 0; s < n_splits; s++) gmax = fmaxf(gmax, pp[s * (size_t)(hd + 2)]);
    float gsum = 0.f, o = 0.f;
    for (unsigned s = 0; s < n_splits; s++) {
        const float *ps = pp + s * (size_t)(hd + 2);
        const float f = (ps[0] == -INFINITY) ? 0.f : expf(ps[0] - gmax);
        gsum += f * ps[1];
        o += f * ps[2 + t];
    }
    const float v = gsum > 0.f ? o / gsum : 0.f;
    if (!FUSED) {
        out_f32[qh * hd + t] = v;
        return;
    }
    // inverse rotation
    const float w = lc_fwht_value(v, sh, hd, t);
    out_f16[qh * hd + t] = __float2half_rn(w * (1.0f / sqrtf((float)hd)) * signs[t]);
}

template <int HD, int BITS, int G>
int launch_split(lc_batch *b, const TqAttnParams &p, dim3 grid) {
    const size_t comb = (size_t)NW * G * HD + 2 * NW * G;
    const size_t floats = (size_t)HD * G + 16 + (size_t)NW * TILE * G + comb;
    const size_t smem = floats * sizeof(float);
    auto kern = tq_attn_split_kernel<HD, BITS, G>;
    static lc_smem_optin optin;
    LC_CUDA_TRY(lc_ensure_smem(kern, optin, b->ctx, smem));
    LC_LAUNCH_CHECKED(lc_launch(kern, dim3(grid), dim3(NT), smem, b, p));
    LC_CHECK_LAUNCH("flash_attention_tq");
    b->dispatch_count++;
    return LC_OK;
}

template <int HD, int BITS>
int launch_split_g(lc_batch *b, const TqAttnParams &p, dim3 grid, int g) {
    switch (g) {
        case 1: return launch_split<HD, BITS, 1>(b, p, grid);
        case 2: return launch_split<HD, BITS, 2>(b, p, grid);
        case 4: return launch_split<HD, BITS, 4>(b, p, grid);
        default: return launch_split<HD, BITS, 8>(b, p, grid);
    }
}

template <int HD>
int launch_split_b(lc_batch *b, const TqAttnParams &p, dim3 grid, int g, unsigned bits) {
    switch (bits) {
        case 2: return launch_split_g<HD, 2>(b, p, grid, g);
        case 3: return launch_split_g<HD, 3>(b, p, grid, g);
        default: return launch_split_g<HD, 4>(b, p, grid, g);
    }
}

// Common host path.  `q_f16`/`out_f16` select the fused form.
int tq_attention(const char *name, lc_kernels *k, lc_batch *b, const lc_buf *rq_or_q, bool fused,
                 const lc_buf *kc, const lc_buf *kn, const lc_buf *vc, const lc_buf *vn, const lc_buf *levels,
                 const lc_buf *signs, lc_buf *out, const lc_buf *positions, uint32_t hd, uint32_t kv_len,
                 uint32_t current_pos, uint32_t lane_capacity, uint32_t n_q, uint32_t n_kv, uint32_t window,
                 uint32_t bits, uint32_t n_lanes, uint32_t ring, float scale, uint32_t n_rows = 0,
                 const lc_buf *qfrag = nullptr) {
    // n_rows != 0: prefill / multi-row verify over one cache: row r at position current_pos + r (n_lanes is ignored)
    const bool prefill = n_rows != 0;
    if (prefill) n_lanes = n_rows;
    if (!k || !b || !rq_or_q || !kc || !kn || !vc || !vn || !levels || !out || (fused && !signs))
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    if (bits < 2 || bits > 4) return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: bits %u not in 2..=4", name, bits);
    if (hd != 64 && hd != 128 && hd != 256 && hd != 512)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: head_dim %u must be 64, 128, 256 or 512", name, hd);
    LC_REQUIRE(n_kv >= 1 && n_q >= 1 && n_q % n_kv == 0, "%s: num_q_heads %u must be a multiple of num_kv_heads %u",
               name, n_q, n_kv);
    if (n_lanes == 0) return LC_OK;
    const size_t cb = (size_t)hd * bits / 8;
    const size_t qn = (size_t)n_lanes * n_q * hd;
    LC_REQUIRE(rq_or_q->bytes >= qn * (fused ? 2 : 4) && out->bytes >= qn * (fused ? 2 : 4),
               "%s: query/output buffers too small", name);
    LC_REQUIRE(levels->bytes >= (4u << bits), "%s: levels buffer too small", name);
    if (fused) LC_REQUIRE(signs->bytes >= hd * 4u, "%s: signs buffer too small", name);
    // Rows a launch may touch: single form reads slots < min(kv_len, pos+1) (or < ring).
    size_t rows;
    uint32_t len_max;
    if (positions) {
        LC_REQUIRE(positions->bytes >= (size_t)n_lanes * 4, "%s: positions buffer too small", name);
        LC_REQUIRE(ring <= lane_capacity, "%s: ring %u exceeds lane capacity %u", name, ring, lane_capacity);
        rows = (size_t)n_lanes * lane_capacity;
        len_max = ring ? ring : lane_capacity;
    } else {
        const uint32_t last_pos = current_pos + (prefill ? n_rows - 1 : 0);   // the row that sees the most keys
        const uint32_t seq_len = kv_len < last_pos + 1 ? kv_len : last_pos + 1;
        rows = ring ? (ring < seq_len ? ring : seq_len) : seq_len;
        const uint32_t ws = (window > 0 && last_pos + 1 > window) ? last_pos + 1 - window : 0;
        len_max = seq_len > ws ? seq_len - ws : 0;
        lane_capacity = 0;
    }
    if (window > 0 && len_max > window) len_max = window;
    LC_REQUIRE(kc->bytes >= rows * n_kv * cb && vc->bytes >= rows * n_kv * cb && kn->bytes >= rows * n_kv * 2 &&
                   vn->bytes >= rows * n_kv * 2,
               "%s: KV buffers hold fewer than %zu rows", name, rows);
    LC_REQUIRE(lc_aligned(kc->dptr, 16) && lc_aligned(vc->dptr, 16), "%s: code buffers must be 16-byte aligned", name);
    LC_REQUIRE(lc_aligned(rq_or_q->dptr, fused ? 2 : 4) && lc_aligned(out->dptr, fused ? 2 : 4) &&
                   lc_aligned(levels->dptr, 4) && (!fused || lc_aligned(signs->dptr, 4)) && lc_aligned(kn->dptr, 2) &&
                   lc_aligned(vn->dptr, 2),
               "%s: a buffer is not aligned to its element size", name);

    const uint32_t group = n_q / n_kv;
    int g = group >= 8 ? 8 : (group > 4 ? 8 : (group > 2 ? 4 : (group > 1 ? 2 : 1)));
    // tq2 at head_dim 256 runs on the tensor-core kernel (8 heads per CTA); LOCAL_CUDA_ATTN_MMA=0 keeps the
    // CUDA-core kernel, which also serves every other head size and bit width.
    static const bool mma_allowed = []() { const char *e = getenv("LOCAL_CUDA_ATTN_MMA"); return !(e && e[0] == '0'); }();
    // (the tensor-core kernel copies norms as aligned 4-byte words)
    const size_t norm_words = ((rows * n_kv + 1) & ~(size_t)1) * 2;
    // (... and loads the query and the signs as 16-byte vectors: buffers wrapped at other offsets take the CUDA-core kernel)
    const bool use_mma = mma_allowed && hd == 256 && bits == 2 && lc_aligned(kn->dptr, 4) && lc_aligned(vn->dptr, 4) &&
                         kn->bytes >= norm_words && vn->bytes >= norm_words && (ring == 0 || ring >= 16) &&
                         lc_aligned(rq_or_q->dptr, 16) && (!fused || lc_aligned(signs->dptr, 16));
    if (use_mma) g = 8;
    const uint32_t gchunks = (group + g - 1) / g;
    const uint32_t base = n_lanes * n_kv * gchunks;
    uint32_t want = (2u * (uint32_t)k->ctx->sm_count + base - 1) / base;
    uint32_t by_len = (len_max + NW * TILE - 1) / (NW * TILE);
    if (by_len < 1) by_len = 1;
    uint32_t n_splits = want < by_len ? want : by_len;
    if (n_splits < 1) n_splits = 1;
    if (n_splits > 64) n_splits = 64;
    if (use_mma) {
        // One CTA per SM (registers), so the launch runs in whole waves; every CTA pays a fixed prologue worth
        // about 320 keys.  Pick the split count that minimises waves x (prologue + keys per split).
        const uint32_t sms = (uint32_t)k->ctx->sm_count;
        uint32_t max_s = len_max / 256u;   // at least two 16-key tiles for each of the 8 warps
        if (max_s < 1) max_s = 1;
        if (max_s > 64) max_s = 64;
        uint64_t best_cost = ~0ull;
        for (uint32_t s = 1; s <= max_s; s++) {
            const uint64_t waves = ((uint64_t)base * s + sms - 1) / sms;
            const uint64_t cost = waves * (320u + (len_max + s - 1) / s);
            if (cost < best_cost) { best_cost = cost; n_splits = s; }
        }
    }
    const bool direct = (n_splits == 1 && !fused);
    // The tensor-core kernel merges up to 8 splits itself (one thread-block cluster per lane and kv head, exchange
    // through distributed shared memory, inverse rotation in the kernel): one launch instead of split + merge, the same
    // arithmetic in the same order, bit-identical output.  Alone 57 vs 59 us at 8193 keys x 64 lanes, 12.4 vs 14.6 us
    // for a 512-key window; inside the decode step 2.314 vs 2.331 ms.  (Before the step's other kernels did their
    // weight prefetch ahead of their dependency wait it was the slower form in situ, 3.48 vs 3.36 ms.)
    // LOCAL_CUDA_ATTN_CLUSTER=0 selects the two-launch form.
    static const bool cluster_allowed = []() { const char *e = getenv("LOCAL_CUDA_ATTN_CLUSTER"); return !(e && e[0] == '0'); }();
    const bool cluster_merge = use_mma && cluster_allowed && n_splits <= 8 &&
                               lc_aligned(out->dptr, 16) && (!fused || lc_aligned(signs->dptr, 16));

    if (!direct && !cluster_merge) {
        int st = lc_reserve_scratch(k, b, qn / hd * n_splits * (size_t)(hd + 2) * sizeof(float), 0);
        if (st != LC_OK) return st;
    }
    TqAttnParams p;
    p.rq = fused ? nullptr : (const float *)rq_or_q->dptr;
    p.q = fused ? (const __half *)rq_or_q->dptr : nullptr;
    p.signs = signs ? (const float *)signs->dptr : nullptr;
    p.kc = (const uint8_t *)kc->dptr;
    p.vc = (const uint8_t *)vc->dptr;
    p.kn = (const __half *)kn->dptr;
    p.vn = (const __half *)vn->dptr;
    p.levels = (const float *)levels->dptr;
    p.out = (direct || (cluster_merge && !fused)) ? (float *)out->dptr : nullptr;
    p.out_f16 = (cluster_merge && fused) ? (__half *)out->dptr : nullptr;
    p.cluster_merge = cluster_merge ? 1 : 0;
    p.partial = (float *)k->scratch;
    p.positions = positions ? (const uint32_t *)positions->dptr : nullptr;
    p.kv_len = kv_len;
    p.current_pos = current_pos;
    p.row_positions = prefill ? 1 : 0;
    p.lane_capacity = lane_capacity;
    p.n_q = n_q;
    p.n_kv = n_kv;
    p.window = window;
    p.ring = ring;
    p.n_splits = n_splits;
    p.group = group;
    p.fused_q = fused ? 1 : 0;
    p.direct_out = direct ? 1 : 0;
    p.scale = scale;
    p.status = k->dev_status;
    p.qfrag = nullptr;
    p.early_kv = (qfrag && use_mma && positions) ? 1u : 0u;   // only the decode step passes fragments: its positions are a step input
    if (qfrag && use_mma && fused && lc_qfrag_supported(hd, bits, n_q, n_kv)) {
        LC_REQUIRE(qfrag->bytes >= qn * 4, "%s: query fragment buffer too small", name);
        p.qfrag = (const uint4 *)qfrag->dptr;
    }
    dim3 grid(n_splits, n_kv * gchunks, n_lanes);
    int st;
    if (use_mma) {
        st = lc_tq2_attn_mma_launch(b, p, grid);
    } else {
        switch (hd) {
            case 64: st = launch_split_b<64>(b, p, grid, g, bits); break;
            case 128: st = launch_split_b<128>(b, p, grid, g, bits); break;
            case 256: st = launch_split_b<256>(b, p, grid, g, bits); break;
            default: st = launch_split_b<512>(b, p, grid, g, bits); break;
        }
    }
    if (st != LC_OK || direct || cluster_merge) return st;
    if (fused)
        LC_LAUNCH_CHECKED(lc_launch(tq_attn_merge_kernel<true>, dim3(n_lanes * n_q), dim3(hd), 0, b, (const float *)k->scratch, (const float *)signs->dptr, nullptr, (__half *)out->dptr, hd, n_splits));
    else
        LC_LAUNCH_CHECKED(lc_launch(tq_attn_merge_kernel<false>, dim3(n_lanes * n_q), dim3(hd), 0, b, (const float *)k->scratch, nullptr, (float *)out->dptr, nullptr, hd, n_splits));
    LC_CHECK_LAUNCH("flash_attention_tq merge");
    b->dispatch_count++;
    return LC_OK;
}

}  // namespace

extern "C" {

int lc_flash_attention_tq_into(lc_kernels *k, lc_batch *b, const lc_buf *rq, const lc_buf *k_codes,
                               const lc_buf *k_norms, const lc_buf *v_codes, const lc_buf *v_norms,
                               const lc_buf *levels, lc_buf *out, uint32_t head_dim, uint32_t kv_len,
                               uint32_t current_pos, uint32_t num_q_heads, uint32_t num_kv_heads, uint32_t window,
                               uint32_t bits, uint32_t ring_capacity, float softmax_scale) {
    return tq_attention("flash_attention_tq", k, b, rq, false, k_codes, k_norms, v_codes, v_norms, levels, nullptr,
                        out, nullptr, head_dim, kv_len, current_pos, 0, num_q_heads, num_kv_heads, window, bits, 1,
                        ring_capacity, softmax_scale);
}

int lc_flash_attention_tq_batched_into(lc_kernels *k, lc_batch *b, const lc_buf *rq, const lc_buf *k_codes,
                                       const lc_buf *k_norms, const lc_buf *v_codes, const lc_buf *v_norms,
                                       const lc_buf *levels, lc_buf *out, const lc_buf *positions,
                                       uint32_t head_dim, uint32_t lane_capacity, uint32_t num_q_heads,
                                       uint32_t num_kv_heads, uint32_t window, uint32_t bits, uint32_t n_lanes,
                                       uint32_t ring_capacity, float softmax_scale) {
    if (!positions) return lc_fail(LC_ERR_INVALID_ARGUMENT, "flash_attention_tq_batched: positions is NULL");
    return tq_attention("flash_attention_tq_batched", k, b, rq, false, k_codes, k_norms, v_codes, v_norms, levels,
                        nullptr, out, positions, head_dim, 0, 0, lane_capacity, num_q_heads, num_kv_heads, window,
                        bits, n_lanes, ring_capacity, softmax_scale);
}

int lc_tq_attention_into(lc_kernels *k, lc_batch *b, const lc_buf *q, const lc_buf *k_codes, const lc_buf *k_norms,
                         const lc_buf *v_codes, const lc_buf *v_norms, const lc_buf *levels, const lc_buf *signs,
                         lc_buf *attn_out, uint32_t head_dim, uint32_t kv_len, uint32_t current_pos,
                         uint32_t num_q_heads, uint32_t num_kv_heads, uint32_t window, uint32_t bits,
                         uint32_t ring_capacity, float softmax_scale) {
    return tq_attention("tq_attention", k, b, q, true, k_codes, k_norms, v_codes, v_norms, levels, signs, attn_out,
                        nullptr, head_dim, kv_len, current_pos, 0, num_q_heads, num_kv_heads, window, bits, 1,
                        ring_capacity, softmax_scale);
}

// Prefill / multi-row verify over codes (shaders/attention_flash_tq.metal:290-556, kernels.rs:5259-5420): row r of the
// chunk is a decode query at position start_pos + r over the one cache that already holds the chunk's rows.  Here both
// reference kernels map onto the decode kernels with the chunk's rows as the grid's third dimension: the tensor-core
// kernel already reads every K/V row once for all q-heads of a kv-head, and the rows of a chunk re-read the cache from
// L2, which is what the reference's query-tiled kernel buys with its threadgroup tiles.  So the "tiled" entry point
// is the same launch; it keeps the reference's name and argument list so callers can switch either way.
int lc_flash_attention_tq_prefill_into(lc_kernels *k, lc_batch *b, const lc_buf *rq, const lc_buf *k_codes,
                                       const lc_buf *k_norms, const lc_buf *v_codes, const lc_buf *v_norms,
                                       const lc_buf *levels, lc_buf *out, uint32_t head_dim, uint32_t kv_len,
                                       uint32_t start_pos, uint32_t n_rows, uint32_t num_q_heads, uint32_t num_kv_heads,
                                       uint32_t window, uint32_t bits, uint32_t ring_capacity, float softmax_scale) {
    if (n_rows == 0) return LC_OK;
    return tq_attention("flash_attention_tq_prefill", k, b, rq, false, k_codes, k_norms, v_codes, v_norms, levels, nullptr,
                        out, nullptr, head_dim, kv_len, start_pos, 0, num_q_heads, num_kv_heads, window, bits, 1,
                        ring_capacity, softmax_scale, n_rows);
}

int lc_flash_attention_tq_prefill_tiled_into(lc_kernels *k, lc_batch *b, const lc_buf *rq, const lc_buf *k_codes,
                                             const lc_buf *k_norms, const lc_buf *v_codes, const lc_buf *v_norms,
                                             const lc_buf *levels, lc_buf *out, uint32_t head_dim, uint32_t kv_len,
                                             uint32_t start_pos, uint32_t n_rows, uint32_t num_q_heads,
                                             uint32_t num_kv_heads, uint32_t window, uint32_t bits,
                                             uint32_t ring_capacity, float softmax_scale) {
    if (n_rows == 0) return LC_OK;
    return tq_attention("flash_attention_tq_prefill_tiled", k, b, rq, false, k_codes, k_norms, v_codes, v_norms, levels,
                        nullptr, out, nullptr, head_dim, kv_len, start_pos, 0, num_q_heads, num_kv_heads, window, bits, 1,
                        ring_capacity, softmax_scale, n_rows);
}

// The three dispatches QuantizedKvCache::fused_attention_batch_into issues (kv_cache/quant_cache.rs:620-700) in one
// call: q f16 [n_rows, n_q, hd] in, attn_out f16 out.
int lc_tq_attention_prefill_into(lc_kernels *k, lc_batch *b, const lc_buf *q, const lc_buf *k_codes, const lc_buf *k_norms,
                                 const lc_buf *v_codes, const lc_buf *v_norms, const lc_buf *levels, const lc_buf *signs,
                                 lc_buf *attn_out, uint32_t head_dim, uint32_t kv_len, uint32_t start_pos, uint32_t n_rows,
                                 uint32_t num_q_heads, uint32_t num_kv_heads, uint32_t window, uint32_t bits,
                                 uint32_t ring_capacity, float softmax_scale) {
    if (n_rows == 0) return LC_OK;
    return tq_attention("tq_attention_prefill", k, b, q, true, k_codes, k_norms, v_codes, v_norms, levels, signs, attn_out,
                        nullptr, head_dim, kv_len, start_pos, 0, num_q_heads, num_kv_heads, window, bits, 1, ring_capacity,
                        softmax_scale, n_rows);
}

int lc_tq_attention_batched_into(lc_kernels *k, lc_batch *b, const lc_buf *q, const lc_buf *k_codes,
                                 const lc_buf *k_norms, const lc_buf *v_codes, const lc_buf *v_norms,
                                 const lc_buf *levels, const lc_buf *signs, lc_buf *attn_out,
                                 const lc_buf *positions, uint32_t head_dim, uint32_t lane_capacity,
                                 uint32_t num_q_heads, uint32_t num_kv_heads, uint32_t window, uint32_t bits,
                                 uint32_t n_lanes, uint32_t ring_capacity, float softmax_scale) {
    if (!positions) return lc_fail(LC_ERR_INVALID_ARGUMENT, "tq_attention_batched: positions is NULL");
    return tq_attention("tq_attention_batched", k, b, q, true, k_codes, k_norms, v_codes, v_norms, levels, signs,
                        attn_out, positions, head_dim, 0, 0, lane_capacity, num_q_heads, num_kv_heads, window, bits,
                        n_lanes, ring_capacity, softmax_scale);
}

}  // extern "C"

bool lc_qfrag_supported(uint32_t head_dim, uint32_t bits, uint32_t n_q_heads, uint32_t n_kv_heads) {
    return head_dim == 256 && bits == 2 && n_kv_heads >= 1 && n_q_heads % n_kv_heads == 0 &&
           (n_q_heads / n_kv_heads) % 8 == 0;
}

int lc_tq_attention_batched_frag(lc_kernels *k, lc_batch *b, const lc_buf *q, const lc_buf *k_codes, const lc_buf *k_norms,
                                 const lc_buf *v_codes, const lc_buf *v_norms, const lc_buf *levels, const lc_buf *signs,
                                 lc_buf *attn_out, const lc_buf *positions, uint32_t head_dim, uint32_t lane_capacity,
                                 uint32_t num_q_heads, uint32_t num_kv_heads, uint32_t window, uint32_t bits,
                                 uint32_t n_lanes, uint32_t ring_capacity, float softmax_scale, const lc_buf *qfrag) {
    if (!positions) return lc_fail(LC_ERR_INVALID_ARGUMENT, "tq_attention_batched: positions is NULL");
    return tq_attention("tq_attention_batched", k, b, q, true, k_codes, k_norms, v_codes, v_norms, levels, signs,
                        attn_out, positions, head_dim, 0, 0, lane_capacity, num_q_heads, num_kv_heads, window, bits,
                        n_lanes, ring_capacity, softmax_scale, 0, qfrag);
}

// ---------------------------------------------------------------------------
// Allocation-free variant of lc_tq_attention_into.
//
// Some callers of this library must not allocate device memory at the moment
// they run attention: a serving thread that has handed every spare byte of HBM
// to its KV pool, or a latency-critical loop where cudaMalloc's implicit device
// synchronisation is unacceptable.  The regular
// entry point keeps its split-K partials in a buffer that the `lc_kernels`
// object grows with cudaMalloc on demand; this one keeps them in the fixed
// array below, which is part of the library image: every GPU that loads the
// library holds these 4 MiB until the process exits.
//
// Rules that follow from sharing one array:
//  * the partials of a call must fit: num_q_heads * splits * (head_dim + 2)
//    floats <= LC_NOALLOC_SCRATCH_FLOATS.  The split count is lowered to fit;
//    if even one split does not fit the call is refused with a status.
//  * nothing in the array has to start at zero: every slot the merge kernel
//    reads is written by the split kernel earlier in the same call, so stale
//    contents of the previous call are never observed;
//  * two calls that overlap on the GPU (different streams, or two host threads)
//    race on the array.  Issue them on one stream, or serialise them.
//  * the first call on each device looks up the array's device address
//    (cudaGetSymbolAddress) and, like every launch site of this library, raises
//    the kernels' shared-memory limit on that device; make that first call
//    before any stream capture begins.
//  * this entry point always runs the CUDA-core split kernel, for every head
//    size and bit width; the regular entry point's tensor-core kernel (tq2 at
//    head_dim 256) is not used here, so at that shape it is the slower of the
//    two, with the same results to within the tests' tolerance.
constexpr size_t LC_NOALLOC_SCRATCH_FLOATS = (size_t)1 << 20;  // 4 MiB
static __device__ __align__(256) float g_noalloc_scratch[LC_NOALLOC_SCRATCH_FLOATS];

namespace {

std::atomic<float *> g_noalloc_ptr[LC_MAX_DEVICES];  // device address of g_noalloc_scratch, per device

// The array's name is a host-side stand-in here, not a device address: resolve
// it once per device, with that device current, and leave the caller's current
// device as it was.  Two threads that race on a device's first call both resolve
// the same address, so the slot only needs to be written atomically.
int noalloc_scratch_for(int device, float **out) {
    if (device < 0 || device >= LC_MAX_DEVICES)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "tq_attention_noalloc: device %d out of range", device);
    float *ptr = g_noalloc_ptr[device].load(std::memory_order_acquire);
    if (!ptr) {
        int prev = -1;
        LC_CUDA_TRY(cudaGetDevice(&prev));
        if (prev != device) LC_CUDA_TRY(cudaSetDevice(device));
        cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_noalloc_scratch);
        if (prev != device) cudaSetDevice(prev);
        if (e != cudaSuccess || !ptr)
            return lc_fail(LC_ERR_CUDA, "tq_attention_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_noalloc_ptr[device].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return LC_OK;
}

}  // namespace

extern "C" int lc_tq_attention_noalloc_into(lc_batch *b, const lc_buf *q, const lc_buf *k_codes,
                                            const lc_buf *k_norms, const lc_buf *v_codes, const lc_buf *v_norms,
                                            const lc_buf *levels, const lc_buf *signs, lc_buf *attn_out,
                                            uint32_t head_dim, uint32_t kv_len, uint32_t current_pos,
                                            uint32_t num_q_heads, uint32_t num_kv_heads, uint32_t window,
                                            uint32_t bits, uint32_t ring_capacity, float softmax_scale) {
    const char *name = "tq_attention_noalloc";
    if (!b || !q || !k_codes || !k_norms || !v_codes || !v_norms || !levels || !signs || !attn_out)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: NULL argument", name);
    if (bits < 2 || bits > 4) return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: bits %u not in 2..=4", name, bits);
    if (head_dim != 64 && head_dim != 128 && head_dim != 256 && head_dim != 512)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: head_dim %u must be 64, 128, 256 or 512", name, head_dim);
    LC_REQUIRE(num_kv_heads >= 1 && num_q_heads >= 1 && num_q_heads % num_kv_heads == 0,
               "%s: num_q_heads %u must be a multiple of num_kv_heads %u", name, num_q_heads, num_kv_heads);
    const size_t cb = (size_t)head_dim * bits / 8, qn = (size_t)num_q_heads * head_dim;
    LC_REQUIRE(q->bytes >= qn * 2 && attn_out->bytes >= qn * 2, "%s: query/output buffers too small", name);
    LC_REQUIRE(levels->bytes >= (4u << bits) && signs->bytes >= head_dim * 4u, "%s: codec buffers too small", name);
    const uint32_t seq_len = kv_len < current_pos + 1 ? kv_len : current_pos + 1;
    const size_t rows = ring_capacity ? (ring_capacity < seq_len ? ring_capacity : seq_len) : seq_len;
    const uint32_t ws = (window > 0 && current_pos + 1 > window) ? current_pos + 1 - window : 0;
    uint32_t len_max = seq_len > ws ? seq_len - ws : 0;
    if (window > 0 && len_max > window) len_max = window;
    LC_REQUIRE(k_codes->bytes >= rows * num_kv_heads * cb && v_codes->bytes >= rows * num_kv_heads * cb &&
                   k_norms->bytes >= rows * num_kv_heads * 2 && v_norms->bytes >= rows * num_kv_heads * 2,
               "%s: KV buffers hold fewer than %zu rows", name, rows);
    LC_REQUIRE(lc_aligned(k_codes->dptr, 16) && lc_aligned(v_codes->dptr, 16),
               "%s: code buffers must be 16-byte aligned", name);

    const size_t per_split = qn / head_dim * (size_t)(head_dim + 2);  // floats of partials per split
    if (per_split > LC_NOALLOC_SCRATCH_FLOATS)
        return lc_fail(LC_ERR_INVALID_ARGUMENT,
                       "%s: %u heads of %u need %zu bytes of partials per split; the built-in scratch holds %zu bytes",
                       name, num_q_heads, head_dim, per_split * sizeof(float), LC_NOALLOC_SCRATCH_FLOATS * sizeof(float));
    float *scratch = nullptr;
    int st = noalloc_scratch_for(b->ctx->device, &scratch);
    if (st != LC_OK) return st;

    const uint32_t group = num_q_heads / num_kv_heads;
    const int g = group > 4 ? 8 : (group > 2 ? 4 : (group > 1 ? 2 : 1));
    const uint32_t gchunks = (group + g - 1) / g;
    const uint32_t base = num_kv_heads * gchunks;
    uint32_t n_splits = (2u * (uint32_t)b->ctx->sm_count + base - 1) / base;
    uint32_t by_len = (len_max + NW * TILE - 1) / (NW * TILE);
    if (by_len < 1) by_len = 1;
    if (n_splits > by_len) n_splits = by_len;
    if (n_splits > 64) n_splits = 64;
    const uint32_t fit = (uint32_t)(LC_NOALLOC_SCRATCH_FLOATS / per_split);
    if (n_splits > fit) n_splits = fit;
    if (n_splits < 1) n_splits = 1;

    TqAttnParams p;
    p.out_f16 = nullptr;
    p.qfrag = nullptr;
    p.early_kv = 0;
    p.cluster_merge = 0;
    p.rq = nullptr;
    p.q = (const __half *)q->dptr;
    p.signs = (const float *)signs->dptr;
    p.kc = (const uint8_t *)k_codes->dptr;
    p.vc = (const uint8_t *)v_codes->dptr;
    p.kn = (const __half *)k_norms->dptr;
    p.vn = (const __half *)v_norms->dptr;
    p.levels = (const float *)levels->dptr;
    p.out = nullptr;
    p.partial = scratch;
    p.positions = nullptr;
    p.kv_len = kv_len;
    p.current_pos = current_pos;
    p.row_positions = 0;
    p.lane_capacity = 0;
    p.n_q = num_q_heads;
    p.n_kv = num_kv_heads;
    p.window = window;
    p.ring = ring_capacity;
    p.n_splits = n_splits;
    p.group = group;
    p.fused_q = 1;
    p.direct_out = 0;
    p.scale = softmax_scale;
    p.status = nullptr;
    dim3 grid(n_splits, num_kv_heads * gchunks, 1);
    switch (head_dim) {
        case 64: st = launch_split_b<64>(b, p, grid, g, bits); break;
        case 128: st = launch_split_b<128>(b, p, grid, g, bits); break;
        case 256: st = launch_split_b<256>(b, p, grid, g, bits); break;
        default: st = launch_split_b<512>(b, p, grid, g, bits); break;
    }
    if (st != LC_OK) return st;
    LC_LAUNCH_CHECKED(lc_launch(tq_attn_merge_kernel<true>, dim3(num_q_heads), dim3(head_dim), 0, b, scratch, (const float *)signs->dptr, nullptr,
                                                                       (__half *)attn_out->dptr, head_dim, n_splits));
    LC_CHECK_LAUNCH("tq_attention_noalloc merge");
    b->dispatch_count++;
    return LC_OK;
}
