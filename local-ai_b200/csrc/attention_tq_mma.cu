// Tensor-core decode attention over TurboQuant tq2 codes, head_dim 256, up to 8 q-heads per kv-head:
// the shape of the synthetic E2B-like decoder and of BASELINE's attention configuration.  Same
// contract, grid and split-K partial layout as tq_attn_split_kernel (attention_tq.cu), which remains
// the general path (other head sizes, tq3 / tq4).
//
// Why a second kernel: with 8 q-heads sharing every K/V row the CUDA-core kernel needs 4096 FMAs per
// 132 bytes of KV, which binds long before HBM does.  Here both contractions run on tensor cores, with
// operands built directly in registers:
//   * a shared-memory table maps one code byte (four 2-bit codes) to four f16 levels with a single
//     8-byte load; the table is replicated per lane so lookups never collide on a bank;
//   * S^T[16 keys x 8 heads] = K[16 x 256] . RQ^T: the contraction index (dims) is free to permute, so
//     thread (g, t) of a warp feeds the MMA with the 64 dims held in its own 16 code bytes of keys g, g+8;
//   * O^T[256 dims x 8 heads] += V^T[256 x 16 keys] . P: the V bytes decode to (key, dim-pair) tiles,
//     which movmatrix transposes into the (dim, key-pair) layout the A operand wants; P reaches the B
//     operand the same way.
// f16 levels: the table stores levels / gamma, with gamma searched (1024 mantissas) so that all levels
// are f16-representable to ~1e-6 relative; gamma is folded into the row norms in f32.  Logits, softmax
// and accumulation stay f32.
#include <math.h>

#include "attention_tq.h"

namespace {

constexpr int HD = 256;
constexpr int CB = 64;           // code bytes per row (tq2)
constexpr int NT = 256;
constexpr int NW = NT / 32;
constexpr int G = 8;             // q-heads per CTA (MMA N)
constexpr int KT = 16;           // keys per warp step (MMA M for QK, MMA K for PV)
constexpr int LUT_BYTES = 256 * 32 * 8;

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t pack_h2(float x, float y) {
    __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t byte_of(const uint4 &q, int s) {
    const uint32_t w = s < 4 ? q.x : (s < 8 ? q.y : (s < 12 ? q.z : q.w));
    return (w >> (8 * (s & 3))) & 0xFFu;
}

template <int HDIM>
__device__ __forceinline__ void fwht_rows_cta(float *sh, int rows) {
    const int pairs = rows * (HDIM / 2);
    for (int len = 1; len < HDIM; len <<= 1) {
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

__global__ void __launch_bounds__(NT) tq2_attn_mma_kernel(const TqAttnParams p) {
    lc_pdl_trigger();
    lc_pdl_wait();
    extern __shared__ __align__(16) uint8_t smem[];
    uint2 *lut = reinterpret_cast<uint2 *>(smem);                       // [256 bytes][32 lanes] x 4 f16
    float *rq_s = reinterpret_cast<float *>(smem + LUT_BYTES);          // [G][HD] rotated, scaled query
    __shared__ float gamma_s;
    __shared__ float cand_err[NW];
    __shared__ int cand_idx[NW];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
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
    } else {
        pos = p.current_pos;
        seq_len = min(p.kv_len, pos + 1u);
    }
    const uint32_t win_start = (p.window > 0u && pos + 1u > p.window) ? (pos + 1u - p.window) : 0u;
    const uint32_t n_keys = seq_len > win_start ? seq_len - win_start : 0u;
    uint32_t per = (n_keys + p.n_splits - 1) / p.n_splits;
    per = (per + KT - 1) & ~(uint32_t)(KT - 1);
    const uint32_t k_begin = win_start + split * per;
    const uint32_t k_end = min(seq_len, k_begin + per);
    const size_t lane_base = (size_t)lane_idx * p.lane_capacity;

    // ---- prologue 1: gamma such that every level / gamma is (almost) exactly an f16 ----
    const float lv0 = p.levels[0], lv1 = p.levels[1], lv2 = p.levels[2], lv3 = p.levels[3];
    {
        const float ref = fmaxf(fmaxf(fabsf(lv0), fabsf(lv1)), fmaxf(fabsf(lv2), fabsf(lv3)));
        float best = INFINITY;
        int besti = 0;
        for (int j = threadIdx.x; j < 1024; j += NT) {
            const float gm = ref > 0.f ? ref / (1.0f + (float)j * (1.0f / 1024.0f)) : 1.0f;  // largest level -> [1, 2)
            float e = 0.f;
            const float ls[4] = {lv0, lv1, lv2, lv3};
#pragma unroll
            for (int l = 0; l < 4; l++) {
                const float back = __half2float(__float2half_rn(ls[l] / gm)) * gm;
                e = fmaxf(e, ls[l] != 0.f ? fabsf(back - ls[l]) / fabsf(ls[l]) : 0.f);
            }
            if (e < best) { best = e; besti = j; }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {   // arg-min inside the warp, lowest index on ties
            const float oe = __shfl_xor_sync(0xffffffffu, best, off);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, off);
            if (oe < best || (oe == best && oi < besti)) { best = oe; besti = oi; }
        }
        if (lane == 0) { cand_err[warp] = best; cand_idx[warp] = besti; }
        __syncthreads();
        if (threadIdx.x == 0) {
            float b = cand_err[0];
            int bi = cand_idx[0];
            for (int i = 1; i < NW; i++)
                if (cand_err[i] < b || (cand_err[i] == b && cand_idx[i] < bi)) { b = cand_err[i]; bi = cand_idx[i]; }
            gamma_s = ref > 0.f ? ref / (1.0f + (float)bi * (1.0f / 1024.0f)) : 1.0f;
        }
        __syncthreads();
    }
    const float gamma = gamma_s;
    // ---- prologue 2: byte -> four f16 levels table, one copy per lane ----
    {
        const float ls[4] = {lv0 / gamma, lv1 / gamma, lv2 / gamma, lv3 / gamma};
        for (int e = threadIdx.x; e < 256 * 32; e += NT) {
            const int byte = e >> 5;
            uint2 v;
            v.x = pack_h2(ls[byte & 3], ls[(byte >> 2) & 3]);
            v.y = pack_h2(ls[(byte >> 4) & 3], ls[(byte >> 6) & 3]);
            lut[e] = v;
        }
    }
    // ---- prologue 3: rotated, scaled query rq_s[g][d] ----
    if (p.fused_q) {
        for (int i = threadIdx.x; i < G * HD; i += NT) {
            const int h = i / HD, d = i - h * HD;
            float v = 0.f;
            if (h < gvalid) v = __half2float(p.q[((size_t)lane_idx * p.n_q + qh0 + h) * HD + d]) * p.signs[d];
            rq_s[i] = v;
        }
        fwht_rows_cta<HD>(rq_s, G);
        const float f = p.scale / sqrtf((float)HD);
        for (int i = threadIdx.x; i < G * HD; i += NT) rq_s[i] *= f;
    } else {
        for (int i = threadIdx.x; i < G * HD; i += NT) {
            const int h = i / HD, d = i - h * HD;
            rq_s[i] = h < gvalid ? p.rq[((size_t)lane_idx * p.n_q + qh0 + h) * HD + d] * p.scale : 0.f;
        }
    }
    __syncthreads();
    // B fragments of the query: thread (g, t) holds head g, dims 64t + 4s + {0,1} and + {2,3}, s = 0..15
    // The query is the one operand f16 cannot hold well enough when logits are large (softmax scale 1.0):
    // it is split into a high f16 part and the f16 of the remainder, and each k-step issues two MMAs.
    uint32_t bq[16][2], bql[16][2];
#pragma unroll
    for (int s = 0; s < 16; s++) {
        const float *r = rq_s + g * HD + 64 * t + 4 * s;
        float hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            hi[e] = __half2float(__float2half_rn(r[e]));
            lo[e] = r[e] - hi[e];
        }
        bq[s][0] = pack_h2(hi[0], hi[1]);
        bq[s][1] = pack_h2(hi[2], hi[3]);
        bql[s][0] = pack_h2(lo[0], lo[1]);
        bql[s][1] = pack_h2(lo[2], lo[3]);
    }
    const uint2 *lut_lane = lut + lane;

    // ---- main loop: each warp takes every 8th 16-key tile of this split ----
    float o[16][4];
#pragma unroll
    for (int s = 0; s < 16; s++) o[s][0] = o[s][1] = o[s][2] = o[s][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_part[2] = {0.f, 0.f};   // heads 2t, 2t+1 (l: this thread's keys only)

    // One tile of codes is always in flight ahead of the one being consumed.
    struct Tile { uint4 kqa, kqb, vqa, vqb; float kna, knb, vna, vnb; };
    auto fetch = [&](uint32_t t0, Tile &tl) {
        const uint32_t ka = t0 + g, kb = t0 + g + 8;
        const uint32_t kca = ka < k_end ? ka : t0, kcb = kb < k_end ? kb : t0;   // t0 is always a valid key
        const size_t slot_a = (lane_base + (p.ring ? kca % p.ring : kca)) * p.n_kv + kv_head;
        const size_t slot_b = (lane_base + (p.ring ? kcb % p.ring : kcb)) * p.n_kv + kv_head;
        tl.kqa = __ldg(reinterpret_cast<const uint4 *>(p.kc + slot_a * CB) + t);
        tl.kqb = __ldg(reinterpret_cast<const uint4 *>(p.kc + slot_b * CB) + t);
        tl.vqa = __ldg(reinterpret_cast<const uint4 *>(p.vc + slot_a * CB) + t);
        tl.vqb = __ldg(reinterpret_cast<const uint4 *>(p.vc + slot_b * CB) + t);
        tl.kna = __half2float(p.kn[slot_a]);
        tl.knb = __half2float(p.kn[slot_b]);
        tl.vna = __half2float(p.vn[slot_a]);
        tl.vnb = __half2float(p.vn[slot_b]);
    };
    Tile nxt;
    const uint32_t t_first = k_begin + warp * KT;
    if (t_first < k_end) fetch(t_first, nxt);
    for (uint32_t t0 = t_first; t0 < k_end; t0 += NW * KT) {
        const Tile cur = nxt;
        if (t0 + NW * KT < k_end) fetch(t0 + NW * KT, nxt);
        const bool va = t0 + g < k_end, vb = t0 + g + 8 < k_end;
        const uint4 kqa = cur.kqa, kqb = cur.kqb, vqa = cur.vqa, vqb = cur.vqb;
        const float kna = cur.kna * gamma, knb = cur.knb * gamma, vna = cur.vna * gamma, vnb = cur.vnb * gamma;

        // S^T[16 keys x 8 heads]
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < 16; s++) {
            const uint2 la = lut_lane[byte_of(kqa, s) * 32], lb = lut_lane[byte_of(kqb, s) * 32];
            const uint32_t a[4] = {la.x, lb.x, la.y, lb.y};
            mma16816(c, a, bq[s]);
            mma16816(c, a, bql[s]);
        }
        // logits of keys g (c0, c1) and g+8 (c2, c3) for heads 2t, 2t+1
        float sA[2] = {va ? c[0] * kna : -INFINITY, va ? c[1] * kna : -INFINITY};
        float sB[2] = {vb ? c[2] * knb : -INFINITY, vb ? c[3] * knb : -INFINITY};
        float pa[2], pb[2], resc[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float tm = fmaxf(sA[h], sB[h]);
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 4));
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 8));
            tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 16));
            const float m_new = fmaxf(m_run[h], tm);    // finite: key t0 is valid
            resc[h] = __expf(m_run[h] - m_new);
            pa[h] = __expf(sA[h] - m_new);
            pb[h] = __expf(sB[h] - m_new);
            l_part[h] = l_part[h] * resc[h] + pa[h] + pb[h];
            m_run[h] = m_new;
        }
        if (__any_sync(0xffffffffu, resc[0] != 1.0f || resc[1] != 1.0f)) {   // the running max moved for some head
#pragma unroll
            for (int s = 0; s < 16; s++) {
                o[s][0] *= resc[0]; o[s][1] *= resc[1]; o[s][2] *= resc[0]; o[s][3] *= resc[1];
            }
        }
        // P (times the value norms) into the B operand: (key g | g+8; heads 2t, 2t+1) -> transposed
        uint32_t bp[2];
        bp[0] = movmatrix_trans(pack_h2(pa[0] * vna, pa[1] * vna));
        bp[1] = movmatrix_trans(pack_h2(pb[0] * vnb, pb[1] * vnb));
        // O^T[256 dims x 8 heads] += V^T . P, one 16-dim tile per code byte index s
#pragma unroll
        for (int s = 0; s < 16; s++) {
            const uint2 la = lut_lane[byte_of(vqa, s) * 32], lb = lut_lane[byte_of(vqb, s) * 32];
            uint32_t a[4];
            a[0] = movmatrix_trans(la.x);   // dims rows 0-7,  keys 0-7
            a[1] = movmatrix_trans(la.y);   // dims rows 8-15, keys 0-7
            a[2] = movmatrix_trans(lb.x);   // dims rows 0-7,  keys 8-15
            a[3] = movmatrix_trans(lb.y);   // dims rows 8-15, keys 8-15
            mma16816(o[s], a, bp);
        }
    }

    // ---- merge the 8 warps; lut memory is reused for the per-warp accumulators ----
    l_part[0] += __shfl_xor_sync(0xffffffffu, l_part[0], 4);
    l_part[0] += __shfl_xor_sync(0xffffffffu, l_part[0], 8);
    l_part[0] += __shfl_xor_sync(0xffffffffu, l_part[0], 16);
    l_part[1] += __shfl_xor_sync(0xffffffffu, l_part[1], 4);
    l_part[1] += __shfl_xor_sync(0xffffffffu, l_part[1], 8);
    l_part[1] += __shfl_xor_sync(0xffffffffu, l_part[1], 16);
    __syncthreads();   // every warp is done with the table
    float *acc_s = reinterpret_cast<float *>(smem);   // [NW][G][HD]
    float *m_s = reinterpret_cast<float *>(smem + LUT_BYTES);   // [NW][G]  (rq_s is dead too)
    float *l_s = m_s + NW * G;
    if (g == 0) {
        m_s[warp * G + 2 * t] = m_run[0];
        m_s[warp * G + 2 * t + 1] = m_run[1];
        l_s[warp * G + 2 * t] = l_part[0];
        l_s[warp * G + 2 * t + 1] = l_part[1];
    }
    // row g of tile s is dim 64*(g>>1) + 4s + (g&1); row g+8 is two dims further
    const int d_lo = 64 * (g >> 1) + (g & 1);
#pragma unroll
    for (int s = 0; s < 16; s++) {
        float *base = acc_s + (size_t)(warp * G) * HD + d_lo + 4 * s;
        base[(2 * t) * HD] = o[s][0];
        base[(2 * t + 1) * HD] = o[s][1];
        base[(2 * t) * HD + 2] = o[s][2];
        base[(2 * t + 1) * HD + 2] = o[s][3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < gvalid * HD; i += NT) {
        const int h = i / HD, d = i - h * HD;
        float gmax = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; w++) gmax = fmaxf(gmax, m_s[w * G + h]);
        float gsum = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) {
            const float mw = m_s[w * G + h];
            const float f = (mw == -INFINITY) ? 0.f : __expf(mw - gmax);
            gsum += f * l_s[w * G + h];
            acc += f * acc_s[(size_t)(w * G + h) * HD + d];
        }
        const size_t qh = (size_t)lane_idx * p.n_q + qh0 + h;
        if (p.direct_out) {
            p.out[qh * HD + d] = gsum > 0.f ? acc / gsum : 0.f;
        } else {
            float *pp = p.partial + (qh * p.n_splits + split) * (size_t)(HD + 2);
            if (d == 0) {
                pp[0] = gmax;
                pp[1] = gsum;
            }
            pp[2 + d] = acc;
        }
    }
}

}  // namespace

int lc_tq2_attn_mma_launch(lc_batch *b, const TqAttnParams &p, dim3 grid) {
    const size_t smem = (size_t)LUT_BYTES + (size_t)G * HD * sizeof(float);
    static bool configured = false;
    if (!configured) {
        LC_CUDA_TRY(cudaFuncSetAttribute(tq2_attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    LC_LAUNCH_CHECKED(lc_launch(tq2_attn_mma_kernel, grid, dim3(NT), smem, b, p));
    b->dispatch_count++;
    return LC_OK;
}
