// Tensor-core decode attention over TurboQuant tq2 codes, head_dim 256, up to 8 q-heads per kv-head:
// the shape of the synthetic E2B-like decoder and of the attention benchmark configuration.  Same
// contract, grid and split-K partial layout as tq_attn_split_kernel (attention_tq.cu), which remains
// the general path (other head sizes, tq3 / tq4).
//
// Why a second kernel: with 8 q-heads sharing every K/V row the CUDA-core kernel needs 4096 FMAs per
// 132 bytes of KV, which binds long before HBM does.  Here both contractions run on tensor cores, with
// operands built directly in registers:
//   * a shared-memory table maps one code byte (four 2-bit codes) to four f16 levels with a single
//     8-byte load; the table is replicated 16 times so the lookups of a half-warp never collide on a bank;
//   * S^T[16 keys x 8 heads] = K[16 x 256] . RQ^T: the contraction index (dims) is free to permute, so
//     thread (g, t) of a warp feeds the MMA with the 64 dims held in its own 16 code bytes of keys g, g+8;
//   * O^T[256 dims x 8 heads] += V^T[256 x 16 keys] . P: the A operand wants (dim; two adjacent keys) per
//     register, so thread (g, t) decodes bytes 8g..8g+7 of keys 2t, 2t+1, 2t+8, 2t+9 itself and pairs the
//     table entries of adjacent keys with byte permutes (no cross-lane traffic); P reaches the B operand
//     through one movmatrix transpose per 8 keys;
//   * codes and norms stream through a per-warp cp.async ring in shared memory (five tiles in flight).
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
constexpr int LUT_COPIES = 16;   // an 8-byte shared load is served per half-warp, so 16 copies are conflict-free
constexpr int LUT_BYTES = 256 * LUT_COPIES * 8;
constexpr int ACC_BYTES = NW * 16 * 4 * 32 * 4;   // merge staging, reuses the front of shared memory
constexpr int DEPTH = 6;         // ring slots per warp (DEPTH - 1 tiles in flight)
constexpr int RING_OFF = LUT_BYTES + G * HD * 4 + 256 * 8;
constexpr int SMEM_BYTES = RING_OFF + NW * DEPTH * (4 * 32 * 16 + 32 * 4);
static_assert(SMEM_BYTES >= ACC_BYTES + 1024 + G * HD * 4, "merge staging must fit");
static_assert(NW == G && NT == 256, "the prologue maps warps to heads and threads to code bytes");

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(void *dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void *dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// a shared-memory word / 16 bytes of CTA `rank` of this cluster (or of this CTA when the launch is not clustered)
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr, uint32_t rank, bool clustered) {
    float v;
    if (clustered) {
        uint32_t ra;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(ra) : "r"(addr), "r"(rank));
        asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(ra));
    } else {
        asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(addr));
    }
    return v;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr, uint32_t rank, bool clustered) {
    float4 v;
    if (clustered) {
        uint32_t ra;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(ra) : "r"(addr), "r"(rank));
        asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(ra));
    } else {
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    }
    return v;
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

// rq_s index of (head h, dim d): the order in which thread (g, t) = lane 4g + t reads its B fragments,
// so that fragment loads are one conflict-free float4 per (s, lane).  d = 64t + 4s + e.
__device__ __forceinline__ int rq_index(int h, int d) {
    return (((d & 63) >> 2) * 32 + h * 4 + (d >> 6)) * 4 + (d & 3);
}

__global__ void __launch_bounds__(NT) tq2_attn_mma_kernel(const TqAttnParams p) {
    lc_pdl_trigger();
    extern __shared__ __align__(16) uint8_t smem[];
    uint2 *lut = reinterpret_cast<uint2 *>(smem);                       // [256 bytes][16 copies] x 4 f16
    float *rq_s = reinterpret_cast<float *>(smem + LUT_BYTES);          // [16 s][32 lanes][4] rotated, scaled query
    uint2 *ent_s = reinterpret_cast<uint2 *>(smem + LUT_BYTES + G * HD * sizeof(float));   // [256] one table copy
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

    // ---- before the dependency wait: everything that depends on the codec's levels only (a constant operand): the
    //      gamma search and the byte table.  A CTA that becomes resident while its predecessor drains does this
    //      part for free. ----
    const float lv0 = p.levels[0], lv1 = p.levels[1], lv2 = p.levels[2], lv3 = p.levels[3];
    // ---- prologue 1: gamma such that every level / gamma is (almost) exactly an f16 ----
    const float ref = fmaxf(fmaxf(fabsf(lv0), fabsf(lv1)), fmaxf(fabsf(lv2), fabsf(lv3)));
    {
        const float ia0 = lv0 != 0.f ? 1.0f / fabsf(lv0) : 0.f, ia1 = lv1 != 0.f ? 1.0f / fabsf(lv1) : 0.f;
        const float ia2 = lv2 != 0.f ? 1.0f / fabsf(lv2) : 0.f, ia3 = lv3 != 0.f ? 1.0f / fabsf(lv3) : 0.f;
        float best = INFINITY;
        int besti = 0;
#pragma unroll
        for (int it = 0; it < 1024 / NT; it++) {
            const int j = threadIdx.x + it * NT;
            const float gm = ref > 0.f ? ref / (1.0f + (float)j * (1.0f / 1024.0f)) : 1.0f;  // largest level -> [1, 2)
            const float inv = __frcp_rn(gm);
            float e = fabsf(__half2float(__float2half_rn(lv0 * inv)) * gm - lv0) * ia0;
            e = fmaxf(e, fabsf(__half2float(__float2half_rn(lv1 * inv)) * gm - lv1) * ia1);
            e = fmaxf(e, fabsf(__half2float(__float2half_rn(lv2 * inv)) * gm - lv2) * ia2);
            e = fmaxf(e, fabsf(__half2float(__float2half_rn(lv3 * inv)) * gm - lv3) * ia3);
            if (e < best) { best = e; besti = j; }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {   // arg-min inside the warp, lowest index on ties
            const float oe = __shfl_xor_sync(0xffffffffu, best, off);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, off);
            if (oe < best || (oe == best && oi < besti)) { best = oe; besti = oi; }
        }
        if (lane == 0) { cand_err[warp] = best; cand_idx[warp] = besti; }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float b2 = cand_err[0];
        int bi = cand_idx[0];
        for (int i = 1; i < NW; i++)
            if (cand_err[i] < b2 || (cand_err[i] == b2 && cand_idx[i] < bi)) { b2 = cand_err[i]; bi = cand_idx[i]; }
        gamma_s = ref > 0.f ? ref / (1.0f + (float)bi * (1.0f / 1024.0f)) : 1.0f;
    }
    __syncthreads();
    const float gamma = gamma_s;
    // ---- prologue 3: byte -> four f16 levels table; one copy first, then one copy per lane ----
    {
        const int byte = threadIdx.x;   // NT == 256
        const float inv_levels[4] = {lv0 / gamma, lv1 / gamma, lv2 / gamma, lv3 / gamma};
        float e4[4];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int c = (byte >> (2 * q)) & 3;
            e4[q] = c == 0 ? inv_levels[0] : (c == 1 ? inv_levels[1] : (c == 2 ? inv_levels[2] : inv_levels[3]));
        }
        uint2 v;
        v.x = pack_h2(e4[0], e4[1]);
        v.y = pack_h2(e4[2], e4[3]);
        ent_s[byte] = v;
    }
    __syncthreads();
#pragma unroll 8
    for (int e = threadIdx.x; e < 256 * LUT_COPIES; e += NT) lut[e] = ent_s[e / LUT_COPIES];

    // Codes and norms of keys below the lanes' positions were written by earlier steps; only the key at the position
    // itself comes from the predecessor.  A caller that also guarantees that `positions` was written before the
    // predecessor kernels started (the decode step: it is an input of the step) sets early_kv, and the first tiles'
    // copies are then in flight while the predecessor finishes.
    const bool early = p.early_kv != 0u && p.positions != nullptr && p.row_positions == 0u;
    if (!early) lc_pdl_wait();
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
    per = (per + KT - 1) & ~(uint32_t)(KT - 1);
    const uint32_t k_begin = win_start + split * per;
    const uint32_t k_end = min(seq_len, k_begin + per);
    const size_t lane_base = (size_t)lane_idx * p.lane_capacity;

    // Each warp keeps DEPTH - 1 tiles of codes and norms in flight.  Every thread copies, with cp.async, exactly the
    // bytes it will consume into its own slots of a shared-memory ring, so no cross-thread synchronisation is needed:
    //   K codes: keys g and g + 8, bytes 16 t .. 16 t + 15 (the thread's 64 dims of the QK contraction);
    //   V codes: keys 2t, 2t + 1, 2t + 8, 2t + 9, bytes 8 g .. 8 g + 7 (the thread's 32 output dims of PV);
    //   one 4-byte word holding one norm (lanes 0-15: key norm of key `lane`; 16-31: value norm of key `lane - 16`).
    uint4 *ring_c = reinterpret_cast<uint4 *>(smem + RING_OFF) + warp * (DEPTH * 4 * 32);
    uint32_t *ring_n = reinterpret_cast<uint32_t *>(smem + RING_OFF + NW * DEPTH * 4 * 32 * 16) + warp * (DEPTH * 32);
    uint32_t parity = 0;   // bit `stage`: which half of the copied word is this lane's norm
    auto issue = [&](uint32_t t0, int stage) {
        const uint32_t r0 = p.ring ? t0 % p.ring : t0;   // ring slot of the tile's first key (ring >= 16)
        auto slot_of = [&](uint32_t off) -> size_t {
            uint32_t r = t0 + off < k_end ? r0 + off : r0;   // t0 is always a valid key
            if (p.ring && r >= p.ring) r -= p.ring;
            return (lane_base + r) * p.n_kv + kv_head;
        };
        const size_t slot_n = slot_of(lane & 15);
        uint4 *dst = ring_c + stage * 4 * 32 + lane;
        cp_async16(dst, p.kc + slot_of(g) * CB + 16 * t);
        cp_async16(dst + 32, p.kc + slot_of(g + 8) * CB + 16 * t);
        uint2 *dv = reinterpret_cast<uint2 *>(dst + 64);
        cp_async8(dv, p.vc + slot_of(2 * t) * CB + 8 * g);
        cp_async8(dv + 1, p.vc + slot_of(2 * t + 1) * CB + 8 * g);
        dv = reinterpret_cast<uint2 *>(dst + 96);
        cp_async8(dv, p.vc + slot_of(2 * t + 8) * CB + 8 * g);
        cp_async8(dv + 1, p.vc + slot_of(2 * t + 9) * CB + 8 * g);
        const __half *nsrc = (lane < 16 ? p.kn : p.vn) + (slot_n & ~(size_t)1);
        cp_async4(ring_n + stage * 32 + lane, nsrc);
        parity = (parity & ~(1u << stage)) | ((uint32_t)(slot_n & 1) << stage);
    };
    const uint32_t t_first = k_begin + warp * KT;
    uint32_t t_issue = t_first;
    // With early_kv the first tiles leave before the dependency wait, up to the tile that holds the key the
    // predecessor is writing (position pos: the last key of the last split); that tile and the ones after it follow
    // the wait.  Groups are committed in tile order either way.
    int issued = 0;
    if (early) {
#pragma unroll
        for (int i = 0; i < DEPTH - 1; i++) {
            if (issued == i && !(t_issue <= pos && pos < t_issue + KT)) {
                if (t_issue < k_end) issue(t_issue, i);
                cp_async_commit();
                t_issue += NW * KT;
                issued = i + 1;
            }
        }
        lc_pdl_wait();
    }
#pragma unroll
    for (int i = 0; i < DEPTH - 1; i++) {
        if (i >= issued) {
            if (t_issue < k_end) issue(t_issue, i);
            cp_async_commit();
            t_issue += NW * KT;
        }
    }

    // ---- after the wait: the query ----
    const size_t q_row = ((size_t)lane_idx * p.n_q + qh0 + warp) * HD + 8 * lane;   // warp w owns head w
    uint4 q_raw = make_uint4(0u, 0u, 0u, 0u);
    float4 q_s0 = make_float4(0.f, 0.f, 0.f, 0.f), q_s1 = q_s0;
    // B fragments of the query: thread (g, t) holds head g, dims 64t + 4s + {0,1} and + {2,3}, s = 0..15.
    // The query is the one operand f16 cannot hold well enough when logits are large (softmax scale 1.0):
    // it is split into a high f16 part and the f16 of the remainder, and each k-step issues two MMAs.
    uint32_t bq[16][2], bql[16][2];
    const bool have_frag = p.qfrag != nullptr;   // the launch that wrote q left the fragments ready (group % 8 == 0)
    if (have_frag) {
        const uint4 *src = p.qfrag + ((size_t)lane_idx * (p.n_q >> 3) + (qh0 >> 3)) * 512 + lane;
#pragma unroll
        for (int s = 0; s < 16; s++) {
            const uint4 v = src[s * 32];
            bq[s][0] = v.x;
            bq[s][1] = v.y;
            bql[s][0] = v.z;
            bql[s][1] = v.w;
        }
    } else if (warp < gvalid) {
        if (p.fused_q) {
            q_raw = *reinterpret_cast<const uint4 *>(p.q + q_row);
            q_s0 = *reinterpret_cast<const float4 *>(p.signs + 8 * lane);
            q_s1 = *reinterpret_cast<const float4 *>(p.signs + 8 * lane + 4);
        } else {
            q_s0 = *reinterpret_cast<const float4 *>(p.rq + q_row);
            q_s1 = *reinterpret_cast<const float4 *>(p.rq + q_row + 4);
        }
    }
    // ---- prologue 2 (independent of gamma): rotated, scaled query; warp w owns head w ----
    if (!have_frag) {
        const int h = warp;   // NW == G
        float x[8];
        if (h < gvalid) {
            if (p.fused_q) {
                const __half2 *hp = reinterpret_cast<const __half2 *>(&q_raw);
                const float sg[8] = {q_s0.x, q_s0.y, q_s0.z, q_s0.w, q_s1.x, q_s1.y, q_s1.z, q_s1.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = __half22float2(hp[e]);
                    x[2 * e] = f.x * sg[2 * e];
                    x[2 * e + 1] = f.y * sg[2 * e + 1];
                }
                // 256-point Walsh-Hadamard butterflies: strides 1, 2, 4 inside the thread, 8..128 across lanes
#pragma unroll
                for (int len = 1; len < 8; len <<= 1) {
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        if (!(i & len)) {
                            const float a = x[i], b2 = x[i + len];
                            x[i] = a + b2;
                            x[i + len] = a - b2;
                        }
                    }
                }
#pragma unroll
                for (int m = 1; m < 32; m <<= 1) {
                    const bool upper = lane & m;
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const float o2 = __shfl_xor_sync(0xffffffffu, x[i], m);
                        x[i] = upper ? o2 - x[i] : x[i] + o2;
                    }
                }
                const float f = p.scale / sqrtf((float)HD);
#pragma unroll
                for (int i = 0; i < 8; i++) x[i] *= f;
            } else {
                const float4 r0 = q_s0, r1 = q_s1;
                x[0] = r0.x * p.scale; x[1] = r0.y * p.scale; x[2] = r0.z * p.scale; x[3] = r0.w * p.scale;
                x[4] = r1.x * p.scale; x[5] = r1.y * p.scale; x[6] = r1.z * p.scale; x[7] = r1.w * p.scale;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) x[i] = 0.f;
        }
        *reinterpret_cast<float4 *>(rq_s + rq_index(h, 8 * lane)) = make_float4(x[0], x[1], x[2], x[3]);
        *reinterpret_cast<float4 *>(rq_s + rq_index(h, 8 * lane + 4)) = make_float4(x[4], x[5], x[6], x[7]);
    }
    __syncthreads();   // the rotated query is in place; so is every copy of the table
    if (!have_frag) {
#pragma unroll
        for (int s = 0; s < 16; s++) {
            const float4 r4 = *reinterpret_cast<const float4 *>(rq_s + (s * 32 + lane) * 4);
            const float r[4] = {r4.x, r4.y, r4.z, r4.w};
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
    }
    const uint2 *lut_lane = lut + (lane & (LUT_COPIES - 1));

    // ---- main loop: each warp takes every 8th 16-key tile of this split ----
    float o[16][4];
#pragma unroll
    for (int s = 0; s < 16; s++) o[s][0] = o[s][1] = o[s][2] = o[s][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_part[2] = {0.f, 0.f};   // heads 2t, 2t+1 (l: this thread's keys only)

    int stage = 0;
    for (uint32_t t0 = t_first; t0 < k_end; t0 += NW * KT) {
        // tile t0 is the oldest group in flight; DEPTH - 2 newer ones may still be pending
        cp_async_wait<DEPTH - 2>();
        const uint4 *src = ring_c + stage * 4 * 32 + lane;
        const uint4 kqa = src[0], kqb = src[32], vqa = src[64], vqb = src[96];
        const uint32_t nw = ring_n[stage * 32 + lane];
        const float n_own = __half2float(__ushort_as_half((unsigned short)((parity >> stage) & 1u ? nw >> 16 : nw & 0xFFFFu))) * gamma;
        const float kna = __shfl_sync(0xffffffffu, n_own, g), knb = __shfl_sync(0xffffffffu, n_own, g + 8);
        const float vna = __shfl_sync(0xffffffffu, n_own, 16 + g), vnb = __shfl_sync(0xffffffffu, n_own, 24 + g);
        // refill: the slot of the tile consumed in the previous iteration is free (its values were used by then)
        {
            const int st_fill = stage == 0 ? DEPTH - 1 : stage - 1;
            if (t_issue < k_end) issue(t_issue, st_fill);
            cp_async_commit();
            t_issue += NW * KT;
        }
        stage = stage + 1 == DEPTH ? 0 : stage + 1;
        const bool va = t0 + g < k_end, vb = t0 + g + 8 < k_end;

        // S^T[16 keys x 8 heads]
        // eight independent accumulation chains (k-step mod 4, high / low query parts)
        float c8[8][4];
#pragma unroll
        for (int i = 0; i < 8; i++) c8[i][0] = c8[i][1] = c8[i][2] = c8[i][3] = 0.f;
#pragma unroll
        for (int s = 0; s < 16; s++) {
            const uint2 la = lut_lane[byte_of(kqa, s) * LUT_COPIES], lb = lut_lane[byte_of(kqb, s) * LUT_COPIES];
            const uint32_t a[4] = {la.x, lb.x, la.y, lb.y};
            mma16816(c8[2 * (s & 3)], a, bq[s]);
            mma16816(c8[2 * (s & 3) + 1], a, bql[s]);
        }
        float c[4];
#pragma unroll
        for (int e = 0; e < 4; e++)
            c[e] = ((c8[0][e] + c8[2][e]) + (c8[4][e] + c8[6][e])) + ((c8[1][e] + c8[3][e]) + (c8[5][e] + c8[7][e]));
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
        // P (times the value norms) into the B operand: (key g | g+8; heads 2t, 2t+1) -> (keys 2t, 2t+1 | +8; head g)
        uint32_t bp[2];
        bp[0] = movmatrix_trans(pack_h2(pa[0] * vna, pa[1] * vna));
        bp[1] = movmatrix_trans(pack_h2(pb[0] * vnb, pb[1] * vnb));
        // O^T[256 dims x 8 heads] += V^T . P.  Code byte u of this thread's 8 (dims 32 g + 4 u .. + 3) of its four keys
        // feeds two MMAs: tile 2u has rows (g, g + 8) = dims (32 g + 4 u, + 1), tile 2u + 1 the next two dims.  The
        // A fragment wants (dim; two adjacent keys) per register: a byte permute of two table entries.
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const uint2 e0 = lut_lane[byte_of(vqa, u) * LUT_COPIES], e1 = lut_lane[byte_of(vqa, 8 + u) * LUT_COPIES];   // keys 2t, 2t+1
            const uint2 e2 = lut_lane[byte_of(vqb, u) * LUT_COPIES], e3 = lut_lane[byte_of(vqb, 8 + u) * LUT_COPIES];   // keys 2t+8, 2t+9
            uint32_t a[4];
            a[0] = __byte_perm(e0.x, e1.x, 0x5410);
            a[1] = __byte_perm(e0.x, e1.x, 0x7632);
            a[2] = __byte_perm(e2.x, e3.x, 0x5410);
            a[3] = __byte_perm(e2.x, e3.x, 0x7632);
            mma16816(o[2 * u], a, bp);
            a[0] = __byte_perm(e0.y, e1.y, 0x5410);
            a[1] = __byte_perm(e0.y, e1.y, 0x7632);
            a[2] = __byte_perm(e2.y, e3.y, 0x5410);
            a[3] = __byte_perm(e2.y, e3.y, 0x7632);
            mma16816(o[2 * u + 1], a, bp);
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
    float *m_s = reinterpret_cast<float *>(smem + ACC_BYTES);   // [NW][G]  (query, table and ring are all dead)
    float *l_s = m_s + NW * G;
    if (g == 0) {
        m_s[warp * G + 2 * t] = m_run[0];
        m_s[warp * G + 2 * t + 1] = m_run[1];
        l_s[warp * G + 2 * t] = l_part[0];
        l_s[warp * G + 2 * t + 1] = l_part[1];
    }
    // Accumulators go to shared memory in fragment order [warp][s][j][lane] (conflict-free both ways).
#pragma unroll
    for (int s = 0; s < 16; s++) {
#pragma unroll
        for (int j = 0; j < 4; j++) acc_s[((warp * 16 + s) * 4 + j) * 32 + lane] = o[s][j];
    }
    __syncthreads();
    // Per (warp, head) weights exp(m_w - max) and the merged (max, sum); thread h < G does head h.
    float *f_s = l_s + NW * G;       // [NW][G]
    float *ml_s = f_s + NW * G;      // [G][2]
    float *cpart = ml_s + 2 * G + 16;  // [G][HD] this CTA's merged, unnormalised tile (cluster merge only)
    if (threadIdx.x < G) {
        const int h = threadIdx.x;
        float gmax = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; w++) gmax = fmaxf(gmax, m_s[w * G + h]);
        float gsum = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) {
            const float mw = m_s[w * G + h];
            const float f = (mw == -INFINITY) ? 0.f : __expf(mw - gmax);
            f_s[w * G + h] = f;
            gsum += f * l_s[w * G + h];
        }
        ml_s[2 * h] = gmax;
        ml_s[2 * h + 1] = gsum;
    }
    __syncthreads();
    // Thread (warp, lane) merges fragment position `lane` of tiles s = 2 warp, 2 warp + 1: element j of tile s is
    // head 2t + (j & 1), dim 32 g + 2 s + (j >> 1).
#pragma unroll
    for (int ss = 0; ss < 2; ss++) {
        const int s = 2 * warp + ss;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int h = 2 * t + (j & 1);
            const int d = 32 * g + 2 * s + (j >> 1);
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < NW; w++) acc += f_s[w * G + h] * acc_s[((w * 16 + s) * 4 + j) * 32 + lane];
            if (p.cluster_merge) {
                cpart[h * HD + d] = acc;
            } else if (h < gvalid) {
                const size_t qh = (size_t)lane_idx * p.n_q + qh0 + h;
                if (p.direct_out) {
                    const float gsum = ml_s[2 * h + 1];
                    p.out[qh * HD + d] = gsum > 0.f ? acc / gsum : 0.f;
                } else {
                    p.partial[(qh * p.n_splits + split) * (size_t)(HD + 2) + 2 + d] = acc;
                }
            }
        }
    }
    if (!p.cluster_merge) {
        if (!p.direct_out && threadIdx.x < 2 * gvalid) {
            const int h = threadIdx.x >> 1;
            const size_t qh = (size_t)lane_idx * p.n_q + qh0 + h;
            p.partial[(qh * p.n_splits + split) * (size_t)(HD + 2) + (threadIdx.x & 1)] = ml_s[threadIdx.x];
        }
        return;
    }
    // ---- splits of this (lane, kv head): one cluster.  Head h is finished by CTA h mod n_splits, one warp per head:
    // the same arithmetic, in the same order, as tq_attn_merge_kernel (attention_tq.cu) ----
    if (p.n_splits > 1) cluster_sync(); else __syncthreads();
    const uint32_t ml_a = smem_u32(ml_s), cp_a = smem_u32(cpart);
    for (int h = (int)split + (int)p.n_splits * warp; h < gvalid; h += (int)p.n_splits * NW) {
        float gmax = -INFINITY;
        for (uint32_t sp = 0; sp < p.n_splits; sp++) gmax = fmaxf(gmax, ld_cluster_f32(ml_a + (2 * h) * 4, sp, p.n_splits > 1));
        float gsum = 0.f, ov[8];
#pragma unroll
        for (int i = 0; i < 8; i++) ov[i] = 0.f;
        for (uint32_t sp = 0; sp < p.n_splits; sp++) {
            const float ms = ld_cluster_f32(ml_a + (2 * h) * 4, sp, p.n_splits > 1);
            const float ls = ld_cluster_f32(ml_a + (2 * h + 1) * 4, sp, p.n_splits > 1);
            const float f = (ms == -INFINITY) ? 0.f : expf(ms - gmax);
            gsum += f * ls;
            const float4 a0 = ld_cluster_f4(cp_a + (h * HD + 8 * lane) * 4, sp, p.n_splits > 1);
            const float4 a1 = ld_cluster_f4(cp_a + (h * HD + 8 * lane + 4) * 4, sp, p.n_splits > 1);
            ov[0] += f * a0.x; ov[1] += f * a0.y; ov[2] += f * a0.z; ov[3] += f * a0.w;
            ov[4] += f * a1.x; ov[5] += f * a1.y; ov[6] += f * a1.z; ov[7] += f * a1.w;
        }
#pragma unroll
        for (int i = 0; i < 8; i++) ov[i] = gsum > 0.f ? ov[i] / gsum : 0.f;
        const size_t qh = (size_t)lane_idx * p.n_q + qh0 + h;
        if (!p.fused_q) {
            *reinterpret_cast<float4 *>(p.out + qh * HD + 8 * lane) = make_float4(ov[0], ov[1], ov[2], ov[3]);
            *reinterpret_cast<float4 *>(p.out + qh * HD + 8 * lane + 4) = make_float4(ov[4], ov[5], ov[6], ov[7]);
            continue;
        }
        // inverse rotation: Walsh-Hadamard butterflies (strides 1, 2, 4 in the thread, 8..128 across lanes), 1/sqrt(d), signs
#pragma unroll
        for (int len = 1; len < 8; len <<= 1) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                if (!(i & len)) {
                    const float a = ov[i], b2 = ov[i + len];
                    ov[i] = a + b2;
                    ov[i + len] = a - b2;
                }
            }
        }
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
            const bool upper = lane & m;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float o2 = __shfl_xor_sync(0xffffffffu, ov[i], m);
                ov[i] = upper ? o2 - ov[i] : ov[i] + o2;
            }
        }
        const float4 s0 = *reinterpret_cast<const float4 *>(p.signs + 8 * lane);
        const float4 s1 = *reinterpret_cast<const float4 *>(p.signs + 8 * lane + 4);
        const float sg[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const float inv = 1.0f / sqrtf((float)HD);
        uint4 packed;
        __half2 *hp = reinterpret_cast<__half2 *>(&packed);
#pragma unroll
        for (int i = 0; i < 4; i++) hp[i] = __floats2half2_rn(ov[2 * i] * inv * sg[2 * i], ov[2 * i + 1] * inv * sg[2 * i + 1]);
        *reinterpret_cast<uint4 *>(p.out_f16 + qh * HD + 8 * lane) = packed;
    }
    if (p.n_splits > 1) cluster_sync();   // no CTA leaves while a peer may still read its shared memory
}

}  // namespace

int lc_tq2_attn_mma_launch(lc_batch *b, const TqAttnParams &p, dim3 grid) {
    const size_t smem = SMEM_BYTES;
    static lc_smem_optin optin;
    LC_CUDA_TRY(lc_ensure_smem(tq2_attn_mma_kernel, optin, b->ctx, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(NT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = b->stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (b->ctx->pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    if (p.cluster_merge && p.n_splits > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = p.n_splits;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    LC_LAUNCH_CHECKED(cudaLaunchKernelEx(&cfg, tq2_attn_mma_kernel, p));
    b->dispatch_count++;
    return LC_OK;
}
