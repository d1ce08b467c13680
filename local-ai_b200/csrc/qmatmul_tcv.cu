// tcgen05 matmul for very tall Q4_0 matrices at decode batch sizes: C[m, n] = A[m, K] (f16) x W[n, K]^T, m <= 64,
// f32 out, n of the order of a vocabulary.  Stands in for the reference's matmul_nt_q4_0 dispatch on the tied
// embedding table (local-engine/src/pipeline/batched.rs:330-352 calls it once per step for all lanes).
//
// One persistent CTA per SM walks 128-row tiles of the table.  Per tile and 128 k ("step"):
//   * a loader thread brings the raw blocks in with TMA: the table is a byte matrix [n][K / 32 * 18], and 256 k of
//     128 rows are one box of 144 bytes x 128 rows (a ring of four boxes; 144 = 9 x 16, so every box starts on a
//     16-byte boundary as the copy engine requires; rows past n read as zero blocks);
//   * eight warps dequantize: thread r of a lane quarter owns operand row r and, per step, two of its four blocks.
//     A Q4_0 weight d (q - 8) needs up to 15 significant bits, so it is written to tensor memory as two f16 operands,
//     hi = f16(d (q - 8)) and lo = d (q - 8) - hi (one fused multiply-add, exact): the sum of the two MMAs is the
//     f32-accumulated product with the exact weight, the contract of the register-direct kernel (qmatmul_mma.cu)
//     that this one replaces for large n;
//   * a second loader thread brings the step's activations (two 64-k boxes, 128-byte swizzle) from L2;
//   * four warps issue the MMAs, weights from tensor memory, activations from shared memory.  An MMA issue costs its
//     thread about 210 cycles whatever the shape, issues of different warps overlap, so the 16 MMAs of a step (eight
//     K = 16 slices x {hi, lo}) are spread over four issuers with one accumulator each;
//   * four more warps read the accumulators back once a tile's last step completes, add the four partial sums in a
//     fixed order and store f32 rows (a warp writes 32 consecutive rows of one batch column: 128 bytes); the issuers
//     start the next tile's MMAs as soon as the loads have left tensor memory, while the dequantizing warps are
//     already ahead by the two weight slots.
// Tensor memory: 4 accumulators x 64 columns + 2 weight slots x (64 hi + 64 lo) columns = 512.
//
// Every wait on an mbarrier is bounded; on expiry the CTA raises the kernels object's status word, lets every role
// run out, frees its tensor memory and returns.
#include <cuda.h>
#include <stdlib.h>

#include "lc_internal.h"
#include "tcgen05_util.cuh"

namespace {

constexpr int V_ROWS = 128;                 // weight rows per tile (UMMA M)
constexpr int V_NB = 64;                    // batch columns (UMMA N)
constexpr int V_KT = 64;                    // k per activation box (one 128-byte swizzled row)
constexpr int V_STEP_K = 128;               // k per pipeline step
constexpr int V_B_TILE = V_NB * V_KT * 2;   // 8 KB
constexpr int V_B_SLOT = (V_STEP_K / V_KT) * V_B_TILE;   // 16 KB
constexpr int V_SB = 4;                     // activation slots
constexpr int V_CHUNK_K = 256;              // k per raw box: 8 blocks
constexpr int V_BB = 18;                    // bytes per Q4_0 block
constexpr int V_CHUNK_RB = V_CHUNK_K / 32 * V_BB;        // 144 bytes per row and box
constexpr int V_RAW_SLOT = V_ROWS * V_CHUNK_RB;          // 18432
constexpr int V_RS = 4;                     // raw slots
constexpr int V_NISS = 4;                   // MMA-issuing warps, one accumulator each
constexpr int V_SA = 2;                     // weight slots in tensor memory
constexpr int V_A_COLS = 128;               // columns per weight slot: 64 hi | 64 lo
constexpr int V_A_BASE = V_NISS * V_NB;     // 256
constexpr int V_TMEM_COLS = V_A_BASE + V_SA * V_A_COLS;  // 512
constexpr int V_NBAR = 8;                   // step-release barriers, one per step index mod 8
constexpr int V_NDQ = 16, V_NDQ_STEP = 8, V_NEPI = 4;   // dequantizing warps in all / per step
constexpr int V_NT = (V_NDQ + 2 + V_NISS + V_NEPI) * 32;   // 832
constexpr uint32_t V_WAIT_LIMIT = 1u << 22;

struct TcvParams {
    float *out;
    int n, m, K, tiles;
    int *status;
    uint32_t wait_limit;
    uint32_t extra_arrivals;   // 0; 1 in the expiry self-test: the readiness barriers then expect an arrival nobody makes
};

// bounded wait by lane 0, result shared with the warp
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, uint32_t limit, int lane) {
    uint32_t ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, limit) ? 1u : 0u;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }

__global__ void __launch_bounds__(V_NT, 1)
qgemm_tcv_kernel(const __grid_constant__ TcvParams p, const __grid_constant__ CUtensorMap x_map,
                 const __grid_constant__ CUtensorMap w_map) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *b_s = smem;                                   // [V_SB][V_B_SLOT]
    uint8_t *raw = b_s + V_SB * V_B_SLOT;                  // [V_RS][V_RAW_SLOT]
    float *stage = reinterpret_cast<float *>(raw + V_RS * V_RAW_SLOT);   // [V_NB][V_ROWS] f32 sums of a tile
    uint64_t *bars = reinterpret_cast<uint64_t *>(stage + V_NB * V_ROWS);
    uint64_t *raw_full = bars;                             // [V_RS]   the box has landed
    uint64_t *raw_empty = raw_full + V_RS;                 // [V_RS]   all dequantizing warps are done with it
    uint64_t *ab_full = raw_empty + V_RS;                  // [V_SB]   a step's weights are in tensor memory and its activations have landed
    uint64_t *step_done = ab_full + V_SB;                   // [V_NBAR] the step's MMAs have completed
    uint64_t *acc_empty = step_done + V_NBAR;              // [1]      the tile's accumulators have been read
    uint64_t *acc_full = acc_empty + 1;                    // [1]      the tile's last MMAs have completed
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    lc_pdl_trigger();
    const int S = p.K / V_STEP_K;                          // steps per tile (even: K is a multiple of 256)
    const int my_tiles = ((int)p.tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total = my_tiles * S;                        // this CTA's steps, numbered across its tiles
    auto tile_of = [&](int j) -> int { return (int)blockIdx.x + j * (int)gridDim.x; };

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)V_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tid == 0) {
        for (int i = 0; i < V_RS; i++) mbar_init(smem_u32(&raw_full[i]), 1);
        for (int i = 0; i < V_RS; i++) mbar_init(smem_u32(&raw_empty[i]), V_NDQ);
        // one barrier per step for both operands, so the issuers test one: eight dequantizing warps arrive, and the
        // activation loader arrives with the byte count of its boxes.  The ring has the depth of the activation ring,
        // the deeper of the two, so no arrival for a later step can reach a barrier before its current phase is over.
        for (int i = 0; i < V_SB; i++) mbar_init(smem_u32(&ab_full[i]), V_NDQ_STEP + 1 + p.extra_arrivals);
        for (int i = 0; i < V_NBAR; i++) mbar_init(smem_u32(&step_done[i]), V_NISS);
        mbar_init(smem_u32(acc_empty), V_NEPI);
        mbar_init(smem_u32(acc_full), V_NISS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t idesc = (1u << 4) | ((uint32_t)(V_NB >> 3) << 17) | ((uint32_t)(V_ROWS >> 4) << 24);

    if (warp < V_NDQ) {
        // =========================== dequantizing warps ===========================
        // Two groups of eight warps take alternate steps, group `grp` always into weight slot `grp`: what a warp
        // does per step besides arithmetic (two barrier tests, stores into tensor memory and the wait for them, an
        // arrival) takes longer than the MMAs of a step, so one group alone cannot keep the issuers busy.
        const int grp = warp >> 3, wq = warp & 7;
        const int r = 32 * (wq & 3) + lane, bq = wq >> 2;
        const uint32_t ta0 = tmem_base + ((uint32_t)(32 * (wq & 3)) << 16) + (uint32_t)(V_A_BASE + grp * V_A_COLS);
        const __half2 c1032 = __float2half2_rn(1032.0f);
        const uint32_t raw_a = smem_u32(raw) + (uint32_t)(r * V_CHUNK_RB + grp * 4 * V_BB + bq * 2 * V_BB);
        bool dead = false;
        for (int g = grp; g < total && !dead; g += 2) {
            const int cg = g >> 1, rs = cg % V_RS;
            if (!warp_wait(smem_u32(&raw_full[rs]), (uint32_t)((cg / V_RS) & 1), p.wait_limit, lane) || *abort_flag) { *abort_flag = 1; dead = true; break; }
#pragma unroll
            for (int bi = 0; bi < 2; bi++) {
                // block 4 grp + 2 bq + bi of the box: f16 scale, then 16 bytes of nibbles (2-byte aligned)
                const uint32_t ba = raw_a + (uint32_t)(rs * V_RAW_SLOT + bi * V_BB);
                const uint32_t dbits = lds16(ba);
                const __half2 d2 = bits_h2(dbits | (dbits << 16));
                const uint32_t ca = ba + 2, sh = (ca & 3u) * 8u, wa = ca & ~3u;
                const uint32_t w0 = lds32(wa), w1 = lds32(wa + 4), w2 = lds32(wa + 8), w3 = lds32(wa + 12), w4 = sh ? lds32(wa + 16) : 0u;
                const uint32_t cw[4] = {__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh), __funnelshift_r(w2, w3, sh),
                                        __funnelshift_r(w3, w4, sh)};
                // low nibbles are elements 0-15 of the block (columns 0-7), high nibbles 16-31 (columns 8-15)
                uint32_t vh[16], vl[16];
#pragma unroll
                for (int part = 0; part < 2; part++) {
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const uint32_t codes = (cw[q] >> (4 * part)) & 0x0F0F0F0Fu;
                        // bytes -> f16 1024 + q by byte placement under exponent 0x64, minus 1032 -> q - 8 (exact)
                        const __half2 q01 = __hsub2(bits_h2(__byte_perm(codes, 0x64u, 0x4140)), c1032);
                        const __half2 q23 = __hsub2(bits_h2(__byte_perm(codes, 0x64u, 0x4342)), c1032);
                        const __half2 h01 = __hmul2(q01, d2), h23 = __hmul2(q23, d2);
                        vh[8 * part + 2 * q] = h2_bits(h01);
                        vh[8 * part + 2 * q + 1] = h2_bits(h23);
                        vl[8 * part + 2 * q] = h2_bits(__hfma2(q01, d2, __hneg2(h01)));
                        vl[8 * part + 2 * q + 1] = h2_bits(__hfma2(q23, d2, __hneg2(h23)));
                    }
                }
                if (bi == 0 && g >= V_SA) {
                    // the first block is in registers; the stores have to wait for the MMAs that read this slot two steps ago
                    const int u = g - V_SA;
                    if (!warp_wait(smem_u32(&step_done[u % V_NBAR]), (uint32_t)((u / V_NBAR) & 1), p.wait_limit, lane)) { *abort_flag = 1; dead = true; break; }
                    tc_fence_after();
                }
                if (bi == 1) {   // every lane of this warp has read its bytes of the box
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&raw_empty[rs]));
                }
                const uint32_t col = (uint32_t)(16 * (2 * bq + bi));
                tmem_st16(ta0 + col, vh);
                tmem_st16(ta0 + col + 64u, vl);
            }
            if (dead) break;
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ab_full[g % V_SB]));
        }
    } else if (warp == V_NDQ) {
        // =========================== activation loader (one thread) ===========================
        if (lane == 0) {
            lc_pdl_wait();   // the activations are the predecessor's output
            bool dead = false;
            int g = 0;
            for (int j = 0; j < my_tiles && !dead; j++) {
                for (int i = 0; i < S; i++, g++) {
                    if (g >= V_SB) {   // its slot was last read by the MMAs of step g - V_SB
                        const int u = g - V_SB;
                        if (!mbar_wait(smem_u32(&step_done[u % V_NBAR]), (uint32_t)((u / V_NBAR) & 1), p.wait_limit) || *abort_flag) { dead = true; break; }
                    }
                    const int k0 = i * V_STEP_K;
                    const uint32_t bar = smem_u32(&ab_full[g % V_SB]), dst = smem_u32(b_s) + (uint32_t)((g % V_SB) * V_B_SLOT);
                    mbar_expect_tx(bar, (uint32_t)V_B_SLOT);
                    tma_load_2d(dst, &x_map, k0, 0, bar);
                    tma_load_2d(dst + V_B_TILE, &x_map, k0 + V_KT, 0, bar);
                }
            }
            if (dead) *abort_flag = 1;
        }
        __syncwarp();
    } else if (warp == V_NDQ + 1) {
        // =========================== raw block loader (one thread); the table does not depend on the predecessor ====
        if (lane == 0) {
            bool dead = false;
            const int cpt = S >> 1;
            int cg = 0;
            for (int j = 0; j < my_tiles && !dead; j++) {
                const int row0 = tile_of(j) * V_ROWS;
                for (int c = 0; c < cpt; c++, cg++) {
                    const int rs = cg % V_RS;
                    if (cg >= V_RS) {   // the box that held this slot has been dequantized
                        if (!mbar_wait(smem_u32(&raw_empty[rs]), (uint32_t)((cg / V_RS - 1) & 1), p.wait_limit) || *abort_flag) { dead = true; break; }
                    }
                    const uint32_t bar = smem_u32(&raw_full[rs]);
                    mbar_expect_tx(bar, (uint32_t)V_RAW_SLOT);
                    tma_load_2d(smem_u32(raw) + (uint32_t)(rs * V_RAW_SLOT), &w_map, c * V_CHUNK_RB, row0, bar);
                }
            }
            if (dead) *abort_flag = 1;
        }
        __syncwarp();
    } else if (warp < V_NDQ + 2 + V_NISS) {
        // =========================== MMA issue (four warps, one thread each) ===========================
        // Issuer iw owns accumulator iw and takes the K = 16 slices iw and iw + 4 of every step, hi then lo
        // (slice ks: weight columns 8 ks of the hi half, + 64 for lo; activations: box ks / 4, 32 bytes per slice).
        const int iw = warp - V_NDQ - 2;
        if (lane == 0) {
            // This loop is the pace of the whole kernel and runs on one thread: nothing in it but the barrier test, the
            // MMAs and the commits (counters instead of divisions; a role that gives up stops arriving, so this
            // thread's own bounded waits are its only failure path).
            const uint64_t bdesc0 = make_desc(smem_u32(b_s) + (uint32_t)((iw & 3) * 32));   // slice iw of the first box
            const uint64_t bdesc1 = bdesc0 + (uint64_t)((uint32_t)V_B_TILE >> 4);              // slice iw + 4: second box
            const uint32_t tmem_acc = tmem_base + (uint32_t)(iw * V_NB);
            const uint32_t ta_first = tmem_base + (uint32_t)(V_A_BASE + 8 * iw);
            const uint32_t ab0 = smem_u32(ab_full), sd0 = smem_u32(step_done);
            bool dead = false;
            uint32_t g = 0;
            for (int j = 0; j < my_tiles && !dead; j++) {
                if (j > 0 && !mbar_wait(smem_u32(acc_empty), (uint32_t)((j - 1) & 1), p.wait_limit)) { dead = true; break; }   // the previous tile's sums have left tensor memory
                for (int i = 0; i < S; i++, g++) {
                    const uint32_t sb = g & (V_SB - 1);
                    if (!mbar_wait(ab0 + 8u * sb, (g / V_SB) & 1u, p.wait_limit)) { dead = true; break; }
                    tc_fence_after();
                    const uint32_t ta = ta_first + (g & (V_SA - 1)) * (uint32_t)V_A_COLS;
                    const uint64_t boff = (uint64_t)((sb * (uint32_t)V_B_SLOT) >> 4);
                    umma_f16_ta(tmem_acc, ta, bdesc0 + boff, idesc, i > 0 ? 1u : 0u);
                    umma_f16_ta(tmem_acc, ta + 64u, bdesc0 + boff, idesc, 1u);
                    umma_f16_ta(tmem_acc, ta + 32u, bdesc1 + boff, idesc, 1u);
                    umma_f16_ta(tmem_acc, ta + 96u, bdesc1 + boff, idesc, 1u);
                    umma_commit(sd0 + 8u * (g & (V_NBAR - 1)));
                }
                // A waiter on a phase must have seen the phase before it complete; the result warps look only once
                // per tile, so they get a barrier of their own rather than the step ring.
                if (!dead) umma_commit(smem_u32(acc_full));
            }
            if (dead) *abort_flag = 1;
        }
        __syncwarp();
    } else {
        // =========================== results (four warps, one per lane quarter) ===========================
        const int qtr = warp & 3;
        bool dead = false;
        for (int j = 0; j < my_tiles && !dead; j++) {
            if (!warp_wait(smem_u32(acc_full), (uint32_t)(j & 1), p.wait_limit, lane) || *abort_flag) { dead = true; break; }
            tc_fence_after();
            // The sums go to shared memory first (a warp writes 32 consecutive floats per batch column), so that the
            // accumulators are handed back after the loads alone; the stores to global memory, 16 bytes per thread,
            // then run beside the next tile's MMAs.  Every warp copies out what it staged itself.
            const uint32_t ta = tmem_base + ((uint32_t)(32 * qtr) << 16);
            float *st_w = stage + 32 * qtr;
#pragma unroll
            for (int cc = 0; cc < V_NB; cc += 8) {
                uint32_t a0[8], a1[8], a2[8], a3[8];
                tmem_ld8(ta + (uint32_t)cc, a0);
                tmem_ld8(ta + (uint32_t)(cc + V_NB), a1);
                tmem_ld8(ta + (uint32_t)(cc + 2 * V_NB), a2);
                tmem_ld8(ta + (uint32_t)(cc + 3 * V_NB), a3);
                tmem_ld_wait();
                if (cc + 8 == V_NB) {   // everything has been read: the next tile's MMAs may overwrite
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(acc_empty));
                }
#pragma unroll
                for (int e = 0; e < 8; e++)
                    st_w[(cc + e) * V_ROWS + lane] =
                        (__uint_as_float(a0[e]) + __uint_as_float(a1[e])) + (__uint_as_float(a2[e]) + __uint_as_float(a3[e]));
            }
            __syncwarp();
            const int row0 = tile_of(j) * V_ROWS + 32 * qtr, r4 = 4 * (lane & 7);
            const bool vec = (p.n & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;   // every (column, 4-row group) then starts on a 16-byte boundary
#pragma unroll 4
            for (int c4 = 0; c4 < V_NB; c4 += 4) {
                const int col = c4 + (lane >> 3);
                if (col >= p.m) break;   // columns ascend with the lane: once a lane is past m, so are the later rounds
                const float4 v = *reinterpret_cast<const float4 *>(st_w + col * V_ROWS + r4);
                float *dst = p.out + (size_t)col * p.n + row0 + r4;
                if (vec && row0 + r4 + 3 < p.n) {
                    *reinterpret_cast<float4 *>(dst) = v;
                } else {
                    const float ev[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int q = 0; q < 4; q++)
                        if (row0 + r4 + q < p.n) dst[q] = ev[q];
                }
            }
            __syncwarp();   // the staging rows are free for the next tile
        }
        if (dead) *abort_flag = 1;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag != 0) tc_wait_expired(p.status, LC_DEV_STATUS_WAIT_EXPIRED_TCD, tid);
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)V_TMEM_COLS) : "memory");
    }
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                    const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_tiled_fn encode_tiled() {
    static encode_tiled_fn fn = []() -> encode_tiled_fn {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<encode_tiled_fn>(ptr);
    }();
    return fn;
}

}  // namespace

// One Q4_0 matrix [n, kk] against activations [m, kk], m <= 64, f32 out.  Returns LC_OK after a launch, a positive
// status on error, or -1 when the shape is outside what this kernel covers (the caller then uses another path).
int lc_qgemm_tcv_launch(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight, lc_buf *output, uint32_t m,
                        uint32_t kk, uint32_t n) {
    if (m < 1 || m > (uint32_t)V_NB || kk % V_CHUNK_K != 0 || kk == 0 || !lc_aligned(input->dptr, 16) ||
        !lc_aligned(weight->dptr, 16) || !lc_aligned(output->dptr, 4))
        return -1;
    // worth it only when every SM gets tiles to walk; smaller matrices stay with the split-K kernels
    if (n < (uint32_t)(V_ROWS * k->ctx->sm_count)) return -1;
    const size_t smem = (size_t)V_SB * V_B_SLOT + (size_t)V_RS * V_RAW_SLOT + (size_t)V_NB * V_ROWS * 4 + (2 * V_RS + V_SB + V_NBAR + 2) * 8 + 16 + 1024;
    if (smem > k->ctx->smem_optin) return -1;
    encode_tiled_fn fn = encode_tiled();
    if (!fn) return -1;
    CUtensorMap x_map, w_map;
    {
        const cuuint64_t dims[2] = {kk, m};
        const cuuint64_t strides[1] = {(cuuint64_t)kk * 2};
        const cuuint32_t box[2] = {V_KT, V_NB};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult r = fn(&x_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, input->dptr, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return lc_fail(LC_ERR_CUDA, "cuTensorMapEncodeTiled (activations) failed (%d)", (int)r);
    }
    {
        const cuuint64_t rb = (cuuint64_t)(kk / 32) * V_BB;   // a multiple of 144
        const cuuint64_t dims[2] = {rb, n};
        const cuuint64_t strides[1] = {rb};
        const cuuint32_t box[2] = {V_CHUNK_RB, V_ROWS};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult r = fn(&w_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, weight->dptr, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return lc_fail(LC_ERR_CUDA, "cuTensorMapEncodeTiled (weights) failed (%d)", (int)r);
    }
    TcvParams p;
    p.out = (float *)output->dptr;
    p.n = (int)n;
    p.m = (int)m;
    p.K = (int)kk;
    p.tiles = (int)((n + V_ROWS - 1) / V_ROWS);
    p.status = k->dev_status;
    p.wait_limit = k->test_wait_expiry ? 4096u : V_WAIT_LIMIT;
    p.extra_arrivals = k->test_wait_expiry ? 1u : 0u;
    static lc_smem_optin optin;
    LC_CUDA_TRY(lc_ensure_smem(qgemm_tcv_kernel, optin, b->ctx, smem));
    const int grid = p.tiles < k->ctx->sm_count ? p.tiles : k->ctx->sm_count;
    LC_LAUNCH_CHECKED(lc_launch(qgemm_tcv_kernel, dim3(grid), dim3(V_NT), smem, b, p, x_map, w_map));
    b->dispatch_count++;
    return LC_OK;
}
