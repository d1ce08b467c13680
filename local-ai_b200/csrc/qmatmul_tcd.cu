// tcgen05 decode matmul: C[m, n] = A[m, K] (f16) x W[n, K]^T with W in GGUF TQ2_0 blocks, m <= 64, f16 out.
// Stands in, at decode batch sizes, for the reference's simdgroup-matrix kernel matmul_nt_tq2_0_mma
// (shaders/matvec_quant.metal:447-577) and, in GeGLU mode, for the pair of projections + gelu_mul of
// local-engine/src/layer.rs:825-838.
//
// A decode projection is a few microseconds of work that sits behind the kernel before it, so the kernel is built
// around the length of the dependent chain after that kernel finishes:
//   * weights take the MMA's M (128 rows per CTA; a GeGLU CTA holds 64 gate rows and the same 64 rows of the up
//     matrix, so gate and up of an output element meet in one CTA), the batch its N (64, zero padded), f32
//     accumulators in tensor memory (TMEM);
//   * at most one CTA per SM and one wave per launch: K is split over a thread-block cluster so that the CTA count
//     stays within the SM count, which also keeps the number of CTAs that re-read the same activations from L2 low;
//   * the weight operand lives in tensor memory, not in shared memory: the dequantizing warps write f16 weights with
//     tcgen05.st (thread r of the four lane quarters owns operand row r; 16 consecutive k are eight 32-bit columns),
//     and the MMA takes A from tensor memory and B, the activations, from shared memory.  All 512 columns are in use:
//     four 64-column accumulators and two weight slots of 128 columns (256 k) each (127 registers x 416 threads
//     keep this kernel at one CTA per SM, so no second CTA ever waits for tensor memory behind a cluster barrier);
//   * before the dependency wait: TMEM allocation, barrier set-up, the raw quantized rows of the CTA's K range
//     brought in by bulk copies (cp.async.bulk, one per row segment, completion counted on an mbarrier), and both
//     weight slots dequantized -- none of it depends on the predecessor;
//   * the pipeline runs in steps of 256 k (one TQ2_0 block per row), because every hand-over costs its thread a few
//     hundred cycles whatever the amount of data behind it: a barrier test ~150, an MMA issue ~210, a commit ~90
//     (measured), and the hand-overs of a step sit in series (slot released -> dequantize -> weights ready ->
//     activations ready -> MMAs -> commit).  With 128-k steps and the weight operand staged in shared memory a launch
//     cost 5.9 us + 0.78 us per step; tensor-memory weights removed the shared-memory stores and made room for twice
//     the k per step (GeGLU 15.2 -> 12.1 us, the batch-64 decode step 2.91 -> 2.70 ms);
//   * after the wait one thread requests the activations of every step with TMA (cp.async.bulk.tensor, four 64-k
//     boxes, 128-byte swizzle applied by the copy engine, rows beyond m zero-filled by the tensor map's bounds) into
//     a ring of up to three slots, the dequantizing warps keep turning code bytes into f16 weights (the four values
//     a 2-bit code can mean, (q - 1) d, sit in two registers as a byte table; one prmt assembles two weights), and
//     four warps issue tcgen05.mma.cta_group::1.kind::f16.  Issuing one MMA costs a warp about 210 cycles whatever its
//     shape (measured: M 64 / 128, N 16 .. 256 all the same), far more than the 32 cycles of arithmetic in a
//     128 x 64 x 16 MMA, but MMAs issued by different warps overlap fully (4 warps: 53 cycles per MMA).  So the four
//     K = 16 slices of a 64-k tile belong to four issuing warps, each with its own TMEM accumulator (four partial
//     sums over interleaved k, added in a fixed order in the epilogue); every issuer commits its MMAs of a step to
//     the step's mbarrier, which hands the slots back after the fourth arrival;
//   * CTAs walk their steps from different starting points so that the CTAs of a launch do not all ask L2 for the
//     same activation lines at the same moment;
//   * the accumulators are read back with tcgen05.ld by all dequantizing warps.  When K is split, the CTAs of a tile
//     add their partial tiles in split order through distributed shared memory, each finishing one contiguous slice.
//
// Numerics: TQ2_0 weights d (q - 1) are exact in f16, accumulation is f32, splits are added in split order:
// the same contract as the register-direct mma.sync kernel (qmatmul_mma.cu), which remains the fallback.
//
// Every wait on an mbarrier is bounded; on expiry the CTA raises the kernels object's status word, skips to the
// TMEM release and returns.
#include <cuda.h>
#include <stdlib.h>

#include "lc_internal.h"
#include "tcgen05_util.cuh"

namespace {

constexpr int TILE_ROWS = 128;   // weight rows per accumulator tile (UMMA M)
constexpr int NB = 64;           // batch columns (UMMA N)
constexpr int KT = 64;           // k per operand tile (one 128-byte swizzled row)
constexpr int STEP_TILES = 4;    // 64-k activation tiles per pipeline step (256 k: one TQ2_0 block per weight row)
constexpr int NBAR = 8;          // step-release barriers, one per step index mod 8
constexpr int NISS = 4;          // MMA-issuing warps, one accumulator each
constexpr int SA = 2;            // weight-operand slots in tensor memory (one step each)
constexpr int A_COLS = 128;      // columns of one weight slot: 256 k as f16 pairs
constexpr int A_BASE = NISS * NB;      // the accumulators take columns 0 .. 255
constexpr int TMEM_COLS = A_BASE + SA * A_COLS;   // 512: all of an SM's tensor memory
// Operand tiles are K-major with the 128-byte swizzle: a row is its 64 k values (128 bytes, eight 16-byte chunks),
// rows follow each other at 128 bytes, and chunk c of row r sits at chunk position c ^ (r % 8) of the row.  Tiles
// start on 1024-byte boundaries (eight rows: the swizzle pattern's period).
constexpr int ROW_BYTES = KT * 2;            // 128
constexpr int B_TILE = NB * ROW_BYTES;          // 8 KB
constexpr int B_SLOT = STEP_TILES * B_TILE;     // activations of one step
constexpr int BB = 66;           // bytes per TQ2_0 block
constexpr int MAX_STEPS = 6;     // steps per CTA (six blocks of 256 k)
constexpr int MAX_GROUPS = 3;
constexpr int MAX_KS = 8;        // portable cluster size
constexpr uint32_t WAIT_LIMIT = 1u << 22;

struct TcdParams {
    const uint8_t *w[MAX_GROUPS];
    __half *out[MAX_GROUPS];
    int n[MAX_GROUPS], tile_end[MAX_GROUPS];
    int ngroups;
    int m, K, nb;        // nb = blocks per weight row
    int ks, bps;         // split-K: grid.z = cluster size = ks, bps = blocks per split
    int raw_rs;          // bytes reserved per row of raw blocks (odd multiple of 16)
    int sa, sb;          // operand slots (one step each): weights in tensor memory (always SA) / activations in shared memory
    int geglu;           // 1: operand rows 0-63 are gate rows, 64-127 the same rows of the up matrix; out[0] = gelu(gate) * up
    int *status;
    uint32_t wait_limit;
    uint32_t extra_arrivals;   // 0; 1 in the expiry self-test: the "weights ready" barriers then expect an arrival nobody makes
};

// gelu_tanh(gate) * up with gate and up rounded to f16 first, as the separate projections would store them, and the
// element-wise kernel's arithmetic (shaders/gelu.metal:23-37)
__device__ __forceinline__ float geglu_f(float gate, float up) {
    const float x = __half2float(__float2half_rn(gate)), u = __half2float(__float2half_rn(up));
    float inner = 0.7978845608f * (x + 0.044715f * (x * x * x));
    inner = fminf(fmaxf(inner, -10.0f), 10.0f);
    return 0.5f * x * (1.0f + tanhf(inner)) * u;
}
__device__ __forceinline__ uint2 pack4(float a, float b, float c, float d) {
    __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
    return make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
}

constexpr int NDQ = 8;                       // dequantizing warps (also the epilogue warps)
constexpr int NT = (NDQ + 1 + NISS) * 32;    // + activation loader warp + MMA issuers

__global__ void __launch_bounds__(NT, 1)
qgemm_tcd_kernel(const __grid_constant__ TcdParams p, const __grid_constant__ CUtensorMap x_map) {
    constexpr int ROWS = TILE_ROWS;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // operand tiles start on 1024-byte boundaries
    const int SB = p.sb;
    uint8_t *b_s = smem;                                   // [SB][B_SLOT]; slot 0 is reused for the split-K exchange
    uint8_t *raw = b_s + SB * B_SLOT;                      // [ROWS][raw_rs]
    uint64_t *bars = reinterpret_cast<uint64_t *>(raw + ROWS * p.raw_rs);
    uint64_t *raw_full = bars;                             // 1
    uint64_t *a_full = bars + 1;                           // [MAX_STEPS] (SA used)
    uint64_t *b_full = a_full + MAX_STEPS;                 // [MAX_STEPS] (SB used)
    uint64_t *step_done = b_full + MAX_STEPS;              // [NBAR]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(step_done + NBAR);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    lc_pdl_trigger();
    int grp = 0;
    while (grp + 1 < p.ngroups && (int)blockIdx.x >= p.tile_end[grp]) grp++;
    const int rows_out = p.geglu ? TILE_ROWS / 2 : TILE_ROWS;                          // output rows of a tile
    const int n0 = ((int)blockIdx.x - (grp ? p.tile_end[grp - 1] : 0)) * rows_out;    // first output row of this tile
    const int n_rows = p.n[grp];
    const size_t rb = (size_t)p.nb * BB, w_bytes = rb * (size_t)n_rows;
    const int kbs = (int)blockIdx.z * p.bps, kbe = min(p.nb, kbs + p.bps), nblk = max(kbe - kbs, 0);
    const int seg = nblk * BB;
    const int total_steps = nblk;                          // 256-k steps of this CTA: one block per row each
    // Step i of this CTA works on block block_of(i) of the CTA's range; the walk starts at a block that differs from
    // CTA to CTA.
    const int start = total_steps ? (int)((blockIdx.x * 5u + blockIdx.z) % (unsigned)total_steps) : 0;
    auto block_of = [&](int i) -> int {
        int bl = i + start;
        if (bl >= total_steps) bl -= total_steps;
        return bl;
    };
    // operand row r of the CTA -> weight matrix and row of it
    auto wmat_of = [&](int r) -> const uint8_t * { return p.geglu ? p.w[r >> 6] : p.w[grp]; };
    auto wrow_of = [&](int r) -> int { return n0 + (p.geglu ? (r & 63) : r); };

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tid == 0) {
        mbar_init(smem_u32(raw_full), ROWS);
        for (int i = 0; i < MAX_STEPS; i++) mbar_init(smem_u32(&a_full[i]), NDQ + p.extra_arrivals);
        for (int i = 0; i < MAX_STEPS; i++) mbar_init(smem_u32(&b_full[i]), 1);
        for (int i = 0; i < NBAR; i++) mbar_init(smem_u32(&step_done[i]), NISS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t idesc = (1u << 4) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(TILE_ROWS >> 4) << 24);

    if (warp < NDQ) {
        // =========================== dequantizing warps ===========================
        // ---- raw rows: thread r < ROWS brings in row r's blocks [kbs, kbe) as one bulk copy of the enclosing
        //      16-byte range (rows are only 2-byte aligned) ----
        if (tid < ROWS) {
            const uint8_t *wm = wmat_of(tid);
            const int row = wrow_of(tid);
            const uint32_t bar = smem_u32(raw_full);
            bool counted = false;
            if (row < n_rows && nblk > 0) {
                const size_t g0 = (size_t)row * rb + (size_t)kbs * BB, a0 = g0 & ~(size_t)15;
                const uint32_t bytes = (uint32_t)(((g0 + seg - a0) + 15) & ~(size_t)15);
                uint8_t *dst = raw + tid * p.raw_rs;
                if (a0 + bytes <= w_bytes) {
                    mbar_arrive_expect_tx(bar, bytes);
                    bulk_g2s(smem_u32(dst), wm + a0, bytes, bar);
                    counted = true;
                } else {   // the last bytes of the matrix: plain loads, nothing is read past its end
                    for (uint32_t i = 0; i < bytes; i++) dst[i] = (a0 + i < w_bytes) ? wm[a0 + i] : 0;
                }
            }
            if (!counted) mbar_arrive(bar);
        }
        bool dead = false;
        {
            uint32_t ok = 1;
            if (lane == 0) ok = mbar_wait(smem_u32(raw_full), 0u, p.wait_limit) ? 1u : 0u;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { *abort_flag = 1; dead = true; }
        }
        // This thread's share of every step: operand row 32 (warp & 3) + lane and, of each 32-byte half h of the row's
        // block, the 16 code bytes 16 bq .. + 15 (bq = warp >> 2): 128 weights.
        const int r = 32 * (warp & 3) + lane, bq = warp >> 2;
        const int row = wrow_of(r);
        const bool rvalid = row < n_rows;
        const size_t g0 = (size_t)row * rb + (size_t)kbs * BB;
        const uint8_t *rrow = raw + r * p.raw_rs + (int)(g0 & 15);
        // tensor-memory address of this warp's lane quarter, first column of the weight slots
        const uint32_t ta0 = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)A_BASE;
        for (int i = 0; i < total_steps && !dead; i++) {
            const int blk = block_of(i), s = i % SA;
            // The four weights a code can mean, (q - 1) d, as a byte table for prmt: lut_lo / lut_hi hold the low /
            // high bytes of {-d, 0, d, 2d}; a selector nibble pair (q, q + 4) then assembles one f16.
            const __half d = rvalid ? *reinterpret_cast<const __half *>(rrow + blk * BB + 64) : __float2half(0.0f);
            const uint32_t p01 = (uint32_t)__half_as_ushort(__hneg(d));
            const uint32_t p23 = (uint32_t)__half_as_ushort(d) | ((uint32_t)__half_as_ushort(__hadd(d, d)) << 16);
            const uint32_t lut_lo = __byte_perm(p01, p23, 0x6420), lut_hi = __byte_perm(p01, p23, 0x7531);
            // The first half block is converted before the wait for the slot (only the stores depend on the MMAs that
            // read the slot SA steps ago); its stores then run beside the conversion of the second half.
#pragma unroll
            for (int h = 0; h < 2; h++) {
                // 16 code bytes, 2-byte aligned: five aligned words, funnel-shifted into place
                const uint32_t ca = smem_u32(rrow + blk * BB + 32 * h + 16 * bq), sh = (ca & 3u) * 8u, wa = ca & ~3u;
                const uint32_t w0 = lds32(wa), w1 = lds32(wa + 4), w2 = lds32(wa + 8), w3 = lds32(wa + 12), w4 = sh ? lds32(wa + 16) : 0u;
                const uint32_t cw[4] = {__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh), __funnelshift_r(w2, w3, sh),
                                        __funnelshift_r(w3, w4, sh)};
                // element k = 128 h + 32 l + j of the block is bit pair l of code byte 32 h + j: for a given l this
                // thread's bytes j = 16 bq .. + 15 are 16 consecutive k, i.e. the eight columns from (128 h + 32 l + 16 bq) / 2
                uint32_t v[4][8];
#pragma unroll
                for (int l = 0; l < 4; l++) {
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const uint32_t sel = ((cw[q] >> (2 * l)) & 0x03030303u) * 0x11u + 0x40404040u;
                        v[l][2 * q] = __byte_perm(lut_lo, lut_hi, sel);
                        v[l][2 * q + 1] = __byte_perm(lut_lo, lut_hi, sel >> 16);
                    }
                }
                if (h == 0 && i >= SA) {   // the MMAs that read this slot SA steps ago have completed
                    uint32_t ok = 1;
                    const int u = i - SA;
                    if (lane == 0) ok = mbar_wait(smem_u32(&step_done[u % NBAR]), (uint32_t)((u / NBAR) & 1), p.wait_limit) ? 1u : 0u;
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok || *abort_flag) { *abort_flag = 1; dead = true; break; }
                    tc_fence_after();
                }
#pragma unroll
                for (int l = 0; l < 4; l++) tmem_st8(ta0 + (uint32_t)(s * A_COLS + 64 * h + 16 * l + 8 * bq), v[l]);
            }
            if (dead) break;
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&a_full[s]));
        }
    } else if (warp == NDQ) {
        // =========================== activation loader (one thread) ===========================
        // Step i needs x[0..64, k .. k + 255], k = 256 (kbs + block): four boxes of the tensor map.
        if (lane == 0) {
            lc_pdl_wait();   // the activations are the predecessor's output
            bool dead = false;
            uint32_t sbi = 0;   // i % SB without the division
            for (int i = 0; i < total_steps && !dead; i++) {
                if (i >= SB) {   // its slot was last read by the MMAs of step i - SB
                    const int u = i - SB;
                    if (!mbar_wait(smem_u32(&step_done[u % NBAR]), (uint32_t)((u / NBAR) & 1), p.wait_limit) || *abort_flag) { dead = true; break; }
                }
                const int k0 = (kbs + block_of(i)) * 256;
                const uint32_t bar = smem_u32(&b_full[sbi]), dst = smem_u32(b_s) + sbi * (uint32_t)B_SLOT;
                if (++sbi == (uint32_t)SB) sbi = 0;
                mbar_expect_tx(bar, (uint32_t)B_SLOT);
#pragma unroll
                for (int lp = 0; lp < STEP_TILES; lp++) tma_load_2d(dst + lp * B_TILE, &x_map, k0 + lp * KT, 0, bar);
            }
            if (dead) *abort_flag = 1;
        }
        __syncwarp();
    } else {
        // =========================== MMA issue (four warps, one thread each) ===========================
        // Issuer iw owns TMEM accumulator iw (columns 64 iw ..) and takes K = 16 slice iw of each of the four 64-k tiles of
        // every step: weights from tensor memory (eight columns per slice), activations from shared memory.
        // One thread per issuer runs the loop: every instruction in it (barrier test, MMA, commit) costs its thread on
        // the order of a hundred cycles or more, so nothing warp-wide is added.
        const int iw = warp - NDQ - 1;
        if (lane == 0) {
            const uint64_t bdesc0 = make_desc(smem_u32(b_s) + (uint32_t)(iw * 32));
            const uint32_t tmem_acc = tmem_base + (uint32_t)(iw * NB);
            const uint32_t ta0 = tmem_base + (uint32_t)(A_BASE + 8 * iw);
            const uint32_t af0 = smem_u32(a_full), bf0 = smem_u32(b_full), sd0 = smem_u32(step_done);
            bool dead = false;
            // counters instead of divisions by the (run-time) ring depth: this thread's loop is the pace of the CTA
            uint32_t sbi = 0, sbp = 0;   // activation slot of step i and the parity of its barrier's phase
            for (int i = 0; i < total_steps; i++) {
                const uint32_t sa = (uint32_t)i & (SA - 1);
                if (!mbar_wait(af0 + 8u * sa, ((uint32_t)i / SA) & 1u, p.wait_limit) || !mbar_wait(bf0 + 8u * sbi, sbp, p.wait_limit)) { dead = true; break; }
                tc_fence_after();
                const uint32_t ta = ta0 + sa * (uint32_t)A_COLS;
                const uint64_t bd = bdesc0 + (uint64_t)((sbi * (uint32_t)B_SLOT) >> 4);
#pragma unroll
                for (int lp = 0; lp < STEP_TILES; lp++)
                    umma_f16_ta(tmem_acc, ta + (uint32_t)(32 * lp), bd + (uint64_t)((uint32_t)(lp * B_TILE) >> 4), idesc, (i > 0 || lp > 0) ? 1u : 0u);
                umma_commit(sd0 + 8u * ((uint32_t)i & (NBAR - 1)));
                if (++sbi == (uint32_t)SB) { sbi = 0; sbp ^= 1u; }
            }
            // drain: the last step's barrier completes when all four issuers' MMAs are done
            if (!dead && total_steps > 0) {
                const int last = total_steps - 1;
                dead = !mbar_wait(smem_u32(&step_done[last % NBAR]), (uint32_t)((last / NBAR) & 1), p.wait_limit);
            }
            if (dead) *abort_flag = 1;
        }
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const bool failed = *abort_flag != 0;

    // ---- results.  Dequantizing warp w reads TMEM lanes 32 (w & 3) .. + 31 (one operand row per thread) and the 32
    //      batch columns starting at 32 (w >> 2); the four partial accumulators are added as (0 + 1) + (2 + 3) ----
    float *red = reinterpret_cast<float *>(b_s);            // staging, reuses the first activation slot: [NB cols][128 rows] f32
    __half *out = p.out[grp];
    const int lrow = 32 * (warp & 3) + lane, c0 = 32 * (warp >> 2);
    float v[32];
    if (warp < NDQ) {
#pragma unroll
        for (int cc = 0; cc < 32; cc += 16) {
            if (!failed && total_steps > 0) {
                const uint32_t ta = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(c0 + cc);
                uint32_t a0[16], a1[16], a2[16], a3[16];   // the four accumulators' loads are in flight together
                tmem_ld16(ta, a0);
                tmem_ld16(ta + NB, a1);
                tmem_ld16(ta + 2 * NB, a2);
                tmem_ld16(ta + 3 * NB, a3);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; j++)
                    v[cc + j] = (__uint_as_float(a0[j]) + __uint_as_float(a1[j])) + (__uint_as_float(a2[j]) + __uint_as_float(a3[j]));
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) v[cc + j] = 0.f;
            }
        }
        if (p.ks > 1 || p.geglu) {   // partial tiles of a split, or the two halves of a GeGLU tile
#pragma unroll
            for (int j = 0; j < 32; j++) red[(c0 + j) * TILE_ROWS + lrow] = v[j];
        } else if (n0 + lrow < n_rows && !failed) {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (c0 + j < p.m) out[(size_t)(c0 + j) * n_rows + n0 + lrow] = __float2half_rn(v[j]);
        }
    }
    if (p.ks == 1 && p.geglu) {
        // Gate rows (operand rows 0-63) meet their up rows (64-127) through shared memory.  All eight warps share the
        // activation: a thread takes two neighbouring output rows of eight batch columns, so a warp stores 128
        // contiguous bytes per column.
        __syncthreads();
        if (warp < NDQ && !failed) {
            const int r2 = 2 * lane, cg = 8 * warp;
            const bool pair_ok = n0 + r2 + 1 < n_rows && ((n_rows | n0) & 1) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int col = cg + j;
                if (col >= p.m) break;
                const float2 gt = *reinterpret_cast<const float2 *>(red + col * TILE_ROWS + r2);
                const float2 up = *reinterpret_cast<const float2 *>(red + col * TILE_ROWS + 64 + r2);
                const float o0 = geglu_f(gt.x, up.x), o1 = geglu_f(gt.y, up.y);
                __half *dst = out + (size_t)col * n_rows + n0 + r2;
                if (pair_ok) {
                    *reinterpret_cast<__half2 *>(dst) = __floats2half2_rn(o0, o1);
                } else {
                    if (n0 + r2 < n_rows) dst[0] = __float2half_rn(o0);
                    if (n0 + r2 + 1 < n_rows) dst[1] = __float2half_rn(o1);
                }
            }
        }
    }
    if (p.ks > 1) {
        // The ks CTAs of this tile are one cluster.  An item is four consecutive output rows of one batch column; CTA
        // `rank` finishes the items [rank, rank + 1) * per: adds the ks partials in split order and stores.  Consecutive
        // threads take consecutive items: consecutive 16-byte pieces of the peers' shared memory, consecutive rows out.
        cluster_sync();
        const int rank = (int)blockIdx.z;
        const uint32_t red_a = smem_u32(red);
        auto gather = [&](int col, int r4) {
            const uint32_t la = red_a + (uint32_t)((col * TILE_ROWS + r4) * 4);
            float4 pv[MAX_KS];
#pragma unroll
            for (int sp = 0; sp < MAX_KS; sp++) pv[sp] = sp < p.ks ? ld_dsmem_f4(la, (uint32_t)sp) : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int sp = 0; sp < MAX_KS; sp++) {
                acc.x += pv[sp].x; acc.y += pv[sp].y; acc.z += pv[sp].z; acc.w += pv[sp].w;
            }
            return acc;
        };
        const int items = p.m * (rows_out / 4), per = (items + p.ks - 1) / p.ks;
        const int it_end = min(items, (rank + 1) * per);
        if (!failed) {
            for (int it = rank * per + tid; it < it_end; it += NT) {
                const int col = it / (rows_out / 4), r4 = (it - col * (rows_out / 4)) * 4;
                float4 a = gather(col, r4);
                if (p.geglu) {
                    const float4 u = gather(col, r4 + 64);
                    a = make_float4(geglu_f(a.x, u.x), geglu_f(a.y, u.y), geglu_f(a.z, u.z), geglu_f(a.w, u.w));
                }
                __half *dst = out + (size_t)col * n_rows + n0 + r4;
                if (n0 + r4 + 3 < n_rows && (((uintptr_t)dst) & 7) == 0) {
                    *reinterpret_cast<uint2 *>(dst) = pack4(a.x, a.y, a.z, a.w);
                } else {
                    const float e[4] = {a.x, a.y, a.z, a.w};
                    for (int q = 0; q < 4; q++)
                        if (n0 + r4 + q < n_rows) dst[q] = __float2half_rn(e[q]);
                }
            }
        }
        cluster_sync();   // no CTA leaves while a peer may still read its shared memory
    }
    if (failed) tc_wait_expired(p.status, LC_DEV_STATUS_WAIT_EXPIRED_TCD, tid);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link-time dependency on the driver).
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

// The activations x[m, K] (f16, row-major) as a 2-D tensor map: boxes of 64 k x 64 rows land as 64 rows of 128 bytes
// with the 128-byte swizzle; rows beyond m read as zero.
int make_x_map(CUtensorMap *map, const void *x, uint32_t m, uint32_t kk) {
    encode_tiled_fn fn = encode_tiled();
    if (!fn) return lc_fail(LC_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    const cuuint64_t dims[2] = {kk, m};
    const cuuint64_t strides[1] = {(cuuint64_t)kk * 2};
    const cuuint32_t box[2] = {KT, NB};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return lc_fail(LC_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return LC_OK;
}

int launch_tcd(lc_batch *b, const TcdParams &p, const CUtensorMap &x_map, int tiles, size_t smem) {
    static lc_smem_optin optin;
    LC_CUDA_TRY(lc_ensure_smem(qgemm_tcd_kernel, optin, b->ctx, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, 1, p.ks);
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
    if (p.ks > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = (unsigned)p.ks;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    LC_LAUNCH_CHECKED(cudaLaunchKernelEx(&cfg, qgemm_tcd_kernel, p, x_map));
    b->dispatch_count++;
    return LC_OK;
}

}  // namespace

// Grouped launch: `ng` TQ2_0 weight matrices [ns[g], kk] sharing the activations `input` [m, kk], 8 < m <= 64, f16 out;
// with `geglu`, two matrices of the same shape and one output gelu_tanh(x Wg^T) * (x Wu^T).  Returns LC_OK after a
// launch, a positive status on error, or -1 when the shape is outside what this kernel covers.
int lc_qgemm_tcd_launch(lc_kernels *k, lc_batch *b, const lc_buf *input, int ng, const lc_buf *const *weights,
                        lc_buf *const *outputs, const uint32_t *ns, uint32_t m, uint32_t kk, bool geglu) {
    if (m < 1 || m > NB || ng < 1 || ng > MAX_GROUPS || kk % 256 != 0 || !lc_aligned(input->dptr, 16)) return -1;
    if (geglu && (ng != 2 || ns[0] != ns[1])) return -1;
    TcdParams p;
    p.m = (int)m;
    p.K = (int)kk;
    p.nb = (int)(kk / 256);
    p.ngroups = geglu ? 1 : ng;
    p.geglu = geglu ? 1 : 0;
    int tiles = 0;
    for (int g = 0; g < MAX_GROUPS; g++) {
        const int gi = g < ng ? g : ng - 1;
        if (!lc_aligned(weights[gi]->dptr, 16)) return -1;
        p.w[g] = (const uint8_t *)weights[gi]->dptr;
        p.out[g] = (__half *)outputs[gi]->dptr;
        p.n[g] = (int)ns[gi];
        const int rows_out = geglu ? TILE_ROWS / 2 : TILE_ROWS;
        if (g < ng && !(geglu && g > 0)) tiles += ((int)ns[g] + rows_out - 1) / rows_out;
        p.tile_end[g] = tiles;
    }
    if (tiles < 1) return -1;
    const int rows = TILE_ROWS;
    // One wave: split K over a cluster of at most 8 CTAs while the CTA count stays within about 7/8 of the SM count
    // (a cluster needs all its SMs in one GPC, so the last few SMs cannot always be used; a launch that does not fit
    // runs a second wave and takes twice as long), no CTA takes more than MAX_STEPS steps (six blocks per row), and,
    // where K allows, every CTA keeps two steps: both weight slots are dequantized before the dependency wait, so a
    // second step costs only its MMAs, while every further split adds a partial tile to the exchange that follows
    // (Q/K/V 3 x 2 steps instead of 6 x 1, O 4 x 2 instead of 8 x 1: step 2.328 -> 2.281 ms; three steps per CTA
    // 2.333 ms, four 2.350 ms; LOCAL_CUDA_TCD_MIN_BPS overrides).
    static const int ks_cap = []() { const char *e = getenv("LOCAL_CUDA_TCD_KS"); const int v = e ? atoi(e) : 0; return v > 0 ? v : MAX_KS; }();
    int ks = (k->ctx->sm_count * 7 / 8) / tiles;
    if (ks > ks_cap) ks = ks_cap;
    if (ks > MAX_KS) ks = MAX_KS;
    if (ks > p.nb) ks = p.nb;
    static const int min_bps = []() { const char *e = getenv("LOCAL_CUDA_TCD_MIN_BPS"); const int v = e ? atoi(e) : 2; return v >= 1 && v <= MAX_STEPS ? v : 2; }();
    if (ks > (p.nb + min_bps - 1) / min_bps) ks = (p.nb + min_bps - 1) / min_bps;
    if (ks < 1) ks = 1;
    int bps = (p.nb + ks - 1) / ks;
    if (bps > MAX_STEPS) bps = MAX_STEPS;
    ks = (p.nb + bps - 1) / bps;
    if (ks > MAX_KS) return -1;   // K too long for one cluster of this kernel
    p.ks = ks;
    p.bps = bps;
    p.raw_rs = ((bps * BB + 15 + 15) / 16) * 16;
    if ((p.raw_rs / 16) % 2 == 0) p.raw_rs += 16;
    p.status = k->dev_status;
    p.wait_limit = k->test_wait_expiry ? 4096u : WAIT_LIMIT;
    p.extra_arrivals = k->test_wait_expiry ? 1u : 0u;
    // Shared memory: the raw rows and up to three activation slots of one step each (the weight operand lives in
    // tensor memory); the first slot doubles as the staging of the split-K / GeGLU exchange (32 KB, exactly one slot).
    const int total = bps;
    const size_t fixed = (size_t)rows * p.raw_rs + (1 + 2 * MAX_STEPS + NBAR) * 8 + 16 + 1024;   // + 1024: tile alignment slack
    const size_t budget = k->ctx->smem_optin > 2048 ? k->ctx->smem_optin - 1024 : 0;
    static const int sb_cap = []() { const char *e = getenv("LOCAL_CUDA_TCD_SB"); const int v = e ? atoi(e) : 0; return v >= 1 && v <= MAX_STEPS ? v : 3; }();
    int sb = total < sb_cap ? total : sb_cap;
    while (sb > 1 && fixed + (size_t)sb * B_SLOT > budget) sb--;
    if (fixed + (size_t)sb * B_SLOT > budget) return -1;
    static_assert((size_t)B_SLOT >= (size_t)NB * TILE_ROWS * 4, "the exchange staging must fit one activation slot");
    p.sa = SA;
    p.sb = sb;
    const size_t smem = fixed + (size_t)sb * B_SLOT;
    CUtensorMap x_map;
    int st = make_x_map(&x_map, input->dptr, m, kk);
    if (st != LC_OK) return st;
    return launch_tcd(b, p, x_map, tiles, smem);
}
