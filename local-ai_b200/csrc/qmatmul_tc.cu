// Tensor-core (tcgen05 + TMEM) path of the quantized batched matmul
//   C[m, n] = A[m, K] (f16) x W[n, K]^T,  W in GGUF Q4_0 / TQ2_0 blocks.
// Stands in for the reference's simdgroup-matrix kernels matmul_nt_{q4_0,tq2_0}_mma
// (shaders/matvec_quant.metal:447-577) for m > 8.
//
// Mapping.  The weights take the MMA's M dimension and the batch its N dimension:
//   D[128 weight rows, NB batch rows] (f32, TMEM) += Wdeq[128, 16] * Act[NB, 16]^T
// (tcgen05.mma.cta_group::1.kind::f16, both operands K-major in shared memory,
// no-swizzle "interleave" layout: 8x16-byte core matrices, SBO = 128 B between
// 8-row groups, LBO between 8-element k-chunks).  One CTA owns a 128-row weight tile and up to
// 128 batch rows, and walks K in phases:
//   1. the phase's raw weight bytes — for each of the 128 rows one contiguous run
//      of blocks — are copied HBM -> shared with 16-byte cp.async (rows are only
//      2-byte aligned, so each run is copied as its enclosing 16-byte range);
//   2. per 128-wide k-tile: the activations are cp.async'ed straight into the
//      operand layout, the weights are unpacked with the 0x6400 magic-number
//      trick (two codes per 32-bit op) into f16 and stored into the operand
//      layout, then one thread issues eight K=16 MMAs and commits them to an
//      mbarrier; the two operand stages alternate so unpacking of tile t+1
//      overlaps the MMAs of tile t.
// The epilogue reads the accumulator with tcgen05.ld (warp w <- TMEM lanes
// 32w..32w+31, one weight row per thread) and stores C transposed.
//
// Numerics: TQ2_0 weights d*(q-1) in {-d, 0, d, 2d} are exact in f16, so the
// result equals the CUDA-core path up to f32 summation order.  Q4_0 weights
// d*(q-8) need up to 15 significant bits; the reference's M > 8 kernel keeps
// them in f32 (matvec_quant.metal:477-506).  Here every 128-k tile of Q4_0 runs
// as two pipeline steps over the same activations: the f16-rounded weights, then
// the f16 of what the rounding dropped (exact but for f16 underflow, ~3e-8
// absolute), so the accumulated product matches the f32-weight one.
//
// Every wait on an mbarrier is bounded; on expiry the CTA records a status
// word, skips to the TMEM release and returns.
#include <stdlib.h>
#include "lc_internal.h"

namespace {

constexpr int FMT_Q4_0 = 0;
constexpr int FMT_TQ2_0 = 1;
constexpr int NT = 256;
constexpr int TILE_ROWS = 128;          // weight rows per CTA (UMMA M)
constexpr int KT = 128;                 // k per operand stage
constexpr int RAW_RS = 448;             // bytes reserved per row of raw blocks (<= 432 data + 15 skew)
constexpr int A_SBO = 128;
constexpr int A_LBO = TILE_ROWS * 16 + 32;   // +32 B: consecutive k-chunks land 8 banks apart
constexpr int A_STAGE = (KT / 8) * A_LBO;
constexpr int MAX_NB = 128;
constexpr uint32_t WAIT_LIMIT = 1u << 24;

template <int FMT> struct TcFmt;
template <> struct TcFmt<FMT_Q4_0> { static constexpr int bytes = 18, elems = 32, phase_blocks = 24; };
template <> struct TcFmt<FMT_TQ2_0> { static constexpr int bytes = 66, elems = 256, phase_blocks = 6; };

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void mbar_init(uint32_t addr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(addr), "r"(count) : "memory");
}
// Bounded wait; false on expiry.
__device__ __forceinline__ bool mbar_wait(uint32_t addr, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// K-major, no swizzle: start address, LBO (between k-chunks), SBO (between 8-row groups), version 1.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}\n"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

__device__ __forceinline__ void store_c(__half *p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void store_c(float *p, float v) { *p = v; }

constexpr int MAX_GROUPS = 3;
struct TcParams {
    // Up to three weight matrices that share the activations and K (Q/K/V, gate/up) run as one launch:
    // row tiles [tile_end[g-1], tile_end[g]) of the grid's x dimension belong to matrix g.
    const uint8_t *w[MAX_GROUPS];
    void *out[MAX_GROUPS];
    int n[MAX_GROUPS], tile_end[MAX_GROUPS];
    int ngroups;
    const __half *x;
    int m, K, nb;          // nb = blocks per row
    int ks, bps;           // split-K: grid.z = ks, bps = blocks per split
    float *partial;        // [tile][split][NB cols][128 rows] f32, used when ks > 1
    unsigned int *counters; // one per tile, zero between launches (the last CTA to arrive resets it)
    int NB;                // batch rows per CTA (multiple of 16, <= 128)
    int sb;                // activation stages (6 when they fit, else 3); weight stages are fixed at 2
    int tmem_cols;         // power of two >= max(32, NB)
    int *status;
    uint32_t wait_limit;   // polls before a barrier wait gives up
    uint32_t extra_arrivals;   // 0; 1 in the expiry self-test: the "weights ready" barriers then expect an arrival nobody makes
};

__device__ __forceinline__ void mbar_arrive(uint32_t addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(addr) : "memory");
}

constexpr int N_UNPACK_WARPS = 16;
constexpr int ROWS_PER_WARP = TILE_ROWS / N_UNPACK_WARPS;  // 8
constexpr int NT2 = (N_UNPACK_WARPS + 1) * 32;              // + one warp: activation loads and MMA issue
constexpr int SA = 2;        // weight (A operand) stages
constexpr int MAX_BAR = 6;   // mma_done barriers, one per tile index mod 6 (>= any activation stage count)
static_assert(N_UNPACK_WARPS == KT / 8, "one unpack warp per k-chunk of the activation tile");

// Warp-specialised pipeline, no CTA-wide barrier inside the k loop:
//   warps 0..15 own 8 weight rows each: cp.async their raw blocks, unpack them into operand
//               stage s, bring in one k-chunk of the activation tile (prefetched one tile ahead) and
//               arrive on a_full[s];
//   warp 16     waits for a_full[s], issues the eight K=16 MMAs of the tile and commits them to
//               mma_done[s], which frees stage s.  Nothing waits on a commit younger than S tiles:
//               the commit -> mbarrier latency is far longer than one tile of work.
template <int FMT, typename OutT>
__global__ void __launch_bounds__(NT2, 1) qgemm_tc_kernel(const TcParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int BB = TcFmt<FMT>::bytes, BE = TcFmt<FMT>::elems, PB = TcFmt<FMT>::phase_blocks;
    const int NB = p.NB, SB = p.sb, PD = p.sb - 2;   // PD: activation tiles kept in flight ahead of the current one
    const int B_LBO = NB * 16, B_STAGE = (KT / 8) * B_LBO;
    uint8_t *raw = smem;                                   // [128][RAW_RS]
    uint8_t *a_s = raw + TILE_ROWS * RAW_RS;               // [SA][A_STAGE]
    uint8_t *b_s = a_s + SA * A_STAGE;                     // [SB][B_STAGE]
    uint64_t *a_full = reinterpret_cast<uint64_t *>(b_s + SB * B_STAGE);  // [SA]
    uint64_t *mma_done = a_full + SA;                                   // [MAX_BAR]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(mma_done + MAX_BAR);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    lc_pdl_trigger();
    int grp = 0;
    while (grp + 1 < p.ngroups && (int)blockIdx.x >= p.tile_end[grp]) grp++;
    const int n0 = ((int)blockIdx.x - (grp ? p.tile_end[grp - 1] : 0)) * TILE_ROWS, m0 = blockIdx.y * MAX_NB;
    const int n_rows = p.n[grp];
    const uint8_t *wmat = p.w[grp];
    const size_t rb = (size_t)p.nb * BB;
    const size_t w_bytes = rb * (size_t)n_rows;
    const int kbs = (int)blockIdx.z * p.bps, kbe = min(p.nb, kbs + p.bps);   // this CTA's K blocks

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tid == 0) {
        for (int i = 0; i < SA; i++) mbar_init(smem_u32(&a_full[i]), N_UNPACK_WARPS + p.extra_arrivals);
        for (int i = 0; i < MAX_BAR; i++) mbar_init(smem_u32(&mma_done[i]), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t idesc = (1u << 4) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(TILE_ROWS >> 4) << 24);
    // pipeline steps per 128-k tile: Q4_0 runs each tile twice (rounded weights, then the rounding remainder)
    constexpr int REP = (FMT == FMT_Q4_0) ? 2 : 1;
    const int nphases = (kbe - kbs + PB - 1) / PB;
    const int total_tiles = ((kbe - kbs) * BE) / KT * REP;
    const int kg_base = kbs * BE;   // first k of this CTA

    if (warp < N_UNPACK_WARPS) {
        // =============================== unpack warps ===============================
        const int r_base = warp * ROWS_PER_WARP;
        int tile = 0;
        bool dead = false;
        // This warp also brings in k-chunk `warp` (8 k values) of every activation tile, one tile ahead:
        // lane walks batch rows lane, lane + 32, ...  Element (mrow, chunk c) lives at c*B_LBO + 16*mrow.
        const __half *x_lane = p.x + (size_t)(m0 + lane) * p.K + kg_base + warp * 8;
        const int rows_valid = p.m - m0;
        auto load_b = [&](int tl) {
            uint32_t dst = smem_u32(b_s + (tl % SB) * B_STAGE) + (uint32_t)(warp * B_LBO + 16 * lane);
            const __half *src = x_lane + (size_t)(tl / REP) * KT;
            for (int mrow = lane; mrow < NB; mrow += 32) {
                const bool ok = mrow < rows_valid;
                cp_async16(dst, ok ? (const void *)src : (const void *)p.x, ok ? 16u : 0u);
                dst += 512;
                src += (size_t)32 * p.K;
            }
        };
        // MMAs of tile tl have completed (frees weight stage tl % SA and activation stage tl % SB).
        auto mma_finished = [&](int tl) -> bool {
            uint32_t ok = 1;
            if (lane == 0) ok = mbar_wait(smem_u32(&mma_done[tl % MAX_BAR]), (uint32_t)((tl / MAX_BAR) & 1), p.wait_limit) ? 1u : 0u;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            return ok && !*abort_flag;
        };
        for (int ph = 0; ph < nphases && !dead; ph++) {
            const int kb0 = kbs + ph * PB, kb1 = min(kbe, kb0 + PB);
            const int seg = (kb1 - kb0) * BB;
            __syncwarp();  // the previous phase's raw bytes are no longer being read by this warp
            for (int rr = 0; rr < ROWS_PER_WARP; rr++) {
                const int r = r_base + rr, row = n0 + r;
                if (row >= n_rows) break;
                const size_t g0 = (size_t)row * rb + (size_t)kb0 * BB;
                const size_t a0 = g0 & ~(size_t)15;
                const int npieces = (int)((g0 + seg - a0 + 15) >> 4);
                for (int pc = lane; pc < npieces; pc += 32) {
                    const size_t g = a0 + ((size_t)pc << 4);
                    uint8_t *dst = raw + r * RAW_RS + (pc << 4);
                    if (g + 16 <= w_bytes) {
                        cp_async16(smem_u32(dst), wmat + g, 16);
                    } else {
                        for (int b = 0; b < 16; b++) dst[b] = (g + b < w_bytes) ? wmat[g + b] : 0;
                    }
                }
            }
            cp_async_commit();
            if (ph == 0) {
                // The weights above do not depend on the previous kernel, so their copies are already in
                // flight; the activations do: wait for the predecessor grid before touching them.
                lc_pdl_wait();
                for (int t = 0; t < PD; t++) {   // activation tiles 0 .. PD-1, one cp.async group each
                    if (t < total_tiles) load_b(t);
                    cp_async_commit();
                }
            }
            cp_async_wait<0>();
            __syncwarp();
            const int ntiles = ((kb1 - kb0) * BE) / KT * REP;
            // Per-thread constants of this phase: where each of its rows starts in the raw area (the row's
            // 16-byte skew differs from row to row) and whether the row exists.
            constexpr int NIT = (FMT == FMT_TQ2_0) ? ROWS_PER_WARP / 2 : ROWS_PER_WARP;
            const int sub = (FMT == FMT_TQ2_0) ? (lane >> 4) : 0;      // TQ2_0: which row of the pair
            const uint8_t *src[NIT];
            bool valid[NIT];
#pragma unroll
            for (int i = 0; i < NIT; i++) {
                const int r = r_base + ((FMT == FMT_TQ2_0) ? 2 * i + sub : i), row = n0 + r;
                const size_t g0 = (size_t)row * rb + (size_t)kb0 * BB;
                src[i] = raw + r * RAW_RS + (int)(g0 & 15);
                valid[i] = row < n_rows;
            }
            for (int t = 0; t < ntiles; t++, tile++) {
                const int s = tile % SA;
                // One wait per tile: the MMAs of tile - 2 are done, which frees weight stage s and the
                // activation stage that tile + PD will use (PD = SB - 2).
                if (tile >= 2 && !mma_finished(tile - 2)) { *abort_flag = 1; dead = true; break; }
                if (tile + PD < total_tiles) load_b(tile + PD);
                cp_async_commit();
                uint8_t *ast = a_s + s * A_STAGE;
                if (FMT == FMT_TQ2_0) {
                    // tile t = half h of block kb (32 code bytes per row). lane = (row of a pair, 2-byte piece u):
                    // 8 weights k = l*32 + 2u + {0,1}, l = 0..3.  Element (r, k) lives at 16 r + (k/8) LBO + 2 (k%8).
                    const int u = lane & 15;
                    const int soff = (t >> 1) * BB + (t & 1) * 32 + 2 * u, doff = (t >> 1) * BB + 64;
                    uint8_t *dst = ast + 16 * (r_base + sub) + (u & 3) * 4 + (u >> 2) * A_LBO;
                    uint32_t w16[NIT];
                    __half dd[NIT];
#pragma unroll
                    for (int i = 0; i < NIT; i++) {
                        w16[i] = *reinterpret_cast<const uint16_t *>(src[i] + soff);
                        dd[i] = *reinterpret_cast<const __half *>(src[i] + doff);
                    }
                    const __half2 c1025 = __float2half2_rn(1025.0f);
#pragma unroll
                    for (int i = 0; i < NIT; i++) {
                        const __half2 d2 = __half2half2(valid[i] ? dd[i] : __float2half(0.0f));
                        const uint32_t tlo = __byte_perm(w16[i], 0u, 0x4140);  // [b0, 0, b1, 0]
#pragma unroll
                        for (int l = 0; l < 4; l++) {
                            const uint32_t hbits = ((tlo >> (2 * l)) & 0x00030003u) | 0x64006400u;   // 1024 + q
                            const __half2 w = __hmul2(__hsub2(bits_h2(hbits), c1025), d2);           // (q - 1) d, exact
                            *reinterpret_cast<uint32_t *>(dst + 32 * i + l * (4 * A_LBO)) = h2_bits(w);
                        }
                    }
                } else {
                    // step t = blocks 4(t/2)..4(t/2)+3 of the phase, rounded weights (t even) or remainder (t odd);
                    // lane = (block b, 2-byte piece hh): low nibbles k = 32b + 2hh + {0,1}, high nibbles 16 further
                    // (two k-chunks on).
                    const int b = lane >> 3, hh = lane & 7;
                    const int boff = (4 * (t >> 1) + b) * BB;
                    const bool rem = t & 1;
                    uint8_t *dst = ast + 16 * r_base + (hh & 3) * 4 + (4 * b + (hh >> 2)) * A_LBO;
                    uint32_t w16[NIT];
                    __half dd[NIT];
#pragma unroll
                    for (int i = 0; i < NIT; i++) {
                        dd[i] = *reinterpret_cast<const __half *>(src[i] + boff);
                        w16[i] = *reinterpret_cast<const uint16_t *>(src[i] + boff + 2 + 2 * hh);
                    }
                    const __half2 c1032 = __float2half2_rn(1032.0f);
#pragma unroll
                    for (int i = 0; i < NIT; i++) {
                        const __half2 d2 = __half2half2(valid[i] ? dd[i] : __float2half(0.0f));
                        const float df = __low2float(d2);
                        const uint32_t tlo = __byte_perm(w16[i], 0u, 0x4140);
                        const __half2 qlo = __hsub2(bits_h2((tlo & 0x000F000Fu) | 0x64006400u), c1032);          // q - 8, exact
                        const __half2 qhi = __hsub2(bits_h2(((tlo >> 4) & 0x000F000Fu) | 0x64006400u), c1032);
                        __half2 lo = __hmul2(qlo, d2), hi = __hmul2(qhi, d2);                                     // rounded weights
                        if (rem) {   // what the rounding dropped: d (q - 8) is exact in f32
                            const float2 ql = __half22float2(qlo), qh = __half22float2(qhi), rl = __half22float2(lo), rh = __half22float2(hi);
                            lo = __floats2half2_rn(ql.x * df - rl.x, ql.y * df - rl.y);
                            hi = __floats2half2_rn(qh.x * df - rh.x, qh.y * df - rh.y);
                        }
                        *reinterpret_cast<uint32_t *>(dst + 16 * i) = h2_bits(lo);
                        *reinterpret_cast<uint32_t *>(dst + 16 * i + 2 * A_LBO) = h2_bits(hi);
                    }
                }
                // this tile's activation chunk has landed; the PD younger groups may still be in flight
                if (PD == 4) cp_async_wait<4>(); else cp_async_wait<1>();
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&a_full[s]));
            }
        }
    } else {
        // ============================ MMA issue (one warp) ============================
        bool dead = false;
        const uint64_t adesc0 = make_desc(smem_u32(a_s), A_LBO, A_SBO), bdesc0 = make_desc(smem_u32(b_s), (uint32_t)B_LBO, 128u);
        for (int tile = 0; tile < total_tiles && !dead; tile++) {
            const int s = tile % SA, use = tile / SA;
            uint32_t ok = 1;
            if (lane == 0) ok = mbar_wait(smem_u32(&a_full[s]), (uint32_t)(use & 1), p.wait_limit) ? 1u : 0u;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok || *abort_flag) { *abort_flag = 1; dead = true; break; }
            if (lane == 0) {
                tc_fence_after();
                // descriptors differ from tile to tile only in the start-address field (bits 0-13, address >> 4)
                uint64_t ad = adesc0 + (uint64_t)((uint32_t)(s * A_STAGE) >> 4);
                uint64_t bd = bdesc0 + (uint64_t)((uint32_t)((tile % SB) * B_STAGE) >> 4);
                const uint64_t bstep = (uint64_t)((uint32_t)(2 * B_LBO) >> 4);
#pragma unroll
                for (int j = 0; j < KT / 16; j++) {
                    umma_f16(tmem_base, ad, bd, idesc, (tile > 0 || j > 0) ? 1u : 0u);
                    ad += (uint64_t)((2 * A_LBO) >> 4);
                    bd += bstep;
                }
                umma_commit(smem_u32(&mma_done[tile % MAX_BAR]));
            }
            __syncwarp();
        }
        // drain: the last commit covers every MMA issued before it
        if (!dead && total_tiles > 0) {
            const int last = total_tiles - 1;
            uint32_t ok = 1;
            if (lane == 0) ok = mbar_wait(smem_u32(&mma_done[last % MAX_BAR]), (uint32_t)((last / MAX_BAR) & 1), p.wait_limit) ? 1u : 0u;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) *abort_flag = 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const bool failed = *abort_flag != 0;
    const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
    if (!failed && warp < 4) {
        const int lrow = warp * 32 + lane, row = n0 + lrow;
        OutT *out = reinterpret_cast<OutT *>(p.out[grp]);
        float *part = p.partial + ((size_t)tile_id * p.ks + blockIdx.z) * (size_t)NB * TILE_ROWS;
        for (int c0 = 0; c0 < NB; c0 += 16) {
            uint32_t v[16];
            tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
            if (p.ks > 1) {
#pragma unroll
                for (int j = 0; j < 16; j++) part[(size_t)(c0 + j) * TILE_ROWS + lrow] = __uint_as_float(v[j]);
            } else if (row < n_rows) {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int gm = m0 + c0 + j;
                    if (gm < p.m) store_c(out + (size_t)gm * n_rows + row, __uint_as_float(v[j]));
                }
            }
        }
    }
    if (p.ks > 1 && !failed) {
        // Deterministic split-K: every split stores its f32 partial tile; the last CTA to arrive adds the
        // partials in split order and writes the result.
        __shared__ unsigned int is_last;
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned int prev = atomicAdd(&p.counters[tile_id], 1u);
            is_last = (prev == (unsigned int)p.ks - 1) ? 1u : 0u;
            if (is_last) p.counters[tile_id] = 0u;
        }
        __syncthreads();
        if (is_last) {
            __threadfence();
            OutT *out = reinterpret_cast<OutT *>(p.out[grp]);
            const float *part = p.partial + (size_t)tile_id * p.ks * (size_t)NB * TILE_ROWS;
            // four rows per thread-step (float4 along the row index), splits summed in order, loads in
            // independent batches of four so several L2 round trips are in flight per thread
            const size_t pstride = (size_t)NB * TILE_ROWS;
            for (int i4 = tid; i4 < NB * TILE_ROWS / 4; i4 += NT2) {
                const int i = i4 * 4;
                const int col = i / TILE_ROWS, lrow = i - col * TILE_ROWS;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int sp = 0; sp < p.ks; sp += 4) {
                    float4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        v[u] = (sp + u < p.ks) ? __ldcg(reinterpret_cast<const float4 *>(part + (size_t)(sp + u) * pstride + i))
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w;
                    }
                }
                const int gm = m0 + col;
                if (gm < p.m) {
                    const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        if (n0 + lrow + u < n_rows) store_c(out + (size_t)gm * n_rows + n0 + lrow + u, a4[u]);
                }
            }
        }
    }
    if (failed && tid == 0) atomicExch(p.status, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                     : "memory");
    }
}

template <int FMT, typename OutT>
int launch_tc(lc_kernels *k, lc_batch *b, TcParams &p, dim3 grid) {
    const size_t bstage = (size_t)(KT / 8) * p.NB * 16;
    auto need = [&](int sb) { return (size_t)TILE_ROWS * RAW_RS + (size_t)SA * A_STAGE + sb * bstage + 128; };
    p.sb = need(6) <= k->ctx->smem_optin ? 6 : 3;
    const size_t smem = need(p.sb);
    auto kern = qgemm_tc_kernel<FMT, OutT>;
    static lc_smem_optin optin;
    LC_CUDA_TRY(lc_ensure_smem(kern, optin, b->ctx, smem));
    LC_LAUNCH_CHECKED(lc_launch(kern, dim3(grid), dim3(NT2), smem, b, p));
    LC_CHECK_LAUNCH("qgemm_tcgen05");
    b->dispatch_count++;
    return LC_OK;
}

}  // namespace

// Grouped launch: `ng` weight matrices [n[g], kk] sharing the activations `input` [m, kk].
// Returns LC_OK after a launch, a positive status on error, or -1 when the shape
// is outside what this kernel covers (the caller then uses the CUDA-core path).
int lc_qgemm_tcgen05_grouped(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input, int ng,
                             const lc_buf *const *weights, lc_buf *const *outputs, const uint32_t *ns, uint32_t m,
                             uint32_t kk) {
    if (kk % KT != 0 || ng < 1 || ng > MAX_GROUPS) return -1;  // Q4_0 with K not a multiple of 128
    TcParams p;
    p.x = (const __half *)input->dptr;
    p.m = (int)m;
    p.K = (int)kk;
    p.nb = fmt == FMT_Q4_0 ? (int)(kk / 32) : (int)(kk / 256);
    p.ngroups = ng;
    int tiles = 0;
    for (int g = 0; g < MAX_GROUPS; g++) {
        const int gi = g < ng ? g : ng - 1;
        p.w[g] = (const uint8_t *)weights[gi]->dptr;
        p.out[g] = outputs[gi]->dptr;
        p.n[g] = (int)ns[gi];
        if (g < ng) tiles += ((int)ns[g] + TILE_ROWS - 1) / TILE_ROWS;
        p.tile_end[g] = tiles;
    }
    const uint32_t mb = m < (uint32_t)MAX_NB ? m : (uint32_t)MAX_NB;
    p.NB = (int)((mb + 15) / 16 * 16);
    int cols = 32;
    while (cols < p.NB) cols <<= 1;
    p.tmem_cols = cols;
    p.sb = 3;
    p.status = k->dev_status;
    p.wait_limit = k->test_wait_expiry ? 4096u : WAIT_LIMIT;
    p.extra_arrivals = k->test_wait_expiry ? 1u : 0u;
    const int mtiles = (int)((m + MAX_NB - 1) / MAX_NB);
    // split-K so that small-n projections still fill the GPU: each split gets whole blocks and at least two k-tiles.
    const int min_blocks = fmt == FMT_Q4_0 ? 8 : 1;   // 8 Q4_0 blocks = 256 k = 2 k-tiles; 1 TQ2_0 block = 2 k-tiles
    int ks = k->ctx->sm_count / (tiles * mtiles);
    const int max_ks = p.nb / min_blocks;
    if (ks > max_ks) ks = max_ks;
    if (ks < 1) ks = 1;
    if (ks > 32) ks = 32;
    int bps = (p.nb + ks - 1) / ks;
    bps = (bps + min_blocks - 1) / min_blocks * min_blocks;   // Q4_0: whole k-tiles (4 blocks) per split
    ks = (p.nb + bps - 1) / bps;
    p.ks = ks;
    p.bps = bps;
    p.partial = nullptr;
    p.counters = nullptr;
    if (ks > 1) {
        const size_t ntile = (size_t)tiles * mtiles;
        int st = lc_reserve_scratch(k, b, ntile * ks * (size_t)p.NB * TILE_ROWS * sizeof(float), ntile);
        if (st != LC_OK) return st;
        p.partial = (float *)k->scratch;
        p.counters = k->counters;
    }
    dim3 grid(tiles, mtiles, ks);
    if (fmt == FMT_Q4_0)
        return f32out ? launch_tc<FMT_Q4_0, float>(k, b, p, grid) : launch_tc<FMT_Q4_0, __half>(k, b, p, grid);
    return f32out ? launch_tc<FMT_TQ2_0, float>(k, b, p, grid) : launch_tc<FMT_TQ2_0, __half>(k, b, p, grid);
}

int lc_qgemm_tcgen05(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                     lc_buf *output, uint32_t m, uint32_t kk, uint32_t n) {
    const lc_buf *ws[1] = {weight};
    lc_buf *os[1] = {output};
    const uint32_t ns[1] = {n};
    return lc_qgemm_tcgen05_grouped(fmt, f32out, k, b, input, 1, ws, os, ns, m, kk);
}

extern "C" int lc_kernels_device_status(lc_kernels *k, int *status) {
    if (!k || !status) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_kernels_device_status: NULL argument");
    LC_CUDA_TRY(cudaMemcpyAsync(status, k->dev_status, sizeof(int), cudaMemcpyDeviceToHost, k->ctx->stream));
    LC_CUDA_TRY(cudaStreamSynchronize(k->ctx->stream));
    if (*status == LC_DEV_STATUS_POSITION)
        return lc_fail(LC_ERR_INVALID_ARGUMENT,
                       "a position in a device buffer pointed past its lane's pool rows (the row was not written / the "
                       "context was clamped)");
    if (*status) return lc_fail(LC_ERR_TIMEOUT, "a device-side bounded wait expired (status %d)", *status);
    return LC_OK;
}
