// tcgen05 decode matmul: C[m, n] = A[m, K] (f16) x W[n, K]^T with W in GGUF TQ2_0 blocks, 8 < m <= 64, f16 out.
// Stands in, at decode batch sizes, for the reference's simdgroup-matrix kernel matmul_nt_tq2_0_mma
// (shaders/matvec_quant.metal:447-577) and, in GeGLU mode, for the pair of projections + gelu_mul of
// local-engine/src/layer.rs:825-838.
//
// A decode projection is a few microseconds of work that sits behind the kernel before it, so the kernel is built
// around the length of the dependent chain after that kernel finishes:
//   * weights take the MMA's M (128 rows per accumulator; a GeGLU CTA holds two accumulators, 128 gate rows and the
//     same 128 rows of the up matrix), the batch its N (64, zero padded), f32 accumulators in TMEM;
//   * at most one CTA per SM and one wave per launch: K is split over a thread-block cluster so that the CTA count
//     stays within the SM count, which also keeps the number of CTAs that re-read the same activations from L2 low;
//   * before the dependency wait: TMEM allocation, barrier set-up, the raw quantized rows of the CTA's K range
//     brought in by bulk copies (cp.async.bulk, one per row segment, completion counted on an mbarrier), and as many
//     operand stages dequantized as shared memory holds -- none of it depends on the predecessor;
//   * after the wait two warps bring in the activations of the CTA's whole K range (every stage in flight at once;
//     the first access after a kernel boundary costs well over a microsecond, so nothing is requested late), the
//     dequantizing warps keep turning code bytes into f16 weights (the four values a 2-bit code can mean, (q - 1) d,
//     sit in two registers as a byte table; one prmt assembles two weights; 16-byte stores into the K-major
//     128-byte-swizzled operand layout), and four warps issue tcgen05.mma.cta_group::1.kind::f16.  Issuing one MMA costs a
//     warp about 210 cycles whatever its shape (measured: M 64 / 128, N 16 .. 256 all the same), far more than the
//     32 cycles of arithmetic in a 128 x 64 x 16 step, but MMAs issued by different warps overlap fully (4 warps: 53
//     cycles per MMA).  So the four K = 16 steps of a 64-k stage belong to four issuing warps, each with its own TMEM
//     accumulator (four partial sums over interleaved k, added in a fixed order in the epilogue); every issuer
//     commits its step to the stage's mbarrier, which hands the stage back after the fourth arrival;
//   * CTAs walk their stages from different starting points so that the CTAs of a launch do not all ask L2 for the
//     same activation lines at the same moment;
//   * the accumulators are read back with tcgen05.ld by all dequantizing warps.  When K is split, the CTAs of a tile
//     add their partial tiles in split order through distributed shared memory, each finishing one contiguous slice.
//
// Numerics: TQ2_0 weights d (q - 1) are exact in f16, accumulation is f32, splits are added in split order:
// the same contract as the register-direct mma.sync kernel (qmatmul_mma.cu), which remains the fallback.
//
// Every wait on an mbarrier is bounded; on expiry the CTA raises the kernels object's status word, skips to the
// TMEM release and returns.
#include <stdlib.h>

#include "lc_internal.h"

namespace {

constexpr int TILE_ROWS = 128;   // weight rows per accumulator (UMMA M)
constexpr int NB = 64;           // batch columns (UMMA N)
constexpr int KT = 64;           // k per operand stage
constexpr int NBAR = 16;         // stage-release barriers, one per stage index mod 16
constexpr int NLOAD = 2;         // activation loader warps
constexpr int NISS = 4;          // MMA-issuing warps, one accumulator each (see below)
constexpr int TMEM_COLS = NISS * NB;   // 256
// Operand tiles are K-major with the 128-byte swizzle: a row is its 64 k values (128 bytes, eight 16-byte chunks),
// rows follow each other at 128 bytes, and chunk c of row r sits at chunk position c ^ (r % 8) of the row.  Tiles
// start on 1024-byte boundaries (eight rows: the swizzle pattern's period).
constexpr int ROW_BYTES = KT * 2;            // 128
constexpr int A_TILE = TILE_ROWS * ROW_BYTES;   // one 128-row operand tile of one stage: 16 KB
constexpr int B_STAGE = NB * ROW_BYTES;         // 8 KB
constexpr int BB = 66;           // bytes per TQ2_0 block
constexpr int MAX_TILES = 12;    // stages per CTA (three blocks of 256 k)
constexpr int MAX_GROUPS = 3;
constexpr int MAX_KS = 8;        // portable cluster size
constexpr uint32_t WAIT_LIMIT = 1u << 22;

struct TcdParams {
    const uint8_t *w[MAX_GROUPS];
    __half *out[MAX_GROUPS];
    int n[MAX_GROUPS], tile_end[MAX_GROUPS];
    int ngroups;
    const __half *x;
    int m, K, nb;        // nb = blocks per weight row
    int ks, bps;         // split-K: grid.z = cluster size = ks, bps = blocks per split
    int raw_rs;          // bytes reserved per row of raw blocks (odd multiple of 16)
    int sa, sb;          // operand stages in shared memory: weights (a ring) / activations (all stages of a CTA)
    int geglu;           // 1 (two accumulators): w[0] = gate, w[1] = up, out[0] = gelu(gate) * up
    int *status;
    uint32_t wait_limit;
};

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
__device__ __forceinline__ void mbar_arrive(uint32_t addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(addr), "r"(bytes) : "memory");
}
// One bulk copy global -> this CTA's shared memory; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t mbar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(mbar)
                 : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
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
// Shared-memory operand descriptor, K-major with the 128-byte swizzle: start address (>> 4), leading-dimension
// offset unused for this layout, 1024 bytes (eight 128-byte rows) between 8-row groups, descriptor version 1,
// layout type 2 (128-byte swizzle).  A K = 16 step inside the 64-k row advances the start address by 32 bytes.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
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
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t local_addr, uint32_t rank) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(ra) : "r"(local_addr), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(ra));
    return v;
}
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

// MT accumulators of 128 weight rows per CTA: 1 for a plain (grouped) projection, 2 for GeGLU.
template <int MT>
__global__ void __launch_bounds__((8 * MT + NLOAD + NISS) * 32, 1) qgemm_tcd_kernel(const TcdParams p) {
    constexpr int ROWS = TILE_ROWS * MT, NDQ = 8 * MT, NT = (NDQ + NLOAD + NISS) * 32;
    constexpr int A_STAGE = MT * A_TILE;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // operand tiles start on 1024-byte boundaries
    const int SA = p.sa, SB = p.sb;   // SB = the CTA's stage count: every activation stage has its own slot
    uint8_t *a_s = smem;                                   // [SA][A_STAGE]; reused for the split-K exchange
    uint8_t *b_s = a_s + SA * A_STAGE;                     // [SB][B_STAGE]
    uint8_t *raw = b_s + SB * B_STAGE;                     // [ROWS][raw_rs]
    uint64_t *bars = reinterpret_cast<uint64_t *>(raw + ROWS * p.raw_rs);
    uint64_t *raw_full = bars;                             // 1
    uint64_t *a_full = bars + 1;                           // [MAX_TILES] (SA used)
    uint64_t *b_all = a_full + MAX_TILES;                  // 1
    uint64_t *mma_done = b_all + 1;                        // [NBAR]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(mma_done + NBAR);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    lc_pdl_trigger();
    int grp = 0;
    if (MT == 1) while (grp + 1 < p.ngroups && (int)blockIdx.x >= p.tile_end[grp]) grp++;
    const int n0 = ((int)blockIdx.x - (grp ? p.tile_end[grp - 1] : 0)) * TILE_ROWS;   // first output row of this tile
    const int n_rows = p.n[grp];
    const size_t rb = (size_t)p.nb * BB, w_bytes = rb * (size_t)n_rows;
    const int kbs = (int)blockIdx.z * p.bps, kbe = min(p.nb, kbs + p.bps), nblk = max(kbe - kbs, 0);
    const int seg = nblk * BB;
    const int total_tiles = nblk * 4;                      // 64-k stages of this CTA
    // Step i of this CTA works on stage tile_of(i): pairs of stages (one 32-byte half block of codes) are walked
    // from a starting pair that differs from CTA to CTA.
    const int npairs = total_tiles >> 1, pair0 = npairs ? (int)((blockIdx.x * 5u + blockIdx.z) % (unsigned)npairs) : 0;
    auto tile_of = [&](int i) -> int {
        int pi = (i >> 1) + pair0;
        if (pi >= npairs) pi -= npairs;
        return 2 * pi + (i & 1);
    };
    // operand row r of the CTA -> weight matrix (accumulator r / 128) and row of it
    auto wmat_of = [&](int r) -> const uint8_t * { return MT == 2 ? p.w[r >> 7] : p.w[grp]; };

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    if (tid == 0) {
        mbar_init(smem_u32(raw_full), ROWS);
        for (int i = 0; i < MAX_TILES; i++) mbar_init(smem_u32(&a_full[i]), NDQ);
        mbar_init(smem_u32(b_all), NLOAD);
        for (int i = 0; i < NBAR; i++) mbar_init(smem_u32(&mma_done[i]), NISS);
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
            const int row = n0 + (tid & (TILE_ROWS - 1));
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
        // This thread's share of every stage: operand row 32 (warp & 3) + lane of accumulator (warp >> 3), the 16 code
        // bytes 16 bq .. + 15 (bq = (warp >> 2) & 1) of the stage's 32-byte half block, two of their four bit pairs.
        const int acc = warp >> 3, r = 32 * (warp & 3) + lane, bq = (warp >> 2) & 1;
        const int row = n0 + r;
        const bool rvalid = row < n_rows;
        const size_t g0 = (size_t)row * rb + (size_t)kbs * BB;
        const uint8_t *rrow = raw + (acc * TILE_ROWS + r) * p.raw_rs + (int)(g0 & 15);
        const uint32_t dst0 = smem_u32(a_s) + (uint32_t)(acc * A_TILE + r * ROW_BYTES);
        const uint32_t swz = (uint32_t)(r & 7);
        uint32_t lut_lo = 0, lut_hi = 0, cw[4] = {0, 0, 0, 0};
        for (int i = 0; i < total_tiles && !dead; i++) {
            const int t = tile_of(i), s = i % SA, blk = t >> 2, h = (t >> 1) & 1, lp = t & 1;
            if (i >= SA) {   // the MMAs that read this stage SA steps ago have completed
                uint32_t ok = 1;
                const int u = i - SA;
                if (lane == 0) ok = mbar_wait(smem_u32(&mma_done[u % NBAR]), (uint32_t)((u / NBAR) & 1), p.wait_limit) ? 1u : 0u;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok || *abort_flag) { *abort_flag = 1; dead = true; break; }
            }
            if (lp == 0) {
                // The four weights a code can mean, (q - 1) d, as a byte table for prmt: lut_lo / lut_hi hold the low /
                // high bytes of {-d, 0, d, 2d}; a selector nibble pair (q, q + 4) then assembles one f16.
                const __half d = rvalid ? *reinterpret_cast<const __half *>(rrow + blk * BB + 64) : __float2half(0.0f);
                const uint32_t p01 = (uint32_t)__half_as_ushort(__hneg(d));
                const uint32_t p23 = (uint32_t)__half_as_ushort(d) | ((uint32_t)__half_as_ushort(__hadd(d, d)) << 16);
                lut_lo = __byte_perm(p01, p23, 0x6420);
                lut_hi = __byte_perm(p01, p23, 0x7531);
                // 16 code bytes, 2-byte aligned: five aligned words, funnel-shifted into place
                const uint32_t ca = smem_u32(rrow + blk * BB + 32 * h + 16 * bq), sh = (ca & 3u) * 8u, wa = ca & ~3u;
                const uint32_t w0 = lds32(wa), w1 = lds32(wa + 4), w2 = lds32(wa + 8), w3 = lds32(wa + 12), w4 = sh ? lds32(wa + 16) : 0u;
                cw[0] = __funnelshift_r(w0, w1, sh);
                cw[1] = __funnelshift_r(w1, w2, sh);
                cw[2] = __funnelshift_r(w2, w3, sh);
                cw[3] = __funnelshift_r(w3, w4, sh);
            }
            // element k = 128 h + 32 l + j of the block is bit pair l of code byte 32 h + j; this stage holds
            // l = 2 lp, 2 lp + 1; chunk 4 (l & 1) + 2 bq + {0, 1} of the row takes bytes j = 16 bq + {0..7, 8..15}
            const uint32_t dst = dst0 + (uint32_t)(s * A_STAGE);
#pragma unroll
            for (int li = 0; li < 2; li++) {
                const int l = 2 * lp + li;
                uint32_t v[8];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint32_t sel = ((cw[q] >> (2 * l)) & 0x03030303u) * 0x11u + 0x40404040u;
                    v[2 * q] = __byte_perm(lut_lo, lut_hi, sel);
                    v[2 * q + 1] = __byte_perm(lut_lo, lut_hi, sel >> 16);
                }
                const uint32_t c0 = (uint32_t)(4 * li + 2 * bq);
                const uint32_t da = dst + (((c0 ^ swz) << 4)), db = dst + ((((c0 + 1) ^ swz) << 4));
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(da), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(db), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&a_full[s]));
        }
    } else if (warp < NDQ + NLOAD) {
        // =========================== activation loaders (two warps) ===========================
        // Stage t holds x[0..64, k0 + 64 t .. + 63]: 64 rows of 128 bytes, chunks swizzled as above.  Every stage of the
        // CTA has its own slot and all are requested at once; loader w takes the steps i with i % 2 == w, each lane
        // copies 16 pieces of 16 bytes per stage.  The loaders report once, when everything has landed.
        const int lw = warp - NDQ;
        lc_pdl_wait();   // the activations are the predecessor's output
        const __half *xk = p.x + (size_t)kbs * 256;
        for (int i = lw; i < total_tiles; i += NLOAD) {
            const int t = tile_of(i);
            const uint32_t base = smem_u32(b_s) + (uint32_t)(i * B_STAGE);
#pragma unroll
            for (int e = 0; e < 16; e++) {
                const int pc = lane + 32 * e, rowb = pc >> 3, c = pc & 7;   // 8 consecutive lanes: 128 contiguous bytes of a row
                const bool ok = rowb < p.m;
                cp_async16(base + (uint32_t)(rowb * ROW_BYTES + ((c ^ (rowb & 7)) << 4)),
                           ok ? (const void *)(xk + (size_t)rowb * p.K + t * KT + c * 8) : (const void *)p.x, ok ? 16u : 0u);
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(b_all));
    } else {
        // =========================== MMA issue (four warps, one thread each) ===========================
        // Issuer iw owns TMEM accumulator iw (columns 64 iw ..).  One accumulator tile per CTA: issuer iw takes K = 16
        // step iw of every stage.  Two (GeGLU): issuers 0, 1 take steps {0, 1}, {2, 3} of the gate tile, issuers 2, 3
        // the same of the up tile.
        const int iw = warp - NDQ - NLOAD;
        const int mt = MT == 2 ? (iw >> 1) : 0, k_first = MT == 2 ? 2 * (iw & 1) : iw, k_count = MT == 2 ? 2 : 1;
        // One thread per issuer runs the loop: every instruction in it (barrier test, MMA, commit) costs its thread on
        // the order of a hundred cycles or more, so nothing warp-wide is added.
        if (lane == 0) {
            const uint64_t adesc0 = make_desc(smem_u32(a_s) + (uint32_t)(mt * A_TILE + k_first * 32));
            const uint64_t bdesc0 = make_desc(smem_u32(b_s) + (uint32_t)(k_first * 32));
            const uint32_t tmem_acc = tmem_base + (uint32_t)(iw * NB);
            bool dead = !mbar_wait(smem_u32(b_all), 0u, p.wait_limit);   // all activations of this CTA have landed
            for (int i = 0; i < total_tiles && !dead; i++) {
                if (!mbar_wait(smem_u32(&a_full[i % SA]), (uint32_t)((i / SA) & 1), p.wait_limit) || *abort_flag) { dead = true; break; }
                tc_fence_after();
                uint64_t ad = adesc0 + (uint64_t)((uint32_t)((i % SA) * A_STAGE) >> 4);
                uint64_t bd = bdesc0 + (uint64_t)((uint32_t)(i * B_STAGE) >> 4);
#pragma unroll
                for (int j = 0; j < k_count; j++) {
                    umma_f16(tmem_acc, ad, bd, idesc, (i > 0 || j > 0) ? 1u : 0u);
                    ad += (uint64_t)(32 >> 4);   // the next K = 16 step: 32 bytes along the row
                    bd += (uint64_t)(32 >> 4);
                }
                umma_commit(smem_u32(&mma_done[i % NBAR]));
            }
            // drain: the last stage's barrier completes when all four issuers' MMAs are done
            if (!dead && total_tiles > 0) {
                const int last = total_tiles - 1;
                dead = !mbar_wait(smem_u32(&mma_done[last % NBAR]), (uint32_t)((last / NBAR) & 1), p.wait_limit);
            }
            if (dead) *abort_flag = 1;
        }
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const bool failed = *abort_flag != 0;

    // ---- results.  Dequantizing warp w reads TMEM lanes 32 (w & 3) .. + 31 (one weight row per thread) and CW batch
    //      columns starting at CW (w >> 2), of every accumulator ----
    constexpr int CW = NB / (NDQ / 4);                      // 32 (one accumulator) or 16 (two)
    float *red = reinterpret_cast<float *>(a_s);            // [MT][NB cols][128 rows] f32 (split K only)
    __half *out = p.out[grp];
    if (warp < NDQ) {
        const int lrow = 32 * (warp & 3) + lane, c0 = CW * (warp >> 2);
#pragma unroll
        for (int cc = 0; cc < CW; cc += 16) {
            // the four partial accumulators, added in a fixed order: (0 + 1) + (2 + 3) for one tile; gate = 0 + 1 and
            // up = 2 + 3 for two
            float v[MT][16];
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int j = 0; j < 16; j++) v[mt][j] = 0.f;
            if (!failed && total_tiles > 0) {
                const uint32_t ta = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(c0 + cc);
                uint32_t a0[16], a1[16];
                tmem_ld16(ta, a0);
                tmem_ld16(ta + NB, a1);
#pragma unroll
                for (int j = 0; j < 16; j++) v[0][j] = __uint_as_float(a0[j]) + __uint_as_float(a1[j]);
                tmem_ld16(ta + 2 * NB, a0);
                tmem_ld16(ta + 3 * NB, a1);
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const float hi = __uint_as_float(a0[j]) + __uint_as_float(a1[j]);
                    if (MT == 2) v[MT - 1][j] = hi; else v[0][j] += hi;
                }
            }
            if (p.ks > 1) {
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int j = 0; j < 16; j++) red[(mt * NB + c0 + cc + j) * TILE_ROWS + lrow] = v[mt][j];
            } else if (n0 + lrow < n_rows && !failed) {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int col = c0 + cc + j;
                    float r = v[0][j];
                    if (MT == 2) r = geglu_f(r, v[MT - 1][j]);
                    if (col < p.m) out[(size_t)col * n_rows + n0 + lrow] = __float2half_rn(r);
                }
            }
        }
    }
    if (p.ks > 1) {
        // The ks CTAs of this tile are one cluster.  An item is four consecutive rows of one batch column; CTA `rank`
        // finishes the items [rank, rank + 1) * per: adds the ks partials in split order and stores.  Consecutive
        // threads take consecutive items: consecutive 16-byte pieces of the peers' shared memory, consecutive rows out.
        cluster_sync();
        const int rank = (int)blockIdx.z;
        const uint32_t red_a = smem_u32(red);
        auto gather = [&](int mt, int col, int r4) {
            const uint32_t la = red_a + (uint32_t)(((mt * NB + col) * TILE_ROWS + r4) * 4);
            float4 v[MAX_KS];
#pragma unroll
            for (int sp = 0; sp < MAX_KS; sp++) v[sp] = sp < p.ks ? ld_dsmem_f4(la, (uint32_t)sp) : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int sp = 0; sp < MAX_KS; sp++) {
                acc.x += v[sp].x; acc.y += v[sp].y; acc.z += v[sp].z; acc.w += v[sp].w;
            }
            return acc;
        };
        const int items = p.m * (TILE_ROWS / 4), per = (items + p.ks - 1) / p.ks;
        const int it_end = min(items, (rank + 1) * per);
        if (!failed) {
            for (int it = rank * per + tid; it < it_end; it += NT) {
                const int col = it / (TILE_ROWS / 4), r4 = (it - col * (TILE_ROWS / 4)) * 4;
                float4 a = gather(0, col, r4);
                if (MT == 2) {
                    const float4 u = gather(MT - 1, col, r4);
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
    if (failed && tid == 0) atomicExch(p.status, LC_DEV_STATUS_WAIT_EXPIRED_TCD);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

template <int MT>
int launch_tcd(lc_batch *b, const TcdParams &p, int tiles, size_t smem) {
    auto kern = qgemm_tcd_kernel<MT>;
    static lc_smem_optin optin;
    LC_CUDA_TRY(lc_ensure_smem(kern, optin, b->ctx, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, 1, p.ks);
    cfg.blockDim = dim3((8 * MT + NLOAD + NISS) * 32);
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
    LC_LAUNCH_CHECKED(cudaLaunchKernelEx(&cfg, kern, p));
    b->dispatch_count++;
    return LC_OK;
}

}  // namespace

// Grouped launch: `ng` TQ2_0 weight matrices [ns[g], kk] sharing the activations `input` [m, kk], 8 < m <= 64, f16 out;
// with `geglu`, two matrices of the same shape and one output gelu_tanh(x Wg^T) * (x Wu^T).  Returns LC_OK after a
// launch, a positive status on error, or -1 when the shape is outside what this kernel covers.
int lc_qgemm_tcd_launch(lc_kernels *k, lc_batch *b, const lc_buf *input, int ng, const lc_buf *const *weights,
                        lc_buf *const *outputs, const uint32_t *ns, uint32_t m, uint32_t kk, bool geglu) {
    if (m <= 8 || m > NB || ng < 1 || ng > MAX_GROUPS || kk % 256 != 0 || !lc_aligned(input->dptr, 16)) return -1;
    if (geglu && (ng != 2 || ns[0] != ns[1])) return -1;
    TcdParams p;
    p.x = (const __half *)input->dptr;
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
        if (g < ng && !(geglu && g > 0)) tiles += ((int)ns[g] + TILE_ROWS - 1) / TILE_ROWS;
        p.tile_end[g] = tiles;
    }
    if (tiles < 1) return -1;
    const int mt = geglu ? 2 : 1, rows = TILE_ROWS * mt;
    // One wave: split K over a cluster of at most 8 CTAs while the CTA count stays within about 7/8 of the SM count
    // (a cluster needs all its SMs in one GPC, so the last few SMs cannot always be used; a launch that does not fit
    // runs a second wave and takes twice as long), and no CTA takes more than MAX_TILES stages (three blocks per row).
    static const int ks_cap = []() { const char *e = getenv("LOCAL_CUDA_TCD_KS"); const int v = e ? atoi(e) : 0; return v > 0 ? v : MAX_KS; }();
    int ks = (k->ctx->sm_count * 7 / 8) / tiles;
    if (ks > ks_cap) ks = ks_cap;
    if (ks > MAX_KS) ks = MAX_KS;
    if (ks > p.nb) ks = p.nb;
    if (ks < 1) ks = 1;
    int bps = (p.nb + ks - 1) / ks;
    if (bps > MAX_TILES / 4) bps = MAX_TILES / 4;
    ks = (p.nb + bps - 1) / bps;
    if (ks > MAX_KS) return -1;   // K too long for one cluster of this kernel
    p.ks = ks;
    p.bps = bps;
    p.raw_rs = ((bps * BB + 15 + 15) / 16) * 16;
    if ((p.raw_rs / 16) % 2 == 0) p.raw_rs += 16;
    p.status = k->dev_status;
    p.wait_limit = WAIT_LIMIT;
    // shared memory: all activation stages of the CTA when they fit, then as many weight stages as the rest holds
    const int total = 4 * bps;
    const size_t fixed = (size_t)rows * p.raw_rs + (2 + MAX_TILES + NBAR) * 8 + 16 + 1024;   // + 1024: tile alignment slack
    const size_t budget = k->ctx->smem_optin > 8192 ? k->ctx->smem_optin - 4096 : 0;
    const size_t a_stage = (size_t)mt * A_TILE;
    const int sb = total;
    if (fixed + (size_t)sb * B_STAGE + 2 * a_stage > budget) return -1;
    int sa = (int)((budget - fixed - (size_t)sb * B_STAGE) / a_stage);
    if (sa > total) sa = total;
    if (ks > 1 && (size_t)sa * a_stage < (size_t)mt * NB * TILE_ROWS * 4) return -1;   // the split-K exchange reuses the weight stages
    p.sa = sa;
    p.sb = sb;
    const size_t smem = fixed + (size_t)sb * B_STAGE + (size_t)sa * a_stage;
    return geglu ? launch_tcd<2>(b, p, tiles, smem) : launch_tcd<1>(b, p, tiles, smem);
}
