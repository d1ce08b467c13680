// Register-direct tensor-core path of the quantized batched matmul for 8 < m <= 64 (decode batches):
//   C[m, n] = A[m, K] (f16) x W[n, K]^T,  W in GGUF TQ2_0 / Q4_0 blocks.
// Stands in, for these m, for the reference's simdgroup-matrix kernels matmul_nt_{q4_0,tq2_0}_mma
// (shaders/matvec_quant.metal:447-577).
//
// At these batch sizes a projection of a decoder layer is a few microseconds of HBM traffic, so what matters
// is the length of the dependent chain inside a launch and how much of it can run before the previous kernel
// has finished.  The kernel therefore has no cross-warp pipeline, no TMEM and no operand staging of weights:
//   * before the dependency wait, every warp copies the raw quantized blocks of its own 16 weight rows (this
//     CTA's K range) into shared memory with 16-byte cp.async (rows are only 2-byte aligned: the enclosing
//     16-byte ranges are copied);
//   * after the wait, the activations [m, K range] stream through two shared-memory buffers of 256 k with
//     cp.async;
//   * each warp walks its rows' blocks: 2-byte pieces of code bytes -> f16 weights in registers, directly in the
//     layout of the m16n8k16 A fragment (thread t of a quad owns bytes 2t, 2t+1 of every 8-byte group, which are
//     the k values 2t, 2t+1 the fragment wants; for TQ2_0 the four values a code can take, (q - 1) d, sit in two
//     registers as a byte table and one prmt assembles two weights), B fragments by ldmatrix, f32 accumulators
//     in registers.
// Weights take the MMA's M dimension, the batch its N dimension.  When K is split (grid.z > 1) the CTAs of a
// tile form a thread-block cluster: each stages its partial tile in its own shared memory and, after a cluster
// barrier, every CTA adds one slice of the tile over all splits in split order through distributed shared
// memory and stores it -- deterministic, with no round trip through global memory.
//
// Numerics: TQ2_0 weights d (q - 1) are exact in f16.  For Q4_0 the MMA operand is the integer q - 8 (exact in
// f16); the two k-steps of a 32-k block accumulate on their own and the block's f32 sum is scaled by d in f32, so
// the weights keep the f32 value d (q - 8) the reference's kernels use (shaders/matvec_quant.metal:25,477-506).
// Accumulation is f32.
#include "lc_internal.h"

namespace {

constexpr int FMT_Q4_0 = 0;
constexpr int FMT_TQ2_0 = 1;
constexpr int NW = 8;              // warps per CTA
constexpr int NT = NW * 32;
constexpr int WROWS = 16;          // weight rows per warp (one MMA tile)
constexpr int CTA_ROWS = NW * WROWS;
constexpr int CHUNK_K = 256;       // k per activation buffer
constexpr int XS = CHUNK_K * 2 + 16;   // bytes per activation row in a buffer (+16: ldmatrix rows spread over banks)
constexpr int MAX_GROUPS = 3;
constexpr int MAX_KS = 8;          // portable cluster size

struct MmaParams {
    const uint8_t *w[MAX_GROUPS];
    void *out[MAX_GROUPS];
    int n[MAX_GROUPS], tile_end[MAX_GROUPS];
    int ngroups;
    const __half *x;
    int m, K, nb;          // nb = blocks per weight row
    int ks, bps;           // split-K: grid.z = cluster size = ks, bps = blocks per split
    int raw_rs;            // bytes reserved per row of raw blocks
    int geglu;             // 1: w[0] = gate, w[1] = up, out[0] = gelu(gate) * up (see lc_qgemm_mma_geglu)
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes = 16u) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
// d = a . b (no accumulator input: the zero operand needs no registers)
__device__ __forceinline__ void mma16816_zero(float (&d)[4], const uint32_t (&a)[4], const uint32_t b0, const uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t b0, const uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
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
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ void store_c(__half *p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void store_c(float *p, float v) { *p = v; }
__device__ __forceinline__ uint32_t lds_u16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }
__device__ __forceinline__ uint32_t lds_u16s(uint32_t addr) {   // by shared-memory address
    uint16_t v;
    asm("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

template <int FMT> struct Fmt;
template <> struct Fmt<FMT_Q4_0> { static constexpr int bytes = 18, elems = 32, chunk_blocks = CHUNK_K / 32; };
template <> struct Fmt<FMT_TQ2_0> { static constexpr int bytes = 66, elems = 256, chunk_blocks = 1; };

// NBT: 8-row batch tiles (m <= 8 NBT).
template <int FMT, int NBT, typename OutT>
__global__ void __launch_bounds__(NT) qgemm_mma_kernel(const MmaParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int BB = Fmt<FMT>::bytes, BE = Fmt<FMT>::elems, CHB = Fmt<FMT>::chunk_blocks;
    constexpr int XBUF = 8 * NBT * XS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    lc_pdl_trigger();
    int grp = 0;
    while (grp + 1 < p.ngroups && (int)blockIdx.x >= p.tile_end[grp]) grp++;
    // GeGLU mode: a CTA owns 64 rows of the gate matrix (warps 0-3) and the same 64 rows of the up matrix (warps 4-7)
    if (p.geglu) grp = warp >> 2;
    const int n0 = p.geglu ? (int)blockIdx.x * (CTA_ROWS / 2) - (warp >> 2) * (CTA_ROWS / 2)
                           : ((int)blockIdx.x - (grp ? p.tile_end[grp - 1] : 0)) * CTA_ROWS;
    const int n_rows = p.n[grp];
    const uint8_t *wmat = p.w[grp];
    const size_t rb = (size_t)p.nb * BB, w_bytes = rb * (size_t)n_rows;
    const int kbs = (int)blockIdx.z * p.bps, kbe = min(p.nb, kbs + p.bps), nblk = max(kbe - kbs, 0);
    const int seg = nblk * BB;
    uint8_t *x_s = smem;                                   // [2][8 NBT][XS]; reused for the split-K exchange
    uint8_t *raw = smem + 2 * XBUF;                        // [128][raw_rs]

    // ---- 1. this warp's raw weight rows -> shared memory (does not depend on the previous kernel) ----
    for (int rr = 0; rr < WROWS && nblk > 0; rr++) {
        const int r = warp * WROWS + rr, row = n0 + r;
        if (row >= n_rows) break;
        const size_t g0 = (size_t)row * rb + (size_t)kbs * BB, a0 = g0 & ~(size_t)15;
        const int npieces = (int)((g0 + seg - a0 + 15) >> 4);
        for (int pc = lane; pc < npieces; pc += 32) {
            const size_t ga = a0 + ((size_t)pc << 4);
            uint8_t *dst = raw + r * p.raw_rs + (pc << 4);
            if (ga + 16 <= w_bytes) {
                cp_async16(smem_u32(dst), wmat + ga);
            } else {
                for (int b = 0; b < 16; b++) dst[b] = (ga + b < w_bytes) ? wmat[ga + b] : 0;
            }
        }
    }
    cp_async_commit();
    lc_pdl_wait();

    // ---- 2. activation chunks: [8 NBT rows][256 k] per buffer, 16-byte pieces, rows beyond m zero-filled ----
    const int nchunks = (nblk + CHB - 1) / CHB;
    auto load_chunk = [&](int ch) {
        const int cb0 = ch * CHB, cblk = min(CHB, nblk - cb0);
        const int ppr = cblk * BE / 8;                      // 16-byte pieces per row
        const __half *src0 = p.x + (size_t)(kbs + cb0) * BE;
        uint8_t *buf = x_s + (ch & 1) * XBUF;
        for (int it = tid; it < 8 * NBT * ppr; it += NT) {
            const int r = it / ppr, pc = it - r * ppr;
            const bool ok = r < p.m;
            cp_async16(smem_u32(buf + r * XS + pc * 16), ok ? (const void *)(src0 + (size_t)r * p.K + pc * 8) : (const void *)p.x,
                       ok ? 16u : 0u);
        }
    };
    if (nchunks > 0) load_chunk(0);
    cp_async_commit();
    if (nchunks > 1) load_chunk(1);
    cp_async_commit();

    // ---- 3. main loop: 16 weight rows x (8 NBT) batch rows per warp ----
    float c[NBT][4];
#pragma unroll
    for (int j = 0; j < NBT; j++) c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f;
    // the two rows this thread dequantizes: warp rows g and g + 8
    const uint8_t *rbase[2];
    bool rvalid[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = warp * WROWS + g + 8 * i, row = n0 + r;
        const size_t g0 = (size_t)row * rb + (size_t)kbs * BB;
        rbase[i] = raw + r * p.raw_rs + (int)(g0 & 15);
        rvalid[i] = row < n_rows;
    }
    // ldmatrix lane address: matrix mi = lane >> 3 is (batch tile j + (mi >> 1), k half mi & 1 of the 16-k step)
    const uint32_t xl = (uint32_t)((8 * (lane >> 4) + (lane & 7)) * XS + ((lane >> 3) & 1) * 16);

    for (int ch = 0; ch < nchunks; ch++) {
        cp_async_wait<1>();          // chunk ch (and the raw rows) have landed for this thread
        __syncthreads();             // ... and for every thread
        const uint32_t xb = smem_u32(x_s + (ch & 1) * XBUF) + xl;
        const int cb0 = ch * CHB, cblk = min(CHB, nblk - cb0);
        if (FMT == FMT_TQ2_0) {
            // one block: element 128 h + 32 l + j of the block is bit pair l of code byte 32 h + j
            // The four weights a code can mean, (q - 1) d, as a byte table for prmt: lut_lo / lut_hi hold the low /
            // high bytes of {-d, 0, d, 2d}; a selector nibble pair (q, q + 4) then assembles one f16.
            uint32_t lut_lo[2], lut_hi[2];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const __half d = rvalid[i] ? *reinterpret_cast<const __half *>(rbase[i] + cb0 * BB + 64) : __float2half(0.0f);
                const uint32_t p01 = (uint32_t)__half_as_ushort(__hneg(d));                       // {-d, 0}
                const uint32_t p23 = (uint32_t)__half_as_ushort(d) | ((uint32_t)__half_as_ushort(__hadd(d, d)) << 16);
                lut_lo[i] = __byte_perm(p01, p23, 0x6420);
                lut_hi[i] = __byte_perm(p01, p23, 0x7531);
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                // pieces: bytes 8 q + 2 t, + 1 of the half (q = 0..3), packed two per word
                uint32_t wq[2][2];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const uint8_t *hp = rbase[i] + cb0 * BB + h * 32 + 2 * t;
                    wq[i][0] = lds_u16(hp) | (lds_u16(hp + 8) << 16);
                    wq[i][1] = lds_u16(hp + 16) | (lds_u16(hp + 24) << 16);
                }
#pragma unroll
                for (int l = 0; l < 4; l++) {
#pragma unroll
                    for (int qp = 0; qp < 2; qp++) {
                        uint32_t a[4];
#pragma unroll
                        for (int i = 0; i < 2; i++) {
                            const uint32_t sel = ((wq[i][qp] >> (2 * l)) & 0x03030303u) * 0x11u + 0x40404040u;
                            a[i] = __byte_perm(lut_lo[i], lut_hi[i], sel);            // k-fragment 2t, 2t+1
                            a[i + 2] = __byte_perm(lut_lo[i], lut_hi[i], sel >> 16);  // k-fragment 2t+8, 2t+9
                        }
                        const uint32_t xk = xb + (uint32_t)((128 * h + 32 * l + 16 * qp) * 2);
#pragma unroll
                        for (int j = 0; j < NBT; j += 2) {
                            uint32_t b[4];
                            ldmatrix_x4(b, xk + (uint32_t)(8 * j * XS));
                            mma16816(c[j], a, b[0], b[1]);
                            mma16816(c[j + 1], a, b[2], b[3]);
                        }
                    }
                }
            }
        } else {
            // up to 8 blocks of 32 k: f16 scale, then byte i holds k = i (low nibble) and k = i + 16 (high nibble).
            // The operand is the integer q - 8; each block's sum is scaled by d in f32 (exact f32 weights).
            const __half2 c1032 = __float2half2_rn(1032.0f);
            for (int bi = 0; bi < cblk; bi++) {
                float df[2];
                uint32_t a[2][4];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const uint8_t *bp = rbase[i] + (cb0 + bi) * BB;
                    df[i] = rvalid[i] ? __half2float(*reinterpret_cast<const __half *>(bp)) : 0.0f;
                    const uint32_t wq = lds_u16(bp + 2 + 2 * t) | (lds_u16(bp + 10 + 2 * t) << 16);
#pragma unroll
                    for (int part = 0; part < 2; part++) {
                        const uint32_t codes = (wq >> (4 * part)) & 0x0F0F0F0Fu;
                        a[part][i] = h2_bits(__hsub2(bits_h2(__byte_perm(codes, 0x64u, 0x4140)), c1032));
                        a[part][i + 2] = h2_bits(__hsub2(bits_h2(__byte_perm(codes, 0x64u, 0x4342)), c1032));
                    }
                }
                const uint32_t xk = xb + (uint32_t)(32 * bi * 2);
#pragma unroll
                for (int j = 0; j < NBT; j += 2) {
                    float t0[4] = {0.f, 0.f, 0.f, 0.f}, t1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int part = 0; part < 2; part++) {
                        uint32_t b[4];
                        ldmatrix_x4(b, xk + (uint32_t)(16 * part * 2 + 8 * j * XS));
                        mma16816(t0, a[part], b[0], b[1]);
                        mma16816(t1, a[part], b[2], b[3]);
                    }
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        c[j][e] = fmaf(df[e >> 1], t0[e], c[j][e]);
                        c[j + 1][e] = fmaf(df[e >> 1], t1[e], c[j + 1][e]);
                    }
                }
            }
        }
        __syncthreads();             // every warp is done with buffer ch & 1
        if (ch + 2 < nchunks) load_chunk(ch + 2);
        cp_async_commit();
    }

    // ---- 4. results.  c[j][e]: weight row 16 warp + g + 8 (e >> 1), batch row 8 j + 2 t + (e & 1) ----
    OutT *out = reinterpret_cast<OutT *>(p.out[p.geglu ? 0 : grp]);
    auto store_tile = [&](const float4 v, int w, int ln, int j) {
        const float e4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int row = n0 + w * WROWS + (ln >> 2) + 8 * (e >> 1), col = 8 * j + 2 * (ln & 3) + (e & 1);
            if (row < n_rows && col < p.m) store_c(out + (size_t)col * n_rows + row, e4[e]);
        }
    };
    // GeGLU: gate and up are rounded to f16 as the separate projections would store them, then
    // gelu_tanh(gate) * up exactly as the element-wise kernel computes it (gelu.metal, layer.rs:825-838)
    auto geglu = [](float gate, float up) {
        const float x = __half2float(__float2half_rn(gate)), u = __half2float(__float2half_rn(up));
        float inner = 0.7978845608f * (x + 0.044715f * (x * x * x));
        inner = fminf(fmaxf(inner, -10.0f), 10.0f);
        return 0.5f * x * (1.0f + tanhf(inner)) * u;
    };
    auto store_geglu = [&](const float4 gt, const float4 up, int w, int ln, int j) {   // w = 0..3: gate warp
        const int row0 = (int)blockIdx.x * (CTA_ROWS / 2) + w * WROWS + (ln >> 2), col0 = 8 * j + 2 * (ln & 3);
        const float g4[4] = {gt.x, gt.y, gt.z, gt.w}, u4[4] = {up.x, up.y, up.z, up.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int row = row0 + 8 * (e >> 1), col = col0 + (e & 1);
            if (row < n_rows && col < p.m) store_c(out + (size_t)col * n_rows + row, geglu(g4[e], u4[e]));
        }
    };
    float4 *red = reinterpret_cast<float4 *>(x_s);           // [NBT][NT]
    if (p.ks == 1) {
        if (!p.geglu) {
#pragma unroll
            for (int j = 0; j < NBT; j++) store_tile(make_float4(c[j][0], c[j][1], c[j][2], c[j][3]), warp, lane, j);
            return;
        }
        cp_async_wait<0>();
        if (warp >= 4) {
#pragma unroll
            for (int j = 0; j < NBT; j++) red[j * NT + tid] = make_float4(c[j][0], c[j][1], c[j][2], c[j][3]);
        }
        __syncthreads();
        if (warp < 4) {
#pragma unroll
            for (int j = 0; j < NBT; j++)
                store_geglu(make_float4(c[j][0], c[j][1], c[j][2], c[j][3]), red[j * NT + tid + 128], warp, lane, j);
        }
        return;
    }
    // Split K: the ks CTAs of this tile are one cluster.  Partial tiles are exchanged through shared memory.
    cp_async_wait<0>();
#pragma unroll
    for (int j = 0; j < NBT; j++) red[j * NT + tid] = make_float4(c[j][0], c[j][1], c[j][2], c[j][3]);
    cluster_sync();
    // items (j, source warp) are dealt round-robin to the CTAs of the cluster; a warp adds the ks partials of an
    // item in split order and stores it
    const int rank = (int)blockIdx.z;
    auto gather = [&](int j, int w) {
        const uint32_t la = smem_u32(red + j * NT + w * 32 + lane);
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
    if (!p.geglu) {
        for (int item = rank + p.ks * warp; item < NBT * NW; item += p.ks * NW) {
            const int j = item / NW, w = item - j * NW;
            store_tile(gather(j, w), w, lane, j);
        }
    } else {
        for (int item = rank + p.ks * warp; item < NBT * 4; item += p.ks * NW) {
            const int j = item / 4, w = item - j * 4;
            const float4 gt = gather(j, w), up = gather(j, w + 4);
            store_geglu(gt, up, w, lane, j);
        }
    }
    cluster_sync();   // no CTA leaves while a peer may still read its shared memory
}

template <int FMT, int NBT, typename OutT>
int launch_mma(lc_batch *b, const MmaParams &p, dim3 grid, size_t smem) {
    auto kern = qgemm_mma_kernel<FMT, NBT, OutT>;
    static lc_smem_optin optin;
    LC_CUDA_TRY(lc_ensure_smem(kern, optin, b->ctx, smem));
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

template <int FMT, typename OutT>
int launch_mma_nbt(lc_batch *b, const MmaParams &p, dim3 grid, size_t smem, int nbt) {
    switch (nbt) {
        case 2: return launch_mma<FMT, 2, OutT>(b, p, grid, smem);
        case 4: return launch_mma<FMT, 4, OutT>(b, p, grid, smem);
        default: return launch_mma<FMT, 8, OutT>(b, p, grid, smem);
    }
}


// ---- wide matrices (the vocabulary projection): Q4_0, 32 < m <= 64, no K split -------------------------------------
// With 128-row tiles every CTA streams the whole activation matrix from L2 once per tile, which for a 262144-row
// table is 2048 x 196 KB.  Here a CTA owns 512 rows (16 warps x 32 rows), so the activations are read a quarter as
// often, is persistent over tiles, and streams raw weights and activations together in 128-k chunks through a
// three-stage cp.async ring (one __syncthreads per chunk).
constexpr int W_NW = 16, W_NT = W_NW * 32, W_ROWS = W_NW * 32;
constexpr int W_CK = 128;                        // k per chunk: 4 Q4_0 blocks
constexpr int W_RAW_RS = 112;                    // 72 bytes of blocks + up to 15 of skew, odd multiple of 16
constexpr int W_XS = W_CK * 2 + 16;
constexpr int W_STAGE = W_ROWS * W_RAW_RS + 64 * W_XS;
constexpr int W_STAGES = 3;

struct WideParams {
    const uint8_t *w;
    void *out;
    const __half *x;
    int n, m, K, nb, tiles;
};

template <typename OutT, int NBT>
__global__ void __launch_bounds__(W_NT, 1) qgemm_mma_wide_kernel(const WideParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int BB = 18;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    lc_pdl_trigger();
    const size_t rb = (size_t)p.nb * BB, w_bytes = rb * (size_t)p.n;
    const int nchunks = p.K / W_CK;
    const int my_tiles = ((int)p.tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total = my_tiles * nchunks;

    // chunk `it` of this CTA's sequence: tile blockIdx.x + (it / nchunks) gridDim.x, k chunk it % nchunks
    auto load_raw = [&](int it) {
        const int tile = (int)blockIdx.x + (it / nchunks) * (int)gridDim.x, ch = it % nchunks;
        uint8_t *st = smem + (it % W_STAGES) * W_STAGE;
        const int row = tile * W_ROWS + tid;        // one row per thread
        if (row < p.n) {
            const size_t g0 = (size_t)row * rb + (size_t)ch * 4 * BB, a0 = g0 & ~(size_t)15;
            const int npieces = (int)((g0 + 4 * BB - a0 + 15) >> 4);
            for (int pc = 0; pc < npieces; pc++) {
                const size_t ga = a0 + ((size_t)pc << 4);
                uint8_t *dst = st + tid * W_RAW_RS + (pc << 4);
                if (ga + 16 <= w_bytes) {
                    cp_async16(smem_u32(dst), p.w + ga);
                } else {
                    for (int b = 0; b < 16; b++) dst[b] = (ga + b < w_bytes) ? p.w[ga + b] : 0;
                }
            }
        }
    };
    auto load_x = [&](int it) {
        const int ch = it % nchunks;
        uint8_t *xs = smem + (it % W_STAGES) * W_STAGE + W_ROWS * W_RAW_RS;
        for (int i = tid; i < 8 * NBT * (W_CK / 8); i += W_NT) {
            const int r = i / (W_CK / 8), pc = i - r * (W_CK / 8);
            const bool ok = r < p.m;
            cp_async16(smem_u32(xs + r * W_XS + pc * 16),
                       ok ? (const void *)(p.x + (size_t)r * p.K + ch * W_CK + pc * 8) : (const void *)p.x, ok ? 16u : 0u);
        }
    };
    // the weights of the first two chunks do not depend on the previous kernel
    if (total > 0) load_raw(0);
    if (total > 1) load_raw(1);
    lc_pdl_wait();
    if (total > 0) load_x(0);
    cp_async_commit();
    if (total > 1) load_x(1);
    cp_async_commit();

    float c[2][NBT][4];
#pragma unroll
    for (int f = 0; f < 2; f++)
#pragma unroll
        for (int j = 0; j < NBT; j++) c[f][j][0] = c[f][j][1] = c[f][j][2] = c[f][j][3] = 0.f;
    const uint32_t xl = (uint32_t)((8 * (lane >> 4) + (lane & 7)) * W_XS + ((lane >> 3) & 1) * 16);
    const __half2 c1032 = __float2half2_rn(1032.0f);
    OutT *out = reinterpret_cast<OutT *>(p.out);

    for (int it = 0; it < total; it++) {
        cp_async_wait<1>();
        __syncthreads();             // chunk `it` has landed everywhere, and everyone is done with chunk it - 1
        if (it + 2 < total) {
            load_raw(it + 2);
            load_x(it + 2);
        }
        cp_async_commit();
        const int tile = (int)blockIdx.x + (it / nchunks) * (int)gridDim.x, ch = it % nchunks;
        const uint8_t *st = smem + (it % W_STAGES) * W_STAGE;
        const uint32_t xb = smem_u32(st + W_ROWS * W_RAW_RS) + xl;
        uint32_t rbase[4];   // shared-memory addresses
        bool rvalid[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = warp * 32 + g + 8 * i, row = tile * W_ROWS + r;
            const size_t g0 = (size_t)row * rb + (size_t)ch * 4 * BB;
            rbase[i] = smem_u32(st) + (uint32_t)(r * W_RAW_RS + (int)(g0 & 15));
            rvalid[i] = row < p.n;
        }
#pragma unroll
        for (int bi = 0; bi < 4; bi++) {
            // the operand is the integer q - 8; the block's sum is scaled by d in f32 (exact f32 weights)
            float df[4];
            uint32_t a[2][2][4];   // [k half of the block][fragment][register]
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t bp = rbase[i] + (uint32_t)(bi * BB);
                df[i] = rvalid[i] ? __half2float(__ushort_as_half((unsigned short)lds_u16s(bp))) : 0.0f;
                const uint32_t wq = lds_u16s(bp + 2 + 2 * t) | (lds_u16s(bp + 10 + 2 * t) << 16);
#pragma unroll
                for (int part = 0; part < 2; part++) {
                    const uint32_t codes = (wq >> (4 * part)) & 0x0F0F0F0Fu;
                    a[part][i >> 1][i & 1] = h2_bits(__hsub2(bits_h2(__byte_perm(codes, 0x64u, 0x4140)), c1032));
                    a[part][i >> 1][(i & 1) + 2] = h2_bits(__hsub2(bits_h2(__byte_perm(codes, 0x64u, 0x4342)), c1032));
                }
            }
            const uint32_t xk = xb + (uint32_t)(32 * bi * 2);
#pragma unroll
            for (int j = 0; j + 1 < NBT; j += 2) {
                uint32_t b[2][4];
                ldmatrix_x4(b[0], xk + (uint32_t)(8 * j * W_XS));
                ldmatrix_x4(b[1], xk + (uint32_t)(32 + 8 * j * W_XS));
#pragma unroll
                for (int f = 0; f < 2; f++) {
                    float t0[4], t1[4];
                    mma16816_zero(t0, a[0][f], b[0][0], b[0][1]);
                    mma16816_zero(t1, a[0][f], b[0][2], b[0][3]);
                    mma16816(t0, a[1][f], b[1][0], b[1][1]);
                    mma16816(t1, a[1][f], b[1][2], b[1][3]);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        c[f][j][e] = fmaf(df[2 * f + (e >> 1)], t0[e], c[f][j][e]);
                        c[f][j + 1][e] = fmaf(df[2 * f + (e >> 1)], t1[e], c[f][j + 1][e]);
                    }
                }
            }
        }
        if (ch == nchunks - 1) {
            // c[f][j][e]: weight row 32 warp + 16 f + g + 8 (e >> 1) of the tile, batch row 8 j + 2 t + (e & 1)
#pragma unroll
            for (int f = 0; f < 2; f++)
#pragma unroll
                for (int j = 0; j < NBT; j++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int row = tile * W_ROWS + warp * 32 + 16 * f + g + 8 * (e >> 1), col = 8 * j + 2 * t + (e & 1);
                        if (row < p.n && col < p.m) store_c(out + (size_t)col * p.n + row, c[f][j][e]);
                        c[f][j][e] = 0.f;
                    }
                }
        }
    }
    cp_async_wait<0>();
}

template <typename OutT, int NBT>
int launch_wide(lc_kernels *k, lc_batch *b, const WideParams &p) {
    auto kern = qgemm_mma_wide_kernel<OutT, NBT>;
    const size_t smem = (size_t)W_STAGES * W_STAGE;
    static lc_smem_optin optin;
    LC_CUDA_TRY(lc_ensure_smem(kern, optin, b->ctx, smem));
    const int grid = p.tiles < k->ctx->sm_count ? p.tiles : k->ctx->sm_count;
    LC_LAUNCH_CHECKED(lc_launch(kern, dim3(grid), dim3(W_NT), smem, b, p));
    b->dispatch_count++;
    return LC_OK;
}

}  // namespace

// Grouped launch: `ng` weight matrices [ns[g], kk] sharing the activations `input` [m, kk], 8 < m <= 64.
// Returns LC_OK after a launch, a positive status on error, or -1 when the shape is outside what this kernel
// covers (the caller then uses another path).
static int qgemm_mma_launch(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input, int ng,
                            const lc_buf *const *weights, lc_buf *const *outputs, const uint32_t *ns, uint32_t m,
                            uint32_t kk, bool geglu) {
    const int be = fmt == FMT_Q4_0 ? 32 : 256, bb = fmt == FMT_Q4_0 ? 18 : 66;
    if (m > 64 || ng < 1 || ng > MAX_GROUPS || kk % be != 0 || !lc_aligned(input->dptr, 16)) return -1;
    if (m <= 8) return -1;   // small batches: qmatvec_mma.cu / qmatvec.cu
    MmaParams p;
    p.x = (const __half *)input->dptr;
    p.m = (int)m;
    p.K = (int)kk;
    p.nb = (int)(kk / be);
    p.ngroups = ng;
    int tiles = 0;
    for (int g = 0; g < MAX_GROUPS; g++) {
        const int gi = g < ng ? g : ng - 1;
        p.w[g] = (const uint8_t *)weights[gi]->dptr;
        p.out[g] = outputs[gi]->dptr;
        p.n[g] = (int)ns[gi];
        if (g < ng) tiles += ((int)ns[g] + CTA_ROWS - 1) / CTA_ROWS;
        p.tile_end[g] = tiles;
    }
    if (!geglu && fmt == FMT_Q4_0 && ng == 1 && m > 32 && kk % W_CK == 0 && ns[0] >= (uint32_t)(W_ROWS * k->ctx->sm_count) &&
        (size_t)W_STAGES * W_STAGE <= k->ctx->smem_optin) {
        WideParams wp;
        wp.w = (const uint8_t *)weights[0]->dptr;
        wp.out = outputs[0]->dptr;
        wp.x = (const __half *)input->dptr;
        wp.n = (int)ns[0];
        wp.m = (int)m;
        wp.K = (int)kk;
        wp.nb = (int)(kk / 32);
        wp.tiles = (int)((ns[0] + W_ROWS - 1) / W_ROWS);
        return f32out ? launch_wide<float, 8>(k, b, wp) : launch_wide<__half, 8>(k, b, wp);
    }
    p.geglu = geglu ? 1 : 0;
    if (geglu) tiles = ((int)ns[0] + CTA_ROWS / 2 - 1) / (CTA_ROWS / 2);
    const int nbt = m <= 16 ? 2 : (m <= 32 ? 4 : 8);
    // Split K (at most 8 ways: one cluster per tile) while the grid stays within 1.5 CTAs per SM (measured optimum:
    // more splits cost more in the exchange than they gain in parallelism); whole 256-k chunks per
    // split, and no more raw bytes per CTA than fit beside the activation buffers.
    const int chb = CHUNK_K / be;                       // blocks per 256 k
    const int nchunk = (p.nb + chb - 1) / chb;
    int ks = (3 * k->ctx->sm_count / 2) / tiles;
    if (ks > MAX_KS) ks = MAX_KS;
    if (ks > nchunk) ks = nchunk;
    if (ks < 1) ks = 1;
    int cps = (nchunk + ks - 1) / ks;                   // chunks per split
    ks = (nchunk + cps - 1) / cps;
    p.ks = ks;
    p.bps = cps * chb;
    p.raw_rs = ((p.bps * bb + 15 + 15) / 16) * 16;
    if ((p.raw_rs / 16) % 2 == 0) p.raw_rs += 16;      // odd multiple of 16 bytes: rows spread over the banks
    const size_t smem = (size_t)2 * 8 * nbt * XS + (size_t)CTA_ROWS * p.raw_rs;
    if (smem > k->ctx->smem_optin) return -1;           // K range too long for one CTA's raw rows (tcgen05 path instead)
    dim3 grid(tiles, 1, ks);
    if (fmt == FMT_Q4_0)
        return f32out ? launch_mma_nbt<FMT_Q4_0, float>(b, p, grid, smem, nbt) : launch_mma_nbt<FMT_Q4_0, __half>(b, p, grid, smem, nbt);
    return f32out ? launch_mma_nbt<FMT_TQ2_0, float>(b, p, grid, smem, nbt) : launch_mma_nbt<FMT_TQ2_0, __half>(b, p, grid, smem, nbt);
}

int lc_qgemm_mma_grouped(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input, int ng,
                         const lc_buf *const *weights, lc_buf *const *outputs, const uint32_t *ns, uint32_t m,
                         uint32_t kk) {
    return qgemm_mma_launch(fmt, f32out, k, b, input, ng, weights, outputs, ns, m, kk, false);
}

// out[m, n] = gelu_tanh(x W_gate^T) * (x W_up^T) in one launch (TQ2_0, f16 out), 8 < m <= 64; -1 when not covered.
int lc_qgemm_mma_geglu(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *w_gate, const lc_buf *w_up,
                       lc_buf *output, uint32_t m, uint32_t kk, uint32_t n) {
    const lc_buf *ws[2] = {w_gate, w_up};
    lc_buf *os[2] = {output, output};
    const uint32_t ns[2] = {n, n};
    return qgemm_mma_launch(FMT_TQ2_0, false, k, b, input, 2, ws, os, ns, m, kk, true);
}
