// Streaming tensor-core matvec / small-batch matmul (m <= 8) over GGUF Q4_0 / TQ2_0 rows:
//   out[m, n] = X[m, K] (f16) x W[n, K]^T.
// Stands in for matvec_q4_0 / matvec_tq2_0 (+ f32out) and the batchm / smallm kernels of
// shaders/matvec_quant.metal (:64-312, :590-916) when the matrix is large enough for bandwidth to matter.
//
// A batch-1 matvec is HBM-bound in principle, but on CUDA cores the dequantisation costs 5-6 instructions per
// weight and binds long before HBM does.  Here the multiply-adds run on mma.sync (the 1..8 batch rows take the
// MMA's N = 8), which leaves about two integer instructions per four weights:
//   * a persistent CTA streams groups of 64 consecutive weight rows -- one contiguous byte range, so every
//     cp.async is a fully coalesced 16-byte piece and DRAM sees sequential reads -- through a three-slot ring;
//   * the activations (8 rows x K) stay in shared memory for the whole launch;
//   * warp (rg, kq) of 16 owns rows 16 rg .. + 15 of the group and quarter kq of K; its threads turn 2-byte pieces
//     of code bytes into A fragments in registers (thread t of a quad owns bytes 2t, 2t+1 of every 8-byte group);
//   * the four K quarters are added through shared memory once per group and stored.
// Numerics keep the exact-weight semantic of the CUDA-core kernels: TQ2_0 weights (q - 1) d are exact in f16;
// for Q4_0 the A operand holds the integers q - 8, every 32-k block is accumulated on its own and scaled by d in
// f32.  Accumulation is f32.
#include "lc_internal.h"

namespace {

constexpr int FMT_Q4_0 = 0;
constexpr int FMT_TQ2_0 = 1;
constexpr int NW = 16, NT = NW * 32;
constexpr int GROUP_ROWS = 64;       // rows per ring slot: 4 row groups of 16
constexpr int SLOTS = 3;
constexpr int UNIT_K = 128;          // K is split over the four warp quarters in units of 128 k

constexpr int MAX_MATRICES = 96;     // matrices of one shape streamed by one launch (lc_matvec_*_group_into)

struct StreamParams {
    const uint8_t *w[MAX_MATRICES];   // n_mat matrices of n rows each, all read against the same activations
    void *out[MAX_MATRICES];
    const __half *x;
    int n, m, K, nb;        // nb = blocks per row
    int gpm;                // 64-row groups per matrix: ceil(n / 64)
    int groups;             // n_mat * gpm
    int xs;                 // bytes per activation row in shared memory
    int slot_bytes;         // bytes reserved per ring slot
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes = 16u) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t b0, const uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t &b0, uint32_t &b1, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];\n" : "=r"(b0), "=r"(b1) : "r"(addr));
}
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ void store_c(__half *p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void store_c(float *p, float v) { *p = v; }
__device__ __forceinline__ uint32_t lds_u16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }

template <int FMT> struct Fmt;
template <> struct Fmt<FMT_Q4_0> { static constexpr int bytes = 18; };
template <> struct Fmt<FMT_TQ2_0> { static constexpr int bytes = 66; };

// UPQ > 0: the warp's K quarter is UPQ units long and its activation fragments (8 k-steps x 2 registers per unit)
// stay in registers for the whole launch; UPQ = 0: any length, fragments re-read from shared memory with ldmatrix.
// MULTI: several matrices (group index -> matrix and group of it); otherwise the one matrix p.w[0].
template <int FMT, typename OutT, int UPQ, bool MULTI>
__global__ void __launch_bounds__(NT, 1) qgemv_mma_stream_kernel(const __grid_constant__ StreamParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int BB = Fmt<FMT>::bytes;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int rg = warp & 3, kq = warp >> 2;
    lc_pdl_trigger();
    const size_t rb = (size_t)p.nb * BB, w_bytes = rb * (size_t)p.n;
    uint8_t *x_s = smem;                                              // [8][xs]
    float4 *red = reinterpret_cast<float4 *>(smem + 8 * p.xs);        // [2][NW][32]
    uint8_t *ring = smem + 8 * p.xs + 2 * NW * 32 * 16;               // [SLOTS][slot_bytes]
    const int my_groups = (p.groups - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

    // group `it` of this CTA: group (blockIdx.x + it gridDim.x) of the launch = rows 64 gi .. of matrix mi; one
    // contiguous byte range
    auto load_group = [&](int it) {
        const int gl = (int)blockIdx.x + it * (int)gridDim.x, mi = MULTI ? gl / p.gpm : 0, grp = gl - mi * p.gpm;
        const uint8_t *wm = p.w[mi];
        const size_t start = (size_t)grp * GROUP_ROWS * rb;
        const size_t len = (size_t)min(GROUP_ROWS, p.n - grp * GROUP_ROWS) * rb;
        const size_t a0 = start & ~(size_t)15;
        const int n16 = (int)((start - a0 + len + 15) >> 4);
        uint8_t *slot = ring + (size_t)(it % SLOTS) * p.slot_bytes;
        for (int i = tid; i < n16; i += NT) {
            const size_t ga = a0 + ((size_t)i << 4);
            if (ga + 16 <= w_bytes) {
                cp_async16(smem_u32(slot + ((size_t)i << 4)), wm + ga);
            } else {
                for (int b = 0; b < 16; b++) slot[((size_t)i << 4) + b] = (ga + b < w_bytes) ? wm[ga + b] : 0;
            }
        }
    };
    // the weights of the first two groups do not depend on the previous kernel
    if (my_groups > 0) load_group(0);
    if (my_groups > 1) load_group(1);
    lc_pdl_wait();
    for (int i = tid; i < 8 * (p.K / 8); i += NT) {
        const int r = i / (p.K / 8), pc = i - r * (p.K / 8);
        const bool ok = r < p.m;
        cp_async16(smem_u32(x_s + r * p.xs + pc * 16), ok ? (const void *)(p.x + (size_t)r * p.K + pc * 8) : (const void *)p.x,
                   ok ? 16u : 0u);
    }
    cp_async_commit();      // group 0: weights of groups 0 and 1 + the activations
    cp_async_commit();      // group 1: empty (keeps the wait arithmetic uniform)

    // this warp's quarter of K, in units of 128 k
    const int nu = p.K / UNIT_K, upq = (nu + 3) / 4;
    const int u0 = kq * upq, u1 = min(nu, u0 + upq);
    // ldmatrix.x2 lane address: lanes 0-7 rows of the first k half, lanes 8-15 the second
    const uint32_t xl = smem_u32(x_s) + (uint32_t)((lane & 7) * p.xs + ((lane >> 3) & 1) * 16);
    uint32_t breg[UPQ > 0 ? UPQ * 8 : 1][2];
    if (UPQ > 0) {
        cp_async_wait<1>();
        __syncthreads();          // the activations have landed
#pragma unroll
        for (int uu = 0; uu < (UPQ > 0 ? UPQ : 1); uu++)
#pragma unroll
            for (int s8 = 0; s8 < 8; s8++) {
                breg[uu * 8 + s8][0] = breg[uu * 8 + s8][1] = 0u;
                if (u0 + uu < u1) ldmatrix_x2(breg[uu * 8 + s8][0], breg[uu * 8 + s8][1], xl + (uint32_t)(((u0 + uu) * UNIT_K + 16 * s8) * 2));
            }
    }

    auto reduce_store = [&](int it) {      // warps kq == 0: add the four quarters of group `it` and store
        const int gl = (int)blockIdx.x + it * (int)gridDim.x, mi = MULTI ? gl / p.gpm : 0, grp = gl - mi * p.gpm;
        OutT *out = reinterpret_cast<OutT *>(p.out[mi]);
        const float4 *rp = red + (size_t)(it & 1) * NW * 32;
        float4 v = rp[(0 * 4 + rg) * 32 + lane];
#pragma unroll
        for (int q = 1; q < 4; q++) {
            const float4 o = rp[(q * 4 + rg) * 32 + lane];
            v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
        }
        const float e4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int row = grp * GROUP_ROWS + rg * 16 + g + 8 * (e >> 1), col = 2 * t + (e & 1);
            if (row < p.n && col < p.m) store_c(out + (size_t)col * p.n + row, e4[e]);
        }
    };

    for (int it = 0; it < my_groups; it++) {
        cp_async_wait<1>();
        __syncthreads();          // group `it` has landed everywhere; everyone is done with group it - 1
        if (it + 2 < my_groups) load_group(it + 2);
        cp_async_commit();
        if (it > 0 && kq == 0) reduce_store(it - 1);

        const int gl = (int)blockIdx.x + it * (int)gridDim.x, grp = MULTI ? gl % p.gpm : gl;
        const size_t start = (size_t)grp * GROUP_ROWS * rb;
        const uint8_t *slot = ring + (size_t)(it % SLOTS) * p.slot_bytes + (start & 15);
        const uint8_t *rbase[2];
        bool rvalid[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int r = rg * 16 + g + 8 * i;
            rbase[i] = slot + (size_t)r * rb;
            rvalid[i] = grp * GROUP_ROWS + r < p.n;
        }
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        if (FMT == FMT_TQ2_0) {
            // unit u = half h of block b: element 128 h + 32 l + j of the block is bit pair l of code byte 32 h + j
#pragma unroll
            for (int uu = 0; uu < (UPQ > 0 ? UPQ : 64); uu++) {
                const int u = u0 + uu;
                if (u >= u1) break;
                const int b = u >> 1, h = u & 1;
                uint32_t lut_lo[2], lut_hi[2], wq[2][2];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const uint8_t *bp = rbase[i] + b * BB;
                    const __half d = rvalid[i] ? *reinterpret_cast<const __half *>(bp + 64) : __float2half(0.0f);
                    const uint32_t p01 = (uint32_t)__half_as_ushort(__hneg(d));                       // {-d, 0}
                    const uint32_t p23 = (uint32_t)__half_as_ushort(d) | ((uint32_t)__half_as_ushort(__hadd(d, d)) << 16);
                    lut_lo[i] = __byte_perm(p01, p23, 0x6420);
                    lut_hi[i] = __byte_perm(p01, p23, 0x7531);
                    const uint8_t *hp = bp + h * 32 + 2 * t;
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
                            a[i] = __byte_perm(lut_lo[i], lut_hi[i], sel);
                            a[i + 2] = __byte_perm(lut_lo[i], lut_hi[i], sel >> 16);
                        }
                        uint32_t b0, b1;
                        if (UPQ > 0) {
                            b0 = breg[uu * 8 + 2 * l + qp][0];
                            b1 = breg[uu * 8 + 2 * l + qp][1];
                        } else {
                            ldmatrix_x2(b0, b1, xl + (uint32_t)((u * UNIT_K + 32 * l + 16 * qp) * 2));
                        }
                        mma16816(c, a, b0, b1);
                    }
                }
            }
        } else {
            // unit u = blocks 4u .. 4u+3; block: f16 scale, then byte i holds k = i (low nibble) and i + 16 (high)
            const __half2 c1032 = __float2half2_rn(1032.0f);
#pragma unroll
            for (int uu = 0; uu < (UPQ > 0 ? UPQ : 64); uu++) {
                const int u = u0 + uu;
                if (u >= u1) break;
#pragma unroll
                for (int bi = 0; bi < 4; bi++) {
                    const int b = 4 * u + bi;
                    float df[2];
                    uint32_t wq[2];
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const uint8_t *bp = rbase[i] + b * BB;
                        df[i] = rvalid[i] ? __half2float(*reinterpret_cast<const __half *>(bp)) : 0.f;
                        wq[i] = lds_u16(bp + 2 + 2 * t) | (lds_u16(bp + 10 + 2 * t) << 16);
                    }
                    float cb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int part = 0; part < 2; part++) {
                        uint32_t a[4];
#pragma unroll
                        for (int i = 0; i < 2; i++) {
                            const uint32_t codes = (wq[i] >> (4 * part)) & 0x0F0F0F0Fu;
                            a[i] = h2_bits(__hsub2(bits_h2(__byte_perm(codes, 0x64u, 0x4140)), c1032));
                            a[i + 2] = h2_bits(__hsub2(bits_h2(__byte_perm(codes, 0x64u, 0x4342)), c1032));
                        }
                        uint32_t b0, b1;
                        if (UPQ > 0) {
                            b0 = breg[uu * 8 + 2 * bi + part][0];
                            b1 = breg[uu * 8 + 2 * bi + part][1];
                        } else {
                            ldmatrix_x2(b0, b1, xl + (uint32_t)((b * 32 + 16 * part) * 2));
                        }
                        mma16816(cb, a, b0, b1);
                    }
                    c[0] = fmaf(df[0], cb[0], c[0]);
                    c[1] = fmaf(df[0], cb[1], c[1]);
                    c[2] = fmaf(df[1], cb[2], c[2]);
                    c[3] = fmaf(df[1], cb[3], c[3]);
                }
            }
        }
        red[((size_t)(it & 1) * NW + kq * 4 + rg) * 32 + lane] = make_float4(c[0], c[1], c[2], c[3]);
    }
    cp_async_wait<0>();
    __syncthreads();
    if (my_groups > 0 && kq == 0) reduce_store(my_groups - 1);
}

template <int FMT, typename OutT, int UPQ, bool MULTI>
int launch_stream_um(lc_kernels *k, lc_batch *b, const StreamParams &p, size_t smem) {
    auto kern = qgemv_mma_stream_kernel<FMT, OutT, UPQ, MULTI>;
    static lc_smem_optin optin;
    LC_CUDA_TRY(lc_ensure_smem(kern, optin, b->ctx, smem));
    const int grid = p.groups < k->ctx->sm_count ? p.groups : k->ctx->sm_count;
    LC_LAUNCH_CHECKED(lc_launch(kern, dim3(grid), dim3(NT), smem, b, p));
    b->dispatch_count++;
    return LC_OK;
}
template <int FMT, typename OutT, int UPQ>
int launch_stream_u(lc_kernels *k, lc_batch *b, const StreamParams &p, size_t smem) {
    return p.groups > p.gpm ? launch_stream_um<FMT, OutT, UPQ, true>(k, b, p, smem)
                            : launch_stream_um<FMT, OutT, UPQ, false>(k, b, p, smem);
}

template <int FMT, typename OutT>
int launch_stream(lc_kernels *k, lc_batch *b, const StreamParams &p, size_t smem) {
    const int upq = (p.K / UNIT_K + 3) / 4;
    switch (upq) {
        case 1: return launch_stream_u<FMT, OutT, 1>(k, b, p, smem);
        case 2: return launch_stream_u<FMT, OutT, 2>(k, b, p, smem);
        case 3: return launch_stream_u<FMT, OutT, 3>(k, b, p, smem);
        default: return launch_stream_u<FMT, OutT, 0>(k, b, p, smem);
    }
}

}  // namespace

// m <= 8; `count` matrices of one shape [n, kk] against the same activations, each with its own output.  Returns
// LC_OK after a launch, a positive status on error, or -1 when the shape is outside what this kernel covers or too
// small for it to pay (the caller then uses the CUDA-core kernel).
int lc_qgemv_mma_stream_group(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input, int count,
                              const lc_buf *const *weights, lc_buf *const *outputs, uint32_t m, uint32_t kk, uint32_t n) {
    const int be = fmt == FMT_Q4_0 ? 32 : 256, bb = fmt == FMT_Q4_0 ? 18 : 66;
    if (count < 1 || count > MAX_MATRICES || m > 8 || kk % UNIT_K != 0 || kk % be != 0 || !lc_aligned(input->dptr, 16)) return -1;
    StreamParams p;
    for (int i = 0; i < MAX_MATRICES; i++) {
        const int j = i < count ? i : count - 1;
        if (!lc_aligned(weights[j]->dptr, 16)) return -1;
        p.w[i] = (const uint8_t *)weights[j]->dptr;
        p.out[i] = outputs[j]->dptr;
    }
    p.x = (const __half *)input->dptr;
    p.n = (int)n;
    p.m = (int)m;
    p.K = (int)kk;
    p.nb = (int)(kk / be);
    p.gpm = (int)((n + GROUP_ROWS - 1) / GROUP_ROWS);
    p.groups = p.gpm * count;
    p.xs = (int)kk * 2 + 16;
    const size_t rb = (size_t)p.nb * bb;
    p.slot_bytes = (int)(((size_t)GROUP_ROWS * rb + 15 + 15) / 16 * 16 + 16);
    const size_t smem = (size_t)8 * p.xs + 2 * NW * 32 * 16 + (size_t)SLOTS * p.slot_bytes;
    if (smem > k->ctx->smem_optin) return -1;
    // worth it only when every SM gets a few groups to stream
    if (p.groups < 2 * k->ctx->sm_count) return -1;
    if (fmt == FMT_Q4_0)
        return f32out ? launch_stream<FMT_Q4_0, float>(k, b, p, smem) : launch_stream<FMT_Q4_0, __half>(k, b, p, smem);
    return f32out ? launch_stream<FMT_TQ2_0, float>(k, b, p, smem) : launch_stream<FMT_TQ2_0, __half>(k, b, p, smem);
}

int lc_qgemv_mma_stream(int fmt, bool f32out, lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                        lc_buf *output, uint32_t m, uint32_t kk, uint32_t n) {
    const lc_buf *ws[1] = {weight};
    lc_buf *os[1] = {output};
    return lc_qgemv_mma_stream_group(fmt, f32out, k, b, input, 1, ws, os, m, kk, n);
}
