// Internal definitions shared by the translation units of liblocal_cuda.so.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <atomic>
#include <string>
#include <vector>

#include "../../include/local_cuda.h"

struct lc_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 0;
    size_t smem_optin = 0;
    size_t l2_bytes = 0;
    size_t total_mem = 0;
    bool pdl = true;  // launch kernels with programmatic stream serialization (LOCAL_CUDA_PDL=0 disables)
};

struct lc_buf {
    lc_ctx *ctx = nullptr;
    void *dptr = nullptr;
    size_t bytes = 0;
    bool owned = false;
};

struct lc_batch {
    lc_ctx *ctx = nullptr;
    cudaStream_t stream = nullptr;
    uint32_t dispatch_count = 0;
    bool capturing = false;
};

struct lc_pending {
    lc_ctx *ctx = nullptr;
    cudaEvent_t ev = nullptr;
};

struct lc_graph {
    lc_ctx *ctx = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

struct lc_kernels {
    lc_ctx *ctx = nullptr;
    // Routing switches, read once like the reference's OnceLock-cached env flags.
    bool batchm = true;  // LOCAL_AI_BATCHM: register-resident small-M path
    bool smallm = true;  // LOCAL_AI_SMALLM
    bool mma = true;     // LOCAL_AI_MMA: tensor-core path for larger M
    bool decode_tc = true;   // LOCAL_CUDA_DECODE_TC: lean tcgen05 kernel for TQ2_0 at small_m < M <= 64
    uint32_t small_m = 0;    // LOCAL_CUDA_SMALL_M (0..8): TQ2_0 matmuls of up to this many rows keep the CUDA-core kernel
    bool vocab_tc = true;    // LOCAL_CUDA_VOCAB_TC: persistent tcgen05 kernel for very tall Q4_0 matrices, f32 out, M <= 64
    bool decode_mma = true;  // LOCAL_CUDA_DECODE_MMA: register-direct mma.sync path for 8 < M <= 64 (0: tcgen05 there too)
    int kv_norm_mode = 0;  // LOCAL_CUDA_TQ_NORM: 0 sequential (Rust codec order), 1 tree (Metal order)
    // Library-owned scratch for split-K partials (grown outside graph capture).
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    unsigned int *counters = nullptr;  // per-(lane,head) arrival counters, zero between launches
    size_t counters_len = 0;
    std::vector<void *> retired;  // outgrown scratch / counter blocks: graphs recorded earlier still point at them
    int *dev_status = nullptr;  // device-side error word (bounded waits report here)
    // LOCAL_CUDA_TEST_WAIT_EXPIRY=1 (read at creation): the tcgen05 matmul's barrier waits use a short limit and wait for
    // an arrival that never comes, so the expiry path (status word, early exit, TMEM release) can be exercised on purpose.
    bool test_wait_expiry = false;
};

// Values of the device-side status word (lc_kernels::dev_status).
constexpr int LC_DEV_STATUS_WAIT_EXPIRED = 1;      // a bounded barrier wait ran out (large-tile tcgen05 matmul)
constexpr int LC_DEV_STATUS_WAIT_EXPIRED_TCD = 2;  // the same in the decode tcgen05 matmul
constexpr int LC_DEV_STATUS_POSITION = 3;          // a device-resident position pointed past its lane's pool rows

// Record a failure for lc_last_error() and return `code`.
int lc_fail(int code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
void lc_clear_error();

#define LC_CUDA_TRY(expr)                                                              \
    do {                                                                               \
        cudaError_t _e = (expr);                                                       \
        if (_e != cudaSuccess)                                                         \
            return lc_fail(LC_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e));      \
    } while (0)

#define LC_REQUIRE(cond, ...)                                          \
    do {                                                               \
        if (!(cond)) return lc_fail(LC_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

#define LC_LAUNCH_CHECKED(expr)                                                        \
    do {                                                                               \
        cudaError_t _le = (expr);                                                      \
        if (_le != cudaSuccess)                                                        \
            return lc_fail(LC_ERR_CUDA, "launch: %s", cudaGetErrorString(_le));         \
    } while (0)

// After a kernel launch: surface launch-configuration errors as a status.
#define LC_CHECK_LAUNCH(name)                                                          \
    do {                                                                               \
        cudaError_t _e = cudaGetLastError();                                           \
        if (_e != cudaSuccess)                                                         \
            return lc_fail(LC_ERR_CUDA, "launch %s: %s", name, cudaGetErrorString(_e)); \
    } while (0)

// Every kernel of this library is launched through lc_launch so that it can start while its
// predecessor on the stream is still draining (programmatic dependent launch): a kernel calls
// lc_pdl_trigger() at its top — its successors may then be scheduled — and lc_pdl_wait() before it
// first touches memory a predecessor may have written.  Work that does not depend on the predecessor
// (streaming constant weights towards the SM) goes before the wait.
template <typename... KArgs, typename... Args>
static inline cudaError_t lc_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, lc_batch *b,
                                    Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = b->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = b->ctx->pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#ifdef __CUDACC__
__device__ __forceinline__ void lc_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void lc_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Walsh-Hadamard transform (unnormalised) over d = 32 .. 512 elements held one per thread of a d-thread block;
// returns the thread's element of the result.  Butterflies run in ascending stride, lower = a + b, upper = a - b.
// The strides below 32 pair lanes of one warp and run as shuffles.  For the strides from 32 up every thread
// publishes its value once in `sh` and rebuilds the butterflies its result depends on from the d / 32 values it
// needs: the same additions on the same operands as stage-by-stage passes through shared memory, hence bit-identical
// to them, with one barrier in all instead of two per stage.  No thread may still be reading `sh` from earlier code
// when the block enters (callers that used it since their last barrier place one), and callers that reuse `sh`
// afterwards synchronise first.
template <int P>
__device__ __forceinline__ float lc_fwht_cross_warp(float v, float *sh, unsigned t) {
    sh[t] = v;
    __syncthreads();
    float a[P];
#pragma unroll
    for (int j = 0; j < P; j++) a[j] = sh[t ^ ((unsigned)j << 5)];
#pragma unroll
    for (int s = 0; (1 << s) < P; s++) {
        const bool upper = t & (32u << s);
#pragma unroll
        for (int j = 0; j < P; j += 2 << s) {
            const float self_v = a[j], other_v = a[j | (1 << s)];
            a[j] = upper ? __fsub_rn(other_v, self_v) : __fadd_rn(self_v, other_v);
        }
    }
    return a[0];
}
__device__ __forceinline__ float lc_fwht_value(float v, float *sh, unsigned d, unsigned t) {
#pragma unroll
    for (unsigned len = 1; len < 32; len <<= 1) {
        const float other_v = __shfl_xor_sync(0xffffffffu, v, len);
        v = (t & len) ? __fsub_rn(other_v, v) : __fadd_rn(v, other_v);
    }
    switch (d) {
        case 64: return lc_fwht_cross_warp<2>(v, sh, t);
        case 128: return lc_fwht_cross_warp<4>(v, sh, t);
        case 256: return lc_fwht_cross_warp<8>(v, sh, t);
        case 512: return lc_fwht_cross_warp<16>(v, sh, t);
        default: return v;   // d == 32
    }
}
#endif

// The opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of a kernel.  One
// lc_smem_optin (a function-local static at each launch site, i.e. one per kernel instantiation) remembers
// the largest size already granted on each device, so every device a context is created on gets its own call.
constexpr int LC_MAX_DEVICES = 64;
struct lc_smem_optin {
    std::atomic<size_t> granted[LC_MAX_DEVICES];
};
template <typename Kern>
static inline cudaError_t lc_ensure_smem(Kern kern, lc_smem_optin &state, const lc_ctx *ctx, size_t smem) {
    if (smem <= 48 * 1024) return cudaSuccess;
    const int dev = ctx->device;
    if (dev >= 0 && dev < LC_MAX_DEVICES && state.granted[dev].load(std::memory_order_relaxed) >= smem) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess && dev >= 0 && dev < LC_MAX_DEVICES) state.granted[dev].store(smem, std::memory_order_relaxed);
    return e;
}

static inline bool lc_aligned(const void *p, size_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

// Grow the kernels object's split-K scratch (no-op when large enough). Fails
// during graph capture if growth would be needed.
int lc_reserve_scratch(lc_kernels *k, lc_batch *b, size_t bytes, size_t counters);

// Run `body(batch)` on a fresh batch and wait: the shape of the reference's
// ctx-taking dispatchers (e.g. kernels.rs:5711-5742).
template <typename F>
static inline int lc_run_and_wait(lc_ctx *ctx, F body) {
    lc_batch *b = nullptr;
    int st = lc_batch_begin(ctx, &b);
    if (st != LC_OK) return st;
    st = body(b);
    int st2 = lc_batch_commit_and_wait(b);
    return st != LC_OK ? st : st2;
}
