// Multi-GPU pieces of the row-split vocabulary projection (one process per GPU):
//   * NCCL behind the C ABI.  libnccl is loaded at run time (dlopen), so the library carries no link-time dependency
//     and a host without NCCL gets LC_ERR_NCCL from these entry points instead of a load failure.  The unique id is
//     created on one rank and carried to the others by the host (any channel: a file, a socket, an existing
//     process group);
//   * per-shard greedy argmax as (max, global index) pairs and their merge with the first-maximum rule of
//     local-engine/src/sampler.rs:148-158 (strict '>' in index order: the lowest index wins ties, NaN never wins),
//     so that a row-split projection needs 8 bytes per lane from every rank instead of its whole logit slice.
#include <dlfcn.h>
#include <math.h>

#include <mutex>

#include "lc_internal.h"

namespace {

// The part of NCCL's public C API this file calls (nccl.h): opaque communicator, 128-byte unique id, result 0 = success.
struct nccl_unique_id { char internal[LC_COMM_ID_BYTES]; };
typedef void *nccl_comm_t;
constexpr int NCCL_UINT8 = 1;   // ncclUint8
typedef int (*get_unique_id_fn)(nccl_unique_id *);
typedef int (*comm_init_rank_fn)(nccl_comm_t *, int, nccl_unique_id, int);
typedef int (*comm_destroy_fn)(nccl_comm_t);
typedef int (*all_gather_fn)(const void *, void *, size_t, int, nccl_comm_t, cudaStream_t);
typedef const char *(*get_error_string_fn)(int);

struct nccl_api {
    void *handle = nullptr;
    get_unique_id_fn get_unique_id = nullptr;
    comm_init_rank_fn comm_init_rank = nullptr;
    comm_destroy_fn comm_destroy = nullptr;
    all_gather_fn all_gather = nullptr;
    get_error_string_fn error_string = nullptr;
    char why[256] = {0};
};

// Loads libnccl once: LOCAL_CUDA_NCCL_LIB if set, else the loader's libnccl.so.2 (already mapped in a process that
// imported a framework bundling it), else libnccl.so.
const nccl_api *nccl() {
    static nccl_api api;
    static std::once_flag once;
    std::call_once(once, []() {
        const char *names[3] = {getenv("LOCAL_CUDA_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
        for (const char *n : names) {
            if (!n || !n[0]) continue;
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
            snprintf(api.why, sizeof api.why, "%s", dlerror());
        }
        if (!api.handle) return;
        api.get_unique_id = (get_unique_id_fn)dlsym(api.handle, "ncclGetUniqueId");
        api.comm_init_rank = (comm_init_rank_fn)dlsym(api.handle, "ncclCommInitRank");
        api.comm_destroy = (comm_destroy_fn)dlsym(api.handle, "ncclCommDestroy");
        api.all_gather = (all_gather_fn)dlsym(api.handle, "ncclAllGather");
        api.error_string = (get_error_string_fn)dlsym(api.handle, "ncclGetErrorString");
        if (!api.get_unique_id || !api.comm_init_rank || !api.comm_destroy || !api.all_gather) {
            snprintf(api.why, sizeof api.why, "libnccl lacks an expected symbol");
            api.handle = nullptr;
        }
    });
    return &api;
}

int nccl_fail(const nccl_api *a, const char *what, int rc) {
    return lc_fail(LC_ERR_NCCL, "%s: %s", what, a->error_string ? a->error_string(rc) : "NCCL error");
}

// (max, first index) of one row; index reported with `offset` added.  An all -inf / NaN row reports (-inf, offset).
__global__ void argmax_pairs_kernel(const float *__restrict__ v, float2 *__restrict__ pairs, unsigned cols, unsigned offset) {
    lc_pdl_trigger();
    lc_pdl_wait();
    __shared__ float bv_s[32];
    __shared__ unsigned bi_s[32];
    const float *row = v + (size_t)blockIdx.x * cols;
    float bv = -INFINITY;
    unsigned bi = 0xffffffffu;
    for (unsigned i = threadIdx.x; i < cols; i += blockDim.x) {
        const float x = __ldcs(row + i);
        if (x > bv) { bv = x; bi = i; }
    }
    auto better = [](float a, unsigned ai, float b, unsigned bi2) { return a > b || (a == b && ai < bi2); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const unsigned oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { bv_s[warp] = bv; bi_s[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = lane < nw ? bv_s[lane] : -INFINITY;
        bi = lane < nw ? bi_s[lane] : 0xffffffffu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const unsigned oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) pairs[blockIdx.x] = make_float2(bv, __uint_as_float(offset + (bi == 0xffffffffu ? 0u : bi)));
    }
}

// pairs_all[s][r], shards in index order: the first maximum over shards (strict '>': an earlier shard keeps ties).
__global__ void merge_argmax_pairs_kernel(const float2 *__restrict__ pairs_all, uint32_t *__restrict__ out, unsigned rows,
                                          unsigned shards) {
    lc_pdl_trigger();
    lc_pdl_wait();
    const unsigned r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float bv = -INFINITY;
    unsigned bi = __float_as_uint(pairs_all[r].y);   // an all -inf / NaN row keeps the first shard's first index
    for (unsigned s = 0; s < shards; s++) {
        const float2 c = pairs_all[(size_t)s * rows + r];
        if (c.x > bv) { bv = c.x; bi = __float_as_uint(c.y); }
    }
    out[r] = bi;
}

}  // namespace

struct lc_comm {
    lc_ctx *ctx = nullptr;
    nccl_comm_t comm = nullptr;
    uint32_t rank = 0, world = 1;
};

extern "C" {

int lc_comm_available(void) {
    const nccl_api *a = nccl();
    if (!a->handle) return lc_fail(LC_ERR_NCCL, "NCCL is not loadable: %s", a->why[0] ? a->why : "no libnccl found");
    return LC_OK;
}

int lc_comm_unique_id(uint8_t *id) {
    if (!id) return lc_fail(LC_ERR_INVALID_ARGUMENT, "comm_unique_id: NULL argument");
    const nccl_api *a = nccl();
    if (!a->handle) return lc_comm_available();
    nccl_unique_id u;
    const int rc = a->get_unique_id(&u);
    if (rc != 0) return nccl_fail(a, "ncclGetUniqueId", rc);
    memcpy(id, u.internal, LC_COMM_ID_BYTES);
    return LC_OK;
}

int lc_comm_create(lc_ctx *ctx, const uint8_t *id, uint32_t rank, uint32_t world, lc_comm **out) {
    if (!ctx || !id || !out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "comm_create: NULL argument");
    LC_REQUIRE(world >= 1 && rank < world, "comm_create: rank %u outside a world of %u", rank, world);
    const nccl_api *a = nccl();
    if (!a->handle) return lc_comm_available();
    LC_CUDA_TRY(cudaSetDevice(ctx->device));
    nccl_unique_id u;
    memcpy(u.internal, id, LC_COMM_ID_BYTES);
    nccl_comm_t c = nullptr;
    const int rc = a->comm_init_rank(&c, (int)world, u, (int)rank);
    if (rc != 0) return nccl_fail(a, "ncclCommInitRank", rc);
    lc_comm *h = new lc_comm;
    h->ctx = ctx;
    h->comm = c;
    h->rank = rank;
    h->world = world;
    *out = h;
    return LC_OK;
}

void lc_comm_destroy(lc_comm *c) {
    if (!c) return;
    const nccl_api *a = nccl();
    if (a->handle && c->comm) a->comm_destroy(c->comm);
    delete c;
}

uint32_t lc_comm_rank(const lc_comm *c) { return c ? c->rank : 0; }
uint32_t lc_comm_world(const lc_comm *c) { return c ? c->world : 0; }

int lc_comm_all_gather_into(lc_batch *b, lc_comm *c, const lc_buf *send, size_t send_offset, lc_buf *recv,
                            size_t bytes_per_rank) {
    if (!b || !c || !send || !recv) return lc_fail(LC_ERR_INVALID_ARGUMENT, "comm_all_gather: NULL argument");
    LC_REQUIRE(send_offset <= send->bytes && send->bytes - send_offset >= bytes_per_rank &&
                   recv->bytes >= bytes_per_rank * (size_t)c->world,
               "comm_all_gather: buffers too small for %zu bytes per rank x %u ranks", bytes_per_rank, c->world);
    if (bytes_per_rank == 0) return LC_OK;
    const nccl_api *a = nccl();
    if (!a->handle) return lc_comm_available();
    const int rc = a->all_gather((const uint8_t *)send->dptr + send_offset, recv->dptr, bytes_per_rank, NCCL_UINT8, c->comm,
                                 b->stream);
    if (rc != 0) return nccl_fail(a, "ncclAllGather", rc);
    b->dispatch_count++;
    return LC_OK;
}

int lc_argmax_pairs_f32_into(lc_kernels *k, lc_batch *b, const lc_buf *values, lc_buf *pairs, uint32_t rows, uint32_t cols,
                             uint32_t index_offset) {
    if (!k || !b || !values || !pairs) return lc_fail(LC_ERR_INVALID_ARGUMENT, "argmax_pairs_f32: NULL argument");
    LC_REQUIRE(cols >= 1, "argmax_pairs_f32: cols must be >= 1");
    LC_REQUIRE(values->bytes >= (size_t)rows * cols * 4 && pairs->bytes >= (size_t)rows * 8, "argmax_pairs_f32: buffers too small");
    LC_REQUIRE(lc_aligned(values->dptr, 4) && lc_aligned(pairs->dptr, 8), "argmax_pairs_f32: a buffer is not aligned to its element size");
    if (rows == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(argmax_pairs_kernel, dim3(rows), dim3(1024), 0, b, (const float *)values->dptr,
                                (float2 *)pairs->dptr, cols, index_offset));
    b->dispatch_count++;
    return LC_OK;
}

int lc_merge_argmax_pairs_into(lc_kernels *k, lc_batch *b, const lc_buf *pairs_all, lc_buf *out_index, uint32_t rows,
                               uint32_t shards) {
    if (!k || !b || !pairs_all || !out_index) return lc_fail(LC_ERR_INVALID_ARGUMENT, "merge_argmax_pairs: NULL argument");
    LC_REQUIRE(shards >= 1, "merge_argmax_pairs: shards must be >= 1");
    LC_REQUIRE(pairs_all->bytes >= (size_t)rows * shards * 8 && out_index->bytes >= (size_t)rows * 4,
               "merge_argmax_pairs: buffers too small");
    LC_REQUIRE(lc_aligned(pairs_all->dptr, 8) && lc_aligned(out_index->dptr, 4), "merge_argmax_pairs: a buffer is not aligned to its element size");
    if (rows == 0) return LC_OK;
    LC_LAUNCH_CHECKED(lc_launch(merge_argmax_pairs_kernel, dim3((rows + 127) / 128), dim3(128), 0, b,
                                (const float2 *)pairs_all->dptr, (uint32_t *)out_index->dptr, rows, shards));
    b->dispatch_count++;
    return LC_OK;
}

}  // extern "C"
