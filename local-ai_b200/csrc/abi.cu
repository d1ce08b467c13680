// Context, buffer, batch and graph objects of the C ABI: the CUDA stand-ins for
// local-metal's MetalContext (context.rs:31-101), MetalBuffer (buffer.rs:17-144),
// CommandBatch / PendingCommandBuffer (batch.rs:120-292) and Error (error.rs:2-32).
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "lc_internal.h"

static thread_local std::string g_last_error;

int lc_fail(int code, const char *fmt, ...) {
    char msg[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof msg, fmt, ap);
    va_end(ap);
    g_last_error = msg;
    return code;
}
void lc_clear_error() { g_last_error.clear(); }

extern "C" {

const char *lc_last_error(void) { return g_last_error.c_str(); }

const char *lc_status_name(int s) {
    switch (s) {
        case LC_OK: return "Ok";
        case LC_ERR_NO_DEVICE: return "NoDevice";
        case LC_ERR_NO_COMMAND_QUEUE: return "NoCommandQueue";
        case LC_ERR_BUFFER_ALLOCATION: return "BufferAllocation";
        case LC_ERR_LIBRARY_CREATION: return "LibraryCreation";
        case LC_ERR_PIPELINE_CREATION: return "PipelineCreation";
        case LC_ERR_SHADER_NOT_FOUND: return "ShaderNotFound";
        case LC_ERR_COMMAND_BUFFER: return "CommandBuffer";
        case LC_ERR_INVALID_ARGUMENT: return "InvalidArgument";
        case LC_ERR_IO: return "Io";
        case LC_ERR_CUDA: return "Cuda";
        case LC_ERR_NCCL: return "Nccl";
        case LC_ERR_TIMEOUT: return "Timeout";
        default: return "Unknown";
    }
}

const char *lc_version(void) { return "local-cuda 0.1 sm_100a"; }

// ---------------------------------------------------------------- context --
int lc_ctx_create(int device, lc_ctx **out) {
    if (!out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_ctx_create: out is NULL");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return lc_fail(LC_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    if (device < 0 || device >= n)
        return lc_fail(LC_ERR_NO_DEVICE, "device %d out of range (have %d)", device, n);
    LC_CUDA_TRY(cudaSetDevice(device));
    lc_ctx *c = new lc_ctx();
    c->device = device;
    e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete c;
        return lc_fail(LC_ERR_NO_COMMAND_QUEUE, "stream: %s", cudaGetErrorString(e));
    }
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device);
    c->sm_count = v;
    cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    c->smem_optin = (size_t)v;
    cudaDeviceGetAttribute(&v, cudaDevAttrL2CacheSize, device);
    c->l2_bytes = (size_t)v;
    size_t fr = 0, tot = 0;
    cudaMemGetInfo(&fr, &tot);
    c->total_mem = tot;
    { const char *e = getenv("LOCAL_CUDA_PDL"); c->pdl = !(e && strcmp(e, "0") == 0); }
    *out = c;
    return LC_OK;
}

void lc_ctx_destroy(lc_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) {
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
    }
    delete ctx;
}

int lc_ctx_caps(const lc_ctx *ctx, int *sm_count, size_t *smem_per_cta, size_t *l2_bytes,
                size_t *total_mem) {
    if (!ctx) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_ctx_caps: ctx is NULL");
    if (sm_count) *sm_count = ctx->sm_count;
    if (smem_per_cta) *smem_per_cta = ctx->smem_optin;
    if (l2_bytes) *l2_bytes = ctx->l2_bytes;
    if (total_mem) *total_mem = ctx->total_mem;
    return LC_OK;
}

void *lc_ctx_stream(const lc_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

int lc_ctx_synchronize(lc_ctx *ctx) {
    if (!ctx) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_ctx_synchronize: ctx is NULL");
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return lc_fail(LC_ERR_COMMAND_BUFFER, "%s", cudaGetErrorString(e));
    return LC_OK;
}

// ----------------------------------------------------------------- buffer --
int lc_buf_alloc(lc_ctx *ctx, size_t bytes, lc_buf **out) {
    if (!ctx || !out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_buf_alloc: NULL argument");
    *out = nullptr;
    LC_CUDA_TRY(cudaSetDevice(ctx->device));
    void *p = nullptr;
    size_t n = bytes ? bytes : 1;
    cudaError_t e = cudaMalloc(&p, n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return lc_fail(LC_ERR_BUFFER_ALLOCATION, "size=%zu: %s", bytes, cudaGetErrorString(e));
    }
    e = cudaMemsetAsync(p, 0, n, ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(p);
        return lc_fail(LC_ERR_CUDA, "memset: %s", cudaGetErrorString(e));
    }
    lc_buf *b = new lc_buf();
    b->ctx = ctx;
    b->dptr = p;
    b->bytes = bytes;
    b->owned = true;
    *out = b;
    return LC_OK;
}

int lc_buf_from_host(lc_ctx *ctx, const void *src, size_t bytes, lc_buf **out) {
    if (!src && bytes) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_buf_from_host: src is NULL");
    int st = lc_buf_alloc(ctx, bytes, out);
    if (st != LC_OK) return st;
    st = lc_buf_upload(*out, 0, src, bytes);
    if (st != LC_OK) {
        lc_buf_free(*out);
        *out = nullptr;
    }
    return st;
}

int lc_buf_wrap(lc_ctx *ctx, void *device_ptr, size_t bytes, lc_buf **out) {
    if (!ctx || !out || (!device_ptr && bytes))
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_buf_wrap: NULL argument");
    lc_buf *b = new lc_buf();
    b->ctx = ctx;
    b->dptr = device_ptr;
    b->bytes = bytes;
    b->owned = false;
    *out = b;
    return LC_OK;
}

void lc_buf_free(lc_buf *buf) {
    if (!buf) return;
    if (buf->owned && buf->dptr) {
        cudaSetDevice(buf->ctx->device);
        cudaStreamSynchronize(buf->ctx->stream);
        cudaFree(buf->dptr);
    }
    delete buf;
}

size_t lc_buf_length(const lc_buf *buf) { return buf ? buf->bytes : 0; }
void *lc_buf_device_ptr(const lc_buf *buf) { return buf ? buf->dptr : nullptr; }

static int range_ok(const lc_buf *buf, size_t off, size_t n, const char *what) {
    if (!buf) return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: buffer is NULL", what);
    if (off > buf->bytes || n > buf->bytes - off)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "%s: range [%zu, +%zu) outside buffer of %zu bytes",
                       what, off, n, buf->bytes);
    return LC_OK;
}

int lc_buf_upload(lc_buf *buf, size_t offset, const void *src, size_t bytes) {
    int st = range_ok(buf, offset, bytes, "lc_buf_upload");
    if (st != LC_OK) return st;
    if (!bytes) return LC_OK;
    if (!src) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_buf_upload: src is NULL");
    cudaStream_t s = buf->ctx->stream;
    LC_CUDA_TRY(cudaMemcpyAsync((char *)buf->dptr + offset, src, bytes, cudaMemcpyHostToDevice, s));
    LC_CUDA_TRY(cudaStreamSynchronize(s));
    return LC_OK;
}

int lc_buf_download(const lc_buf *buf, size_t offset, void *dst, size_t bytes) {
    int st = range_ok(buf, offset, bytes, "lc_buf_download");
    if (st != LC_OK) return st;
    if (!bytes) return LC_OK;
    if (!dst) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_buf_download: dst is NULL");
    cudaStream_t s = buf->ctx->stream;
    LC_CUDA_TRY(cudaMemcpyAsync(dst, (const char *)buf->dptr + offset, bytes, cudaMemcpyDeviceToHost, s));
    LC_CUDA_TRY(cudaStreamSynchronize(s));
    return LC_OK;
}

int lc_buf_zero(lc_buf *buf, size_t offset, size_t bytes) {
    int st = range_ok(buf, offset, bytes, "lc_buf_zero");
    if (st != LC_OK) return st;
    if (!bytes) return LC_OK;
    LC_CUDA_TRY(cudaMemsetAsync((char *)buf->dptr + offset, 0, bytes, buf->ctx->stream));
    return LC_OK;
}

int lc_buf_fill(lc_buf *buf, size_t offset, size_t bytes, int value) {
    int st = range_ok(buf, offset, bytes, "lc_buf_fill");
    if (st != LC_OK) return st;
    if (!bytes) return LC_OK;
    LC_CUDA_TRY(cudaMemsetAsync((char *)buf->dptr + offset, value & 0xFF, bytes, buf->ctx->stream));
    return LC_OK;
}

// ------------------------------------------------------------------ batch --
int lc_batch_begin(lc_ctx *ctx, lc_batch **out) {
    if (!ctx || !out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_batch_begin: NULL argument");
    LC_CUDA_TRY(cudaSetDevice(ctx->device));
    lc_batch *b = new lc_batch();
    b->ctx = ctx;
    b->stream = ctx->stream;
    *out = b;
    return LC_OK;
}

uint32_t lc_batch_dispatch_count(const lc_batch *batch) { return batch ? batch->dispatch_count : 0; }

int lc_batch_copy(lc_batch *batch, const lc_buf *src, size_t src_off, lc_buf *dst, size_t dst_off,
                  size_t bytes) {
    if (!batch) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_batch_copy: batch is NULL");
    int st = range_ok(src, src_off, bytes, "lc_batch_copy(src)");
    if (st != LC_OK) return st;
    st = range_ok(dst, dst_off, bytes, "lc_batch_copy(dst)");
    if (st != LC_OK) return st;
    if (!bytes) return LC_OK;
    LC_CUDA_TRY(cudaMemcpyAsync((char *)dst->dptr + dst_off, (const char *)src->dptr + src_off, bytes,
                                cudaMemcpyDeviceToDevice, batch->stream));
    batch->dispatch_count++;
    return LC_OK;
}

int lc_batch_upload(lc_batch *batch, lc_buf *dst, size_t dst_off, const void *src, size_t bytes) {
    if (!batch) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_batch_upload: batch is NULL");
    int st = range_ok(dst, dst_off, bytes, "lc_batch_upload");
    if (st != LC_OK) return st;
    if (!bytes) return LC_OK;
    if (!src) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_batch_upload: src is NULL");
    LC_CUDA_TRY(cudaMemcpyAsync((char *)dst->dptr + dst_off, src, bytes, cudaMemcpyHostToDevice,
                                batch->stream));
    return LC_OK;
}

int lc_batch_download(lc_batch *batch, const lc_buf *src, size_t src_off, void *dst, size_t bytes) {
    if (!batch) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_batch_download: batch is NULL");
    int st = range_ok(src, src_off, bytes, "lc_batch_download");
    if (st != LC_OK) return st;
    if (!bytes) return LC_OK;
    if (!dst) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_batch_download: dst is NULL");
    LC_CUDA_TRY(cudaMemcpyAsync(dst, (const char *)src->dptr + src_off, bytes, cudaMemcpyDeviceToHost,
                                batch->stream));
    return LC_OK;
}

int lc_batch_commit_and_wait(lc_batch *batch) {
    if (!batch) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_batch_commit_and_wait: batch is NULL");
    if (batch->capturing) {
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "batch is capturing: use lc_batch_end_capture");
    }
    cudaError_t e = cudaStreamSynchronize(batch->stream);
    delete batch;
    if (e != cudaSuccess) return lc_fail(LC_ERR_COMMAND_BUFFER, "%s", cudaGetErrorString(e));
    return LC_OK;
}

int lc_batch_commit_async(lc_batch *batch, lc_pending **out) {
    if (!batch || !out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_batch_commit_async: NULL argument");
    if (batch->capturing)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "batch is capturing: use lc_batch_end_capture");
    lc_pending *p = new lc_pending();
    p->ctx = batch->ctx;
    cudaError_t e = cudaEventCreateWithFlags(&p->ev, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventRecord(p->ev, batch->stream);
    delete batch;
    if (e != cudaSuccess) {
        if (p->ev) cudaEventDestroy(p->ev);
        delete p;
        return lc_fail(LC_ERR_COMMAND_BUFFER, "%s", cudaGetErrorString(e));
    }
    *out = p;
    return LC_OK;
}

int lc_pending_wait(lc_pending *pending) {
    if (!pending) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_pending_wait: pending is NULL");
    cudaError_t e = cudaEventSynchronize(pending->ev);
    cudaEventDestroy(pending->ev);
    delete pending;
    if (e != cudaSuccess) return lc_fail(LC_ERR_COMMAND_BUFFER, "%s", cudaGetErrorString(e));
    return LC_OK;
}

int lc_batch_begin_capture(lc_ctx *ctx, lc_batch **out) {
    int st = lc_batch_begin(ctx, out);
    if (st != LC_OK) return st;
    cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) {
        delete *out;
        *out = nullptr;
        return lc_fail(LC_ERR_CUDA, "begin capture: %s", cudaGetErrorString(e));
    }
    (*out)->capturing = true;
    return LC_OK;
}

int lc_batch_end_capture(lc_batch *batch, lc_graph **out) {
    if (!batch || !out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_batch_end_capture: NULL argument");
    if (!batch->capturing) return lc_fail(LC_ERR_INVALID_ARGUMENT, "batch is not capturing");
    lc_ctx *ctx = batch->ctx;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(batch->stream, &g);
    delete batch;
    if (e != cudaSuccess || !g) {
        cudaGetLastError();
        return lc_fail(LC_ERR_CUDA, "end capture: %s", cudaGetErrorString(e));
    }
    cudaGraphExec_t ex = nullptr;
    e = cudaGraphInstantiate(&ex, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        return lc_fail(LC_ERR_CUDA, "graph instantiate: %s", cudaGetErrorString(e));
    }
    lc_graph *gr = new lc_graph();
    gr->ctx = ctx;
    gr->graph = g;
    gr->exec = ex;
    *out = gr;
    return LC_OK;
}

int lc_graph_launch(lc_graph *graph) {
    if (!graph) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_graph_launch: graph is NULL");
    LC_CUDA_TRY(cudaGraphLaunch(graph->exec, graph->ctx->stream));
    return LC_OK;
}

void lc_graph_destroy(lc_graph *graph) {
    if (!graph) return;
    if (graph->exec) cudaGraphExecDestroy(graph->exec);
    if (graph->graph) cudaGraphDestroy(graph->graph);
    delete graph;
}

int lc_host_alloc(size_t bytes, void **out) {
    if (!out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_host_alloc: out is NULL");
    cudaError_t e = cudaMallocHost(out, bytes ? bytes : 1);
    if (e != cudaSuccess) {
        *out = nullptr;
        return lc_fail(LC_ERR_BUFFER_ALLOCATION, "pinned size=%zu: %s", bytes, cudaGetErrorString(e));
    }
    return LC_OK;
}

void lc_host_free(void *ptr) {
    if (ptr) cudaFreeHost(ptr);
}

// ---------------------------------------------------------------- kernels --
static bool env_enabled(const char *name) {
    // Same rule as kernels.rs:6277-6304: only an explicit "0" disables.
    const char *v = getenv(name);
    return !(v && strcmp(v, "0") == 0);
}

int lc_kernels_create(lc_ctx *ctx, lc_kernels **out) {
    if (!ctx || !out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_kernels_create: NULL argument");
    LC_CUDA_TRY(cudaSetDevice(ctx->device));
    lc_kernels *k = new lc_kernels();
    k->ctx = ctx;
    k->batchm = env_enabled("LOCAL_AI_BATCHM");
    k->smallm = env_enabled("LOCAL_AI_SMALLM");
    k->mma = env_enabled("LOCAL_AI_MMA");
    k->decode_mma = env_enabled("LOCAL_CUDA_DECODE_MMA");
    k->decode_tc = env_enabled("LOCAL_CUDA_DECODE_TC");
    k->vocab_tc = env_enabled("LOCAL_CUDA_VOCAB_TC");
    if (const char *e = getenv("LOCAL_CUDA_SMALL_M")) {
        const long v = strtol(e, nullptr, 10);
        if (v >= 0 && v <= 8) k->small_m = (uint32_t)v;
    }
    { const char *e = getenv("LOCAL_CUDA_TEST_WAIT_EXPIRY"); k->test_wait_expiry = e && strcmp(e, "1") == 0; }
    const char *nm = getenv("LOCAL_CUDA_TQ_NORM");
    k->kv_norm_mode = (nm && strcmp(nm, "tree") == 0) ? 1 : 0;
    cudaError_t e = cudaMalloc((void **)&k->dev_status, 128);  // status word + tuning stamps
    if (e == cudaSuccess) e = cudaMemsetAsync(k->dev_status, 0, 128, ctx->stream);
    if (e != cudaSuccess) {
        delete k;
        return lc_fail(LC_ERR_PIPELINE_CREATION, "status word: %s", cudaGetErrorString(e));
    }
    *out = k;
    return LC_OK;
}

void lc_kernels_destroy(lc_kernels *k) {
    if (!k) return;
    cudaSetDevice(k->ctx->device);
    cudaStreamSynchronize(k->ctx->stream);
    if (k->scratch) cudaFree(k->scratch);
    if (k->counters) cudaFree(k->counters);
    for (void *p : k->retired) cudaFree(p);
    if (k->dev_status) cudaFree(k->dev_status);
    delete k;
}

}  // extern "C"

// A captured graph keeps the scratch and counter addresses it was recorded with, so a block that has
// ever been handed out is never freed before lc_kernels_destroy: growth allocates a new block and retires
// the old one (kept alive in `retired`).  Graphs recorded earlier go on using their own, still valid, block.
int lc_reserve_scratch(lc_kernels *k, lc_batch *b, size_t bytes, size_t counters) {
    if (bytes > k->scratch_bytes) {
        if (b && b->capturing)
            return lc_fail(LC_ERR_INVALID_ARGUMENT,
                           "split-K scratch must grow to %zu bytes during graph capture; run the "
                           "same call once outside capture first", bytes);
        size_t want = bytes + bytes / 2;
        void *fresh = nullptr;
        cudaError_t e = cudaMalloc(&fresh, want);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return lc_fail(LC_ERR_BUFFER_ALLOCATION, "scratch size=%zu: %s", want, cudaGetErrorString(e));
        }
        if (k->scratch) k->retired.push_back(k->scratch);
        k->scratch = fresh;
        k->scratch_bytes = want;
    }
    if (counters > k->counters_len) {
        if (b && b->capturing)
            return lc_fail(LC_ERR_INVALID_ARGUMENT,
                           "split-K counters must grow during graph capture; run the same call once "
                           "outside capture first");
        size_t want = counters * 2;
        unsigned int *fresh = nullptr;
        cudaError_t e = cudaMalloc((void **)&fresh, want * sizeof(unsigned int));
        if (e != cudaSuccess) {
            cudaGetLastError();
            return lc_fail(LC_ERR_BUFFER_ALLOCATION, "counters: %s", cudaGetErrorString(e));
        }
        // zeroed in stream order, before any kernel that is enqueued after this call can use them
        cudaStream_t s = b ? b->stream : k->ctx->stream;
        e = cudaMemsetAsync(fresh, 0, want * sizeof(unsigned int), s);
        if (e != cudaSuccess) {
            cudaFree(fresh);
            return lc_fail(LC_ERR_CUDA, "counters memset: %s", cudaGetErrorString(e));
        }
        if (k->counters) k->retired.push_back(k->counters);
        k->counters = fresh;
        k->counters_len = want;
    }
    return LC_OK;
}
