/*
 * local_cuda.h — C ABI of the B200 (sm_100a) backend for local-ai's decode hot path.
 *
 * Every entry point replaces one item of the reference's `local-metal` crate
 * (the kernel-dispatch layer local-engine's forward pass calls).  The citation
 * after each declaration is the reference interface it stands in for, as
 * file:line relative to the reference project root.  Argument order and meaning
 * follow the Rust method of the same name; buffers are opaque handles
 * (`MetalBuffer` -> `lc_buf`), scalars are uint32_t / float, the result is an
 * `lc_status` (`local_metal::Error` -> integer code + `lc_last_error()` text).
 *
 * Conventions
 *  - `*_into` entry points enqueue onto the batch's stream and return at once
 *    (the reference encodes into a `CommandBatch`); the same name without
 *    `_into` takes the context, runs and waits (the reference's `ctx` variants).
 *  - All device work of one context is issued in call order on one stream, the
 *    serial-encoder semantics of batch.rs:59-66.
 *  - Buffers must outlive the batch / graph that references them.
 *  - Handles are not thread-safe; use one context per host thread, one per GPU.
 *    lc_batch_begin makes its context's device current on the calling thread; a
 *    thread that drives contexts of several GPUs must not interleave the enqueues
 *    of batches that belong to different devices.
 *  - Kernels start copying their constant operands (weights, norm weights,
 *    levels, signs) while the previous kernel of the stream is still running
 *    (programmatic dependent launch).  Such a buffer must therefore not be
 *    written by the kernel enqueued immediately before the call that reads it as
 *    a constant operand; callers that build weights on the device in the preceding
 *    dispatch set LOCAL_CUDA_PDL=0 (no early start) or enqueue any other dispatch
 *    in between.  Activations, positions and KV pools carry no such rule.
 *  - Split-K scratch owned by an `lc_kernels` grows on demand, outside graph
 *    capture only.  A block that was handed out once stays allocated until
 *    lc_kernels_destroy, so a captured graph keeps working after later, larger
 *    eager calls on the same object.
 *  - There is no CPU fallback: every compute entry point launches a CUDA kernel
 *    or fails with a status.
 */
#ifndef LOCAL_CUDA_H
#define LOCAL_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LC_API __attribute__((visibility("default")))

/* local-metal/src/error.rs:2-32 (+ CUDA / NCCL / TIMEOUT, which have no Metal twin) */
typedef enum lc_status {
    LC_OK = 0,
    LC_ERR_NO_DEVICE = 1,          /* NoMetalDevice / NoDevice */
    LC_ERR_NO_COMMAND_QUEUE = 2,   /* NoCommandQueue */
    LC_ERR_BUFFER_ALLOCATION = 3,  /* BufferAllocation{size,reason} */
    LC_ERR_LIBRARY_CREATION = 4,   /* LibraryCreation */
    LC_ERR_PIPELINE_CREATION = 5,  /* PipelineCreation */
    LC_ERR_SHADER_NOT_FOUND = 6,   /* ShaderNotFound */
    LC_ERR_COMMAND_BUFFER = 7,     /* CommandBuffer */
    LC_ERR_INVALID_ARGUMENT = 8,   /* InvalidArgument */
    LC_ERR_IO = 9,                 /* Io */
    LC_ERR_CUDA = 10,
    LC_ERR_NCCL = 11,
    LC_ERR_TIMEOUT = 12
} lc_status;

typedef struct lc_ctx lc_ctx;         /* MetalContext    local-metal/src/context.rs:31-101 */
typedef struct lc_buf lc_buf;         /* MetalBuffer     local-metal/src/buffer.rs:17-144 */
typedef struct lc_batch lc_batch;     /* CommandBatch    local-metal/src/batch.rs:147-292 */
typedef struct lc_pending lc_pending; /* PendingCommandBuffer  batch.rs:120-145 */
typedef struct lc_graph lc_graph;     /* no twin: a captured batch that can be replayed */
typedef struct lc_kernels lc_kernels; /* Kernels         local-metal/src/kernels.rs:18-219 */

/* Text of the last failure on the calling thread ("" if none). */
LC_API const char *lc_last_error(void);
LC_API const char *lc_status_name(int status);
/* Build identification: "local-cuda <ver> sm_100a". */
LC_API const char *lc_version(void);

/* ------------------------------------------------------------- context -- */
/* MetalContext::new (context.rs:37-62). `device` is the CUDA ordinal. */
LC_API int lc_ctx_create(int device, lc_ctx **out);
LC_API void lc_ctx_destroy(lc_ctx *ctx);
/* MetalContext::caps (context.rs:70-90): SM count, opt-in shared memory per
 * CTA, L2 bytes, total device memory. Any out pointer may be NULL. */
LC_API int lc_ctx_caps(const lc_ctx *ctx, int *sm_count, size_t *smem_per_cta,
                       size_t *l2_bytes, size_t *total_mem);
/* The context's stream as a cudaStream_t, for callers that time with events. */
LC_API void *lc_ctx_stream(const lc_ctx *ctx);
LC_API int lc_ctx_synchronize(lc_ctx *ctx);

/* -------------------------------------------------------------- buffer -- */
/* MetalBuffer::empty (buffer.rs:45-62): zero-filled device allocation. */
LC_API int lc_buf_alloc(lc_ctx *ctx, size_t bytes, lc_buf **out);
/* MetalBuffer::from_slice (buffer.rs:21-43): allocate + copy from host. */
LC_API int lc_buf_from_host(lc_ctx *ctx, const void *src, size_t bytes, lc_buf **out);
/* Wrap device memory the caller owns (never freed by the library). */
LC_API int lc_buf_wrap(lc_ctx *ctx, void *device_ptr, size_t bytes, lc_buf **out);
LC_API void lc_buf_free(lc_buf *buf);
LC_API size_t lc_buf_length(const lc_buf *buf);   /* MetalBuffer::length buffer.rs:64-67 */
LC_API void *lc_buf_device_ptr(const lc_buf *buf); /* MetalBuffer::raw    buffer.rs:139-143 */
/* MetalBuffer::copy_from_bytes (buffer.rs:112-131); out of range -> status, not a panic. */
LC_API int lc_buf_upload(lc_buf *buf, size_t offset, const void *src, size_t bytes);
/* MetalBuffer::as_slice (buffer.rs:78-94): the CPU read of GPU results. */
LC_API int lc_buf_download(const lc_buf *buf, size_t offset, void *dst, size_t bytes);
/* Zero a byte range (the containers' reset paths, kv_cache/quant_cache.rs:364-380). */
LC_API int lc_buf_zero(lc_buf *buf, size_t offset, size_t bytes);
/* Set every byte of a range to `value` (synthetic pool contents for benchmarks). */
LC_API int lc_buf_fill(lc_buf *buf, size_t offset, size_t bytes, int value);

/* --------------------------------------------------------------- batch -- */
LC_API int lc_batch_begin(lc_ctx *ctx, lc_batch **out);           /* CommandBatch::new batch.rs:160-172 */
LC_API uint32_t lc_batch_dispatch_count(const lc_batch *batch);   /* batch.rs:174-182 */
/* CommandBatch::blit_buffer_copies (batch.rs:196-226), one copy per call. */
LC_API int lc_batch_copy(lc_batch *batch, const lc_buf *src, size_t src_off, lc_buf *dst,
                         size_t dst_off, size_t bytes);
/* Async host<->device copies in batch order (host memory should be pinned). */
LC_API int lc_batch_upload(lc_batch *batch, lc_buf *dst, size_t dst_off, const void *src,
                           size_t bytes);
LC_API int lc_batch_download(lc_batch *batch, const lc_buf *src, size_t src_off, void *dst,
                             size_t bytes);
LC_API int lc_batch_commit_and_wait(lc_batch *batch);             /* batch.rs:258-272; frees batch */
LC_API int lc_batch_commit_async(lc_batch *batch, lc_pending **out); /* batch.rs:274-291; frees batch */
LC_API int lc_pending_wait(lc_pending *pending);                  /* batch.rs:126-144; frees pending */
/* Record everything enqueued between begin_capture and end_capture into a CUDA
 * graph instead of running it; lc_graph_launch replays it on the context's
 * stream (the reference re-encodes every token; a graph removes that cost). */
LC_API int lc_batch_begin_capture(lc_ctx *ctx, lc_batch **out);
LC_API int lc_batch_end_capture(lc_batch *batch, lc_graph **out); /* frees batch */
LC_API int lc_graph_launch(lc_graph *graph);
LC_API void lc_graph_destroy(lc_graph *graph);
/* Pinned host memory for lc_batch_upload / lc_batch_download. */
LC_API int lc_host_alloc(size_t bytes, void **out);
LC_API void lc_host_free(void *ptr);

/* ------------------------------------------------------------- kernels -- */
/* Kernels::new (kernels.rs:116-219). Reads the routing switches LOCAL_AI_BATCHM,
 * LOCAL_AI_SMALLM, LOCAL_AI_MMA once (kernels.rs:6277-6304). */
LC_API int lc_kernels_create(lc_ctx *ctx, lc_kernels **out);
LC_API void lc_kernels_destroy(lc_kernels *k);

/* Device-side status word, for what the host cannot see before a launch.  Kernels that wait on
 * hardware barriers bound every wait and record 1 or 2 here instead of hanging (-> LC_ERR_TIMEOUT).
 * The per-lane entry points read positions from a device buffer: a position that points past its
 * lane's pool rows (ring_capacity == 0 and position >= lane_capacity) writes no KV row and attends
 * only over the rows that exist, and records 3 (-> LC_ERR_INVALID_ARGUMENT).  *status receives the
 * word; LC_OK when it is 0.  The word stays set until the object is destroyed. */
LC_API int lc_kernels_device_status(lc_kernels *k, int *status);

/* Quantized matvec: output[rows] = matrix[rows, cols] x vector[cols], f16 input,
 * f32 accumulate.  matrix holds verbatim GGUF blocks (Q4_0: 18 B / 32 weights,
 * cols % 32 == 0; TQ2_0: 66 B / 256 weights, cols % 256 == 0), else
 * LC_ERR_INVALID_ARGUMENT. */
LC_API int lc_matvec_q4_0(lc_kernels *k, lc_ctx *ctx, const lc_buf *matrix, const lc_buf *vector,
                          lc_buf *output, uint32_t rows, uint32_t cols);           /* kernels.rs:5711 */
LC_API int lc_matvec_q4_0_into(lc_kernels *k, lc_batch *b, const lc_buf *matrix,
                               const lc_buf *vector, lc_buf *output, uint32_t rows,
                               uint32_t cols);                                      /* kernels.rs:5744 */
LC_API int lc_matvec_q4_0_f32out(lc_kernels *k, lc_ctx *ctx, const lc_buf *matrix,
                                 const lc_buf *vector, lc_buf *output, uint32_t rows,
                                 uint32_t cols);                                    /* kernels.rs:5778 */
LC_API int lc_matvec_q4_0_f32out_into(lc_kernels *k, lc_batch *b, const lc_buf *matrix,
                                      const lc_buf *vector, lc_buf *output, uint32_t rows,
                                      uint32_t cols);                               /* kernels.rs:5811 */
LC_API int lc_matvec_tq2_0(lc_kernels *k, lc_ctx *ctx, const lc_buf *matrix, const lc_buf *vector,
                           lc_buf *output, uint32_t rows, uint32_t cols);          /* kernels.rs:5848 */
LC_API int lc_matvec_tq2_0_into(lc_kernels *k, lc_batch *b, const lc_buf *matrix,
                                const lc_buf *vector, lc_buf *output, uint32_t rows,
                                uint32_t cols);                                     /* kernels.rs:5881 */
LC_API int lc_matvec_tq2_0_f32out(lc_kernels *k, lc_ctx *ctx, const lc_buf *matrix,
                                  const lc_buf *vector, lc_buf *output, uint32_t rows,
                                  uint32_t cols);                                   /* kernels.rs:5978 */
LC_API int lc_matvec_tq2_0_f32out_into(lc_kernels *k, lc_batch *b, const lc_buf *matrix,
                                       const lc_buf *vector, lc_buf *output, uint32_t rows,
                                       uint32_t cols);                              /* kernels.rs:6011 */
/* Grouped form: `count` (1..=96) matrices of one shape [rows, cols] against the same vector, output i = matrix i x
 * vector, f16 out.  One launch when the streaming kernel applies (it walks the matrices as one run of 64-row groups,
 * so a set of small projections streams at the rate of one large matrix), else one launch per matrix.  The decode-time
 * access pattern the reference's own microbenchmark models with 35 distinct weight sets
 * (local-metal/src/kernels.rs:8886-9136). */
LC_API int lc_matvec_q4_0_group_into(lc_kernels *k, lc_batch *b, const lc_buf *const *matrices, uint32_t count,
                                     const lc_buf *vector, lc_buf *const *outputs, uint32_t rows, uint32_t cols);
LC_API int lc_matvec_tq2_0_group_into(lc_kernels *k, lc_batch *b, const lc_buf *const *matrices, uint32_t count,
                                      const lc_buf *vector, lc_buf *const *outputs, uint32_t rows, uint32_t cols);
/* SoA TQ2_0: qs = rows*blocks*64 bytes, scales = rows*blocks f16. */
LC_API int lc_matvec_tq2_0_soa_into(lc_kernels *k, lc_batch *b, const lc_buf *qs,
                                    const lc_buf *scales, const lc_buf *vector, lc_buf *output,
                                    uint32_t rows, uint32_t cols);                  /* kernels.rs:5919 */

/* Quantized batched matmul: output[m, n] (f16) = input[m, k] (f16) x weight[n, k]^T.
 * Routing by m follows kernels.rs:6459-6563 (register-resident small-M path,
 * then the tensor-core path). */
LC_API int lc_matmul_nt_q4_0_into(lc_kernels *k, lc_batch *b, const lc_buf *input,
                                  const lc_buf *weight, lc_buf *output, uint32_t m, uint32_t kk,
                                  uint32_t n);                                      /* kernels.rs:6459 */
LC_API int lc_matmul_nt_tq2_0_into(lc_kernels *k, lc_batch *b, const lc_buf *input,
                                   const lc_buf *weight, lc_buf *output, uint32_t m, uint32_t kk,
                                   uint32_t n);                                     /* kernels.rs:6509 */
/* 1 <= m <= 16, one pass over the weights for all m rows. */
LC_API int lc_multivec_nt_q4_0_into(lc_kernels *k, lc_batch *b, const lc_buf *input,
                                    const lc_buf *weight, lc_buf *output, uint32_t m, uint32_t kk,
                                    uint32_t n);                                    /* kernels.rs:6378 */
LC_API int lc_multivec_nt_tq2_0_into(lc_kernels *k, lc_batch *b, const lc_buf *input,
                                     const lc_buf *weight, lc_buf *output, uint32_t m,
                                     uint32_t kk, uint32_t n);                      /* kernels.rs:6419 */
/* Same contraction with f32 output: the vocabulary projection of n_lanes rows
 * in ONE pass over the table.  The reference issues one matvec_q4_0_f32out per
 * lane (pipeline/batched.rs:427-447), re-reading the table n_lanes times. */
LC_API int lc_matmul_nt_q4_0_f32out_into(lc_kernels *k, lc_batch *b, const lc_buf *input,
                                         const lc_buf *weight, lc_buf *output, uint32_t m,
                                         uint32_t kk, uint32_t n);

/* out[i] = scales[i/4] * ((packed[i/4] >> 2(i%4)) & 3), f16.  The reference
 * launches a single threadgroup of <= 256 threads whatever num_elements is
 * (kernels.rs:6788-6797); this entry point covers all num_elements. */
LC_API int lc_tq2_dequant(lc_kernels *k, lc_ctx *ctx, const lc_buf *packed, const lc_buf *scales,
                          lc_buf *output, uint32_t num_elements);                   /* kernels.rs:6753 */

/* ---------------------------------------------------------- TurboQuant -- */
/* Host-side codec set-up, what TurboQuant::new computes on the CPU
 * (local-engine/src/turboquant.rs:187-199): the caller uploads the results as
 * the `levels` / `signs` buffers below. */
LC_API size_t lc_tq_code_bytes(uint32_t head_dim, uint32_t bits);          /* turboquant.rs:203-205 */
LC_API int lc_tq_signs(uint32_t dim, uint64_t seed, float *signs);         /* turboquant.rs:66-80 */
LC_API int lc_tq_levels(uint32_t dim, uint32_t bits, float *levels);       /* turboquant.rs:114-166,187-192 */
LC_API size_t lc_swa_ring_capacity(size_t window, size_t max_positions);   /* kv_cache/quant_cache.rs:48-54 */
LC_API uint32_t lc_kv_bits_from_env(void);                                 /* kv_cache/quant_cache.rs:60-66 */
#define LC_TQ_SEED 0x7459C0DEull                                           /* kv_cache/quant_cache.rs:30 */
/* Summation order of the row norm in the encode kernels: 0 (default) = the Rust
 * codec's sequential order, bit-exact with TurboQuant::encode_into
 * (turboquant.rs:241-276); 1 = the Metal kernel's pairwise tree
 * (shaders/dequantize_kv.metal:247-257).  Also read once from LOCAL_CUDA_TQ_NORM=tree. */
LC_API int lc_kernels_set_kv_norm_mode(lc_kernels *k, int mode);

/* input f16 [num_tokens, n_kv_heads, head_dim] -> packed codes + f16 norms at slot
 * ((position + tok) % ring) * n_kv + head, or (position + tok) * n_kv + head when ring == 0. */
LC_API int lc_encode_kv_turboquant_into(lc_kernels *k, lc_batch *b, const lc_buf *input,
                                        const lc_buf *levels, const lc_buf *signs, lc_buf *packed,
                                        lc_buf *norms, uint32_t head_dim, uint32_t n_kv_heads,
                                        uint32_t num_tokens, uint32_t bits, uint32_t position,
                                        uint32_t ring_capacity);                    /* kernels.rs:4819 */
LC_API int lc_encode_kv_turboquant(lc_kernels *k, lc_ctx *ctx, const lc_buf *input,
                                   const lc_buf *levels, const lc_buf *signs, lc_buf *packed,
                                   lc_buf *norms, uint32_t head_dim, uint32_t n_kv_heads,
                                   uint32_t num_tokens, uint32_t bits, uint32_t position,
                                   uint32_t ring_capacity);                         /* kernels.rs:4988 */
/* One new row per lane: slot (lane * lane_capacity + positions[lane] % ring) * n_kv + head. */
LC_API int lc_encode_kv_turboquant_batched_into(lc_kernels *k, lc_batch *b, const lc_buf *input,
                                                const lc_buf *levels, const lc_buf *signs,
                                                lc_buf *packed, lc_buf *norms, const lc_buf *positions,
                                                uint32_t head_dim, uint32_t n_kv_heads,
                                                uint32_t lane_capacity, uint32_t bits, uint32_t n_lanes,
                                                uint32_t ring_capacity);            /* kernels.rs:4901 */
LC_API int lc_dequantize_kv_turboquant_into(lc_kernels *k, lc_batch *b, const lc_buf *packed,
                                            const lc_buf *norms, const lc_buf *levels,
                                            const lc_buf *signs, lc_buf *output, uint32_t head_dim,
                                            uint32_t n_kv_heads, uint32_t num_tokens, uint32_t bits,
                                            uint32_t token_start, uint32_t ring_capacity); /* kernels.rs:4732 */
LC_API int lc_dequantize_kv_turboquant(lc_kernels *k, lc_ctx *ctx, const lc_buf *packed,
                                       const lc_buf *norms, const lc_buf *levels, const lc_buf *signs,
                                       lc_buf *output, uint32_t head_dim, uint32_t n_kv_heads,
                                       uint32_t num_tokens, uint32_t bits, uint32_t token_start,
                                       uint32_t ring_capacity);                     /* kernels.rs:4641 */
/* y = (1/sqrt d) H(pre_sign ? s*x : x), then * s when post_sign; f32->f32, f16->f32, f32->f16. */
LC_API int lc_hadamard_rotate_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *signs,
                                   lc_buf *output, uint32_t head_dim, uint32_t num_heads,
                                   uint32_t pre_sign, uint32_t post_sign);          /* kernels.rs:5032 */
LC_API int lc_hadamard_rotate_hf_into(lc_kernels *k, lc_batch *b, const lc_buf *input,
                                      const lc_buf *signs, lc_buf *output, uint32_t head_dim,
                                      uint32_t num_heads, uint32_t pre_sign, uint32_t post_sign); /* kernels.rs:5060 */
LC_API int lc_hadamard_rotate_fh_into(lc_kernels *k, lc_batch *b, const lc_buf *input,
                                      const lc_buf *signs, lc_buf *output, uint32_t head_dim,
                                      uint32_t num_heads, uint32_t pre_sign, uint32_t post_sign); /* kernels.rs:5088 */

/* ------------------------------------------------- attention over codes -- */
/* Decode attention of one query position over packed TurboQuant rows.
 * rq = rotated query f32 [n_q, hd]; out = rotated-space accumulation f32 [n_q, hd].
 * Same arguments as the reference plus a trailing softmax_scale (the reference
 * hard-codes 1.0: attention_flash_tq.metal has no scale); pass 1.0f for the
 * reference's behaviour.  Split-K partials live in scratch owned by `k`. */
LC_API int lc_flash_attention_tq_into(lc_kernels *k, lc_batch *b, const lc_buf *rq,
                                      const lc_buf *k_codes, const lc_buf *k_norms,
                                      const lc_buf *v_codes, const lc_buf *v_norms, const lc_buf *levels,
                                      lc_buf *out, uint32_t head_dim, uint32_t kv_len,
                                      uint32_t current_pos, uint32_t num_q_heads, uint32_t num_kv_heads,
                                      uint32_t window, uint32_t bits, uint32_t ring_capacity,
                                      float softmax_scale);                         /* kernels.rs:5176 */
/* Per-lane form over a unified pool [n_lanes, lane_capacity, n_kv, code_bytes]. */
LC_API int lc_flash_attention_tq_batched_into(lc_kernels *k, lc_batch *b, const lc_buf *rq,
                                              const lc_buf *k_codes, const lc_buf *k_norms,
                                              const lc_buf *v_codes, const lc_buf *v_norms,
                                              const lc_buf *levels, lc_buf *out, const lc_buf *positions,
                                              uint32_t head_dim, uint32_t lane_capacity,
                                              uint32_t num_q_heads, uint32_t num_kv_heads, uint32_t window,
                                              uint32_t bits, uint32_t n_lanes, uint32_t ring_capacity,
                                              float softmax_scale);                 /* kernels.rs:5434 */
/* Fused rotate -> attend -> inverse-rotate: q f16 [n_q, hd] in, attn_out f16 out.
 * One call for the three dispatches QuantizedKvCache::fused_attention_into
 * always issues together (kv_cache/quant_cache.rs:548-598). */
LC_API int lc_tq_attention_into(lc_kernels *k, lc_batch *b, const lc_buf *q, const lc_buf *k_codes,
                                const lc_buf *k_norms, const lc_buf *v_codes, const lc_buf *v_norms,
                                const lc_buf *levels, const lc_buf *signs, lc_buf *attn_out,
                                uint32_t head_dim, uint32_t kv_len, uint32_t current_pos,
                                uint32_t num_q_heads, uint32_t num_kv_heads, uint32_t window, uint32_t bits,
                                uint32_t ring_capacity, float softmax_scale);
/* The same for QuantizedUnifiedKvPool::attention_into (kv_cache/quant_unified_pool.rs:194-258). */
LC_API int lc_tq_attention_batched_into(lc_kernels *k, lc_batch *b, const lc_buf *q,
                                        const lc_buf *k_codes, const lc_buf *k_norms,
                                        const lc_buf *v_codes, const lc_buf *v_norms, const lc_buf *levels,
                                        const lc_buf *signs, lc_buf *attn_out, const lc_buf *positions,
                                        uint32_t head_dim, uint32_t lane_capacity, uint32_t num_q_heads,
                                        uint32_t num_kv_heads, uint32_t window, uint32_t bits,
                                        uint32_t n_lanes, uint32_t ring_capacity, float softmax_scale);

/* Prefill / multi-row verify attention over codes: query row r of the chunk (rq / out f32 [n_rows, n_q, hd]) sits at
 * absolute position start_pos + r and attends the keys of its own causal window of the ONE cache that already holds
 * the chunk's rows: exactly a decode call with current_pos = start_pos + r per row.  The second entry point is the
 * reference's query-tiled kernel; here both run the same launch (rows of a chunk share the cache through L2). */
LC_API int lc_flash_attention_tq_prefill_into(lc_kernels *k, lc_batch *b, const lc_buf *rq, const lc_buf *k_codes,
                                              const lc_buf *k_norms, const lc_buf *v_codes, const lc_buf *v_norms,
                                              const lc_buf *levels, lc_buf *out, uint32_t head_dim, uint32_t kv_len,
                                              uint32_t start_pos, uint32_t n_rows, uint32_t num_q_heads,
                                              uint32_t num_kv_heads, uint32_t window, uint32_t bits,
                                              uint32_t ring_capacity, float softmax_scale);   /* kernels.rs:5259 */
LC_API int lc_flash_attention_tq_prefill_tiled_into(lc_kernels *k, lc_batch *b, const lc_buf *rq, const lc_buf *k_codes,
                                                    const lc_buf *k_norms, const lc_buf *v_codes,
                                                    const lc_buf *v_norms, const lc_buf *levels, lc_buf *out,
                                                    uint32_t head_dim, uint32_t kv_len, uint32_t start_pos,
                                                    uint32_t n_rows, uint32_t num_q_heads, uint32_t num_kv_heads,
                                                    uint32_t window, uint32_t bits, uint32_t ring_capacity,
                                                    float softmax_scale);                      /* kernels.rs:5345 */
/* Rotate -> prefill attention -> inverse-rotate for a chunk: q f16 [n_rows, n_q, hd] in, attn_out f16 out
 * (QuantizedKvCache::fused_attention_batch_into, kv_cache/quant_cache.rs:620-700). */
LC_API int lc_tq_attention_prefill_into(lc_kernels *k, lc_batch *b, const lc_buf *q, const lc_buf *k_codes,
                                        const lc_buf *k_norms, const lc_buf *v_codes, const lc_buf *v_norms,
                                        const lc_buf *levels, const lc_buf *signs, lc_buf *attn_out, uint32_t head_dim,
                                        uint32_t kv_len, uint32_t start_pos, uint32_t n_rows, uint32_t num_q_heads,
                                        uint32_t num_kv_heads, uint32_t window, uint32_t bits, uint32_t ring_capacity,
                                        float softmax_scale);

/* No counterpart in the reference.  lc_tq_attention_into for callers that must not
 * allocate device memory when they run attention (an HBM budget fully handed to the KV
 * pool, or a latency-critical serving loop that cannot take cudaMalloc's stall): the split-K
 * partials live in a 4 MiB array built into the library instead of the cudaMalloc'ed
 * scratch of `lc_kernels`, so no `lc_kernels` is needed and nothing is allocated or freed.
 * Limit: num_q_heads * (head_dim + 2) * 4 bytes per split must fit in 4 MiB (the split count
 * is lowered to fit, else LC_ERR_INVALID_ARGUMENT).  All calls share the array: calls that
 * overlap on the GPU race, so keep them on one stream.  The first call on each device
 * resolves the array's address and should be made before any stream capture.  Always runs the
 * CUDA-core split kernel (the tensor-core kernel of the regular entry point is not used here). */
LC_API int lc_tq_attention_noalloc_into(lc_batch *b, const lc_buf *q, const lc_buf *k_codes,
                                        const lc_buf *k_norms, const lc_buf *v_codes,
                                        const lc_buf *v_norms, const lc_buf *levels, const lc_buf *signs,
                                        lc_buf *attn_out, uint32_t head_dim, uint32_t kv_len,
                                        uint32_t current_pos, uint32_t num_q_heads, uint32_t num_kv_heads,
                                        uint32_t window, uint32_t bits, uint32_t ring_capacity,
                                        float softmax_scale);

/* ---------------------------------------------------- FP16-KV attention -- */
/* K/V f16 [kv_len, n_kv, hd]; q, output f16 [n_q, hd]; softmax scale 1.0 as in the shaders. */
LC_API uint32_t lc_flash_split_count(const lc_kernels *k, uint32_t eff_seq_len);    /* kernels.rs:1265 */
LC_API int lc_flash_attention_windowed_split_into(lc_kernels *k, lc_batch *b, const lc_buf *q,
                                                  const lc_buf *kk, const lc_buf *v, lc_buf *output,
                                                  lc_buf *partial_max, lc_buf *partial_sum,
                                                  lc_buf *partial_acc, uint32_t head_dim, uint32_t kv_len,
                                                  uint32_t current_pos, uint32_t num_q_heads,
                                                  uint32_t num_kv_heads, uint32_t window,
                                                  uint32_t num_splits);             /* kernels.rs:1292 */
LC_API int lc_flash_decoding_into(lc_kernels *k, lc_ctx *ctx, lc_batch *b, const lc_buf *q,
                                  const lc_buf *kk, const lc_buf *v, lc_buf *output, uint32_t head_dim,
                                  uint32_t kv_len, uint32_t current_pos, uint32_t num_q_heads,
                                  uint32_t num_kv_heads);                           /* kernels.rs:1397 */
LC_API int lc_attention_sliding(lc_kernels *k, lc_ctx *ctx, const lc_buf *q, const lc_buf *kk,
                                const lc_buf *v, lc_buf *output, uint32_t head_dim, uint32_t kv_len,
                                uint32_t current_pos, uint32_t window, uint32_t num_q_heads,
                                uint32_t num_kv_heads);                             /* kernels.rs:691 */

/* ------------------------------------------------------ per-layer small ops -- */
LC_API int lc_rms_norm_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                            lc_buf *output, uint32_t dim, uint32_t rows, float eps); /* kernels.rs:2142 */
LC_API int lc_rms_norm_add_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                                const lc_buf *residual, lc_buf *output, uint32_t dim, uint32_t rows,
                                float eps);                                         /* kernels.rs:6663 */
LC_API int lc_qk_norm_gpu_into(lc_kernels *k, lc_batch *b, lc_buf *qk_data, const lc_buf *weight,
                               uint32_t head_dim, uint32_t num_heads, float eps);   /* kernels.rs:2215 */
LC_API int lc_rope_into(lc_kernels *k, lc_batch *b, const lc_buf *input, lc_buf *output,
                        uint32_t head_dim, uint32_t position, float theta, float partial_rotary_factor,
                        uint32_t num_heads);                                        /* kernels.rs:509 */
LC_API int lc_rope_batch_decode_into(lc_kernels *k, lc_batch *b, lc_buf *qk, const lc_buf *positions,
                                     float theta, uint32_t head_dim, uint32_t num_heads, uint32_t seq_len,
                                     float partial_rotary_factor);                  /* kernels.rs:4311 */
LC_API int lc_gelu_mul_into(lc_kernels *k, lc_batch *b, const lc_buf *a, const lc_buf *bb, lc_buf *out,
                            uint32_t count);                                        /* kernels.rs:6648 */
LC_API int lc_residual_add_into(lc_kernels *k, lc_batch *b, const lc_buf *a, const lc_buf *bb,
                                lc_buf *output, uint32_t count);                    /* kernels.rs:2592 */
LC_API int lc_scale_in_place_gpu_into(lc_kernels *k, lc_batch *b, lc_buf *data, float scalar,
                                      uint32_t count);                              /* kernels.rs:2845 */
LC_API int lc_logit_softcap_gpu_into(lc_kernels *k, lc_batch *b, lc_buf *data, float cap,
                                     uint32_t count);                               /* kernels.rs:2749 */
LC_API int lc_gather_strided_f16_into(lc_kernels *k, lc_batch *b, const lc_buf *src, lc_buf *dst,
                                      uint32_t row_stride, uint32_t base_off, uint32_t pld,
                                      uint32_t n_rows);                             /* kernels.rs:2801 */
/* Fused forms of dispatch pairs the forward pass always issues back to back; each keeps the f16
 * rounding points of the unfused sequence.
 *  - qk_norm + rope_batch_decode in place (the reference's own fusion: qk_norm_rope_into, kernels.rs:2302);
 *  - rms_norm_add followed by rms_norm of its result (layer.rs:808-822, 843-853): two outputs;
 *  - the KV write of a decode step: k_norm, V rms_norm with unit weights, RoPE on K, TurboQuant encode of
 *    both rows into the per-lane pools (layer.rs:773-790 + kv_cache/quant_unified_pool.rs:138-181). */
LC_API int lc_qk_norm_rope_batch_decode_into(lc_kernels *k, lc_batch *b, lc_buf *qk, const lc_buf *weight,
                                             const lc_buf *positions, float theta, uint32_t head_dim,
                                             uint32_t num_heads, uint32_t seq_len, float eps,
                                             float partial_rotary_factor);
LC_API int lc_rms_norm_add_norm_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *weight,
                                     const lc_buf *residual, lc_buf *out_residual, const lc_buf *weight2,
                                     lc_buf *out_normed, uint32_t dim, uint32_t rows, float eps);
LC_API int lc_kv_write_batched_into(lc_kernels *k, lc_batch *b, const lc_buf *k_in, const lc_buf *v_in,
                                    const lc_buf *k_norm_weight, const lc_buf *positions, const lc_buf *levels,
                                    const lc_buf *signs, lc_buf *k_packed, lc_buf *k_norms, lc_buf *v_packed,
                                    lc_buf *v_norms, uint32_t head_dim, uint32_t n_kv_heads,
                                    uint32_t lane_capacity, uint32_t bits, uint32_t n_lanes,
                                    uint32_t ring_capacity, float eps, float rope_theta,
                                    float partial_rotary_factor);
/* The GeGLU half of the feed-forward block, gelu_mul(matmul_nt_tq2_0(x, W_gate), matmul_nt_tq2_0(x, W_up))
 * (local-engine/src/layer.rs:825-838), as one launch for decode batches (8 < m <= 64); other m run the two
 * projections into gate_tmp / up_tmp [m, n] and lc_gelu_mul_into.  `output` may alias `gate_tmp`. */
LC_API int lc_matmul_nt_tq2_0_geglu_into(lc_kernels *k, lc_batch *b, const lc_buf *input, const lc_buf *w_gate,
                                         const lc_buf *w_up, lc_buf *gate_tmp, lc_buf *up_tmp, lc_buf *output,
                                         uint32_t m, uint32_t kk, uint32_t n);
/* lc_qk_norm_rope_batch_decode_into on the queries and lc_kv_write_batched_into in one launch: everything
 * between the Q/K/V projections and attention of a decode step (layer.rs:757-790). */
LC_API int lc_qkv_post_batched_into(lc_kernels *k, lc_batch *b, lc_buf *q, const lc_buf *q_norm_weight,
                                    uint32_t n_q_heads, const lc_buf *k_in, const lc_buf *v_in,
                                    const lc_buf *k_norm_weight, const lc_buf *positions, const lc_buf *levels,
                                    const lc_buf *signs, lc_buf *k_packed, lc_buf *k_norms, lc_buf *v_packed,
                                    lc_buf *v_norms, uint32_t head_dim, uint32_t n_kv_heads,
                                    uint32_t lane_capacity, uint32_t bits, uint32_t n_lanes,
                                    uint32_t ring_capacity, float eps, float rope_theta,
                                    float partial_rotary_factor);
/* Device-side stand-ins for two CPU steps the reference performs through unified
 * memory: the embedding-row gather (QuantWeight::dequant_row, local-engine/src/layer.rs:255-281,
 * followed by scale_in_place) and greedy first-max argmax (sampler.rs:148-158). */
LC_API int lc_embed_rows_q4_0_into(lc_kernels *k, lc_batch *b, const lc_buf *table, const lc_buf *tokens,
                                   lc_buf *output, uint32_t n_rows, uint32_t cols, uint32_t vocab,
                                   float scale);
LC_API int lc_argmax_rows_f32_into(lc_kernels *k, lc_batch *b, const lc_buf *values, lc_buf *out_index,
                                   uint32_t rows, uint32_t cols);

/* Row-split vocabulary projection (the 262144-row table split across GPUs, one process per GPU): per-shard greedy
 * argmax as pairs {f32 max, u32 first index + index_offset} and their merge over shards laid out [shards][rows] in
 * index order, with the first-maximum rule of local-engine/src/sampler.rs:148-158 (strict '>' in index order; an
 * all -inf / NaN row yields the first shard's first index).  8 bytes per lane cross the links instead of a logit slice. */
LC_API int lc_argmax_pairs_f32_into(lc_kernels *k, lc_batch *b, const lc_buf *values, lc_buf *pairs, uint32_t rows,
                                    uint32_t cols, uint32_t index_offset);
LC_API int lc_merge_argmax_pairs_into(lc_kernels *k, lc_batch *b, const lc_buf *pairs_all, lc_buf *out_index,
                                      uint32_t rows, uint32_t shards);

/* ------------------------------------------------------------- multi-GPU -- */
/* NCCL behind the ABI, for the all-gather of the row-split vocabulary projection.  The reference is single-GPU; these
 * entry points exist for the sharded configuration only.  libnccl is loaded at run time (LOCAL_CUDA_NCCL_LIB, else the
 * loader's libnccl.so.2): without it every call returns LC_ERR_NCCL, as does any NCCL error.  lc_comm_unique_id runs on
 * one rank; the host carries the 128 bytes to the others; every rank then calls lc_comm_create (collective, blocking).
 * lc_comm_all_gather_into enqueues on the batch's stream: bytes_per_rank bytes at send + send_offset go to
 * recv + rank * bytes_per_rank on every rank (send may be recv itself: in place). */
#define LC_COMM_ID_BYTES 128
typedef struct lc_comm lc_comm;
LC_API int lc_comm_available(void);
LC_API int lc_comm_unique_id(uint8_t *id);                      /* out: LC_COMM_ID_BYTES bytes */
LC_API int lc_comm_create(lc_ctx *ctx, const uint8_t *id, uint32_t rank, uint32_t world, lc_comm **out);
LC_API void lc_comm_destroy(lc_comm *c);
LC_API uint32_t lc_comm_rank(const lc_comm *c);
LC_API uint32_t lc_comm_world(const lc_comm *c);
LC_API int lc_comm_all_gather_into(lc_batch *b, lc_comm *c, const lc_buf *send, size_t send_offset, lc_buf *recv,
                                   size_t bytes_per_rank);

/* ----------------------------------------------------------- decode step -- */
/* One batched decode step of the dense decoder in the op order of
 * TransformerLayer::forward_decode_batch_turbo (local-engine/src/layer.rs:731-868) inside
 * Pipeline::decode_batch_step (local-engine/src/pipeline/batched.rs:271-456).  The model
 * object owns the per-lane KV pools (QuantizedUnifiedKvPool, kv_cache/quant_unified_pool.rs:33-181)
 * and the scratch (BatchScratch, layer.rs:960-1036); weights are borrowed buffers that must
 * outlive it.  Layer i is a full-attention layer iff i % full_every == full_every - 1 (or
 * swa_window == 0), otherwise a sliding-window layer with a ring of swa_ring rows
 * (0 = swa_ring_capacity(window, max_context)). */
typedef struct lc_model lc_model;
typedef struct lc_model_config {
    uint32_t hidden, n_q_heads, n_kv_heads, head_dim, inter, vocab, n_layers, kv_bits;
    uint32_t max_lanes, max_context, swa_window, swa_ring, full_every;
    float rms_eps, rope_theta, softmax_scale, embed_scale;
} lc_model_config;

LC_API int lc_model_create(lc_ctx *ctx, lc_kernels *k, const lc_model_config *cfg, lc_model **out);
LC_API void lc_model_destroy(lc_model *m);
/* TQ2_0 projections [out, in] and f16 norm weights of one layer (LayerWeights, layer.rs:284-352). */
LC_API int lc_model_set_layer(lc_model *m, uint32_t layer, const lc_buf *wq, const lc_buf *wk,
                              const lc_buf *wv, const lc_buf *wo, const lc_buf *wgate, const lc_buf *wup,
                              const lc_buf *wdown, const lc_buf *attn_norm, const lc_buf *q_norm,
                              const lc_buf *k_norm, const lc_buf *post_attn_norm, const lc_buf *ffn_norm,
                              const lc_buf *post_ffn_norm);
/* Q4_0 [vocab, hidden] table, tied with the output projection, and the final norm. */
LC_API int lc_model_set_embedding(lc_model *m, const lc_buf *embed_q4_0, const lc_buf *final_norm);
/* The pool buffers of a layer (owned by the model), for prefill / snapshots / tests. */
LC_API int lc_model_kv_buffers(lc_model *m, uint32_t layer, lc_buf **k_codes, lc_buf **k_norms,
                               lc_buf **v_codes, lc_buf **v_norms, uint32_t *lane_rows, uint32_t *ring,
                               uint32_t *window);
LC_API int lc_model_logits_buffer(lc_model *m, lc_buf **logits);   /* f32 [max_lanes, vocab] */
LC_API int lc_model_hidden_buffer(lc_model *m, lc_buf **hidden);   /* f16 [max_lanes, hidden]: final normed rows */
LC_API int lc_model_reset_lane(lc_model *m, uint32_t lane);         /* quant_unified_pool.rs:316-346 */
/* tokens, positions: u32 [n_lanes] device buffers.  want_logits != 0 or next_tokens != NULL runs the
 * vocabulary projection into the model's logits buffer; next_tokens (u32 [n_lanes]) receives the
 * greedy first-max argmax. */
LC_API int lc_model_decode_batch_step_into(lc_model *m, lc_batch *b, const lc_buf *tokens,
                                           const lc_buf *positions, uint32_t n_lanes, uint32_t want_logits,
                                           lc_buf *next_tokens);                    /* batched.rs:271 */

/* ------------------------------------------------------------ KV containers -- */
/* QuantizedKvCache (local-engine/src/kv_cache/quant_cache.rs:73-91): the TurboQuant cache of one layer of one
 * sequence -- packed K / V codes [rows, n_kv, code_bytes], f16 norms [rows, n_kv], and the codec's levels / signs
 * (TurboQuant::new with LC_TQ_SEED).  physical_positions < max_positions makes it a sliding-window ring (logical
 * position p in row p % physical_positions); the constructor's checks are the reference's: bits in 2..=4, head_dim a
 * power of two <= 512, ring >= sliding_window + 255 (room for a 256-row prefill chunk, quant_cache.rs:191-209). */
typedef struct lc_kv_cache lc_kv_cache;
LC_API int lc_kv_cache_create(lc_ctx *ctx, uint32_t n_kv_heads, uint32_t head_dim, uint32_t max_positions,
                              uint32_t physical_positions, uint32_t sliding_window, uint32_t bits,
                              lc_kv_cache **out);                                   /* quant_cache.rs:182-228 */
LC_API void lc_kv_cache_destroy(lc_kv_cache *cache);
LC_API uint32_t lc_kv_cache_physical_positions(const lc_kv_cache *cache);           /* quant_cache.rs:243-246 */
LC_API uint32_t lc_kv_cache_ring_capacity(const lc_kv_cache *cache);                /* quant_cache.rs:258-266 */
LC_API size_t lc_kv_cache_code_bytes(const lc_kv_cache *cache);                     /* quant_cache.rs:278-280 */
/* The owned buffers (borrowed; any out pointer may be NULL). */
LC_API int lc_kv_cache_buffers(lc_kv_cache *cache, lc_buf **keys_q, lc_buf **key_norms, lc_buf **values_q,
                               lc_buf **value_norms, lc_buf **levels, lc_buf **signs); /* quant_cache.rs:283-300 */
LC_API int lc_kv_cache_reset(lc_kv_cache *cache);                                   /* quant_cache.rs:364-380 */
/* k_src / v_src: f16 [n_rows, n_kv_heads, head_dim]; position + n_rows <= max_positions. */
LC_API int lc_kv_cache_write_kv_gpu_into(lc_kv_cache *cache, lc_batch *b, lc_kernels *k, const lc_buf *k_src,
                                         const lc_buf *v_src, uint32_t position, uint32_t n_rows); /* quant_cache.rs:391-444 */
/* q, attn_out: f16 [n_q_heads, head_dim].  The reference's rq / vacc scratch arguments are gone: rotate, attend and
 * rotate back run as one fused call.  softmax_scale: 1.0 for the reference's behaviour. */
LC_API int lc_kv_cache_fused_attention_into(lc_kv_cache *cache, lc_batch *b, lc_kernels *k, const lc_buf *q,
                                            lc_buf *attn_out, uint32_t seq_len, uint32_t current_pos,
                                            uint32_t n_q_heads, uint32_t window, float softmax_scale); /* quant_cache.rs:548-598 */
/* q, attn_out: f16 [n_rows, n_q_heads, head_dim]; row r at position start_pos + r. */
LC_API int lc_kv_cache_fused_attention_batch_into(lc_kv_cache *cache, lc_batch *b, lc_kernels *k, const lc_buf *q,
                                                  lc_buf *attn_out, uint32_t kv_len, uint32_t start_pos,
                                                  uint32_t n_rows, uint32_t n_q_heads, uint32_t window,
                                                  float softmax_scale);             /* quant_cache.rs:620-700 */
/* Prefix snapshots for prompt reuse: rows [0, positions) of the four buffers to / from host memory; `positions` is
 * clamped to lc_kv_cache_max_snapshot_positions (the ring capacity for a ringed cache). */
LC_API uint32_t lc_kv_cache_max_snapshot_positions(const lc_kv_cache *cache);       /* quant_cache.rs:311-318 */
LC_API int lc_kv_cache_snapshot_prefix(const lc_kv_cache *cache, uint32_t positions, void *keys_q, void *values_q,
                                       void *key_norms, void *value_norms);         /* quant_cache.rs:327-340 */
LC_API int lc_kv_cache_restore_prefix(lc_kv_cache *cache, uint32_t positions, const void *keys_q,
                                      const void *values_q, const void *key_norms,
                                      const void *value_norms);                     /* quant_cache.rs:343-362 */

/* The lane admit / recycle loop of batched decode (Pipeline::run_batched_to_completion,
 * local-engine/src/pipeline/runner.rs:123-214) over the per-lane pools of an lc_model: more requests than lanes is the
 * normal case; as lanes finish they are zeroed (lc_model_reset_lane) and the next queued request is admitted.  A round
 * is: lc_lane_sched_prepare (finalize, admit, fill the host arrays tokens / positions [n_lanes]; idle lanes carry token 0
 * at position 0), upload + lc_model_decode_batch_step_into with next_tokens, download, lc_lane_sched_consume.  An
 * admitted lane is fed its prompt one token per step through the same decode step (outputs discarded until the last
 * prompt token); the reference runs a separate prefill pipeline for that.  `model` may be NULL (no pools to zero). */
typedef struct lc_lane_sched lc_lane_sched;
typedef enum lc_stop_reason { LC_STOP_NONE = 0, LC_STOP_EOS = 1, LC_STOP_MAX_TOKENS = 2, LC_STOP_CAPACITY = 3 } lc_stop_reason;
LC_API int lc_lane_sched_create(lc_model *model, uint32_t n_lanes, uint32_t lane_capacity, uint32_t eos_token,
                                lc_lane_sched **out);
LC_API void lc_lane_sched_destroy(lc_lane_sched *s);
LC_API int lc_lane_sched_submit(lc_lane_sched *s, uint64_t id, const uint32_t *prompt, uint32_t prompt_len,
                                uint32_t max_new_tokens);
LC_API int lc_lane_sched_prepare(lc_lane_sched *s, uint32_t *tokens, uint32_t *positions, uint32_t *n_active);
LC_API int lc_lane_sched_consume(lc_lane_sched *s, const uint32_t *next_tokens);    /* runner.rs:196-208, 100-109 */
/* Pop one completed request in completion order; *n_out = 0 and *reason = 0 when none is ready.  With out_tokens NULL
 * only *n_out / *reason / *id are reported and the request stays queued. */
LC_API int lc_lane_sched_pop_finished(lc_lane_sched *s, uint64_t *id, uint32_t *out_tokens, uint32_t capacity,
                                      uint32_t *n_out, int *reason);
LC_API uint32_t lc_lane_sched_pending(const lc_lane_sched *s);   /* queued + running requests */

#ifdef __cplusplus
}
#endif
#endif /* LOCAL_CUDA_H */
