// Parameters shared by the code-space attention kernels (CUDA-core and tensor-core variants).
#pragma once
#include "lc_internal.h"

struct TqAttnParams {
    const float *rq;      // rotated query f32 [lanes, n_q, HD]   (fused_q == 0)
    const __half *q;      // query f16 [lanes, n_q, HD]            (fused_q == 1)
    const float *signs;   // [HD]
    const uint8_t *kc, *vc;
    const __half *kn, *vn;
    const float *levels;  // [1 << BITS]
    float *out;           // f32 [lanes, n_q, HD], written when n_splits == 1 and !fused
    float *partial;       // [lanes * n_q * n_splits] x (2 + HD) floats
    const uint32_t *positions;  // per-lane positions, or NULL for the single-sequence form
    uint32_t kv_len, current_pos;
    // row_positions (prefill / multi-row verify): the grid's z index is a query ROW of one sequence, row r at position
    // current_pos + r; all rows read the same cache (lane_capacity = 0) and row r sees min(kv_len, its position + 1) keys.
    uint32_t row_positions;
    uint32_t lane_capacity, n_q, n_kv, window, ring, n_splits, group;  // group = n_q / n_kv
    uint32_t fused_q, direct_out;
    float scale;
    // cluster_merge: the n_splits CTAs of a (lane, kv head) are one thread-block cluster; they exchange their partials
    // through distributed shared memory and write the final result themselves (f32 rotated-space `out`, or, with
    // fused_q, the inverse-rotated f16 `out_f16`) -- no partial buffer, no merge launch.
    __half *out_f16;
    uint32_t cluster_merge;
    // Device-resident positions cannot be checked on the host: a lane whose position lies beyond its pool rows
    // (ring == 0 and position >= lane_capacity) is clamped to the rows that exist and *status is set to
    // LC_DEV_STATUS_POSITION (NULL: no report).
    int *status;
    // Optional (tensor-core kernel, fused_q, group a multiple of 8): the query already rotated, scaled and split into
    // the kernel's B fragments by the launch that wrote q (lc_qkv_post_frag): uint4 {hi01, hi23, lo01, lo23} at
    // [(lane * n_q / 8 + head / 8) * 512 + s * 32 + 4 * (head % 8) + t] for dims 64 t + 4 s + 0..3.  NULL: build from q.
    const uint4 *qfrag;
    // 1: `positions` and every key below the lanes' positions were complete before the predecessor kernels started, so
    // the kernel may read them ahead of its dependency wait (tensor-core kernel, per-lane positions only).
    uint32_t early_kv;
};

// Tensor-core variant for tq2 / head_dim 256 (attention_tq_mma.cu). Same grid and partial layout as the
// CUDA-core split kernel: grid = (n_splits, n_kv * gchunks, n_lanes) with 8 q-heads per chunk.
int lc_tq2_attn_mma_launch(lc_batch *b, const TqAttnParams &p, dim3 grid);

// Library-internal forms used by the decode step: lc_qkv_post_batched_into that also leaves the query fragments
// described at TqAttnParams::qfrag in `qfrag` (n_lanes * n_q_heads * head_dim * 4 bytes; requires head_dim 256, 2-bit codes and n_q_heads / n_kv_heads a multiple of 8), and lc_tq_attention_batched_into that reads them.
// The fragments hold exactly the values the attention kernel would derive from q, so results do not change.
bool lc_qfrag_supported(uint32_t head_dim, uint32_t bits, uint32_t n_q_heads, uint32_t n_kv_heads);
int lc_qkv_post_frag(lc_kernels *k, lc_batch *b, lc_buf *q, const lc_buf *q_norm_weight, uint32_t n_q_heads,
                     const lc_buf *k_in, const lc_buf *v_in, const lc_buf *k_norm_weight, const lc_buf *positions,
                     const lc_buf *levels, const lc_buf *signs, lc_buf *k_packed, lc_buf *k_norms, lc_buf *v_packed,
                     lc_buf *v_norms, uint32_t head_dim, uint32_t n_kv_heads, uint32_t lane_capacity, uint32_t bits,
                     uint32_t n_lanes, uint32_t ring_capacity, float eps, float rope_theta, float partial_rotary_factor,
                     lc_buf *qfrag, float softmax_scale);
int lc_tq_attention_batched_frag(lc_kernels *k, lc_batch *b, const lc_buf *q, const lc_buf *k_codes, const lc_buf *k_norms,
                                 const lc_buf *v_codes, const lc_buf *v_norms, const lc_buf *levels, const lc_buf *signs,
                                 lc_buf *attn_out, const lc_buf *positions, uint32_t head_dim, uint32_t lane_capacity,
                                 uint32_t num_q_heads, uint32_t num_kv_heads, uint32_t window, uint32_t bits,
                                 uint32_t n_lanes, uint32_t ring_capacity, float softmax_scale, const lc_buf *qfrag);
