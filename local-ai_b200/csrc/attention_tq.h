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
};

// Tensor-core variant for tq2 / head_dim 256 (attention_tq_mma.cu). Same grid and partial layout as the
// CUDA-core split kernel: grid = (n_splits, n_kv * gchunks, n_lanes) with 8 q-heads per chunk.
int lc_tq2_attn_mma_launch(lc_batch *b, const TqAttnParams &p, dim3 grid);
