// The containers around the KV kernels: the single-sequence TurboQuant cache and the lane admit / recycle loop of
// batched decode.  Host logic only; every device operation goes through the kernel entry points of this library.
//
//  * lc_kv_cache: QuantizedKvCache (local-engine/src/kv_cache/quant_cache.rs:73-91): owns the packed K / V codes, the
//    f16 row norms and the codec's levels / signs buffers of one layer of one sequence; a sliding-window layer is a
//    ring of `physical_positions` rows (logical position p lives in row p % physical_positions, :258-274).
//  * lc_lane_sched: the request loop of Pipeline::run_batched_to_completion (local-engine/src/pipeline/runner.rs:
//    123-214) over the per-lane pools of an lc_model: admit queued requests into free lanes (zeroing the lane,
//    kv_cache/quant_unified_pool.rs:333-346), build the token / position arrays of a full-width step (idle lanes carry
//    token 0 at position 0), consume the greedy tokens, apply the stop rules (:100-109) and recycle finished lanes.
//    The reference prefills a prompt through its prefill pipeline, which is outside this library; here an admitted
//    lane consumes its prompt one token per step through the same batched decode step (its outputs are discarded
//    until the last prompt token has been fed), which writes the same KV rows.
#include <deque>
#include <vector>

#include "lc_internal.h"

constexpr uint32_t LC_MAX_PREFILL_CHUNK = 256;   // quant_cache.rs:42-46: rows one multi-row write may add

struct lc_kv_cache {
    lc_ctx *ctx = nullptr;
    lc_buf *keys_q = nullptr, *values_q = nullptr, *key_norms = nullptr, *value_norms = nullptr;
    lc_buf *levels = nullptr, *signs = nullptr;
    uint32_t n_kv_heads = 0, head_dim = 0, bits = 0;
    uint32_t max_positions = 0, physical_positions = 0;
    size_t code_bytes = 0;
};

namespace {

bool pow2(uint32_t v) { return v && !(v & (v - 1)); }
uint32_t ring_of(const lc_kv_cache *c) { return c->physical_positions < c->max_positions ? c->physical_positions : 0; }

}  // namespace

extern "C" {

// QuantizedKvCache::new_with_bits_and_ring (quant_cache.rs:182-228).  physical_positions == max_positions and
// sliding_window == 0 give the full-attention (absolute) layout.
int lc_kv_cache_create(lc_ctx *ctx, uint32_t n_kv_heads, uint32_t head_dim, uint32_t max_positions,
                       uint32_t physical_positions, uint32_t sliding_window, uint32_t bits, lc_kv_cache **out) {
    if (!ctx || !out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_kv_cache_create: NULL argument");
    *out = nullptr;
    if (bits < 2 || bits > 4) return lc_fail(LC_ERR_INVALID_ARGUMENT, "TurboQuant bits must be 2..=4, got %u", bits);
    if (!pow2(head_dim) || head_dim > 512 || head_dim < 32)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "TurboQuant head_dim must be a power of two <= 512, got %u", head_dim);
    LC_REQUIRE(n_kv_heads >= 1 && max_positions >= 1, "lc_kv_cache_create: n_kv_heads and max_positions must be >= 1");
    uint32_t phys = physical_positions < max_positions ? physical_positions : max_positions;
    if (phys < 1) phys = 1;
    const bool is_ring = phys < max_positions;
    if (is_ring && phys < sliding_window + LC_MAX_PREFILL_CHUNK - 1)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "ring capacity %u too small for window %u + prefill slack %u", phys,
                       sliding_window, LC_MAX_PREFILL_CHUNK - 1);
    lc_kv_cache *c = new lc_kv_cache();
    c->ctx = ctx;
    c->n_kv_heads = n_kv_heads;
    c->head_dim = head_dim;
    c->bits = bits;
    c->max_positions = max_positions;
    c->physical_positions = phys;
    c->code_bytes = lc_tq_code_bytes(head_dim, bits);
    const size_t slots = (size_t)phys * n_kv_heads;
    std::vector<float> lv(1u << bits), sg(head_dim);
    lc_tq_levels(head_dim, bits, lv.data());
    lc_tq_signs(head_dim, LC_TQ_SEED, sg.data());
    int st;
    if ((st = lc_buf_alloc(ctx, slots * c->code_bytes, &c->keys_q)) || (st = lc_buf_alloc(ctx, slots * c->code_bytes, &c->values_q)) ||
        (st = lc_buf_alloc(ctx, slots * 2, &c->key_norms)) || (st = lc_buf_alloc(ctx, slots * 2, &c->value_norms)) ||
        (st = lc_buf_from_host(ctx, lv.data(), lv.size() * 4, &c->levels)) ||
        (st = lc_buf_from_host(ctx, sg.data(), sg.size() * 4, &c->signs))) {
        lc_kv_cache_destroy(c);
        return st;
    }
    *out = c;
    return LC_OK;
}

void lc_kv_cache_destroy(lc_kv_cache *c) {
    if (!c) return;
    lc_buf_free(c->keys_q);
    lc_buf_free(c->values_q);
    lc_buf_free(c->key_norms);
    lc_buf_free(c->value_norms);
    lc_buf_free(c->levels);
    lc_buf_free(c->signs);
    delete c;
}

// quant_cache.rs:230-274.
uint32_t lc_kv_cache_physical_positions(const lc_kv_cache *c) { return c ? c->physical_positions : 0; }
uint32_t lc_kv_cache_ring_capacity(const lc_kv_cache *c) { return c ? ring_of(c) : 0; }
size_t lc_kv_cache_code_bytes(const lc_kv_cache *c) { return c ? c->code_bytes : 0; }

int lc_kv_cache_buffers(lc_kv_cache *c, lc_buf **keys_q, lc_buf **key_norms, lc_buf **values_q, lc_buf **value_norms,
                        lc_buf **levels, lc_buf **signs) {
    if (!c) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_kv_cache_buffers: cache is NULL");
    if (keys_q) *keys_q = c->keys_q;
    if (key_norms) *key_norms = c->key_norms;
    if (values_q) *values_q = c->values_q;
    if (value_norms) *value_norms = c->value_norms;
    if (levels) *levels = c->levels;
    if (signs) *signs = c->signs;
    return LC_OK;
}

// QuantizedKvCache::reset (quant_cache.rs:364-380): zero codes and norms; a zero norm annihilates a stale row.
int lc_kv_cache_reset(lc_kv_cache *c) {
    if (!c) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_kv_cache_reset: cache is NULL");
    int st;
    if ((st = lc_buf_zero(c->keys_q, 0, c->keys_q->bytes)) || (st = lc_buf_zero(c->values_q, 0, c->values_q->bytes)) ||
        (st = lc_buf_zero(c->key_norms, 0, c->key_norms->bytes)) || (st = lc_buf_zero(c->value_norms, 0, c->value_norms->bytes)))
        return st;
    return LC_OK;
}

// QuantizedKvCache::write_kv_gpu_into (quant_cache.rs:391-444): encode n_rows fresh K / V rows
// [n_rows, n_kv_heads, head_dim] f16 into the cache at `position`.
int lc_kv_cache_write_kv_gpu_into(lc_kv_cache *c, lc_batch *b, lc_kernels *k, const lc_buf *k_src, const lc_buf *v_src,
                                  uint32_t position, uint32_t n_rows) {
    if (!c || !b || !k || !k_src || !v_src) return lc_fail(LC_ERR_INVALID_ARGUMENT, "kv_cache write: NULL argument");
    if ((uint64_t)position + n_rows > c->max_positions)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "KV write [%u..%llu) exceeds capacity %u", position,
                       (unsigned long long)position + n_rows, c->max_positions);
    const uint32_t ring = ring_of(c);
    int st = lc_encode_kv_turboquant_into(k, b, k_src, c->levels, c->signs, c->keys_q, c->key_norms, c->head_dim, c->n_kv_heads,
                                          n_rows, c->bits, position, ring);
    if (st != LC_OK) return st;
    return lc_encode_kv_turboquant_into(k, b, v_src, c->levels, c->signs, c->values_q, c->value_norms, c->head_dim,
                                        c->n_kv_heads, n_rows, c->bits, position, ring);
}

// QuantizedKvCache::fused_attention_into (quant_cache.rs:548-598): rotate, attend over codes, rotate back, as one
// call of the fused kernel (the reference's rq / vacc scratch buffers are not needed).
int lc_kv_cache_fused_attention_into(lc_kv_cache *c, lc_batch *b, lc_kernels *k, const lc_buf *q, lc_buf *attn_out,
                                     uint32_t seq_len, uint32_t current_pos, uint32_t n_q_heads, uint32_t window,
                                     float softmax_scale) {
    if (!c || !b || !k || !q || !attn_out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "kv_cache attention: NULL argument");
    return lc_tq_attention_into(k, b, q, c->keys_q, c->key_norms, c->values_q, c->value_norms, c->levels, c->signs, attn_out,
                                c->head_dim, seq_len, current_pos, n_q_heads, c->n_kv_heads, window, c->bits, ring_of(c),
                                softmax_scale);
}

// QuantizedKvCache::fused_attention_batch_into (quant_cache.rs:620-700): the prefill / multi-row verify analogue; call
// it after lc_kv_cache_write_kv_gpu_into of the same rows in the same batch.
int lc_kv_cache_fused_attention_batch_into(lc_kv_cache *c, lc_batch *b, lc_kernels *k, const lc_buf *q, lc_buf *attn_out,
                                           uint32_t kv_len, uint32_t start_pos, uint32_t n_rows, uint32_t n_q_heads,
                                           uint32_t window, float softmax_scale) {
    if (!c || !b || !k || !q || !attn_out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "kv_cache attention: NULL argument");
    return lc_tq_attention_prefill_into(k, b, q, c->keys_q, c->key_norms, c->values_q, c->value_norms, c->levels, c->signs,
                                        attn_out, c->head_dim, kv_len, start_pos, n_rows, n_q_heads, c->n_kv_heads, window,
                                        c->bits, ring_of(c), softmax_scale);
}

// QuantizedKvCache::max_snapshot_positions / snapshot_prefix / restore_prefix (quant_cache.rs:311-362): rows
// [0, positions) of the four buffers to / from host memory (codes: positions * n_kv * code_bytes bytes per buffer,
// norms: positions * n_kv * 2).
uint32_t lc_kv_cache_max_snapshot_positions(const lc_kv_cache *c) {
    return c ? (c->physical_positions < c->max_positions ? c->physical_positions : c->max_positions) : 0;
}

int lc_kv_cache_snapshot_prefix(const lc_kv_cache *c, uint32_t positions, void *keys_q, void *values_q, void *key_norms,
                                void *value_norms) {
    if (!c || !keys_q || !values_q || !key_norms || !value_norms)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "kv_cache snapshot: NULL argument");
    const uint32_t lim = lc_kv_cache_max_snapshot_positions(c);
    if (positions > lim) positions = lim;
    const size_t cb = (size_t)positions * c->n_kv_heads * c->code_bytes, nb = (size_t)positions * c->n_kv_heads * 2;
    int st;
    if ((st = lc_buf_download(c->keys_q, 0, keys_q, cb)) || (st = lc_buf_download(c->values_q, 0, values_q, cb)) ||
        (st = lc_buf_download(c->key_norms, 0, key_norms, nb)) || (st = lc_buf_download(c->value_norms, 0, value_norms, nb)))
        return st;
    return LC_OK;
}

int lc_kv_cache_restore_prefix(lc_kv_cache *c, uint32_t positions, const void *keys_q, const void *values_q,
                               const void *key_norms, const void *value_norms) {
    if (!c || !keys_q || !values_q || !key_norms || !value_norms)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "kv_cache restore: NULL argument");
    const uint32_t lim = lc_kv_cache_max_snapshot_positions(c);
    if (positions > lim) positions = lim;
    const size_t cb = (size_t)positions * c->n_kv_heads * c->code_bytes, nb = (size_t)positions * c->n_kv_heads * 2;
    int st;
    if ((st = lc_buf_upload(c->keys_q, 0, keys_q, cb)) || (st = lc_buf_upload(c->values_q, 0, values_q, cb)) ||
        (st = lc_buf_upload(c->key_norms, 0, key_norms, nb)) || (st = lc_buf_upload(c->value_norms, 0, value_norms, nb)))
        return st;
    return LC_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------ lane scheduler --
struct lc_lane_request {
    uint64_t id = 0;
    std::vector<uint32_t> prompt;
    uint32_t max_new_tokens = 1;
};

struct lc_lane_state {
    bool active = false;
    uint64_t id = 0;
    std::vector<uint32_t> prompt, output;
    uint32_t fed = 0;          // prompt tokens already fed
    uint32_t pos = 0;          // position the next fed token occupies
    uint32_t last_token = 0;
    uint32_t max_new_tokens = 1;
    int stop = 0;              // 0 running, else an lc_stop_reason
};

struct lc_finished {
    uint64_t id;
    std::vector<uint32_t> output;
    int reason;
};

struct lc_lane_sched {
    lc_model *model = nullptr;   // may be NULL (host logic only: no pools to zero)
    uint32_t n_lanes = 0, lane_capacity = 0, eos = 0;
    std::vector<lc_lane_state> lanes;
    std::deque<lc_lane_request> queue;
    std::deque<lc_finished> finished;
    uint64_t steps = 0, admitted = 0;
};

namespace {

// LaneState::check_stop (runner.rs:100-109), applied after a generated token.
void check_stop(lc_lane_state &s, bool is_eos, uint32_t capacity) {
    if (is_eos) s.stop = LC_STOP_EOS;
    else if (s.output.size() >= s.max_new_tokens) s.stop = LC_STOP_MAX_TOKENS;
    else if (s.pos >= capacity) s.stop = LC_STOP_CAPACITY;
}

}  // namespace

extern "C" {

int lc_lane_sched_create(lc_model *model, uint32_t n_lanes, uint32_t lane_capacity, uint32_t eos_token, lc_lane_sched **out) {
    if (!out || n_lanes == 0 || lane_capacity == 0)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_lane_sched_create: out is NULL or an empty lane pool");
    lc_lane_sched *s = new lc_lane_sched();
    s->model = model;
    s->n_lanes = n_lanes;
    s->lane_capacity = lane_capacity;
    s->eos = eos_token;
    s->lanes.resize(n_lanes);
    *out = s;
    return LC_OK;
}

void lc_lane_sched_destroy(lc_lane_sched *s) { delete s; }

int lc_lane_sched_submit(lc_lane_sched *s, uint64_t id, const uint32_t *prompt, uint32_t prompt_len, uint32_t max_new_tokens) {
    if (!s || !prompt || prompt_len == 0) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_lane_sched_submit: an empty prompt");
    if (prompt_len > s->lane_capacity)   // "a prompt longer than the lane capacity fails that request's prefill"
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "prompt of %u tokens exceeds the lane capacity %u", prompt_len, s->lane_capacity);
    lc_lane_request r;
    r.id = id;
    r.prompt.assign(prompt, prompt + prompt_len);
    r.max_new_tokens = max_new_tokens ? max_new_tokens : 1;
    s->queue.push_back(std::move(r));
    return LC_OK;
}

// One scheduling round before a decode step: finished lanes are finalized and zeroed, queued requests are admitted
// into free lanes (zeroed first), then tokens[n_lanes] / positions[n_lanes] are filled for a full-width step.
// *n_active = lanes that carry a request; 0 with an empty queue means everything has completed.
int lc_lane_sched_prepare(lc_lane_sched *s, uint32_t *tokens, uint32_t *positions, uint32_t *n_active) {
    if (!s || !tokens || !positions || !n_active) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_lane_sched_prepare: NULL argument");
    for (uint32_t l = 0; l < s->n_lanes; l++) {
        lc_lane_state &ls = s->lanes[l];
        if (ls.active && ls.stop) {
            if (s->model) {
                int st = lc_model_reset_lane(s->model, l);
                if (st != LC_OK) return st;
            }
            s->finished.push_back({ls.id, std::move(ls.output), ls.stop});
            ls = lc_lane_state();
        }
    }
    for (uint32_t l = 0; l < s->n_lanes && !s->queue.empty(); l++) {
        lc_lane_state &ls = s->lanes[l];
        if (ls.active) continue;
        if (s->model) {
            int st = lc_model_reset_lane(s->model, l);
            if (st != LC_OK) return st;
        }
        lc_lane_request r = std::move(s->queue.front());
        s->queue.pop_front();
        ls.active = true;
        ls.id = r.id;
        ls.prompt = std::move(r.prompt);
        ls.max_new_tokens = r.max_new_tokens;
        ls.fed = 0;
        ls.pos = 0;
        ls.stop = 0;
        s->admitted++;
    }
    uint32_t act = 0;
    for (uint32_t l = 0; l < s->n_lanes; l++) {
        const lc_lane_state &ls = s->lanes[l];
        if (!ls.active) {   // idle lanes carry a filler token at position 0; their outputs are discarded
            tokens[l] = 0;
            positions[l] = 0;
            continue;
        }
        tokens[l] = ls.fed < ls.prompt.size() ? ls.prompt[ls.fed] : ls.last_token;
        positions[l] = ls.pos;
        act++;
    }
    *n_active = act;
    return LC_OK;
}

// After the step: next_tokens[n_lanes] are the greedy tokens of the step lc_lane_sched_prepare set up.
int lc_lane_sched_consume(lc_lane_sched *s, const uint32_t *next_tokens) {
    if (!s || !next_tokens) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_lane_sched_consume: NULL argument");
    s->steps++;
    for (uint32_t l = 0; l < s->n_lanes; l++) {
        lc_lane_state &ls = s->lanes[l];
        if (!ls.active || ls.stop) continue;
        const bool in_prompt = ls.fed < ls.prompt.size();
        if (in_prompt) ls.fed++;
        ls.pos++;
        if (in_prompt && ls.fed < ls.prompt.size()) continue;   // still feeding the prompt: this output is discarded
        const uint32_t tok = next_tokens[l];
        ls.output.push_back(tok);
        ls.last_token = tok;
        // after the first generated token `pos` is the position the next token would occupy (runner.rs:160-163)
        check_stop(ls, tok == s->eos, ls.output.size() == 1 ? s->lane_capacity - 1 : s->lane_capacity);
    }
    return LC_OK;
}

// Pop one completed request (completion order).  Returns LC_OK with *n_out = 0 and *reason = 0 when none is ready;
// out_tokens may be NULL to query *n_out only (the request then stays queued).
int lc_lane_sched_pop_finished(lc_lane_sched *s, uint64_t *id, uint32_t *out_tokens, uint32_t capacity, uint32_t *n_out,
                               int *reason) {
    if (!s || !n_out || !reason) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_lane_sched_pop_finished: NULL argument");
    // lanes that stopped on the last consume are finalized here as well, so a caller can drain without another prepare
    for (uint32_t l = 0; l < s->n_lanes; l++) {
        lc_lane_state &ls = s->lanes[l];
        if (ls.active && ls.stop) {
            if (s->model) {
                int st = lc_model_reset_lane(s->model, l);
                if (st != LC_OK) return st;
            }
            s->finished.push_back({ls.id, std::move(ls.output), ls.stop});
            ls = lc_lane_state();
        }
    }
    if (s->finished.empty()) {
        *n_out = 0;
        *reason = 0;
        return LC_OK;
    }
    lc_finished &f = s->finished.front();
    *n_out = (uint32_t)f.output.size();
    *reason = f.reason;
    if (id) *id = f.id;
    if (!out_tokens) return LC_OK;
    if (capacity < f.output.size()) return lc_fail(LC_ERR_INVALID_ARGUMENT, "output buffer holds %u tokens, need %zu", capacity, f.output.size());
    for (size_t i = 0; i < f.output.size(); i++) out_tokens[i] = f.output[i];
    s->finished.pop_front();
    return LC_OK;
}

uint32_t lc_lane_sched_pending(const lc_lane_sched *s) {
    if (!s) return 0;
    uint32_t n = (uint32_t)s->queue.size();
    for (const lc_lane_state &ls : s->lanes) n += ls.active ? 1u : 0u;
    return n;
}

}  // extern "C"
