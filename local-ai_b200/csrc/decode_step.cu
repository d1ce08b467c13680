// One batched decode step of the dense decoder, composed from the kernels of
// this library in the op order of TransformerLayer::forward_decode_batch_turbo
// (local-engine/src/layer.rs:731-868) inside Pipeline::decode_batch_step
// (local-engine/src/pipeline/batched.rs:271-456):
//
//   embed gather (device-side) -> * sqrt(hidden)
//   per layer: rms_norm -> Q -> q_norm -> rope | K, V -> k_norm, v rms_norm(ones) -> rope(K)
//              -> KV encode into the per-lane pool -> attention over codes (rotate, attend, rotate back)
//              -> O -> rms_norm_add -> rms_norm -> gate, up -> gelu_mul -> down -> rms_norm_add
//   final rms_norm -> vocabulary projection (all lanes in one pass) -> optional greedy argmax
// Launch count is cut by issuing Q/K/V and gate/up as grouped matmuls and by the fused forms of
// q_norm+rope, the KV write, and rms_norm_add+rms_norm; the arithmetic and its f16 rounding points
// are those of the unfused sequence.
//
// Everything between ops is f16, as the reference's scratch buffers are
// (layer.rs:873-1036).  The model object owns the KV pools (QuantizedUnifiedKvPool,
// kv_cache/quant_unified_pool.rs:33-181: [n_lanes, lane_rows, n_kv, code_bytes] with
// lane_rows = ring capacity on sliding-window layers) and the scratch; weights are
// borrowed buffers.  The whole step can be captured into one CUDA graph.
#include <math.h>
#include <stdlib.h>
#include <vector>

#include "lc_internal.h"
#include "attention_tq.h"

int lc_matmul_nt_tq2_0_grouped(lc_kernels *k, lc_batch *b, const lc_buf *input, int ng, const lc_buf *const *weights,
                               lc_buf *const *outputs, const uint32_t *ns, uint32_t m, uint32_t kk);

constexpr uint32_t LC_MAX_CHAINS = 4;

struct lc_model_layer {
    const lc_buf *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *wgate = nullptr, *wup = nullptr,
                 *wdown = nullptr;
    const lc_buf *attn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr, *post_attn_norm = nullptr,
                 *ffn_norm = nullptr, *post_ffn_norm = nullptr;
    lc_buf *k_codes = nullptr, *k_norms = nullptr, *v_codes = nullptr, *v_norms = nullptr;
    uint32_t window = 0, ring = 0, lane_rows = 0;
};

struct lc_model {
    lc_ctx *ctx = nullptr;
    lc_kernels *k = nullptr;
    lc_model_config cfg;
    std::vector<lc_model_layer> layers;
    const lc_buf *embed = nullptr, *final_norm = nullptr;
    lc_buf *levels = nullptr, *signs = nullptr, *ones = nullptr;
    lc_buf *x = nullptr, *x2 = nullptr, *normed = nullptr, *q = nullptr, *qfrag = nullptr, *kbuf = nullptr, *vbuf = nullptr,
           *attn = nullptr, *resid = nullptr, *gate = nullptr, *up = nullptr, *ffn = nullptr, *logits = nullptr;
    std::vector<lc_buf *> owned;
    // lane-group chains (see chain_count): side streams, their own kernels objects (split-K scratch is per object) and
    // the fork / join events
    uint32_t default_chains = 1;
    cudaStream_t side_s[LC_MAX_CHAINS - 1] = {};
    lc_kernels *side_k[LC_MAX_CHAINS - 1] = {};
    cudaEvent_t fork_ev = nullptr, join_ev[LC_MAX_CHAINS - 1] = {};
};

namespace {

int alloc(lc_model *m, size_t bytes, lc_buf **out) {
    int st = lc_buf_alloc(m->ctx, bytes, out);
    if (st == LC_OK) m->owned.push_back(*out);
    return st;
}

}  // namespace

extern "C" {

int lc_model_create(lc_ctx *ctx, lc_kernels *k, const lc_model_config *cfg, lc_model **out) {
    if (!ctx || !k || !cfg || !out) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_model_create: NULL argument");
    *out = nullptr;
    const lc_model_config &c = *cfg;
    LC_REQUIRE(c.hidden % 256 == 0 && c.inter % 256 == 0 && (c.n_q_heads * c.head_dim) % 256 == 0,
               "lc_model_create: hidden, inter and n_q*head_dim must be multiples of 256 (TQ2_0 blocks)");
    LC_REQUIRE(c.n_kv_heads >= 1 && c.n_q_heads % c.n_kv_heads == 0, "lc_model_create: n_q_heads %% n_kv_heads != 0");
    LC_REQUIRE(c.kv_bits >= 2 && c.kv_bits <= 4, "lc_model_create: kv_bits %u not in 2..=4", c.kv_bits);
    LC_REQUIRE(c.n_layers >= 1 && c.max_lanes >= 1 && c.max_context >= 1 && c.full_every >= 1,
               "lc_model_create: empty model");
    LC_REQUIRE(c.swa_ring == 0 || c.swa_ring >= c.swa_window, "lc_model_create: ring %u smaller than window %u",
               c.swa_ring, c.swa_window);
    lc_model *m = new lc_model();
    m->ctx = ctx;
    m->k = k;
    m->cfg = c;
    m->layers.resize(c.n_layers);
    const size_t cb = lc_tq_code_bytes(c.head_dim, c.kv_bits);
    int st = LC_OK;
    auto fail = [&](int s) {
        lc_model_destroy(m);
        return s;
    };
    for (uint32_t i = 0; i < c.n_layers; i++) {
        lc_model_layer &L = m->layers[i];
        const bool full = (i % c.full_every) == c.full_every - 1 || c.swa_window == 0;
        L.window = full ? 0 : c.swa_window;
        L.ring = full ? 0 : (c.swa_ring ? c.swa_ring : (uint32_t)lc_swa_ring_capacity(c.swa_window, c.max_context));
        if (L.ring > c.max_context) L.ring = 0, L.window = c.swa_window;  // window never fills: absolute rows
        L.lane_rows = L.ring ? L.ring : c.max_context;
        const size_t rows = (size_t)c.max_lanes * L.lane_rows * c.n_kv_heads;
        if ((st = alloc(m, rows * cb, &L.k_codes)) || (st = alloc(m, rows * cb, &L.v_codes)) ||
            (st = alloc(m, rows * 2, &L.k_norms)) || (st = alloc(m, rows * 2, &L.v_norms)))
            return fail(st);
    }
    // codec constants (TurboQuant::new, turboquant.rs:187-199; seed quant_cache.rs:30)
    std::vector<float> lv(1u << c.kv_bits), sg(c.head_dim);
    lc_tq_levels(c.head_dim, c.kv_bits, lv.data());
    lc_tq_signs(c.head_dim, LC_TQ_SEED, sg.data());
    std::vector<__half> ones(c.head_dim, __float2half(1.0f));
    if ((st = alloc(m, lv.size() * 4, &m->levels)) || (st = alloc(m, sg.size() * 4, &m->signs)) ||
        (st = alloc(m, ones.size() * 2, &m->ones)))
        return fail(st);
    if ((st = lc_buf_upload(m->levels, 0, lv.data(), lv.size() * 4)) ||
        (st = lc_buf_upload(m->signs, 0, sg.data(), sg.size() * 4)) ||
        (st = lc_buf_upload(m->ones, 0, ones.data(), ones.size() * 2)))
        return fail(st);
    const size_t n = c.max_lanes, qd = (size_t)c.n_q_heads * c.head_dim, kd = (size_t)c.n_kv_heads * c.head_dim;
    if ((st = alloc(m, n * c.hidden * 2, &m->x)) || (st = alloc(m, n * c.hidden * 2, &m->x2)) ||
        (st = alloc(m, n * c.hidden * 2, &m->normed)) || (st = alloc(m, n * qd * 2, &m->q)) ||
        (st = alloc(m, n * kd * 2, &m->kbuf)) || (st = alloc(m, n * kd * 2, &m->vbuf)) ||
        (st = alloc(m, n * qd * 2, &m->attn)) || (st = alloc(m, n * c.hidden * 2, &m->resid)) ||
        (st = alloc(m, n * c.inter * 2, &m->gate)) || (st = alloc(m, n * c.inter * 2, &m->up)) ||
        (st = alloc(m, n * c.hidden * 2, &m->ffn)) || (st = alloc(m, n * (size_t)c.vocab * 4, &m->logits)))
        return fail(st);
    // LOCAL_CUDA_QFRAG=0 keeps the attention kernel's own query prologue (same results; for A/B timing and tests)
    const char *qf_env = getenv("LOCAL_CUDA_QFRAG");
    if (!(qf_env && qf_env[0] == '0') && lc_qfrag_supported(c.head_dim, c.kv_bits, c.n_q_heads, c.n_kv_heads) &&
        (st = alloc(m, n * qd * 4, &m->qfrag)))
        return fail(st);
    {
        const char *e = getenv("LOCAL_CUDA_DECODE_CHAINS");
        const long v = e ? strtol(e, nullptr, 10) : 1;
        m->default_chains = v < 1 ? 1u : (v > (long)LC_MAX_CHAINS ? LC_MAX_CHAINS : (uint32_t)v);
    }
    if (cudaEventCreateWithFlags(&m->fork_ev, cudaEventDisableTiming) != cudaSuccess)
        return fail(lc_fail(LC_ERR_CUDA, "lc_model_create: event"));
    for (uint32_t i = 0; i + 1 < LC_MAX_CHAINS; i++) {
        if (cudaStreamCreateWithFlags(&m->side_s[i], cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&m->join_ev[i], cudaEventDisableTiming) != cudaSuccess)
            return fail(lc_fail(LC_ERR_CUDA, "lc_model_create: side stream"));
        if ((st = lc_kernels_create(ctx, &m->side_k[i])) != LC_OK) return fail(st);
    }
    *out = m;
    return LC_OK;
}

void lc_model_destroy(lc_model *m) {
    if (!m) return;
    cudaSetDevice(m->ctx->device);
    for (uint32_t i = 0; i + 1 < LC_MAX_CHAINS; i++) {
        if (m->side_s[i]) {
            cudaStreamSynchronize(m->side_s[i]);
            cudaStreamDestroy(m->side_s[i]);
        }
        if (m->join_ev[i]) cudaEventDestroy(m->join_ev[i]);
        if (m->side_k[i]) lc_kernels_destroy(m->side_k[i]);
    }
    if (m->fork_ev) cudaEventDestroy(m->fork_ev);
    for (lc_buf *b : m->owned) lc_buf_free(b);
    delete m;
}

int lc_model_set_layer(lc_model *m, uint32_t layer, const lc_buf *wq, const lc_buf *wk, const lc_buf *wv,
                       const lc_buf *wo, const lc_buf *wgate, const lc_buf *wup, const lc_buf *wdown,
                       const lc_buf *attn_norm, const lc_buf *q_norm, const lc_buf *k_norm,
                       const lc_buf *post_attn_norm, const lc_buf *ffn_norm, const lc_buf *post_ffn_norm) {
    if (!m || layer >= m->layers.size()) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_model_set_layer: bad layer");
    if (!wq || !wk || !wv || !wo || !wgate || !wup || !wdown || !attn_norm || !q_norm || !k_norm || !post_attn_norm ||
        !ffn_norm || !post_ffn_norm)
        return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_model_set_layer: NULL tensor");
    const lc_model_config &c = m->cfg;
    const size_t qd = (size_t)c.n_q_heads * c.head_dim, kd = (size_t)c.n_kv_heads * c.head_dim;
    auto tq = [](size_t rows, size_t cols) { return rows * (cols / 256) * 66; };
    LC_REQUIRE(wq->bytes >= tq(qd, c.hidden) && wk->bytes >= tq(kd, c.hidden) && wv->bytes >= tq(kd, c.hidden) &&
                   wo->bytes >= tq(c.hidden, qd) && wgate->bytes >= tq(c.inter, c.hidden) &&
                   wup->bytes >= tq(c.inter, c.hidden) && wdown->bytes >= tq(c.hidden, c.inter),
               "lc_model_set_layer: a TQ2_0 tensor is smaller than its shape");
    LC_REQUIRE(attn_norm->bytes >= c.hidden * 2u && post_attn_norm->bytes >= c.hidden * 2u &&
                   ffn_norm->bytes >= c.hidden * 2u && post_ffn_norm->bytes >= c.hidden * 2u &&
                   q_norm->bytes >= c.head_dim * 2u && k_norm->bytes >= c.head_dim * 2u,
               "lc_model_set_layer: a norm weight is smaller than its shape");
    lc_model_layer &L = m->layers[layer];
    L.wq = wq; L.wk = wk; L.wv = wv; L.wo = wo; L.wgate = wgate; L.wup = wup; L.wdown = wdown;
    L.attn_norm = attn_norm; L.q_norm = q_norm; L.k_norm = k_norm; L.post_attn_norm = post_attn_norm;
    L.ffn_norm = ffn_norm; L.post_ffn_norm = post_ffn_norm;
    return LC_OK;
}

int lc_model_set_embedding(lc_model *m, const lc_buf *embed_q4_0, const lc_buf *final_norm) {
    if (!m || !embed_q4_0 || !final_norm) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_model_set_embedding: NULL argument");
    LC_REQUIRE(embed_q4_0->bytes >= (size_t)m->cfg.vocab * (m->cfg.hidden / 32) * 18 &&
                   final_norm->bytes >= m->cfg.hidden * 2u,
               "lc_model_set_embedding: tensor smaller than its shape");
    m->embed = embed_q4_0;
    m->final_norm = final_norm;
    return LC_OK;
}

int lc_model_kv_buffers(lc_model *m, uint32_t layer, lc_buf **k_codes, lc_buf **k_norms, lc_buf **v_codes,
                        lc_buf **v_norms, uint32_t *lane_rows, uint32_t *ring, uint32_t *window) {
    if (!m || layer >= m->layers.size()) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_model_kv_buffers: bad layer");
    lc_model_layer &L = m->layers[layer];
    if (k_codes) *k_codes = L.k_codes;
    if (k_norms) *k_norms = L.k_norms;
    if (v_codes) *v_codes = L.v_codes;
    if (v_norms) *v_norms = L.v_norms;
    if (lane_rows) *lane_rows = L.lane_rows;
    if (ring) *ring = L.ring;
    if (window) *window = L.window;
    return LC_OK;
}

int lc_model_logits_buffer(lc_model *m, lc_buf **logits) {
    if (!m || !logits) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_model_logits_buffer: NULL argument");
    *logits = m->logits;
    return LC_OK;
}

int lc_model_hidden_buffer(lc_model *m, lc_buf **hidden) {
    if (!m || !hidden) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_model_hidden_buffer: NULL argument");
    *hidden = m->normed;
    return LC_OK;
}

// QuantizedUnifiedKvPool::reset_lane (quant_unified_pool.rs:316-346): zero one lane's rows in every layer
// ("a zero norm annihilates the row").
int lc_model_reset_lane(lc_model *m, uint32_t lane) {
    if (!m || lane >= m->cfg.max_lanes) return lc_fail(LC_ERR_INVALID_ARGUMENT, "lc_model_reset_lane: bad lane");
    const size_t cb = lc_tq_code_bytes(m->cfg.head_dim, m->cfg.kv_bits);
    for (lc_model_layer &L : m->layers) {
        const size_t rows = (size_t)L.lane_rows * m->cfg.n_kv_heads;
        int st;
        if ((st = lc_buf_zero(L.k_codes, lane * rows * cb, rows * cb)) || (st = lc_buf_zero(L.v_codes, lane * rows * cb, rows * cb)) ||
            (st = lc_buf_zero(L.k_norms, lane * rows * 2, rows * 2)) || (st = lc_buf_zero(L.v_norms, lane * rows * 2, rows * 2)))
            return st;
    }
    return LC_OK;
}

// The per-layer part of the step for lanes [lane0, lane0 + n): every buffer is addressed through a view that starts
// at the chain's first lane, so the kernels see an ordinary n-lane step.
static int run_layers(lc_model *m, lc_kernels *k, lc_batch *b, const lc_buf *positions, uint32_t lane0, uint32_t n) {
    const lc_model_config &c = m->cfg;
    const uint32_t H = c.hidden, HD = c.head_dim, NQ = c.n_q_heads, NKV = c.n_kv_heads, I = c.inter;
    const uint32_t qd = NQ * HD, kd = NKV * HD;
    const size_t cb = lc_tq_code_bytes(c.head_dim, c.kv_bits);
    auto view = [](const lc_buf *src, size_t off) {
        lc_buf v = *src;
        v.dptr = (char *)src->dptr + off;
        v.bytes = src->bytes - off;
        v.owned = false;
        return v;
    };
    lc_buf pos = view(positions, (size_t)lane0 * 4);
    lc_buf xa = view(m->x, (size_t)lane0 * H * 2), xb = view(m->x2, (size_t)lane0 * H * 2);
    lc_buf normed = view(m->normed, (size_t)lane0 * H * 2), q = view(m->q, (size_t)lane0 * qd * 2);
    lc_buf kbuf = view(m->kbuf, (size_t)lane0 * kd * 2), vbuf = view(m->vbuf, (size_t)lane0 * kd * 2);
    lc_buf attn = view(m->attn, (size_t)lane0 * qd * 2), resid = view(m->resid, (size_t)lane0 * H * 2);
    lc_buf gate = view(m->gate, (size_t)lane0 * I * 2), up = view(m->up, (size_t)lane0 * I * 2);
    lc_buf ffn = view(m->ffn, (size_t)lane0 * H * 2);
    lc_buf qfrag_v = m->qfrag ? view(m->qfrag, (size_t)lane0 * qd * 4) : lc_buf();
    // Worth it while the attention launch is a wave or two (2.34 vs 2.39 ms at 64 lanes); at 512 lanes the KV-write
    // launch's extra transform costs more than the attention prologue saves (11.90 vs 11.85 ms).
    lc_buf *qf = (m->qfrag && n <= 128) ? &qfrag_v : nullptr;
    lc_buf *x = &xa, *xn = &xb;
    const size_t nl = m->layers.size();
    int st;
#define STEP(call) do { if ((st = (call)) != LC_OK) return st; } while (0)
    for (size_t li = 0; li < nl; li++) {
        lc_model_layer &L = m->layers[li];
        const size_t row0 = (size_t)lane0 * L.lane_rows * NKV;
        lc_buf kc = view(L.k_codes, row0 * cb), vc = view(L.v_codes, row0 * cb);
        lc_buf kn = view(L.k_norms, row0 * 2), vn = view(L.v_norms, row0 * 2);
        // Q, K, V in one grouped launch (same activations); q_norm + RoPE fused; the KV write fused
        {
            const lc_buf *ws[3] = {L.wq, L.wk, L.wv};
            lc_buf *os[3] = {&q, &kbuf, &vbuf};
            const uint32_t ns[3] = {qd, kd, kd};
            STEP(lc_matmul_nt_tq2_0_grouped(k, b, &normed, 3, ws, os, ns, n, H));
        }
        // where the tensor-core attention kernel runs, the launch that finishes q also leaves its rotated, scaled
        // fragments, so attention starts on the keys as soon as it may read them
        STEP(lc_qkv_post_frag(k, b, &q, L.q_norm, NQ, &kbuf, &vbuf, L.k_norm, &pos, m->levels, m->signs, &kc, &kn, &vc, &vn,
                              HD, NKV, L.lane_rows, c.kv_bits, n, L.ring, c.rms_eps, c.rope_theta, 1.0f, qf, c.softmax_scale));
        STEP(lc_tq_attention_batched_frag(k, b, &q, &kc, &kn, &vc, &vn, m->levels, m->signs, &attn, &pos, HD, L.lane_rows,
                                          NQ, NKV, L.window, c.kv_bits, n, L.ring, c.softmax_scale, qf));
        STEP(lc_matmul_nt_tq2_0_into(k, b, &attn, L.wo, &ffn, n, qd, H));
        // resid = rms_norm(ffn, post_attn) + x ; normed = rms_norm(resid, ffn_norm)
        STEP(lc_rms_norm_add_norm_into(k, b, &ffn, L.post_attn_norm, x, &resid, L.ffn_norm, &normed, H, n, c.rms_eps));
        STEP(lc_matmul_nt_tq2_0_geglu_into(k, b, &normed, L.wgate, L.wup, &gate, &up, &gate, n, H, I));
        STEP(lc_matmul_nt_tq2_0_into(k, b, &gate, L.wdown, &ffn, n, I, H));
        // x' = rms_norm(ffn, post_ffn) + resid ; normed = rms_norm(x', next layer's attention norm | final norm)
        const lc_buf *next_norm = li + 1 < nl ? m->layers[li + 1].attn_norm : m->final_norm;
        STEP(lc_rms_norm_add_norm_into(k, b, &ffn, L.post_ffn_norm, &resid, xn, next_norm, &normed, H, n, c.rms_eps));
        lc_buf *t = x; x = xn; xn = t;
    }
#undef STEP
    return LC_OK;
}

// How many independent lane groups ("chains") the layers of a step are issued as.  The per-layer kernels of a decode
// step are short and strictly dependent, so one chain leaves most SMs idle most of the time; lanes are independent
// between the embedding and the vocabulary projection, so two or four chains on forked streams fill the gaps (each
// re-reads the layer's weights, from L2 when the chains stay close).  LOCAL_CUDA_DECODE_CHAINS overrides.
static uint32_t chain_count(const lc_model *m, uint32_t n_lanes) {
    uint32_t want = m->default_chains;
    if (n_lanes < 32) want = 1;
    else if (n_lanes < 64 && want > 2) want = 2;
    if (want > LC_MAX_CHAINS) want = LC_MAX_CHAINS;
    return want < 1 ? 1 : want;
}

int lc_model_decode_batch_step_into(lc_model *m, lc_batch *b, const lc_buf *tokens, const lc_buf *positions,
                                    uint32_t n_lanes, uint32_t want_logits, lc_buf *next_tokens) {
    if (!m || !b || !tokens || !positions) return lc_fail(LC_ERR_INVALID_ARGUMENT, "decode_batch_step: NULL argument");
    const lc_model_config &c = m->cfg;
    LC_REQUIRE(n_lanes >= 1 && n_lanes <= c.max_lanes, "decode_batch_step: n_lanes %u not in 1..=%u", n_lanes, c.max_lanes);
    LC_REQUIRE(m->embed && m->final_norm, "decode_batch_step: embedding not set");
    LC_REQUIRE(tokens->bytes >= (size_t)n_lanes * 4 && positions->bytes >= (size_t)n_lanes * 4,
               "decode_batch_step: tokens / positions hold fewer than %u entries", n_lanes);
    for (const lc_model_layer &L : m->layers) LC_REQUIRE(L.wq, "decode_batch_step: a layer has no weights");
    lc_kernels *k = m->k;
    const uint32_t H = c.hidden, n = n_lanes;
    int st;
#define STEP(call) do { if ((st = (call)) != LC_OK) return st; } while (0)
    STEP(lc_embed_rows_q4_0_into(k, b, m->embed, tokens, m->x, n, H, c.vocab, c.embed_scale));
    STEP(lc_rms_norm_into(k, b, m->x, m->layers[0].attn_norm, m->normed, H, n, c.rms_eps));
    const uint32_t chains = chain_count(m, n);
    if (chains <= 1) {
        STEP(run_layers(m, k, b, positions, 0, n));
    } else {
        // fork: chain 0 stays on the batch's stream, chains 1.. run on the model's side streams (captured into the same
        // graph when the batch is capturing); join before the vocabulary projection
        const uint32_t per = ((n + chains - 1) / chains + 7) & ~7u;
        cudaStream_t main_s = b->stream;
        LC_CUDA_TRY(cudaEventRecord(m->fork_ev, main_s));
        uint32_t lane0 = per;
        for (uint32_t ci = 1; ci < chains && lane0 < n; ci++, lane0 += per) {
            lc_kernels *kc = m->side_k[ci - 1];
            kc->batchm = k->batchm; kc->smallm = k->smallm; kc->mma = k->mma; kc->decode_mma = k->decode_mma; kc->decode_tc = k->decode_tc;
            kc->kv_norm_mode = k->kv_norm_mode;
            lc_batch side = *b;
            side.stream = m->side_s[ci - 1];
            side.dispatch_count = 0;
            LC_CUDA_TRY(cudaStreamWaitEvent(side.stream, m->fork_ev, 0));
            st = run_layers(m, kc, &side, positions, lane0, (lane0 + per <= n ? per : n - lane0));
            b->dispatch_count += side.dispatch_count;
            // join even after a failure so that a capture in progress stays well-formed
            cudaEventRecord(m->join_ev[ci - 1], side.stream);
            cudaStreamWaitEvent(main_s, m->join_ev[ci - 1], 0);
            if (st != LC_OK) return st;
        }
        STEP(run_layers(m, k, b, positions, 0, per < n ? per : n));
    }
    if (want_logits || next_tokens) {
        STEP(lc_matmul_nt_q4_0_f32out_into(k, b, m->normed, m->embed, m->logits, n, H, c.vocab));
        if (next_tokens) STEP(lc_argmax_rows_f32_into(k, b, m->logits, next_tokens, n, c.vocab));
    }
#undef STEP
    return LC_OK;
}

}  // extern "C"
