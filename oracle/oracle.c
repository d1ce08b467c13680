/*
 * CPU oracle for the decode hot path of local-ai.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE. It is a plain-C restatement of
 * the reference's own arithmetic (its Rust CPU code where that exists, the
 * Metal shader math elsewhere). Only the test-suite, the smoke check and the
 * benchmark's cpu-baseline leg may load it; the CUDA library never does.
 *
 * Parity status: PINNED against every known-answer test the reference holds
 * for this path (TQ2_0 / Q4_0 block bytes, code_bytes, ring capacity,
 * encode==encode_into, zero vector, FWHT involution ...) — see
 * tests/test_oracle_golden.py.  The reference ships no stored output arrays,
 * and its own toolchain (Rust, Metal) is absent here, so values beyond those
 * known answers are pinned by restating the reference tests' CPU checkers.
 *
 * Each function cites the reference file:line it follows (paths are relative
 * to the reference project root).
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see build.py).
 * -ffp-contract=off matters: the Rust code never fuses a*b+c unless it says
 * mul_add, and bit-exact TurboQuant codes depend on that.
 */
#include <math.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ f16 -- */
/* IEEE binary16, round-to-nearest-even: what crate `half` 2.7.1 does
 * (Cargo.lock:885; call sites qat_recover.rs:38,46,82,93, turboquant.rs:275). */
static inline float h2f(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}
static inline uint16_t f2h(float f) {
    _Float16 v = (_Float16)f;
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}
ORC_API float orc_f16_to_f32(uint16_t h) { return h2f(h); }
ORC_API uint16_t orc_f32_to_f16(float f) { return f2h(f); }

/* ------------------------------------------------- weight block layouts -- */
enum { ORC_Q4_0 = 0, ORC_TQ2_0 = 1 };

/* local-engine/src/qat_recover.rs:23-52 — TQ2_0: 66-byte block = 64 qs bytes
 * then f16 d; element order j in {0,32}, l in 0..4, m in 0..32;
 * q = (qs[j+m] >> 2l) & 3; value = f16(d * (q - 1)). */
ORC_API void orc_dequant_tq2_0(const uint8_t *data, size_t nbytes,
                               size_t num_elements, uint16_t *out) {
    size_t blocks = nbytes / 66, n = 0;
    for (size_t b = 0; b < blocks; b++) {
        const uint8_t *qs = data + b * 66;
        uint16_t dh;
        memcpy(&dh, qs + 64, 2);
        float d = h2f(dh);
        for (int j = 0; j < 64; j += 32)
            for (int l = 0; l < 4; l++)
                for (int m = 0; m < 32; m++) {
                    if (n >= num_elements) return;
                    int q = (qs[j + m] >> (l * 2)) & 3;
                    out[n++] = f2h(d * ((float)q - 1.0f));
                }
    }
}

/* local-engine/src/qat_recover.rs:70-97 — Q4_0: 18-byte block = f16 d then 16
 * bytes; low nibbles are elements 0..15, high nibbles 16..31;
 * value = f16((nibble - 8) * d). */
ORC_API void orc_dequant_q4_0(const uint8_t *data, size_t nbytes,
                              size_t num_elements, uint16_t *out) {
    size_t blocks = nbytes / 18, n = 0;
    for (size_t b = 0; b < blocks; b++) {
        const uint8_t *p = data + b * 18;
        uint16_t dh;
        memcpy(&dh, p, 2);
        float d = h2f(dh);
        float block[32];
        for (int j = 0; j < 16; j++) {
            uint8_t q = p[2 + j];
            block[j] = ((float)(q & 0x0F) - 8.0f) * d;
            block[j + 16] = ((float)(q >> 4) - 8.0f) * d;
        }
        for (int j = 0; j < 32; j++) {
            if (n >= num_elements) return;
            out[n++] = f2h(block[j]);
        }
    }
}

/* f32 expansion exactly as the GPU kernels and the reference's kernel tests
 * see a weight: d*(q-8) / d*(q-1) kept in f32, NOT rounded to f16
 * (shaders/matvec_quant.metal:20-38; local-metal/src/kernels.rs:8804-8805,8834). */
static void expand_row_f32(int fmt, const uint8_t *row, size_t cols, float *dq) {
    if (fmt == ORC_Q4_0) {
        for (size_t b = 0; b < cols / 32; b++) {
            const uint8_t *p = row + b * 18;
            uint16_t dh;
            memcpy(&dh, p, 2);
            float d = h2f(dh);
            for (int i = 0; i < 16; i++) {
                uint8_t q = p[2 + i];
                dq[b * 32 + i] = ((float)(q & 0x0F) - 8.0f) * d;
                dq[b * 32 + 16 + i] = ((float)(q >> 4) - 8.0f) * d;
            }
        }
    } else {
        for (size_t b = 0; b < cols / 256; b++) {
            const uint8_t *qs = row + b * 66;
            uint16_t dh;
            memcpy(&dh, qs + 64, 2);
            float d = h2f(dh);
            for (int j = 0; j < 64; j++) {
                size_t base = b * 256 + (size_t)(j >> 5) * 128 + (size_t)(j & 31);
                for (int l = 0; l < 4; l++)
                    dq[base + (size_t)l * 32] = ((float)((qs[j] >> (2 * l)) & 3) - 1.0f) * d;
            }
        }
    }
}
static size_t row_bytes(int fmt, size_t cols) {
    return fmt == ORC_Q4_0 ? cols / 32 * 18 : cols / 256 * 66;
}
ORC_API void orc_expand_f32(int fmt, const uint8_t *w, size_t rows, size_t cols, float *dq) {
    size_t rb = row_bytes(fmt, cols);
    for (size_t r = 0; r < rows; r++) expand_row_f32(fmt, w + r * rb, cols, dq + r * cols);
}

/* The reference's checker for every quantized matvec/matmul is the naive dot
 * of the f32 expansion with the f16 activations (kernels.rs:8865-8869 cpu_matvec,
 * kernels.rs:9536-9544 cpu_matmul_nt).  The oracle accumulates in f64 so that it
 * is the exact value the fp32-accumulating kernels are compared to.
 * c[m,n] = sum_k a[m,k] * W[n,k]. */
ORC_API void orc_matmul_nt_quant(int fmt, const uint16_t *a, const uint8_t *w,
                                 size_t m, size_t k, size_t n, float *c) {
    size_t rb = row_bytes(fmt, k);
    float *af = (float *)malloc(sizeof(float) * m * k);
    for (size_t i = 0; i < m * k; i++) af[i] = h2f(a[i]);
#pragma omp parallel
    {
        float *dq = (float *)malloc(sizeof(float) * k);
#pragma omp for schedule(static)
        for (long j = 0; j < (long)n; j++) {
            expand_row_f32(fmt, w + (size_t)j * rb, k, dq);
            for (size_t i = 0; i < m; i++) {
                double s = 0.0;
                const float *ar = af + i * k;
                for (size_t p = 0; p < k; p++) s += (double)ar[p] * (double)dq[p];
                c[i * n + (size_t)j] = (float)s;
            }
        }
        free(dq);
    }
    free(af);
}
ORC_API void orc_matvec_quant(int fmt, const uint8_t *w, const uint16_t *x,
                              size_t rows, size_t cols, float *out) {
    orc_matmul_nt_quant(fmt, x, w, 1, cols, rows, out);
}

/* CPU baseline = what the reference can do on a CPU for this op: dequantise the
 * row to f16 with qat_recover (rounding each weight to f16), then the test
 * checker's naive f32 dot in k order (kernels.rs:8865-8869).  Timed by bench.py;
 * `threads` <= 0 means all OpenMP threads. */
ORC_API void orc_baseline_matmul_nt(int fmt, const uint16_t *a, const uint8_t *w,
                                    size_t m, size_t k, size_t n, float *c, int threads) {
    size_t rb = row_bytes(fmt, k);
    float *af = (float *)malloc(sizeof(float) * m * k);
    for (size_t i = 0; i < m * k; i++) af[i] = h2f(a[i]);
    int nt = threads > 0 ? threads : omp_get_max_threads();
#pragma omp parallel num_threads(nt)
    {
        uint16_t *dq = (uint16_t *)malloc(sizeof(uint16_t) * k);
        float *dqf = (float *)malloc(sizeof(float) * k);
#pragma omp for schedule(static)
        for (long j = 0; j < (long)n; j++) {
            if (fmt == ORC_Q4_0) orc_dequant_q4_0(w + (size_t)j * rb, rb, k, dq);
            else orc_dequant_tq2_0(w + (size_t)j * rb, rb, k, dq);
            for (size_t p = 0; p < k; p++) dqf[p] = h2f(dq[p]);
            for (size_t i = 0; i < m; i++) {
                float s = 0.0f;
                const float *ar = af + i * k;
                for (size_t p = 0; p < k; p++) s += dqf[p] * ar[p];
                c[i * n + (size_t)j] = s;
            }
        }
        free(dq);
        free(dqf);
    }
    free(af);
}

/* shaders/tq2_dequant.metal:4-16 — out[i] = scale[i/4] * ((packed[i/4] >> 2(i%4)) & 3).
 * No zero point, one scale per byte; result rounded to f16. */
ORC_API void orc_tq2_dequant(const uint8_t *packed, const uint16_t *scales,
                             uint16_t *out, size_t n) {
    for (size_t i = 0; i < n; i++) {
        size_t bi = i / 4;
        unsigned q = (packed[bi] >> (2 * (i % 4))) & 3u;
        out[i] = f2h(h2f(scales[bi]) * (float)q);
    }
}

/* ------------------------------------------------------------ TurboQuant -- */
/* local-engine/src/turboquant.rs:30-51 */
ORC_API void orc_fwht_normalized(float *v, size_t n) {
    for (size_t len = 1; len < n; len <<= 1)
        for (size_t i = 0; i < n; i += len << 1)
            for (size_t j = i; j < i + len; j++) {
                float a = v[j], b = v[j + len];
                v[j] = a + b;
                v[j + len] = a - b;
            }
    float inv = 1.0f / sqrtf((float)n);
    for (size_t i = 0; i < n; i++) v[i] *= inv;
}

/* local-engine/src/turboquant.rs:66-80 — splitmix64 from state = seed | 1;
 * sign = +1 when the output's low bit is 0. */
ORC_API void orc_tq_signs(size_t dim, uint64_t seed, float *signs) {
    uint64_t state = seed | 1ull;
    for (size_t i = 0; i < dim; i++) {
        state += 0x9E3779B97F4A7C15ull;
        uint64_t z = state;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        signs[i] = (z & 1ull) == 0 ? 1.0f : -1.0f;
    }
}

static int cmp_f32(const void *a, const void *b) {
    float x = *(const float *)a, y = *(const float *)b;
    return (x > y) - (x < y);
}

/* local-engine/src/turboquant.rs:114-166 — Lloyd–Max for N(0,1): 8192-point
 * grid on [-6,6], 100 iterations, f32 throughout, fused mul_add at :121 and
 * :155, nearest centroid with strict '<', final sort. */
ORC_API void orc_lloyd_max_gaussian(unsigned bits, float *levels) {
    enum { N = 8192 };
    const float LO = -6.0f, HI = 6.0f;
    size_t k = (size_t)1 << bits;
    float dx = (HI - LO) / (float)N;
    float *xs = (float *)malloc(sizeof(float) * N);
    float *pdf = (float *)malloc(sizeof(float) * N);
    for (int i = 0; i < N; i++) xs[i] = fmaf((float)i + 0.5f, dx, LO);
    const float frac_1_sqrt_2 = 0.70710678118654752440f;
    const float frac_2_sqrt_pi = 1.12837916709551257390f;
    for (int i = 0; i < N; i++) {
        float x = xs[i];
        pdf[i] = expf(-0.5f * x * x) * frac_1_sqrt_2 * frac_2_sqrt_pi / 2.0f;
    }
    for (size_t i = 0; i < k; i++) {
        float t = ((float)i + 0.5f) / (float)k;
        levels[i] = 6.0f * (t - 0.5f);
    }
    float sum[16], wsum[16];
    for (int it = 0; it < 100; it++) {
        for (size_t j = 0; j < k; j++) sum[j] = wsum[j] = 0.0f;
        for (int i = 0; i < N; i++) {
            float x = xs[i], w = pdf[i];
            size_t best = 0;
            float bd = INFINITY;
            for (size_t j = 0; j < k; j++) {
                float d = fabsf(x - levels[j]);
                if (d < bd) { bd = d; best = j; }
            }
            sum[best] = fmaf(w, x, sum[best]);
            wsum[best] += w;
        }
        for (size_t j = 0; j < k; j++)
            if (wsum[j] > 1e-12f) levels[j] = sum[j] / wsum[j];
    }
    qsort(levels, k, sizeof(float), cmp_f32);
    free(xs);
    free(pdf);
}

/* local-engine/src/turboquant.rs:187-199 — levels pre-scaled by 1/sqrt(dim). */
ORC_API void orc_tq_levels(size_t dim, unsigned bits, float *levels) {
    float scale = 1.0f / sqrtf((float)dim);
    orc_lloyd_max_gaussian(bits, levels);
    for (size_t i = 0; i < ((size_t)1 << bits); i++) levels[i] *= scale;
}

ORC_API size_t orc_tq_code_bytes(size_t dim, unsigned bits) { /* turboquant.rs:203-205 */
    return (dim * bits + 7) / 8;
}

/* local-engine/src/turboquant.rs:293-304 */
static unsigned nearest_level(float v, const float *levels, unsigned k) {
    unsigned best = 0;
    float bd = INFINITY;
    for (unsigned i = 0; i < k; i++) {
        float d = fabsf(v - levels[i]);
        if (d < bd) { bd = d; best = i; }
    }
    return best;
}

/* Encode one vector.  norm_mode 0 follows the Rust codec bit for bit
 * (local-engine/src/turboquant.rs:241-276: sequential f32 sum of squares,
 * x *= 1/norm only when norm > 0, sign flip, FWHT, LSB-first packing).
 * norm_mode 1 follows the Metal kernel's summation order instead
 * (shaders/dequantize_kv.metal:247-257: pairwise tree, stride d/2 .. 1); every
 * other step is arithmetically identical (same butterflies, same operand order).
 * Returns the f16 bit pattern of the norm. */
ORC_API uint16_t orc_tq_encode(const float *x, size_t dim, unsigned bits,
                               const float *signs, const float *levels,
                               uint8_t *codes, int norm_mode) {
    float rot[512], red[512];
    float norm;
    if (norm_mode == 0) {
        float s = 0.0f;
        for (size_t i = 0; i < dim; i++) s += x[i] * x[i];
        norm = sqrtf(s);
    } else {
        for (size_t i = 0; i < dim; i++) red[i] = x[i] * x[i];
        for (size_t stride = dim >> 1; stride > 0; stride >>= 1)
            for (size_t i = 0; i < stride; i++) red[i] += red[i + stride];
        norm = sqrtf(red[0]);
    }
    float inv = norm > 0.0f ? 1.0f / norm : (norm_mode == 0 ? 1.0f : 0.0f);
    for (size_t i = 0; i < dim; i++) {
        float v = x[i];
        if (norm > 0.0f || norm_mode == 1) v = v * inv;
        rot[i] = v * signs[i];
    }
    orc_fwht_normalized(rot, dim);
    size_t cb = orc_tq_code_bytes(dim, bits);
    memset(codes, 0, cb);
    uint32_t acc = 0, nbits = 0;
    size_t idx = 0;
    unsigned k = 1u << bits;
    for (size_t i = 0; i < dim; i++) {
        acc |= nearest_level(rot[i], levels, k) << nbits;
        nbits += bits;
        while (nbits >= 8) {
            codes[idx++] = (uint8_t)(acc & 0xFF);
            acc >>= 8;
            nbits -= 8;
        }
    }
    if (nbits > 0) codes[idx] = (uint8_t)(acc & 0xFF);
    return f2h(norm);
}

/* shaders/attention_flash_tq.metal:33-48 == turboquant.rs BitReader:308-337 */
static inline unsigned unpack_code(const uint8_t *codes, size_t d, unsigned bits) {
    size_t bit_off = d * bits;
    size_t byte = bit_off >> 3;
    unsigned shift = (unsigned)(bit_off & 7);
    unsigned v = codes[byte];
    if (shift + bits > 8) v |= (unsigned)codes[byte + 1] << 8;
    return (v >> shift) & ((1u << bits) - 1u);
}

/* local-engine/src/turboquant.rs:280-291 */
ORC_API void orc_tq_decode(const uint8_t *codes, uint16_t norm, size_t dim, unsigned bits,
                           const float *signs, const float *levels, float *out) {
    for (size_t i = 0; i < dim; i++) out[i] = levels[unpack_code(codes, i, bits)];
    orc_fwht_normalized(out, dim);
    float r = h2f(norm);
    for (size_t i = 0; i < dim; i++) out[i] = out[i] * signs[i] * r;
}

/* KV write, single sequence: shaders/dequantize_kv.metal:216-308 with the slot
 * rule of :236-244 (dispatcher local-metal/src/kernels.rs:4819-4890):
 * input f16 [num_tokens, n_kv, hd]; slot = ((position + tok) % ring)*n_kv + head
 * when ring != 0, else (position + tok)*n_kv + head. */
ORC_API void orc_encode_kv(const uint16_t *input, const float *levels, const float *signs,
                           uint8_t *packed, uint16_t *norms, unsigned hd, unsigned n_kv,
                           unsigned num_tokens, unsigned bits, unsigned position,
                           unsigned ring, int norm_mode) {
    size_t cb = orc_tq_code_bytes(hd, bits);
    float x[512];
    for (unsigned g = 0; g < num_tokens * n_kv; g++) {
        unsigned tok = g / n_kv, head = g % n_kv;
        unsigned logical = position + tok;
        size_t slot = (size_t)(ring ? logical % ring : logical) * n_kv + head;
        for (unsigned i = 0; i < hd; i++) x[i] = h2f(input[(size_t)g * hd + i]);
        norms[slot] = orc_tq_encode(x, hd, bits, signs, levels, packed + slot * cb, norm_mode);
    }
}

/* KV write, one new token per lane: shaders/dequantize_kv.metal:327-407
 * (dispatcher kernels.rs:4901-4979): slot = (lane*lane_capacity + pos%ring)*n_kv + head. */
ORC_API void orc_encode_kv_batched(const uint16_t *input, const float *levels,
                                   const float *signs, uint8_t *packed, uint16_t *norms,
                                   const uint32_t *positions, unsigned hd, unsigned n_kv,
                                   unsigned lane_capacity, unsigned bits, unsigned n_lanes,
                                   unsigned ring, int norm_mode) {
    size_t cb = orc_tq_code_bytes(hd, bits);
    float x[512];
    for (unsigned g = 0; g < n_lanes * n_kv; g++) {
        unsigned lane = g / n_kv, head = g % n_kv;
        unsigned pos = positions[lane];
        unsigned ppos = ring ? pos % ring : pos;
        size_t slot = ((size_t)lane * lane_capacity + ppos) * n_kv + head;
        for (unsigned i = 0; i < hd; i++) x[i] = h2f(input[(size_t)g * hd + i]);
        norms[slot] = orc_tq_encode(x, hd, bits, signs, levels, packed + slot * cb, norm_mode);
    }
}

/* shaders/dequantize_kv.metal:132-189 (dispatcher kernels.rs:4641-4804): logical
 * slots [token_start, num_tokens) x n_kv are written to the f16 output at their
 * logical place; codes are read from the ring slot when ring != 0. */
ORC_API void orc_dequantize_kv(const uint8_t *packed, const uint16_t *norms,
                               const float *levels, const float *signs, uint16_t *out,
                               unsigned hd, unsigned n_kv, unsigned num_tokens,
                               unsigned bits, unsigned token_start, unsigned ring) {
    size_t cb = orc_tq_code_bytes(hd, bits);
    float y[512];
    for (unsigned tok = token_start; tok < num_tokens; tok++)
        for (unsigned head = 0; head < n_kv; head++) {
            size_t g = (size_t)tok * n_kv + head;
            size_t src = (size_t)(ring ? tok % ring : tok) * n_kv + head;
            orc_tq_decode(packed + src * cb, norms[src], hd, bits, signs, levels, y);
            for (unsigned i = 0; i < hd; i++) out[g * hd + i] = f2h(y[i]);
        }
}

/* shaders/attention_flash_tq.metal:58-89: y = (1/sqrt d) H(pre ? s*x : x),
 * then *s when post. */
ORC_API void orc_hadamard_rotate(const float *in, const float *signs, float *out,
                                 unsigned hd, unsigned heads, int pre, int post) {
    for (unsigned h = 0; h < heads; h++) {
        float *o = out + (size_t)h * hd;
        for (unsigned i = 0; i < hd; i++) {
            float x = in[(size_t)h * hd + i];
            o[i] = pre ? x * signs[i] : x;
        }
        orc_fwht_normalized(o, hd);
        if (post)
            for (unsigned i = 0; i < hd; i++) o[i] *= signs[i];
    }
}

/* One (lane, q-head) of attention over packed codes.
 * shaders/attention_flash_tq.metal:154-274 (single) and :569-690 (batched):
 * logit_t = norm_k[t] * sum_d rq_d * levels[Kcode], softmax over the window
 * (pos-window, pos], out_d = sum_t p_t * norm_v[t] * levels[Vcode] / sum p.
 * The shader uses an online softmax split over 8 SIMD-groups; the result is
 * order-independent up to rounding, so the oracle evaluates it in f64.
 * `scale` multiplies the logits (the reference hard-codes 1.0). */
static void attn_codes_one(const float *rq, const uint8_t *kc, const uint16_t *kn,
                           const uint8_t *vc, const uint16_t *vn, const float *levels,
                           float *out, unsigned hd, unsigned bits, size_t slot_base,
                           unsigned n_kv, unsigned kv_head, unsigned win_start,
                           unsigned seq_len, unsigned ring, float scale) {
    size_t cb = orc_tq_code_bytes(hd, bits);
    for (unsigned d = 0; d < hd; d++) out[d] = 0.0f;
    if (seq_len <= win_start) return;
    unsigned n = seq_len - win_start;
    double *logit = (double *)malloc(sizeof(double) * n);
    double mx = -INFINITY;
    for (unsigned t = win_start; t < seq_len; t++) {
        size_t slot = (slot_base + (ring ? t % ring : t)) * n_kv + kv_head;
        const uint8_t *c = kc + slot * cb;
        double dot = 0.0;
        for (unsigned d = 0; d < hd; d++)
            dot += (double)rq[d] * (double)levels[unpack_code(c, d, bits)];
        dot *= (double)h2f(kn[slot]) * (double)scale;
        logit[t - win_start] = dot;
        if (dot > mx) mx = dot;
    }
    double *acc = (double *)calloc(hd, sizeof(double));
    double sum = 0.0;
    for (unsigned t = win_start; t < seq_len; t++) {
        size_t slot = (slot_base + (ring ? t % ring : t)) * n_kv + kv_head;
        const uint8_t *c = vc + slot * cb;
        double w = exp(logit[t - win_start] - mx);
        sum += w;
        double wn = w * (double)h2f(vn[slot]);
        for (unsigned d = 0; d < hd; d++)
            acc[d] += wn * (double)levels[unpack_code(c, d, bits)];
    }
    double inv = sum > 0.0 ? 1.0 / sum : 0.0;
    for (unsigned d = 0; d < hd; d++) out[d] = (float)(acc[d] * inv);
    free(acc);
    free(logit);
}

ORC_API void orc_flash_attention_tq(const float *rq, const uint8_t *kc, const uint16_t *kn,
                                    const uint8_t *vc, const uint16_t *vn,
                                    const float *levels, float *out, unsigned hd,
                                    unsigned kv_len, unsigned current_pos, unsigned n_q,
                                    unsigned n_kv, unsigned window, unsigned bits,
                                    unsigned ring, float scale) {
    unsigned seq_len = kv_len < current_pos + 1 ? kv_len : current_pos + 1;
    unsigned win_start = (window > 0 && current_pos + 1 > window) ? current_pos + 1 - window : 0;
#pragma omp parallel for schedule(dynamic)
    for (int qh = 0; qh < (int)n_q; qh++)
        attn_codes_one(rq + (size_t)qh * hd, kc, kn, vc, vn, levels, out + (size_t)qh * hd,
                       hd, bits, 0, n_kv, (unsigned)qh / (n_q / n_kv), win_start, seq_len,
                       ring, scale);
}

ORC_API void orc_flash_attention_tq_batched(const float *rq, const uint8_t *kc,
                                            const uint16_t *kn, const uint8_t *vc,
                                            const uint16_t *vn, const float *levels,
                                            float *out, const uint32_t *positions,
                                            unsigned hd, unsigned lane_capacity,
                                            unsigned n_q, unsigned n_kv, unsigned window,
                                            unsigned bits, unsigned n_lanes, unsigned ring,
                                            float scale) {
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (int lane = 0; lane < (int)n_lanes; lane++)
        for (int qh = 0; qh < (int)n_q; qh++) {
            unsigned pos = positions[lane];
            unsigned seq_len = pos + 1;
            unsigned win_start = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
            size_t qb = ((size_t)lane * n_q + (size_t)qh) * hd;
            attn_codes_one(rq + qb, kc, kn, vc, vn, levels, out + qb, hd, bits,
                           (size_t)lane * lane_capacity, n_kv, (unsigned)qh / (n_q / n_kv),
                           win_start, seq_len, ring, scale);
        }
}

/* Prefill / multi-row verify attention over codes, shaders/attention_flash_tq.metal:290-423
 * (flash_attention_tq_prefill): query row r sits at absolute position start_pos + r, attends
 * t in [win_start(r), min(kv_len, start_pos + r + 1)) of ONE cache (slot = (t % ring) * n_kv +
 * kv_head), i.e. exactly the single-position kernel with current_pos = start_pos + r.
 * rq, out: [n_rows, n_q, hd] f32. */
ORC_API void orc_flash_attention_tq_prefill(const float *rq, const uint8_t *kc, const uint16_t *kn,
                                            const uint8_t *vc, const uint16_t *vn,
                                            const float *levels, float *out, unsigned hd,
                                            unsigned kv_len, unsigned start_pos, unsigned n_rows,
                                            unsigned n_q, unsigned n_kv, unsigned window,
                                            unsigned bits, unsigned ring, float scale) {
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (int r = 0; r < (int)n_rows; r++)
        for (int qh = 0; qh < (int)n_q; qh++) {
            unsigned pos = start_pos + (unsigned)r;
            unsigned seq_len = kv_len < pos + 1 ? kv_len : pos + 1;
            unsigned win_start = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
            size_t qb = ((size_t)r * n_q + (size_t)qh) * hd;
            attn_codes_one(rq + qb, kc, kn, vc, vn, levels, out + qb, hd, bits, 0, n_kv,
                           (unsigned)qh / (n_q / n_kv), win_start, seq_len, ring, scale);
        }
}

/* The query-tiled variant, shaders/attention_flash_tq.metal:425-556
 * (flash_attention_tq_prefill_tiled): same rows and windows, but every K / V element is first
 * rounded to half as `half(norm * levels[code])` (:497-498) and the dot products run over those
 * rounded tiles; the shader's own test holds it to 5e-3 of the non-tiled kernel
 * (local-metal/src/kernels.rs:10287-10448).  Evaluated in f64 over the f16-rounded elements. */
ORC_API void orc_flash_attention_tq_prefill_tiled(const float *rq, const uint8_t *kc,
                                                  const uint16_t *kn, const uint8_t *vc,
                                                  const uint16_t *vn, const float *levels,
                                                  float *out, unsigned hd, unsigned kv_len,
                                                  unsigned start_pos, unsigned n_rows, unsigned n_q,
                                                  unsigned n_kv, unsigned window, unsigned bits,
                                                  unsigned ring, float scale) {
    size_t cb = orc_tq_code_bytes(hd, bits);
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (int r = 0; r < (int)n_rows; r++)
        for (int qh = 0; qh < (int)n_q; qh++) {
            unsigned pos = start_pos + (unsigned)r, kvh = (unsigned)qh / (n_q / n_kv);
            unsigned seq_len = kv_len < pos + 1 ? kv_len : pos + 1;
            unsigned win_start = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
            size_t qb = ((size_t)r * n_q + (size_t)qh) * hd;
            float *o = out + qb;
            for (unsigned d = 0; d < hd; d++) o[d] = 0.0f;
            if (seq_len <= win_start) continue;
            unsigned n = seq_len - win_start;
            double *logit = (double *)malloc(sizeof(double) * n);
            double *acc = (double *)calloc(hd, sizeof(double));
            double mx = -INFINITY, sum = 0.0;
            for (unsigned t = win_start; t < seq_len; t++) {
                size_t slot = (size_t)(ring ? t % ring : t) * n_kv + kvh;
                const uint8_t *c = kc + slot * cb;
                float nk = h2f(kn[slot]);
                double dot = 0.0;
                for (unsigned d = 0; d < hd; d++)
                    dot += (double)rq[qb + d] * (double)h2f(f2h(nk * levels[unpack_code(c, d, bits)]));
                dot *= (double)scale;
                logit[t - win_start] = dot;
                if (dot > mx) mx = dot;
            }
            for (unsigned t = win_start; t < seq_len; t++) {
                size_t slot = (size_t)(ring ? t % ring : t) * n_kv + kvh;
                const uint8_t *c = vc + slot * cb;
                float nv = h2f(vn[slot]);
                double w = exp(logit[t - win_start] - mx);
                sum += w;
                for (unsigned d = 0; d < hd; d++)
                    acc[d] += w * (double)h2f(f2h(nv * levels[unpack_code(c, d, bits)]));
            }
            double inv = sum > 0.0 ? 1.0 / sum : 0.0;
            for (unsigned d = 0; d < hd; d++) o[d] = (float)(acc[d] * inv);
            free(acc);
            free(logit);
        }
}

/* The call sequence the KV containers always issue around the code-space
 * kernel (local-engine/src/kv_cache/quant_cache.rs:565-596,
 * quant_unified_pool.rs:218-256): rq = R(q) from f16 q, attention in rotated
 * space, out = f16(R^-1(acc)).  positions == NULL means the single-sequence
 * form with n_lanes == 1 and current_pos / kv_len given. */
ORC_API void orc_tq_attention_fused(const uint16_t *q, const uint8_t *kc, const uint16_t *kn,
                                    const uint8_t *vc, const uint16_t *vn,
                                    const float *levels, const float *signs, uint16_t *out,
                                    const uint32_t *positions, unsigned hd,
                                    unsigned lane_capacity, unsigned n_q, unsigned n_kv,
                                    unsigned window, unsigned bits, unsigned n_lanes,
                                    unsigned ring, float scale, unsigned kv_len,
                                    unsigned current_pos) {
    size_t total = (size_t)n_lanes * n_q * hd;
    float *qf = (float *)malloc(sizeof(float) * total);
    float *rq = (float *)malloc(sizeof(float) * total);
    float *acc = (float *)malloc(sizeof(float) * total);
    for (size_t i = 0; i < total; i++) qf[i] = h2f(q[i]);
    orc_hadamard_rotate(qf, signs, rq, hd, n_lanes * n_q, 1, 0);
    if (positions)
        orc_flash_attention_tq_batched(rq, kc, kn, vc, vn, levels, acc, positions, hd,
                                       lane_capacity, n_q, n_kv, window, bits, n_lanes, ring,
                                       scale);
    else
        orc_flash_attention_tq(rq, kc, kn, vc, vn, levels, acc, hd, kv_len, current_pos, n_q,
                               n_kv, window, bits, ring, scale);
    orc_hadamard_rotate(acc, signs, qf, hd, n_lanes * n_q, 0, 1);
    for (size_t i = 0; i < total; i++) out[i] = f2h(qf[i]);
    free(qf);
    free(rq);
    free(acc);
}

/* FP16-KV causal / windowed attention for one query position.  This is the
 * math shared by shaders/flash_decoding.metal:10-189, attention_flash.metal
 * :398-503 (windowed split) and attention_sliding.metal:18-78, and it is the
 * CPU softmax reference the reference's own tests use (kernels.rs:8497-8528):
 * scores over t in [win_start, seq_len), softmax scale 1.0 unless `scale` says
 * otherwise, K/V f16 [kv_len, n_kv, hd], output f16. */
ORC_API void orc_attention_f16(const uint16_t *q, const uint16_t *k, const uint16_t *v,
                               uint16_t *out, unsigned hd, unsigned kv_len,
                               unsigned current_pos, unsigned n_q, unsigned n_kv,
                               unsigned window, float scale) {
    unsigned seq_len = kv_len < current_pos + 1 ? kv_len : current_pos + 1;
    unsigned win_start = (window > 0 && current_pos + 1 > window) ? current_pos + 1 - window : 0;
#pragma omp parallel for schedule(dynamic)
    for (int qh = 0; qh < (int)n_q; qh++) {
        unsigned kvh = (unsigned)qh / (n_q / n_kv);
        uint16_t *o = out + (size_t)qh * hd;
        if (seq_len <= win_start) {
            for (unsigned d = 0; d < hd; d++) o[d] = 0;
            continue;
        }
        unsigned n = seq_len - win_start;
        double *logit = (double *)malloc(sizeof(double) * n);
        double *acc = (double *)calloc(hd, sizeof(double));
        double mx = -INFINITY, sum = 0.0;
        for (unsigned t = win_start; t < seq_len; t++) {
            const uint16_t *kr = k + ((size_t)t * n_kv + kvh) * hd;
            double dot = 0.0;
            for (unsigned d = 0; d < hd; d++)
                dot += (double)h2f(q[(size_t)qh * hd + d]) * (double)h2f(kr[d]);
            dot *= (double)scale;
            logit[t - win_start] = dot;
            if (dot > mx) mx = dot;
        }
        for (unsigned t = win_start; t < seq_len; t++) {
            const uint16_t *vr = v + ((size_t)t * n_kv + kvh) * hd;
            double w = exp(logit[t - win_start] - mx);
            sum += w;
            for (unsigned d = 0; d < hd; d++) acc[d] += w * (double)h2f(vr[d]);
        }
        for (unsigned d = 0; d < hd; d++) o[d] = f2h((float)(acc[d] / sum));
        free(acc);
        free(logit);
    }
}

/* local-engine/src/kv_cache/quant_cache.rs:39-54 */
ORC_API size_t orc_swa_ring_capacity(size_t window, size_t max_positions) {
    size_t min_safe = window + 256 - 1;
    size_t v = window * 2 > min_safe ? window * 2 : min_safe;
    size_t p = 1;
    while (p < v) p <<= 1;
    return p < max_positions ? p : max_positions;
}

/* ------------------------------------------------- per-layer small ops -- */
/* shaders/rms_norm.metal:4-43 (+ :48-88 with residual): out = f16(x * rsqrt(mean(x^2)+eps) * w [+ r]).
 * The shader reduces in f32 in an unspecified order; the oracle sums in f64
 * and forms the scale in f32 as the shader does. `residual` may be NULL. */
ORC_API void orc_rms_norm(const uint16_t *in, const uint16_t *weight, const uint16_t *residual,
                          uint16_t *out, unsigned dim, unsigned rows, float eps) {
    for (unsigned r = 0; r < rows; r++) {
        const uint16_t *x = in + (size_t)r * dim;
        double s = 0.0;
        for (unsigned i = 0; i < dim; i++) { double v = h2f(x[i]); s += v * v; }
        float rms = 1.0f / sqrtf((float)s / (float)dim + eps);
        for (unsigned i = 0; i < dim; i++) {
            float val = h2f(x[i]) * rms * h2f(weight[i]);
            if (residual) val += h2f(residual[(size_t)r * dim + i]);
            out[(size_t)r * dim + i] = f2h(val);
        }
    }
}

/* shaders/qk_norm.metal:6-55: per-head RMSNorm in place with learned weights. */
ORC_API void orc_qk_norm(uint16_t *qk, const uint16_t *weight, unsigned hd, unsigned heads,
                         float eps) {
    orc_rms_norm(qk, weight, NULL, qk, hd, heads, eps);
}

/* shaders/rope.metal:14-53 (one position) and :157-196 (per-lane positions):
 * NEOX half-split pairs (i, i+hd/2), freq = theta^(-2i/hd), only the first
 * floor(hd*factor)/2 pairs rotate.  qk is [rows, heads, hd]; positions has one
 * entry per row. */
ORC_API void orc_rope(uint16_t *qk, const uint32_t *positions, float theta, unsigned hd,
                      unsigned heads, unsigned rows, float factor) {
    unsigned half = hd / 2;
    unsigned angles = (unsigned)((float)hd * factor) / 2;
    for (unsigned r = 0; r < rows; r++)
        for (unsigned h = 0; h < heads; h++) {
            uint16_t *p = qk + ((size_t)r * heads + h) * hd;
            for (unsigned i = 0; i < angles && i < half; i++) {
                float x0 = h2f(p[i]), x1 = h2f(p[i + half]);
                float freq = 1.0f / powf(theta, (float)(2 * i) / (float)hd);
                float ang = (float)positions[r] * freq;
                float c = cosf(ang), s = sinf(ang);
                p[i] = f2h(x0 * c - x1 * s);
                p[i + half] = f2h(x0 * s + x1 * c);
            }
        }
}

/* shaders/gelu.metal:23-37: tanh-form GELU(a) * b, inner clamped to +-10. */
ORC_API void orc_gelu_mul(const uint16_t *a, const uint16_t *b, uint16_t *out, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float x = h2f(a[i]);
        float x3 = x * x * x;
        float inner = 0.7978845608f * (x + 0.044715f * x3);
        inner = inner < -10.0f ? -10.0f : (inner > 10.0f ? 10.0f : inner);
        float g = 0.5f * x * (1.0f + tanhf(inner));
        out[i] = f2h(g * h2f(b[i]));
    }
}

/* shaders/residual_add.metal:5-15: half + half, one rounding. */
ORC_API void orc_residual_add(const uint16_t *a, const uint16_t *b, uint16_t *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = f2h(h2f(a[i]) + h2f(b[i]));
}

/* shaders/scale_in_place.metal:5-15 */
ORC_API void orc_scale_in_place(uint16_t *data, float scalar, size_t n) {
    for (size_t i = 0; i < n; i++) data[i] = f2h(h2f(data[i]) * scalar);
}

/* shaders/scale_in_place.metal:22-37 */
ORC_API void orc_gather_strided_f16(const uint16_t *src, uint16_t *dst, unsigned row_stride,
                                    unsigned base_off, unsigned pld, unsigned n_rows) {
    for (unsigned i = 0; i < n_rows; i++)
        for (unsigned p = 0; p < pld; p++)
            dst[(size_t)i * pld + p] = src[(size_t)i * row_stride + base_off + p];
}

/* shaders/scale_in_place.metal:39-48 */
ORC_API void orc_logit_softcap(float *data, float cap, size_t n) {
    for (size_t i = 0; i < n; i++) data[i] = cap * tanhf(data[i] / cap);
}

/* local-engine/src/sampler.rs:148-158: first maximum wins. */
ORC_API uint32_t orc_argmax(const float *v, size_t n) {
    size_t best = 0;
    float bv = -INFINITY;
    for (size_t i = 0; i < n; i++)
        if (v[i] > bv) { bv = v[i]; best = i; }
    return (uint32_t)best;
}

/* Embedding row gather: the reference dequantises the token's row of the
 * Q4_0 table on the CPU (local-engine/src/layer.rs:255-281 via
 * qat_recover::dequant_into), i.e. f16((q-8)*d). */
ORC_API void orc_embed_rows_q4_0(const uint8_t *table, const uint32_t *tokens, unsigned n,
                                 unsigned cols, uint16_t *out) {
    size_t rb = (size_t)cols / 32 * 18;
    for (unsigned i = 0; i < n; i++)
        orc_dequant_q4_0(table + (size_t)tokens[i] * rb, rb, cols, out + (size_t)i * cols);
}

/* ---------------------------------------------- decode step (composition) -- */
/* One decoder layer's tensors.  TQ2_0 matrices are [out, in] row-major blocks. */
typedef struct {
    const uint8_t *wq, *wk, *wv, *wo, *wgate, *wup, *wdown;
    const uint16_t *attn_norm, *q_norm, *k_norm, *post_attn_norm, *ffn_norm, *post_ffn_norm;
    uint8_t *k_codes, *v_codes; /* pool [n_lanes, lane_rows, n_kv, code_bytes] */
    uint16_t *k_norms, *v_norms; /* [n_lanes, lane_rows, n_kv] */
    uint32_t window;             /* 0 = full attention */
    uint32_t ring;               /* 0 = absolute rows */
    uint32_t lane_rows;          /* physical rows per lane */
} orc_layer;

typedef struct {
    uint32_t hidden, n_q, n_kv, hd, inter, vocab, n_layers, bits;
    float eps, rope_theta, softmax_scale, embed_scale;
    const uint8_t *embed; /* Q4_0 [vocab, hidden], tied with the output projection */
    const uint16_t *final_norm;
    const float *levels, *signs;
    const orc_layer *layers;
} orc_model;

/* Which arithmetic the decode step's projections use: 0 = the f64-accumulating checker (orc_matmul_nt_quant),
 * 1 = the CPU baseline's (orc_baseline_matmul_nt: weights rounded to f16, naive f32 dot), which is what the
 * reference would run on a CPU and what the bench times. */
static int g_step_baseline_matmul = 0;
ORC_API void orc_set_step_baseline_matmul(int on) { g_step_baseline_matmul = on; }
static void step_matmul(int fmt, const uint16_t *a, const uint8_t *w, size_t m, size_t k, size_t n, float *c) {
    if (g_step_baseline_matmul) orc_baseline_matmul_nt(fmt, a, w, m, k, n, c, 0);
    else orc_matmul_nt_quant(fmt, a, w, m, k, n, c);
}

static void f32_to_f16_vec(const float *s, uint16_t *d, size_t n) {
    for (size_t i = 0; i < n; i++) d[i] = f2h(s[i]);
}

/* One batched decode step in the op order of
 * TransformerLayer::forward_decode_batch_turbo (local-engine/src/layer.rs:731-868)
 * inside Pipeline::decode_batch_step (local-engine/src/pipeline/batched.rs:271-456):
 * embed gather, *sqrt(hidden), per layer {rms_norm, Q, q_norm, rope, K, V,
 * k_norm, v rms_norm(ones), rope(K), KV encode, code-space attention, O,
 * rms_norm_add, rms_norm, gate, up, gelu_mul, down, rms_norm_add}, final
 * rms_norm, vocab projection to f32 logits.  Every activation between ops is
 * f16, as the reference's scratch buffers are (layer.rs:873-1036).
 * The per-layer-embedding branch, layer scalars and the logit soft-cap are not
 * part of the synthetic model.  `hidden_out` (f16 [n, hidden], may be NULL)
 * receives the final normed rows. */
ORC_API void orc_decode_batch_step(const orc_model *m, const uint32_t *tokens,
                                   const uint32_t *positions, unsigned n, float *logits,
                                   uint16_t *hidden_out, int norm_mode) {
    unsigned H = m->hidden, HD = m->hd, NQ = m->n_q, NKV = m->n_kv, I = m->inter;
    size_t qd = (size_t)NQ * HD, kd = (size_t)NKV * HD;
    uint16_t *x = malloc(2 * (size_t)n * H), *normed = malloc(2 * (size_t)n * H);
    uint16_t *q = malloc(2 * n * qd), *k = malloc(2 * n * kd), *v = malloc(2 * n * kd);
    uint16_t *attn = malloc(2 * n * qd), *resid = malloc(2 * (size_t)n * H);
    uint16_t *gate = malloc(2 * (size_t)n * I), *up = malloc(2 * (size_t)n * I);
    uint16_t *ffn = malloc(2 * (size_t)n * H), *ones = malloc(2 * (size_t)HD);
    size_t big = (size_t)n * (I > qd ? I : qd);
    float *tmp = malloc(sizeof(float) * big);
    for (unsigned i = 0; i < HD; i++) ones[i] = f2h(1.0f);

    orc_embed_rows_q4_0(m->embed, tokens, n, H, x);
    orc_scale_in_place(x, m->embed_scale, (size_t)n * H);
    for (unsigned li = 0; li < m->n_layers; li++) {
        const orc_layer *L = &m->layers[li];
        orc_rms_norm(x, L->attn_norm, NULL, normed, H, n, m->eps);
        step_matmul(ORC_TQ2_0, normed, L->wq, n, H, qd, tmp);
        f32_to_f16_vec(tmp, q, n * qd);
        orc_qk_norm(q, L->q_norm, HD, n * NQ, m->eps);
        orc_rope(q, positions, m->rope_theta, HD, NQ, n, 1.0f);
        step_matmul(ORC_TQ2_0, normed, L->wk, n, H, kd, tmp);
        f32_to_f16_vec(tmp, k, n * kd);
        step_matmul(ORC_TQ2_0, normed, L->wv, n, H, kd, tmp);
        f32_to_f16_vec(tmp, v, n * kd);
        orc_qk_norm(k, L->k_norm, HD, n * NKV, m->eps);
        orc_rms_norm(v, ones, NULL, v, HD, n * NKV, m->eps);
        orc_rope(k, positions, m->rope_theta, HD, NKV, n, 1.0f);
        orc_encode_kv_batched(k, m->levels, m->signs, L->k_codes, L->k_norms, positions, HD,
                              NKV, L->lane_rows, m->bits, n, L->ring, norm_mode);
        orc_encode_kv_batched(v, m->levels, m->signs, L->v_codes, L->v_norms, positions, HD,
                              NKV, L->lane_rows, m->bits, n, L->ring, norm_mode);
        orc_tq_attention_fused(q, L->k_codes, L->k_norms, L->v_codes, L->v_norms, m->levels,
                               m->signs, attn, positions, HD, L->lane_rows, NQ, NKV, L->window,
                               m->bits, n, L->ring, m->softmax_scale, 0, 0);
        step_matmul(ORC_TQ2_0, attn, L->wo, n, qd, H, tmp);
        f32_to_f16_vec(tmp, ffn, (size_t)n * H);
        orc_rms_norm(ffn, L->post_attn_norm, x, resid, H, n, m->eps);
        orc_rms_norm(resid, L->ffn_norm, NULL, normed, H, n, m->eps);
        step_matmul(ORC_TQ2_0, normed, L->wgate, n, H, I, tmp);
        f32_to_f16_vec(tmp, gate, (size_t)n * I);
        step_matmul(ORC_TQ2_0, normed, L->wup, n, H, I, tmp);
        f32_to_f16_vec(tmp, up, (size_t)n * I);
        orc_gelu_mul(gate, up, gate, (size_t)n * I);
        step_matmul(ORC_TQ2_0, gate, L->wdown, n, I, H, tmp);
        f32_to_f16_vec(tmp, ffn, (size_t)n * H);
        orc_rms_norm(ffn, L->post_ffn_norm, resid, x, H, n, m->eps);
    }
    orc_rms_norm(x, m->final_norm, NULL, normed, H, n, m->eps);
    if (hidden_out) memcpy(hidden_out, normed, 2 * (size_t)n * H);
    if (logits) step_matmul(ORC_Q4_0, normed, m->embed, n, H, m->vocab, logits);
    free(x); free(normed); free(q); free(k); free(v); free(attn); free(resid);
    free(gate); free(up); free(ffn); free(ones); free(tmp);
}

ORC_API int orc_num_threads(void) { return omp_get_max_threads(); }
/* The bench sets the thread count itself (a launcher may export OMP_NUM_THREADS=1 to every rank). */
ORC_API void orc_set_num_threads(int n) { if (n > 0) omp_set_num_threads(n); }
