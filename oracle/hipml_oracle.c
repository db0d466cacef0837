/*
 * CPU oracle for the hipml full-attention hot path: TEST INFRASTRUCTURE ONLY
 * (see hipml_oracle.h). Scalar f32, the reference's loop and summation order,
 * no fused multiply-add (compile with -ffp-contract=off).
 */
#include "hipml_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------- f16 <-> f32
 * crates/hipml-core/src/kv.rs:94-165. */

static float bits_to_f32(uint32_t b) {
    float f;
    memcpy(&f, &b, 4);
    return f;
}

static uint32_t f32_to_bits(float f) {
    uint32_t b;
    memcpy(&b, &f, 4);
    return b;
}

float hipml_oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu;
    if (e == 0) {
        /* zero or subnormal: m * 2^-24 is exact in f32 */
        float mag = (float)m * bits_to_f32((127u - 24u) << 23);
        return sign ? -mag : mag;
    }
    if (e == 0x1f) return bits_to_f32(sign | 0x7f800000u | (m << 13));
    return bits_to_f32(sign | ((e + 112u) << 23) | (m << 13));
}

/* Round-to-nearest-even of `mant` shifted right by `shift` bits. */
static uint32_t rne_shift(uint32_t mant, int shift) {
    uint32_t kept = mant >> shift;
    uint32_t rem = mant & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (kept & 1u))) kept += 1;
    return kept;
}

uint16_t hipml_oracle_f32_to_f16(float v) {
    uint32_t x = f32_to_bits(v);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    int e = (int)((x >> 23) & 0xffu);
    uint32_t mant = x & 0x007fffffu;

    if (e == 0xff) { /* inf / nan: keep a nan a nan */
        uint16_t payload = mant ? (uint16_t)((mant >> 13) | 1u) : 0;
        return (uint16_t)(sign | 0x7c00u | payload);
    }
    e -= 112; /* rebias 127 -> 15 */
    if (e >= 0x1f) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return sign; /* below half the smallest subnormal */
        /* subnormal result: shift the 24-bit significand down */
        return (uint16_t)(sign | rne_shift(mant | 0x00800000u, 14 - e));
    }
    uint32_t m = rne_shift(mant, 13);
    if (m == 0x400u) { /* mantissa carried into the exponent */
        m = 0;
        e += 1;
        if (e >= 0x1f) return (uint16_t)(sign | 0x7c00u);
    }
    return (uint16_t)(sign | ((uint32_t)e << 10) | m);
}

/* -------------------------------------------------------------- q8_0 blocks
 * crates/hipml-core/src/kv.rs:176-200, 238-290, 306-329. */

void hipml_oracle_quantize_block_q8(const float *xs, uint8_t *out) {
    float amax = 0.0f;
    for (int j = 0; j < HIPML_KV_BLOCK; j++) {
        float a = fabsf(xs[j]);
        /* Rust's f32::max: a NaN operand is ignored */
        if (a > amax) amax = a;
    }
    float d = amax / 127.0f;
    float id = d > 0.0f ? 1.0f / d : 0.0f; /* from the f32 d, not the rounded scale */
    uint16_t hs = hipml_oracle_f32_to_f16(d);
    out[0] = (uint8_t)(hs & 0xff);
    out[1] = (uint8_t)(hs >> 8);
    for (int j = 0; j < HIPML_KV_BLOCK; j++) {
        float r = roundf(xs[j] * id); /* f32::round: half away from zero */
        if (r < -127.0f) r = -127.0f;
        if (r > 127.0f) r = 127.0f;
        /* `as i8` of a NaN is 0 in Rust */
        int8_t q = (r != r) ? 0 : (int8_t)r;
        out[2 + j] = (uint8_t)q;
    }
}

void hipml_oracle_quantize_q8(const float *values, size_t n, uint8_t *out) {
    for (size_t b = 0; b < n / HIPML_KV_BLOCK; b++)
        hipml_oracle_quantize_block_q8(values + b * HIPML_KV_BLOCK, out + b * HIPML_Q8_BLOCK_BYTES);
}

static void block_f32_q8(const uint8_t *src, float *out) {
    float d = hipml_oracle_f16_to_f32((uint16_t)(src[0] | (src[1] << 8)));
    for (int j = 0; j < HIPML_KV_BLOCK; j++) out[j] = d * (float)(int8_t)src[2 + j];
}

void hipml_oracle_dequantize_q8(const uint8_t *bytes, size_t n_bytes, float *out) {
    for (size_t b = 0; b < n_bytes / HIPML_Q8_BLOCK_BYTES; b++)
        block_f32_q8(bytes + b * HIPML_Q8_BLOCK_BYTES, out + b * HIPML_KV_BLOCK);
}

static uint64_t xorshift64star(uint64_t *state) {
    uint64_t x = *state;
    x ^= x >> 12;
    x ^= x << 25;
    x ^= x >> 27;
    *state = x;
    return x * 0x2545F4914F6CDD1DULL;
}

void hipml_oracle_synthetic_blocks_q8(size_t n_blocks, uint64_t seed, uint8_t *out) {
    uint64_t s = seed | 1;
    for (size_t b = 0; b < n_blocks; b++) {
        uint8_t *blk = out + b * HIPML_Q8_BLOCK_BYTES;
        /* scale in [0.01, 0.05): a normal f16 */
        float d = 0.01f + (float)(xorshift64star(&s) % 1000) * 0.00004f;
        uint16_t hs = hipml_oracle_f32_to_f16(d);
        blk[0] = (uint8_t)(hs & 0xff);
        blk[1] = (uint8_t)(hs >> 8);
        for (int j = 0; j < HIPML_KV_BLOCK; j++) blk[2 + j] = (uint8_t)(xorshift64star(&s) >> 24);
    }
}

/* ------------------------------------------------------------------------ rng
 * crates/hipml-core/src/rng.rs:13-49. */

uint64_t hipml_oracle_rng_new(uint64_t seed) { return seed | 1; }

uint64_t hipml_oracle_rng_next_u64(uint64_t *state) { return xorshift64star(state); }

float hipml_oracle_rng_uniform(uint64_t *state) {
    return (float)(xorshift64star(state) >> 40) / 16777216.0f;
}

float hipml_oracle_rng_normal(uint64_t *state) {
    float u1 = hipml_oracle_rng_uniform(state);
    if (!(u1 > 1e-7f)) u1 = 1e-7f;
    float u2 = hipml_oracle_rng_uniform(state);
    const float tau = 6.28318530717958647692528676655900577f;
    return sqrtf(-2.0f * logf(u1)) * cosf(tau * u2);
}

void hipml_oracle_rng_fill_normal(uint64_t *state, float std, float *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = hipml_oracle_rng_normal(state) * std;
}

/* ------------------------------------------------------------ f32 attention
 * crates/hipml-core/src/attention.rs:56-102. */

static void attn_causal_row(const float *q, const float *k_cache, const float *v_cache,
                            int n_heads, int n_kv, int head_dim, int seq, float scale, float *out,
                            float *scores) {
    const size_t width = (size_t)n_kv * head_dim;
    const int group = n_heads / n_kv;
    for (size_t i = 0; i < (size_t)n_heads * head_dim; i++) out[i] = 0.0f;
    for (int h = 0; h < n_heads; h++) {
        const float *qh = q + (size_t)h * head_dim;
        const size_t col = (size_t)(h / group) * head_dim;
        float mx = -INFINITY;
        for (int t = 0; t < seq; t++) {
            const float *kr = k_cache + (size_t)t * width + col;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; d++) dot += qh[d] * kr[d];
            float s = dot * scale;
            scores[t] = s;
            if (s > mx) mx = s;
        }
        float sum = 0.0f;
        for (int t = 0; t < seq; t++) {
            float w = expf(scores[t] - mx);
            scores[t] = w;
            sum += w;
        }
        float inv = 1.0f / sum;
        float *ob = out + (size_t)h * head_dim;
        for (int t = 0; t < seq; t++) {
            float w = scores[t] * inv;
            const float *vr = v_cache + (size_t)t * width + col;
            for (int d = 0; d < head_dim; d++) ob[d] += w * vr[d];
        }
    }
}

void hipml_oracle_attn_causal_f32(const float *q, const float *k_cache, const float *v_cache,
                                  int n_heads, int n_kv, int head_dim, int seq, float scale,
                                  float *out) {
    float *scores = (float *)malloc(sizeof(float) * (size_t)(seq > 0 ? seq : 1));
    attn_causal_row(q, k_cache, v_cache, n_heads, n_kv, head_dim, seq, scale, out, scores);
    free(scores);
}

struct chunk_job {
    const float *q, *k, *v;
    float *out;
    int n_heads, n_kv, head_dim, pos0, tokens;
    float scale;
    int first, step; /* rows first, first+step, ... */
};

static void *chunk_worker(void *arg) {
    struct chunk_job *j = (struct chunk_job *)arg;
    const size_t nhd = (size_t)j->n_heads * j->head_dim;
    float *scores = (float *)malloc(sizeof(float) * (size_t)(j->pos0 + j->tokens + 1));
    for (int t = j->first; t < j->tokens; t += j->step)
        attn_causal_row(j->q + (size_t)t * nhd, j->k, j->v, j->n_heads, j->n_kv, j->head_dim,
                        j->pos0 + t + 1, j->scale, j->out + (size_t)t * nhd, scores);
    free(scores);
    return NULL;
}

void hipml_oracle_attn_chunk_f32(const float *q, const float *k_cache, const float *v_cache,
                                 int n_heads, int n_kv, int head_dim, int pos0, int tokens,
                                 float scale, float *out, int row0, int row_step, int threads) {
    if (row_step < 1) row_step = 1;
    if (threads < 1) threads = 1;
    if (threads > 256) threads = 256;
    struct chunk_job jobs[256];
    pthread_t tids[256];
    for (int i = 0; i < threads; i++) {
        struct chunk_job j = {q, k_cache, v_cache, out, n_heads, n_kv, head_dim, pos0, tokens,
                              scale, row0 + i * row_step, row_step * threads};
        jobs[i] = j;
    }
    if (threads == 1) {
        chunk_worker(&jobs[0]);
        return;
    }
    for (int i = 0; i < threads; i++) pthread_create(&tids[i], NULL, chunk_worker, &jobs[i]);
    for (int i = 0; i < threads; i++) pthread_join(tids[i], NULL);
}

/* ------------------------------------------------- decode over a q8_0 cache
 * crates/hipml-core/src/ops.rs:449-518. */

static void block_f32_q4(const uint8_t *src, float *out);

/* dtype 0 = q8_0 (34-byte blocks), 1 = q4_0 (18-byte blocks). */
void hipml_oracle_attn_decode_kv_strided(const float *q, const uint8_t *k, const uint8_t *v, int dtype,
                                         int n_heads, int n_kv, int head_dim, int seq, int stride,
                                         float scale, float *out) {
    const int nb = head_dim / HIPML_KV_BLOCK;
    const size_t bb = dtype == 1 ? HIPML_Q4_BLOCK_BYTES : HIPML_Q8_BLOCK_BYTES;
    const size_t row = (size_t)nb * bb;
    const int group = n_heads / n_kv;
    float *acc = (float *)malloc(sizeof(float) * (size_t)head_dim);
    float blk[HIPML_KV_BLOCK];

    for (int h = 0; h < n_heads; h++) {
        const float *qh = q + (size_t)h * head_dim;
        const size_t base = (size_t)(h / group) * stride * row;
        for (int d = 0; d < head_dim; d++) acc[d] = 0.0f;
        float m = -INFINITY;
        float l = 0.0f;
        for (int pos = 0; pos < seq; pos++) {
            const uint8_t *kr = k + base + (size_t)pos * row;
            float dot = 0.0f;
            for (int c = 0; c < nb; c++) {
                if (dtype == 1) block_f32_q4(kr + (size_t)c * bb, blk);
                else block_f32_q8(kr + (size_t)c * bb, blk);
                const float *qc = qh + c * HIPML_KV_BLOCK;
                for (int j = 0; j < HIPML_KV_BLOCK; j++) dot += qc[j] * blk[j];
            }
            float s = dot * scale;
            float m_new = s > m ? s : m; /* f32::max: a NaN score is ignored */
            float corr = expf(m - m_new);
            float p = expf(s - m_new);
            l = l * corr + p;
            m = m_new;
            const uint8_t *vr = v + base + (size_t)pos * row;
            for (int c = 0; c < nb; c++) {
                if (dtype == 1) block_f32_q4(vr + (size_t)c * bb, blk);
                else block_f32_q8(vr + (size_t)c * bb, blk);
                float *a = acc + c * HIPML_KV_BLOCK;
                for (int j = 0; j < HIPML_KV_BLOCK; j++) a[j] = a[j] * corr + p * blk[j];
            }
        }
        float inv = 1.0f / l;
        for (int d = 0; d < head_dim; d++) out[(size_t)h * head_dim + d] = acc[d] * inv;
    }
    free(acc);
}

void hipml_oracle_attn_decode_kv_q8_strided(const float *q, const uint8_t *k, const uint8_t *v,
                                            int n_heads, int n_kv, int head_dim, int seq,
                                            int stride, float scale, float *out) {
    hipml_oracle_attn_decode_kv_strided(q, k, v, 0, n_heads, n_kv, head_dim, seq, stride, scale, out);
}

void hipml_oracle_attn_decode_kv_q8(const float *q, const uint8_t *k, const uint8_t *v,
                                    int n_heads, int n_kv, int head_dim, int seq, float scale,
                                    float *out) {
    hipml_oracle_attn_decode_kv_q8_strided(q, k, v, n_heads, n_kv, head_dim, seq, seq, scale, out);
}

/* crates/hipml-core/src/ops.rs:530-588. */
void hipml_oracle_attn_decode_f32(const float *q, const float *k, const float *v, int n_heads,
                                  int n_kv, int head_dim, int seq, float scale, float *out) {
    const int group = n_heads / n_kv;
    float *scores = (float *)malloc(sizeof(float) * (size_t)(seq > 0 ? seq : 1));
    for (int h = 0; h < n_heads; h++) {
        const float *qh = q + (size_t)h * head_dim;
        const size_t kbase = (size_t)(h / group) * seq * head_dim;
        float *o = out + (size_t)h * head_dim;
        for (int d = 0; d < head_dim; d++) o[d] = 0.0f;
        float mx = -INFINITY;
        for (int r = 0; r < seq; r++) {
            const float *kr = k + kbase + (size_t)r * head_dim;
            float dot = 0.0f;
            for (int d = 0; d < head_dim; d++) dot += qh[d] * kr[d];
            float s = dot * scale;
            scores[r] = s;
            if (s > mx) mx = s;
        }
        float sum = 0.0f;
        for (int r = 0; r < seq; r++) {
            float w = expf(scores[r] - mx);
            scores[r] = w;
            sum += w;
        }
        float inv = 1.0f / sum;
        for (int r = 0; r < seq; r++) {
            float w = scores[r] * inv;
            const float *vr = v + kbase + (size_t)r * head_dim;
            for (int d = 0; d < head_dim; d++) o[d] += w * vr[d];
        }
    }
    free(scores);
}

/* crates/hipml-core/src/ops.rs:366-386 (done in place on the two caches). */
void hipml_oracle_kv_append_f32(float *k_cache, float *v_cache, const float *k, const float *v,
                                size_t off, size_t width) {
    memcpy(k_cache + off * width, k, width * sizeof(float));
    memcpy(v_cache + off * width, v, width * sizeof(float));
}

/* crates/hipml-core/src/parity.rs:58-80. */
void hipml_oracle_compare(const float *expected, const float *actual, size_t n, float *max_abs,
                          float *max_rel) {
    float ma = 0.0f, mr = 0.0f;
    for (size_t i = 0; i < n; i++) {
        float abs = fabsf(expected[i] - actual[i]);
        float denom = fabsf(expected[i]);
        if (!(denom > 1e-12f)) denom = 1e-12f;
        if (abs > ma) ma = abs;
        float rel = abs / denom;
        if (rel > mr) mr = rel;
    }
    *max_abs = ma;
    *max_rel = mr;
}

/* ---- attention front end and tail ------------------------------------------------------ */

/* crates/hipml-core/src/ops.rs:181-187: y = x * (1 / sqrt(mean(x^2) + eps)) * w, the sum in
 * f32 in index order. */
void hipml_oracle_rmsnorm_f32(const float *x, const float *w, int n, float eps, float *out) {
    float sum = 0.0f;
    for (int i = 0; i < n; i++) sum += x[i] * x[i];
    float mean_sq = sum / (float)n;
    float scale = 1.0f / sqrtf(mean_sq + eps);
    for (int i = 0; i < n; i++) out[i] = x[i] * scale * w[i];
}

/* crates/hipml-core/src/ops.rs:334-350: every head row normalised with the shared w. */
void hipml_oracle_head_rmsnorm_f32(const float *x, const float *w, int n_heads, int head_dim,
                                   float eps, float *out) {
    for (int h = 0; h < n_heads; h++)
        hipml_oracle_rmsnorm_f32(x + (size_t)h * head_dim, w, head_dim, eps,
                                 out + (size_t)h * head_dim);
}

/* crates/hipml-core/src/ops.rs:260-309: M-RoPE. Only the first n_rot channels rotate, NeoX
 * pair k against k + n_rot/2, frequency theta_base^(-2k/n_rot), the angle in f64; the section
 * table picks which of the four position ids feeds pair k. */
void hipml_oracle_rope_multi_f32(const float *x, int n_heads, int head_dim, int n_rot,
                                 const int sections[4], const int pos[4], float theta_base,
                                 float *out) {
    const int half = n_rot / 2;
    const int sect = sections[0] + sections[1] + sections[2] + sections[3];
    memcpy(out, x, (size_t)n_heads * head_dim * sizeof(float));
    for (int h = 0; h < n_heads; h++) {
        const size_t base = (size_t)h * head_dim;
        for (int k = 0; k < half; k++) {
            int p = pos[0];
            if (sect != 0) {
                const int s = k % sect;
                if (s < sections[0]) p = pos[0];
                else if (s < sections[0] + sections[1]) p = pos[1];
                else if (s < sections[0] + sections[1] + sections[2]) p = pos[2];
                else p = pos[3];
            }
            const double freq = pow((double)theta_base, -2.0 * (double)k / (double)n_rot);
            const double ang = (double)p * freq;
            const float sn = (float)sin(ang), cs = (float)cos(ang);
            const float x1 = x[base + k], x2 = x[base + half + k];
            out[base + k] = x1 * cs - x2 * sn;
            out[base + half + k] = x1 * sn + x2 * cs;
        }
    }
}

/* crates/hipml-core/src/ops.rs:195-224: plain NeoX rope over the whole head. */
void hipml_oracle_rope_neox_f32(const float *x, int n_heads, int head_dim, int pos,
                                float theta_base, float *out) {
    const int sections[4] = {0, 0, 0, 0};
    const int p[4] = {pos, pos, pos, pos};
    hipml_oracle_rope_multi_f32(x, n_heads, head_dim, head_dim, sections, p, theta_base, out);
}

/* crates/hipml-core/src/ops.rs:315-329: joint [n_heads][2*head_dim] -> q then gate. */
void hipml_oracle_qg_split_f32(const float *qg, int n_heads, int head_dim, float *q, float *gate) {
    for (int h = 0; h < n_heads; h++) {
        memcpy(q + (size_t)h * head_dim, qg + (size_t)h * 2 * head_dim, head_dim * sizeof(float));
        memcpy(gate + (size_t)h * head_dim, qg + (size_t)h * 2 * head_dim + head_dim,
               head_dim * sizeof(float));
    }
}

/* crates/hipml-core/src/ops.rs:354-360: y = q * (1 / (1 + exp(-gate))). */
void hipml_oracle_q_gate_f32(const float *q, const float *gate, size_t n, float *out) {
    for (size_t i = 0; i < n; i++) out[i] = q[i] * (1.0f / (1.0f + expf(-gate[i])));
}

/* ---- q4_0 (crates/hipml-core/src/kv.rs:201-218, 238-290, 306-320) ---------------------------
 * Block = f16 scale + 16 bytes; byte j holds value j in its low nibble and value j + 16 in its
 * high nibble; value = d * (nibble - 8). ggml's convention: the scale takes the sign of the
 * element of largest magnitude (the first one on ties), d = -vmax / 8, so that element lands
 * exactly on nibble 0 or 15. */

void hipml_oracle_quantize_block_q4(const float *xs, uint8_t *out) {
    float vmax = 0.0f;
    for (int j = 0; j < HIPML_KV_BLOCK; j++)
        if (fabsf(xs[j]) > fabsf(vmax)) vmax = xs[j];
    float d = -vmax / 8.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    uint16_t hs = hipml_oracle_f32_to_f16(d);
    out[0] = (uint8_t)(hs & 0xff);
    out[1] = (uint8_t)(hs >> 8);
    uint8_t q[HIPML_KV_BLOCK];
    for (int j = 0; j < HIPML_KV_BLOCK; j++) {
        float r = roundf(xs[j] * id) + 8.0f; /* f32::round: half away from zero */
        if (r < 0.0f) r = 0.0f;
        if (r > 15.0f) r = 15.0f;
        q[j] = (r != r) ? 0 : (uint8_t)r;    /* `as u8` of a NaN is 0 in Rust */
    }
    for (int j = 0; j < HIPML_KV_BLOCK / 2; j++)
        out[2 + j] = (uint8_t)(q[j] | (q[j + HIPML_KV_BLOCK / 2] << 4));
}

void hipml_oracle_quantize_q4(const float *values, size_t n, uint8_t *out) {
    for (size_t b = 0; b < n / HIPML_KV_BLOCK; b++)
        hipml_oracle_quantize_block_q4(values + b * HIPML_KV_BLOCK, out + b * HIPML_Q4_BLOCK_BYTES);
}

static void block_f32_q4(const uint8_t *src, float *out) {
    const float d = hipml_oracle_f16_to_f32((uint16_t)(src[0] | (src[1] << 8)));
    for (int j = 0; j < HIPML_KV_BLOCK / 2; j++) {
        const uint8_t byte = src[2 + j];
        out[j] = d * ((float)(byte & 0x0f) - 8.0f);
        out[j + HIPML_KV_BLOCK / 2] = d * ((float)(byte >> 4) - 8.0f);
    }
}

void hipml_oracle_dequantize_q4(const uint8_t *bytes, size_t n_bytes, float *out) {
    for (size_t b = 0; b < n_bytes / HIPML_Q4_BLOCK_BYTES; b++)
        block_f32_q4(bytes + b * HIPML_Q4_BLOCK_BYTES, out + b * HIPML_KV_BLOCK);
}

void hipml_oracle_synthetic_blocks_q4(size_t n_blocks, uint64_t seed, uint8_t *out) {
    uint64_t s = seed | 1;
    for (size_t b = 0; b < n_blocks; b++) {
        uint8_t *blk = out + b * HIPML_Q4_BLOCK_BYTES;
        float d = 0.01f + (float)(xorshift64star(&s) % 1000) * 0.00004f;
        uint16_t hs = hipml_oracle_f32_to_f16(d);
        blk[0] = (uint8_t)(hs & 0xff);
        blk[1] = (uint8_t)(hs >> 8);
        for (int j = 0; j < HIPML_Q4_BLOCK_BYTES - 2; j++) blk[2 + j] = (uint8_t)(xorshift64star(&s) >> 24);
    }
}
