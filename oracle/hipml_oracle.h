/*
 * CPU oracle for the hipml full-attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the reference's
 * own CPU definition of the path (crates/hipml-core of pgmharikrishnan/hipml);
 * nothing in the product (the CUDA library, its host layer) links, loads or
 * calls it. Only the test-suite, the smoke check and the bench's CPU-baseline
 * leg use it, and there only as the checker / the reported CPU number.
 *
 * Pinning: the restatement is checked against every known-answer vector the
 * reference's CPU tests hold for this path (crates/hipml-core/tests/
 * kv_formats.rs, crates/hipml-core/tests/parity_reference.rs); the Rust
 * original cannot be compiled where this was written (no rustc), so there are
 * no reference-generated output tensors beyond those vectors.
 *
 * Build: gcc -O2 -ffp-contract=off (Rust never contracts a*b+c into an fma, and
 * the summation order below is the reference's, so results are bit-comparable
 * on the same libm).
 */
#ifndef HIPML_ORACLE_H
#define HIPML_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HIPML_KV_BLOCK 32
#define HIPML_Q8_BLOCK_BYTES 34
#define HIPML_Q4_BLOCK_BYTES 18

/* crates/hipml-core/src/kv.rs:94-116 */
float hipml_oracle_f16_to_f32(uint16_t h);
/* crates/hipml-core/src/kv.rs:119-165 */
uint16_t hipml_oracle_f32_to_f16(float v);

/* crates/hipml-core/src/kv.rs:187-200 (Q8 arm): one block of 32 values -> 34 bytes. */
void hipml_oracle_quantize_block_q8(const float *xs, uint8_t *out);
/* crates/hipml-core/src/kv.rs:176-184: n values (multiple of 32) -> n/32*34 bytes. */
void hipml_oracle_quantize_q8(const float *values, size_t n, uint8_t *out);
/* crates/hipml-core/src/kv.rs:268-290 (Q8 arm): n_bytes (multiple of 34) -> n_bytes/34*32 values. */
void hipml_oracle_dequantize_q8(const uint8_t *bytes, size_t n_bytes, float *out);
/* crates/hipml-core/src/kv.rs:306-329 (Q8): format-valid filler for bandwidth benches. */
void hipml_oracle_synthetic_blocks_q8(size_t n_blocks, uint64_t seed, uint8_t *out);

/* crates/hipml-core/src/rng.rs:13-49. The generator is its 64-bit state. */
uint64_t hipml_oracle_rng_new(uint64_t seed);
uint64_t hipml_oracle_rng_next_u64(uint64_t *state);
float hipml_oracle_rng_uniform(uint64_t *state);
float hipml_oracle_rng_normal(uint64_t *state);
/* n draws of normal()*std in flat-index order (crates/hipml-core/src/tensor.rs:43-49). */
void hipml_oracle_rng_fill_normal(uint64_t *state, float std, float *out, size_t n);

/* crates/hipml-core/src/attention.rs:56-102: one query position over the
 * position-major f32 cache [n_ctx][n_kv*head_dim]; out is [n_heads][head_dim]. */
void hipml_oracle_attn_causal_f32(const float *q, const float *k_cache, const float *v_cache,
                                  int n_heads, int n_kv, int head_dim, int seq, float scale,
                                  float *out);

/* Chunk prefill as the reference's parity harness drives it
 * (crates/hipml-cli/src/attn_chunk_parity.rs:44-58,193-207): row t of the
 * chunk calls attn_causal_f32 with seq = pos0 + t + 1. q and out are
 * [tokens][n_heads*head_dim]. Rows row0, row0+row_step, ... < tokens are
 * computed; others are left untouched. threads <= 1 is the reference's own
 * single-threaded loop; threads > 1 parallelises over rows. */
void hipml_oracle_attn_chunk_f32(const float *q, const float *k_cache, const float *v_cache,
                                 int n_heads, int n_kv, int head_dim, int pos0, int tokens,
                                 float scale, float *out, int row0, int row_step, int threads);

/* crates/hipml-core/src/ops.rs:449-518 (Q8 arm): decode over the quantised
 * head-major cache [n_kv][seq][head_dim/32] blocks, online softmax. */
void hipml_oracle_attn_decode_kv_q8(const float *q, const uint8_t *k, const uint8_t *v,
                                    int n_heads, int n_kv, int head_dim, int seq, float scale,
                                    float *out);
/* Same arithmetic over a cache whose per-head row stride is larger than the
 * live length (the engine's layout: stride = n_ctx, crates/hipml-model/src/gpu/
 * deep_kv.rs:40-44). With stride == seq it is exactly the function above. */
void hipml_oracle_attn_decode_kv_q8_strided(const float *q, const uint8_t *k, const uint8_t *v,
                                            int n_heads, int n_kv, int head_dim, int seq,
                                            int stride, float scale, float *out);

/* crates/hipml-core/src/ops.rs:530-588: two-pass decode over [n_kv][seq][head_dim] f32. */
void hipml_oracle_attn_decode_f32(const float *q, const float *k, const float *v, int n_heads,
                                  int n_kv, int head_dim, int seq, float scale, float *out);

/* crates/hipml-core/src/ops.rs:366-386: append one row into position-major caches (in place). */
void hipml_oracle_kv_append_f32(float *k_cache, float *v_cache, const float *k, const float *v,
                                size_t off, size_t width);

/* crates/hipml-core/src/parity.rs:58-80: max_abs and max_rel (denominator max(|e|,1e-12)). */
void hipml_oracle_compare(const float *expected, const float *actual, size_t n, float *max_abs,
                          float *max_rel);

/* q4_0 (crates/hipml-core/src/kv.rs:201-218, 238-290, 306-320) and the decode over either
 * quantised format (ops.rs:449-518; dtype 0 = q8_0, 1 = q4_0). */
void hipml_oracle_quantize_block_q4(const float *xs, uint8_t *out);
void hipml_oracle_quantize_q4(const float *values, size_t n, uint8_t *out);
void hipml_oracle_dequantize_q4(const uint8_t *bytes, size_t n_bytes, float *out);
void hipml_oracle_synthetic_blocks_q4(size_t n_blocks, uint64_t seed, uint8_t *out);
void hipml_oracle_attn_decode_kv_strided(const float *q, const uint8_t *k, const uint8_t *v, int dtype,
                                         int n_heads, int n_kv, int head_dim, int seq, int stride,
                                         float scale, float *out);

/* Attention front end and tail (crates/hipml-core/src/ops.rs:181-187, 195-224, 260-360). */
void hipml_oracle_rmsnorm_f32(const float *x, const float *w, int n, float eps, float *out);
void hipml_oracle_head_rmsnorm_f32(const float *x, const float *w, int n_heads, int head_dim,
                                   float eps, float *out);
void hipml_oracle_rope_multi_f32(const float *x, int n_heads, int head_dim, int n_rot,
                                 const int sections[4], const int pos[4], float theta_base,
                                 float *out);
void hipml_oracle_rope_neox_f32(const float *x, int n_heads, int head_dim, int pos,
                                float theta_base, float *out);
void hipml_oracle_qg_split_f32(const float *qg, int n_heads, int head_dim, float *q, float *gate);
void hipml_oracle_q_gate_f32(const float *q, const float *gate, size_t n, float *out);

#ifdef __cplusplus
}
#endif
#endif
