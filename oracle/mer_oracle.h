/*
 * mer_oracle.h -- CPU restatement of the Micro-Expert-Router routed expert-FFN path.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the parity checker and the timed
 * CPU baseline.  Nothing on the product path links, loads or calls it; the
 * CUDA library must fail loudly on its own when it cannot run.
 *
 * Parity pinning: the reference is Rust and cannot be compiled in this
 * environment (no cargo/rustc, dependencies not vendored).  The oracle is
 * therefore pinned against the literal fixtures and closed-form expectations
 * stated in the reference's own unit tests (transcribed under tests/golden/),
 * not against outputs of a reference binary.
 *
 * Every function cites the reference file:line (paths relative to
 * rust-engine/src/) whose arithmetic it follows.
 */
#ifndef MER_ORACLE_H
#define MER_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Weight block formats (inference.rs:725-747 Q4_0, kernels/mod.rs:74-75 Q8_0). */
#define MER_ORACLE_Q4_0 0
#define MER_ORACLE_Q8_0 1
#define MER_ORACLE_BLOCK_ELEMS 32
#define MER_ORACLE_Q4_0_BLOCK_BYTES 18
#define MER_ORACLE_Q8_0_BLOCK_BYTES 34

/* Expert forward variants: same values, different fp32 rounding order. */
#define MER_ORACLE_FWD_AUTHORITATIVE 0 /* dequantise -> sequential fp32 dot (inference.rs:3291-3306, 1481-1634; kernels/scalar.rs:10-17) */
#define MER_ORACLE_FWD_Q8_SCALAR     1 /* acc += scale*q*x left to right (inference.rs:3539-3572) */
#define MER_ORACLE_FWD_BLOCK_PARTIAL 2 /* sum += d * sum_j (q-8)*x per block (backend/wgpu_shaders/matmul_q4_0.wgsl:65-85) */
#define MER_ORACLE_FWD_F64           3 /* double accumulation; apportions error between oracle and kernel */
#define MER_ORACLE_FWD_SIMD8X4       4 /* 4 x 8-lane FMA accumulators reduced once (kernels/avx2.rs:98-187) */

#define MER_ORACLE_SCORE_SOFTMAX 0
#define MER_ORACLE_SCORE_SIGMOID 1

/* Status codes returned by the oracle. */
#define MER_ORACLE_OK 0
#define MER_ORACLE_ERR_INVALID_LAYOUT 1   /* ExpertWeightsError::InvalidLayout   (inference.rs:1153-1188) */
#define MER_ORACLE_ERR_BUFFER_TOO_SMALL 2 /* ExpertWeightsError::BufferTooSmall */
#define MER_ORACLE_ERR_TRUNCATED 3        /* ExpertWeightsError::TruncatedPayload */

/* IEEE binary16 <-> binary32 (half::f16::{to_f32,from_f32}; round to nearest even). */
float mer_oracle_f16_to_f32(uint16_t h);
uint16_t mer_oracle_f32_to_f16(float f);

/* Block codecs: inference.rs:762-784, 797-841 (Q4_0); 894-914, 920-957 (Q8_0). */
void mer_oracle_dequant_q4_0_block(const uint8_t *src, float *dst);
void mer_oracle_quant_q4_0_block(const float *src, size_t n, uint8_t *dst);
void mer_oracle_dequant_q8_0_block(const uint8_t *src, float *dst);
void mer_oracle_quant_q8_0_block(const float *src, size_t n, uint8_t *dst);

/* Stream decode with tail truncation: inference.rs:852-868, 963-979. */
int mer_oracle_dequant_stream(int dtype, const uint8_t *src, size_t src_len,
                              size_t n_weights, float *dst);

/* Bytes of one projection / one gate||up||down expert blob: inference.rs:1096-1114. */
size_t mer_oracle_projection_bytes(int dtype, size_t d_model, size_t d_ff);
size_t mer_oracle_expert_bytes(int dtype, size_t d_model, size_t d_ff);

/* silu(x) = x / (1 + exp(-x)): inference.rs:1632-1634. */
float mer_oracle_silu(float x);

/*
 * One expert SwiGLU FFN over a resident gate||up||down block stream.
 * swiglu_limit <= 0 or non-finite disables the gate clamp (inference.rs:86-112).
 * gated_out (optional, d_ff floats) receives silu(gate)*up.
 */
int mer_oracle_expert_forward(int dtype, int variant, const uint8_t *blob,
                              size_t blob_len, const float *x, size_t d_model,
                              size_t d_ff, float swiglu_limit, float *y,
                              float *gated_out);

/* Row-chunk threaded zero-copy forward (parallel.rs:432-468 fan-out over rows;
 * row kernels as kernels/avx2.rs:98-187 when AVX2+FMA is available, scalar
 * otherwise).  This is the timed CPU baseline.  Returns threads used (>0) or
 * a negative status. */
int mer_oracle_expert_forward_mt(int dtype, const uint8_t *blob, size_t blob_len,
                                 const float *x, size_t d_model, size_t d_ff,
                                 float swiglu_limit, float *y, int n_threads);
int mer_oracle_has_avx2_fma(void);

/* Raw Q4_0 matvec used by the canonical parity cases: q4_parity.rs:591-619. */
int mer_oracle_q4_matvec(const uint8_t *weights, size_t weights_len,
                         const float *input, size_t rows, size_t columns,
                         size_t w_block_off, float *out);

/* Q8_0 row dot, scalar order: kernels/avx2.rs:232-246 (test oracle), inference.rs:3539-3551. */
float mer_oracle_q8_row_dot_scalar(const uint8_t *row_blocks, const float *x, size_t width);
float mer_oracle_q8_row_dot_simd8x4(const uint8_t *row_blocks, const float *x, size_t width);

/* LinearGate: gating.rs:118-143. */
typedef struct {
  const float *weights;          /* [num_experts x d_model] row-major */
  size_t num_experts;
  size_t d_model;
  size_t top_k;
  int normalise_topk;
  int scoring_func;
  const float *correction_bias;  /* NULL or [num_experts] */
  size_t n_group;
  size_t topk_group;
  float routed_scaling_factor;
  const float *logit_bias;       /* harness extension: added to the logits before scoring; NULL = none */
} mer_oracle_gate;

/* softmax_inplace: transformer.rs:2767-2819 (non-finite row -> uniform). */
void mer_oracle_softmax_inplace(float *v, size_t n);

/*
 * LinearGate::route_with_scratch: gating.rs:395-476.
 * experts/weights hold top_k entries; *n_selected may be < top_k when scores
 * are non-finite.  scores_out (optional, num_experts) receives the post-score
 * values; gap_out (optional) the selection-score gap between the last kept
 * and the best rejected expert (+inf when none was rejected).
 */
int mer_oracle_route(const mer_oracle_gate *gate, const float *x,
                     uint32_t *experts, float *weights, size_t *n_selected,
                     float *scores_out, float *gap_out);

/* Stable-sort second implementation: gating.rs:684-764 (reference_route_stable). */
int mer_oracle_route_stable(const mer_oracle_gate *gate, const float *x,
                            uint32_t *experts, float *weights, size_t *n_selected);

/* combine_outputs_into: inference.rs:4472-4491; skip_zero follows engine.rs:5575-5581. */
void mer_oracle_combine(const float *outputs, const float *scores, size_t k,
                        size_t d, float *out, int skip_zero);

/* RmsNorm::forward_inplace (transformer.rs:62-74), the shared expert's sigmoid gate scalar
 * (transformer.rs:2224-2231) and add_residual_into (transformer.rs:2006-2011). */
void mer_oracle_rmsnorm(const float *x, const float *weight, size_t n, float eps, float *y);
float mer_oracle_shared_gate_scale(const float *gate_inp, const float *x, size_t n);
void mer_oracle_add_residual(const float *a, const float *b, size_t n, float *out);

/* accumulate_ordered_f16_outputs: engine.rs:1651-1673.  Returns 1 on success, 0 on length mismatch. */
int mer_oracle_accumulate_ordered_f16(const uint16_t *outputs, size_t outputs_len,
                                      const float *weights, size_t n_weights,
                                      size_t d_model, float *out);

/* synth_hidden_state (splitmix64 -> [-1,1)): inference.rs:3064-3082. */
void mer_oracle_synth_hidden_state(uint64_t token_idx, size_t d_model,
                                   uint64_t seed, float *out);

/* randomized_q8_expert (xorshift64 test fixture): inference.rs:5905-5926. */
void mer_oracle_randomized_q8_expert(size_t d_model, size_t d_ff, uint64_t state,
                                     uint8_t *out);

/*
 * One MoE layer over B tokens, token by token as the reference does
 * (model.rs:2716-2750 -> engine.rs:5174, 5575-5581): route, run each selected
 * expert (authoritative variant unless `variant` says otherwise), accumulate
 * weight*y in slot order.  expert_blobs[e] points at expert e's block stream.
 * Optional shared expert (transformer.rs:2094-2238) is added with weight 1.
 */
int mer_oracle_moe_layer_forward(int dtype, int variant, const mer_oracle_gate *gate,
                                 const uint8_t *const *expert_blobs, size_t blob_len,
                                 const uint8_t *shared_blob, const float *x,
                                 size_t n_tokens, size_t d_ff, float swiglu_limit,
                                 float *out, uint32_t *topk_ids, float *topk_w,
                                 float *gaps, int n_threads);

/*
 * Production-shaped timing form of the same layer: zero-copy fused row kernels
 * (kernels/avx2.rs:98-187 when AVX2+FMA is present).  Tokens fan out over the
 * threads when n_tokens >= n_threads; otherwise each expert's rows do
 * (parallel.rs:432-468), one token at a time as batch_scheduler.rs:1378-1382 runs them.
 */
int mer_oracle_moe_layer_forward_production(int dtype, const mer_oracle_gate *gate,
                                            const uint8_t *const *expert_blobs, size_t blob_len,
                                            const uint8_t *shared_blob, const float *x,
                                            size_t n_tokens, size_t d_ff, float swiglu_limit,
                                            float *out, int n_threads);

#ifdef __cplusplus
}
#endif
#endif
