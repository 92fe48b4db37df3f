/*
 * mer_oracle.c -- CPU restatement of the reference's routed quantized SwiGLU
 * expert-FFN path.  TEST INFRASTRUCTURE ONLY (see mer_oracle.h).
 *
 * Build with -ffp-contract=off: the reference is Rust, which never fuses
 * a*b+c unless the source says mul_add / _mm256_fmadd_ps, so every place that
 * must round twice is written as separate operations here and every fused
 * place uses fmaf() explicitly.
 *
 * All file:line citations are relative to rust-engine/src/ of the reference.
 */
#include "mer_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

#define BLK MER_ORACLE_BLOCK_ELEMS
#define Q4B MER_ORACLE_Q4_0_BLOCK_BYTES
#define Q8B MER_ORACLE_Q8_0_BLOCK_BYTES
/* EXPERT_SIZE_TOLERANCE_BYTES: one O_DIRECT page (inference.rs: validate_q8_direct_layout, 3349-3418). */
#define SIZE_TOLERANCE_BYTES 4096

/* ------------------------------------------------------------------ f16 */

float mer_oracle_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal: normalise */
      int e = -1;
      do {
        man <<= 1;
        e++;
      } while ((man & 0x400u) == 0);
      man &= 0x3ffu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 0x1f) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

uint16_t mer_oracle_f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t exp = (x >> 23) & 0xffu;
  uint32_t man = x & 0x7fffffu;
  if (exp == 0xff) { /* inf / nan (quiet bit kept so nan stays nan) */
    if (man == 0) return (uint16_t)(sign | 0x7c00u);
    return (uint16_t)(sign | 0x7c00u | 0x0200u | (man >> 13));
  }
  int32_t e = (int32_t)exp - 127 + 15;
  if (e >= 0x1f) return (uint16_t)(sign | 0x7c00u); /* overflow -> inf */
  if (e <= 0) {
    if (e < -10) return (uint16_t)sign; /* underflow -> signed zero */
    man |= 0x800000u;
    uint32_t shift = (uint32_t)(14 - e);
    uint32_t half_man = man >> shift;
    uint32_t round_bit = 1u << (shift - 1);
    if ((man & round_bit) && ((man & (round_bit - 1)) || (half_man & 1))) half_man++;
    return (uint16_t)(sign | half_man);
  }
  uint32_t half_man = man >> 13;
  uint16_t out = (uint16_t)(sign | ((uint32_t)e << 10) | half_man);
  uint32_t round_bit = 0x1000u;
  if ((man & round_bit) && ((man & (round_bit - 1)) || (half_man & 1))) out++; /* carries into exponent correctly */
  return out;
}

static inline float scale_at(const uint8_t *block) {
  return mer_oracle_f16_to_f32((uint16_t)(block[0] | ((uint16_t)block[1] << 8)));
}

/* --------------------------------------------------------------- codecs */

/* inference.rs:762-784 */
void mer_oracle_dequant_q4_0_block(const uint8_t *src, float *dst) {
  float d = scale_at(src);
  const uint8_t *qs = src + 2;
  for (int j = 0; j < BLK / 2; j++) {
    uint8_t byte = qs[j];
    dst[j] = d * (float)((int)(byte & 0x0f) - 8);
    dst[j + BLK / 2] = d * (float)((int)(byte >> 4) - 8);
  }
}

static inline int32_t rust_round_to_i32(float v) {
  /* f32::round (half away from zero) then `as i32` (saturating, NaN -> 0). */
  float r = roundf(v);
  if (r != r) return 0;
  if (r >= 2147483648.0f) return INT32_MAX;
  if (r <= -2147483648.0f) return INT32_MIN;
  return (int32_t)r;
}

/* inference.rs:797-841 */
void mer_oracle_quant_q4_0_block(const float *src, size_t n, uint8_t *dst) {
  float max_abs = 0.0f;
  for (size_t i = 0; i < n; i++) {
    float a = fabsf(src[i]);
    if (a > max_abs) max_abs = a;
  }
  float d = max_abs / 7.0f;
  uint16_t bits = mer_oracle_f32_to_f16(d);
  dst[0] = (uint8_t)(bits & 0xff);
  dst[1] = (uint8_t)(bits >> 8);
  for (int j = 0; j < BLK / 2; j++) dst[2 + j] = 0x88;
  if (d == 0.0f) return;
  float inv_d = 1.0f / d;
  for (int j = 0; j < BLK / 2; j++) {
    float lo_v = (size_t)j < n ? src[j] : 0.0f;
    float hi_v = (size_t)(j + BLK / 2) < n ? src[j + BLK / 2] : 0.0f;
    int32_t lo = rust_round_to_i32(lo_v * inv_d);
    int32_t hi = rust_round_to_i32(hi_v * inv_d);
    /* saturating add of 8 is irrelevant after the clamp for finite inputs */
    lo = lo > INT32_MAX - 8 ? 15 : lo + 8;
    hi = hi > INT32_MAX - 8 ? 15 : hi + 8;
    if (lo < 0) lo = 0;
    if (lo > 15) lo = 15;
    if (hi < 0) hi = 0;
    if (hi > 15) hi = 15;
    dst[2 + j] = (uint8_t)(lo | (hi << 4));
  }
}

/* inference.rs:894-914 */
void mer_oracle_dequant_q8_0_block(const uint8_t *src, float *dst) {
  float d = scale_at(src);
  for (int i = 0; i < BLK; i++) dst[i] = d * (float)(int8_t)src[2 + i];
}

/* inference.rs:920-957 */
void mer_oracle_quant_q8_0_block(const float *src, size_t n, uint8_t *dst) {
  float max_abs = 0.0f;
  for (size_t i = 0; i < n; i++) {
    float a = fabsf(src[i]);
    if (a > max_abs) max_abs = a;
  }
  float d = max_abs / 127.0f;
  uint16_t bits = mer_oracle_f32_to_f16(d);
  dst[0] = (uint8_t)(bits & 0xff);
  dst[1] = (uint8_t)(bits >> 8);
  if (d == 0.0f) {
    memset(dst + 2, 0, BLK);
    return;
  }
  float inv_d = 1.0f / d;
  for (int i = 0; i < BLK; i++) {
    float v = (size_t)i < n ? src[i] : 0.0f;
    int32_t q = rust_round_to_i32(v * inv_d);
    if (q < -128) q = -128;
    if (q > 127) q = 127;
    dst[2 + i] = (uint8_t)(int8_t)q;
  }
}

static inline size_t block_bytes_of(int dtype) { return dtype == MER_ORACLE_Q4_0 ? Q4B : Q8B; }

static inline void dequant_block(int dtype, const uint8_t *src, float *dst) {
  if (dtype == MER_ORACLE_Q4_0)
    mer_oracle_dequant_q4_0_block(src, dst);
  else
    mer_oracle_dequant_q8_0_block(src, dst);
}

/* inference.rs:852-868, 963-979 */
int mer_oracle_dequant_stream(int dtype, const uint8_t *src, size_t src_len,
                              size_t n_weights, float *dst) {
  size_t bb = block_bytes_of(dtype);
  size_t blocks = (n_weights + BLK - 1) / BLK;
  if (src_len < blocks * bb) return MER_ORACLE_ERR_BUFFER_TOO_SMALL;
  float tmp[BLK];
  for (size_t b = 0; b < blocks; b++) {
    dequant_block(dtype, src + b * bb, tmp);
    size_t base = b * BLK;
    size_t n = n_weights - base < BLK ? n_weights - base : BLK;
    memcpy(dst + base, tmp, n * sizeof(float));
  }
  return MER_ORACLE_OK;
}

/* inference.rs:1096-1114: each projection is padded to whole blocks on its own. */
size_t mer_oracle_projection_bytes(int dtype, size_t d_model, size_t d_ff) {
  size_t one = d_model * d_ff;
  return (one + BLK - 1) / BLK * block_bytes_of(dtype);
}
size_t mer_oracle_expert_bytes(int dtype, size_t d_model, size_t d_ff) {
  return 3 * mer_oracle_projection_bytes(dtype, d_model, d_ff);
}

/* inference.rs:1632-1634 */
float mer_oracle_silu(float x) { return x / (1.0f + expf(-x)); }

static inline float clamp_gate(float g, float limit) {
  /* swiglu_limit(): Some(l) only for finite l > 0 (inference.rs:94-112); f32::clamp keeps NaN. */
  if (limit > 0.0f && isfinite(limit)) {
    if (g < -limit) return -limit;
    if (g > limit) return limit;
  }
  return g;
}

/* ------------------------------------------------------- flat matvecs */

/*
 * y[r] = sum_c W[r,c] * x[c] over a flat block stream (a block covers 32
 * consecutive weights of the flattened row-major matrix, so a row may start
 * inside a block when cols % 32 != 0).  `variant` selects the rounding order.
 */
static void matvec_flat(int dtype, int variant, const uint8_t *bytes, size_t rows,
                        size_t cols, const float *x, float *y) {
  size_t bb = block_bytes_of(dtype);
  float tmp[BLK];
  if (cols % BLK != 0 || variant == MER_ORACLE_FWD_AUTHORITATIVE || variant == MER_ORACLE_FWD_F64 ||
      variant == MER_ORACLE_FWD_Q8_SCALAR) {
    /* Row-sequential accumulation, element by element (kernels/scalar.rs:10-17;
     * q8_0_matvec_scalar_flat inference.rs:3618-3632 accumulates in the same
     * per-row order). */
    for (size_t r = 0; r < rows; r++) {
      float acc = 0.0f;
      double acc64 = 0.0;
      size_t flat = r * cols;
      size_t c = 0;
      while (c < cols) {
        size_t b = (flat + c) / BLK;
        size_t off = (flat + c) % BLK;
        size_t n = BLK - off;
        if (n > cols - c) n = cols - c;
        const uint8_t *blk = bytes + b * bb;
        if (variant == MER_ORACLE_FWD_Q8_SCALAR) {
          /* (scale * q) * x, then add: two roundings per term (inference.rs:3546-3548). */
          float scale = scale_at(blk);
          for (size_t i = 0; i < n; i++) {
            float q;
            size_t e = off + i;
            if (dtype == MER_ORACLE_Q8_0) {
              q = (float)(int8_t)blk[2 + e];
            } else {
              uint8_t byte = blk[2 + (e % 16)];
              q = (float)((int)(e < 16 ? (byte & 0x0f) : (byte >> 4)) - 8);
            }
            acc += scale * q * x[c + i];
          }
        } else {
          dequant_block(dtype, blk, tmp);
          if (variant == MER_ORACLE_FWD_F64) {
            for (size_t i = 0; i < n; i++) acc64 += (double)tmp[off + i] * (double)x[c + i];
          } else {
            for (size_t i = 0; i < n; i++) acc += tmp[off + i] * x[c + i];
          }
        }
        c += n;
      }
      y[r] = variant == MER_ORACLE_FWD_F64 ? (float)acc64 : acc;
    }
    return;
  }
  size_t bpr = cols / BLK;
  for (size_t r = 0; r < rows; r++) {
    const uint8_t *row = bytes + r * bpr * bb;
    if (variant == MER_ORACLE_FWD_BLOCK_PARTIAL) {
      /* matmul_q4_0.wgsl:65-85: partial = sum_j q_j * x_j; sum += d * partial. */
      float sum = 0.0f;
      for (size_t b = 0; b < bpr; b++) {
        const uint8_t *blk = row + b * bb;
        float d = scale_at(blk);
        float partial = 0.0f;
        const float *xb = x + b * BLK;
        if (dtype == MER_ORACLE_Q4_0) {
          for (int j = 0; j < 16; j++) {
            uint8_t byte = blk[2 + j];
            partial += (float)((int)(byte & 0x0f) - 8) * xb[j];
            partial += (float)((int)(byte >> 4) - 8) * xb[j + 16];
          }
        } else {
          for (int j = 0; j < BLK; j++) partial += (float)(int8_t)blk[2 + j] * xb[j];
        }
        sum += d * partial;
      }
      y[r] = sum;
    } else { /* MER_ORACLE_FWD_SIMD8X4: kernels/avx2.rs:98-126 lane for lane */
      y[r] = dtype == MER_ORACLE_Q8_0 ? mer_oracle_q8_row_dot_simd8x4(row, x, cols) : 0.0f;
      if (dtype == MER_ORACLE_Q4_0) {
        float acc[4][8];
        memset(acc, 0, sizeof acc);
        for (size_t b = 0; b < bpr; b++) {
          dequant_block(dtype, row + b * bb, tmp);
          for (int l = 0; l < 4; l++)
            for (int i = 0; i < 8; i++)
              acc[l][i] = fmaf(tmp[l * 8 + i], x[b * BLK + l * 8 + i], acc[l][i]);
        }
        float v[8];
        for (int i = 0; i < 8; i++) v[i] = (acc[0][i] + acc[1][i]) + (acc[2][i] + acc[3][i]);
        float s0 = v[0] + v[4], s1 = v[1] + v[5], s2 = v[2] + v[6], s3 = v[3] + v[7];
        y[r] = (s0 + s1) + (s2 + s3);
      }
    }
  }
}

float mer_oracle_q8_row_dot_scalar(const uint8_t *row, const float *x, size_t width) {
  float out = 0.0f;
  for (size_t b = 0; b < width / BLK; b++) {
    const uint8_t *blk = row + b * Q8B;
    float scale = scale_at(blk);
    for (int i = 0; i < BLK; i++) out += scale * (float)(int8_t)blk[2 + i] * x[b * BLK + i];
  }
  return out;
}

float mer_oracle_q8_row_dot_simd8x4(const uint8_t *row, const float *x, size_t width) {
  /* kernels/avx2.rs:98-126: w = cvt(q) * scale (one rounding); acc[lane] = fma(w, x, acc[lane]);
   * reduce (a0+a1)+(a2+a3), then the horizontal sum of avx2.rs:76-84. */
  float acc[4][8];
  memset(acc, 0, sizeof acc);
  for (size_t b = 0; b < width / BLK; b++) {
    const uint8_t *blk = row + b * Q8B;
    float scale = scale_at(blk);
    for (int l = 0; l < 4; l++)
      for (int i = 0; i < 8; i++) {
        float w = (float)(int8_t)blk[2 + l * 8 + i] * scale;
        acc[l][i] = fmaf(w, x[b * BLK + l * 8 + i], acc[l][i]);
      }
  }
  float v[8];
  for (int i = 0; i < 8; i++) v[i] = (acc[0][i] + acc[1][i]) + (acc[2][i] + acc[3][i]);
  float s0 = v[0] + v[4], s1 = v[1] + v[5], s2 = v[2] + v[6], s3 = v[3] + v[7];
  return (s0 + s1) + (s2 + s3);
}

/* q4_parity.rs:591-619 */
int mer_oracle_q4_matvec(const uint8_t *weights, size_t weights_len, const float *input,
                         size_t rows, size_t columns, size_t w_block_off, float *out) {
  if (rows == 0 || columns == 0 || columns % BLK != 0) return MER_ORACLE_ERR_INVALID_LAYOUT;
  size_t bpr = columns / BLK;
  size_t need = (w_block_off + rows * bpr) * Q4B;
  if (weights_len < need || weights_len % Q4B != 0) return MER_ORACLE_ERR_BUFFER_TOO_SMALL;
  float dec[BLK];
  for (size_t r = 0; r < rows; r++) {
    float sum = 0.0f;
    for (size_t b = 0; b < bpr; b++) {
      mer_oracle_dequant_q4_0_block(weights + (w_block_off + r * bpr + b) * Q4B, dec);
      for (int c = 0; c < BLK; c++) sum += dec[c] * input[b * BLK + c];
    }
    out[r] = sum;
  }
  return MER_ORACLE_OK;
}

/* ----------------------------------------------------- expert forward */

static int check_expert_layout(int dtype, size_t blob_len, size_t d_model, size_t d_ff,
                               size_t *proj_bytes) {
  if (d_model == 0 || d_ff == 0) return MER_ORACLE_ERR_INVALID_LAYOUT;
  size_t proj = mer_oracle_projection_bytes(dtype, d_model, d_ff);
  size_t need = 3 * proj;
  if (blob_len < need) {
    /* inference.rs:3381-3399: a shortfall within one page is a truncated payload. */
    if (need > SIZE_TOLERANCE_BYTES && need - blob_len <= SIZE_TOLERANCE_BYTES)
      return MER_ORACLE_ERR_TRUNCATED;
    return MER_ORACLE_ERR_BUFFER_TOO_SMALL;
  }
  *proj_bytes = proj;
  return MER_ORACLE_OK;
}

int mer_oracle_expert_forward(int dtype, int variant, const uint8_t *blob, size_t blob_len,
                              const float *x, size_t d_model, size_t d_ff, float swiglu_limit,
                              float *y, float *gated_out) {
  size_t proj;
  int rc = check_expert_layout(dtype, blob_len, d_model, d_ff, &proj);
  if (rc) return rc;
  float *g = (float *)malloc(sizeof(float) * d_ff * 2);
  if (!g) return MER_ORACLE_ERR_BUFFER_TOO_SMALL;
  float *u = g + d_ff;
  matvec_flat(dtype, variant, blob, d_ff, d_model, x, g);
  matvec_flat(dtype, variant, blob + proj, d_ff, d_model, x, u);
  for (size_t i = 0; i < d_ff; i++) u[i] = mer_oracle_silu(clamp_gate(g[i], swiglu_limit)) * u[i];
  if (gated_out) memcpy(gated_out, u, sizeof(float) * d_ff);
  matvec_flat(dtype, variant, blob + 2 * proj, d_model, d_ff, u, y);
  free(g);
  return MER_ORACLE_OK;
}

/* ------------------------------------------- threaded zero-copy forward */

int mer_oracle_has_avx2_fma(void) {
#if defined(__x86_64__)
  return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
#else
  return 0;
#endif
}

#if defined(__x86_64__)
__attribute__((target("avx2,fma"))) static inline float hsum256(__m256 acc) {
  __m128 lo = _mm256_castps256_ps128(acc);
  __m128 hi = _mm256_extractf128_ps(acc, 1);
  __m128 s = _mm_add_ps(lo, hi);
  __m128 sh = _mm_movehdup_ps(s);
  __m128 sums = _mm_add_ps(s, sh);
  sh = _mm_movehl_ps(sh, sums);
  return _mm_cvtss_f32(_mm_add_ss(sums, sh));
}

/* Eight dequantised weights of lane group l (0..3) of one block, as f32 = cvt(q) * scale. */
__attribute__((target("avx2,fma"))) static inline __m256 lane_weights(int dtype, const uint8_t *blk,
                                                                      int l, __m256 scale) {
  __m256i q;
  if (dtype == MER_ORACLE_Q8_0) {
    q = _mm256_cvtepi8_epi32(_mm_loadl_epi64((const __m128i *)(blk + 2 + l * 8)));
  } else {
    /* elements l*8..l*8+7: low nibbles of bytes 0..15 for l<2, high nibbles for l>=2 */
    __m128i bytes = _mm_loadl_epi64((const __m128i *)(blk + 2 + (l & 1) * 8));
    __m256i w = _mm256_cvtepu8_epi32(bytes);
    if (l >= 2) w = _mm256_srli_epi32(w, 4);
    q = _mm256_sub_epi32(_mm256_and_si256(w, _mm256_set1_epi32(0x0f)), _mm256_set1_epi32(8));
  }
  return _mm256_mul_ps(_mm256_cvtepi32_ps(q), scale);
}

/* One or two rows against one activation vector (kernels/avx2.rs:98-187 shape). */
__attribute__((target("avx2,fma"))) static void two_rows_avx2(int dtype, const uint8_t *ra,
                                                              const uint8_t *rb, const float *x,
                                                              size_t width, float *oa, float *ob) {
  size_t bb = block_bytes_of(dtype);
  __m256 a[4], b[4];
  for (int l = 0; l < 4; l++) a[l] = b[l] = _mm256_setzero_ps();
  for (size_t blk = 0; blk < width / BLK; blk++) {
    const uint8_t *pa = ra + blk * bb;
    __m256 sa = _mm256_set1_ps(scale_at(pa));
    if (rb) {
      const uint8_t *pb = rb + blk * bb;
      __m256 sb = _mm256_set1_ps(scale_at(pb));
      for (int l = 0; l < 4; l++) {
        __m256 xv = _mm256_loadu_ps(x + blk * BLK + l * 8);
        a[l] = _mm256_fmadd_ps(lane_weights(dtype, pa, l, sa), xv, a[l]);
        b[l] = _mm256_fmadd_ps(lane_weights(dtype, pb, l, sb), xv, b[l]);
      }
    } else {
      for (int l = 0; l < 4; l++) {
        __m256 xv = _mm256_loadu_ps(x + blk * BLK + l * 8);
        a[l] = _mm256_fmadd_ps(lane_weights(dtype, pa, l, sa), xv, a[l]);
      }
    }
  }
  *oa = hsum256(_mm256_add_ps(_mm256_add_ps(a[0], a[1]), _mm256_add_ps(a[2], a[3])));
  if (rb) *ob = hsum256(_mm256_add_ps(_mm256_add_ps(b[0], b[1]), _mm256_add_ps(b[2], b[3])));
}
#endif

static void two_rows_scalar(int dtype, const uint8_t *ra, const uint8_t *rb, const float *x,
                            size_t width, float *oa, float *ob) {
  /* q8_0_gate_up_row_scalar order, inference.rs:3553-3572 */
  size_t bb = block_bytes_of(dtype);
  float a = 0.0f, b = 0.0f, ta[BLK], tb[BLK];
  for (size_t blk = 0; blk < width / BLK; blk++) {
    dequant_block(dtype, ra + blk * bb, ta);
    if (rb) dequant_block(dtype, rb + blk * bb, tb);
    for (int i = 0; i < BLK; i++) {
      a += ta[i] * x[blk * BLK + i];
      if (rb) b += tb[i] * x[blk * BLK + i];
    }
  }
  *oa = a;
  if (rb) *ob = b;
}

static void two_rows(int dtype, const uint8_t *ra, const uint8_t *rb, const float *x, size_t width,
                     float *oa, float *ob) {
#if defined(__x86_64__)
  if (mer_oracle_has_avx2_fma()) {
    two_rows_avx2(dtype, ra, rb, x, width, oa, ob);
    return;
  }
#endif
  two_rows_scalar(dtype, ra, rb, x, width, oa, ob);
}

typedef struct {
  int dtype;
  const uint8_t *gate, *up, *down;
  const float *x;
  float *gated, *y;
  size_t d_model, d_ff, row0, row1;
  float limit;
  int phase;
} mt_job;

static void *mt_worker(void *arg) {
  mt_job *j = (mt_job *)arg;
  size_t bb = block_bytes_of(j->dtype);
  if (j->phase == 0) {
    size_t rb = j->d_model / BLK * bb;
    for (size_t r = j->row0; r < j->row1; r++) {
      float g = 0.0f, u = 0.0f;
      two_rows(j->dtype, j->gate + r * rb, j->up + r * rb, j->x, j->d_model, &g, &u);
      j->gated[r] = mer_oracle_silu(clamp_gate(g, j->limit)) * u;
    }
  } else {
    size_t rb = j->d_ff / BLK * bb;
    for (size_t r = j->row0; r < j->row1; r++) {
      float v, unused;
      two_rows(j->dtype, j->down + r * rb, NULL, j->gated, j->d_ff, &v, &unused);
      j->y[r] = v;
    }
  }
  return NULL;
}

/* forward_q8_0_direct_into_with_kernel shape (inference.rs:3659-3746): rows of d_ff fan out
 * over the pool, then rows of d_model.  Q4_0 runs through the same fused zero-copy row kernels. */
int mer_oracle_expert_forward_mt(int dtype, const uint8_t *blob, size_t blob_len, const float *x,
                                 size_t d_model, size_t d_ff, float swiglu_limit, float *y,
                                 int n_threads) {
  size_t proj;
  int rc = check_expert_layout(dtype, blob_len, d_model, d_ff, &proj);
  if (rc) return -rc;
  if (d_model % BLK || d_ff % BLK) return -MER_ORACLE_ERR_INVALID_LAYOUT;
  if (n_threads < 1) n_threads = 1;
  if (n_threads > 256) n_threads = 256;
  float *gated = (float *)malloc(sizeof(float) * d_ff);
  pthread_t *tids = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)n_threads);
  mt_job *jobs = (mt_job *)malloc(sizeof(mt_job) * (size_t)n_threads);
  if (!gated || !tids || !jobs) {
    free(gated), free(tids), free(jobs);
    return -MER_ORACLE_ERR_BUFFER_TOO_SMALL;
  }
  for (int phase = 0; phase < 2; phase++) {
    size_t rows = phase == 0 ? d_ff : d_model;
    for (int t = 0; t < n_threads; t++) {
      mt_job *j = &jobs[t];
      j->dtype = dtype, j->gate = blob, j->up = blob + proj, j->down = blob + 2 * proj;
      j->x = x, j->gated = gated, j->y = y, j->d_model = d_model, j->d_ff = d_ff;
      j->limit = swiglu_limit, j->phase = phase;
      j->row0 = rows * (size_t)t / (size_t)n_threads;
      j->row1 = rows * (size_t)(t + 1) / (size_t)n_threads;
      if (t > 0) pthread_create(&tids[t], NULL, mt_worker, j);
    }
    mt_worker(&jobs[0]);
    for (int t = 1; t < n_threads; t++) pthread_join(tids[t], NULL);
  }
  free(gated), free(tids), free(jobs);
  return n_threads;
}

/* -------------------------------------------------------------- router */

/* transformer.rs:2747-2819 */
void mer_oracle_softmax_inplace(float *v, size_t n) {
  if (n == 0) return;
  float max = -INFINITY;
  int saw_nan = 0;
  for (size_t i = 0; i < n; i++) {
    if (v[i] != v[i])
      saw_nan = 1;
    else if (v[i] > max)
      max = v[i];
  }
  if (saw_nan || !isfinite(max)) {
    float uniform = 1.0f / (float)n;
    for (size_t i = 0; i < n; i++) v[i] = uniform;
    return;
  }
  float sum = 0.0f;
  for (size_t i = 0; i < n; i++) {
    v[i] = expf(v[i] - max);
    sum += v[i];
  }
  if (sum > 0.0f)
    for (size_t i = 0; i < n; i++) v[i] /= sum;
}

/* f32::total_cmp (gating.rs:289): order by sign-magnitude bit pattern. */
static inline int32_t total_key(float f) {
  int32_t b;
  memcpy(&b, &f, 4);
  b ^= (int32_t)(((uint32_t)(b >> 31)) >> 1);
  return b;
}
/* gating.rs:283-294 */
static inline int score_id_is_better(float cs, size_t cid, float is, size_t iid) {
  int32_t a = total_key(cs), b = total_key(is);
  if (a > b) return 1;
  if (a == b) return cid < iid;
  return 0;
}

/* gating.rs:335-345 */
static int group_filter_shape(const mer_oracle_gate *g, size_t *n_group, size_t *group_size) {
  size_t ng = g->n_group < 1 ? 1 : g->n_group;
  if (ng <= 1 || g->topk_group == 0 || g->topk_group >= ng || g->num_experts % ng != 0) return 0;
  *n_group = ng;
  *group_size = g->num_experts / ng;
  return 1;
}

static void gate_scores(const mer_oracle_gate *g, const float *x, float *scores) {
  /* DenseWeight::matvec_into -> dot_f32 per row (dense_tensor.rs:422-441, kernels/scalar.rs:10-17). */
  for (size_t e = 0; e < g->num_experts; e++) {
    float acc = 0.0f;
    const float *row = g->weights + e * g->d_model;
    for (size_t i = 0; i < g->d_model; i++) acc += row[i] * x[i];
    if (g->logit_bias) acc += g->logit_bias[e];
    scores[e] = acc;
  }
  /* gating.rs:271-280 */
  if (g->scoring_func == MER_ORACLE_SCORE_SOFTMAX) {
    mer_oracle_softmax_inplace(scores, g->num_experts);
  } else {
    for (size_t e = 0; e < g->num_experts; e++) scores[e] = 1.0f / (1.0f + expf(-scores[e]));
  }
}

static void finish_weights(const mer_oracle_gate *g, float *weights, size_t n) {
  /* gating.rs:455-474 */
  if (g->normalise_topk) {
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) sum += weights[i];
    if (isfinite(sum) && sum > 0.0f)
      for (size_t i = 0; i < n; i++) weights[i] /= sum;
  }
  if (g->routed_scaling_factor != 1.0f && isfinite(g->routed_scaling_factor))
    for (size_t i = 0; i < n; i++) weights[i] *= g->routed_scaling_factor;
}

/* gating.rs:395-476 */
int mer_oracle_route(const mer_oracle_gate *g, const float *x, uint32_t *experts, float *weights,
                     size_t *n_selected, float *scores_out, float *gap_out) {
  size_t E = g->num_experts;
  if (g->top_k == 0 || g->top_k > E) return MER_ORACLE_ERR_INVALID_LAYOUT;
  float *scores = (float *)malloc(sizeof(float) * E * 2);
  if (!scores) return MER_ORACLE_ERR_BUFFER_TOO_SMALL;
  float *selection = scores + E;
  gate_scores(g, x, scores);
  for (size_t e = 0; e < E; e++)
    selection[e] = g->correction_bias ? scores[e] + g->correction_bias[e] : scores[e];

  /* select_top_groups: gating.rs:352-376 (insertion by score desc, id asc: 296-313) */
  size_t n_group = 0, group_size = 0, n_top_groups = 0;
  size_t top_groups[64];
  float top_group_scores[64];
  int grouped = group_filter_shape(g, &n_group, &group_size);
  if (grouped && g->topk_group > 64) {
    free(scores);
    return MER_ORACLE_ERR_INVALID_LAYOUT;
  }
  if (grouped) {
    for (size_t gi = 0; gi < n_group; gi++) {
      float top1 = -INFINITY, top2 = -INFINITY;
      for (size_t i = 0; i < group_size; i++) {
        float s = selection[gi * group_size + i];
        if (s > top1) {
          top2 = top1;
          top1 = s;
        } else if (s > top2) {
          top2 = s;
        }
      }
      float sum = top1 + (isfinite(top2) ? top2 : 0.0f);
      size_t pos = n_top_groups;
      for (size_t p = 0; p < n_top_groups; p++)
        if (score_id_is_better(sum, gi, top_group_scores[p], top_groups[p])) {
          pos = p;
          break;
        }
      if (pos < n_top_groups || n_top_groups < g->topk_group) {
        size_t last = n_top_groups < g->topk_group ? n_top_groups : g->topk_group - 1;
        for (size_t p = last; p > pos; p--) {
          top_groups[p] = top_groups[p - 1];
          top_group_scores[p] = top_group_scores[p - 1];
        }
        top_groups[pos] = gi;
        top_group_scores[pos] = sum;
        if (n_top_groups < g->topk_group) n_top_groups++;
      }
    }
  }

  /* insert_top_expert over allowed experts: gating.rs:315-333, 429-441 */
  size_t n = 0;
  float *top_scores = weights; /* reuse caller storage for selection scores during insertion */
  float best_rejected = -INFINITY;
  for (size_t e = 0; e < E; e++) {
    if (grouped) {
      int allowed = 0;
      for (size_t p = 0; p < n_top_groups; p++) allowed |= top_groups[p] == e / group_size;
      if (!allowed) continue;
    }
    float s = selection[e];
    if (!isfinite(s)) continue;
    size_t pos = n;
    for (size_t p = 0; p < n; p++)
      if (score_id_is_better(s, e, top_scores[p], experts[p])) {
        pos = p;
        break;
      }
    if (pos < n || n < g->top_k) {
      if (n == g->top_k && top_scores[n - 1] > best_rejected) best_rejected = top_scores[n - 1];
      size_t last = n < g->top_k ? n : g->top_k - 1;
      for (size_t p = last; p > pos; p--) {
        experts[p] = experts[p - 1];
        top_scores[p] = top_scores[p - 1];
      }
      experts[pos] = (uint32_t)e;
      top_scores[pos] = s;
      if (n < g->top_k) n++;
    } else if (s > best_rejected) {
      best_rejected = s;
    }
  }
  if (gap_out) *gap_out = n ? top_scores[n - 1] - best_rejected : INFINITY;
  for (size_t i = 0; i < n; i++) weights[i] = scores[experts[i]];
  finish_weights(g, weights, n);
  if (n_selected) *n_selected = n;
  if (scores_out) memcpy(scores_out, scores, sizeof(float) * E);
  free(scores);
  return MER_ORACLE_OK;
}

typedef struct {
  uint32_t id;
  float sel;
} sel_entry;
static int sel_cmp(const void *a, const void *b) {
  const sel_entry *x = (const sel_entry *)a, *y = (const sel_entry *)b;
  int32_t kx = total_key(x->sel), ky = total_key(y->sel);
  if (kx != ky) return kx > ky ? -1 : 1;
  return x->id < y->id ? -1 : (x->id > y->id ? 1 : 0);
}

/* gating.rs:684-764 */
int mer_oracle_route_stable(const mer_oracle_gate *g, const float *x, uint32_t *experts,
                            float *weights, size_t *n_selected) {
  size_t E = g->num_experts;
  float *scores = (float *)malloc(sizeof(float) * E);
  sel_entry *sel = (sel_entry *)malloc(sizeof(sel_entry) * E);
  if (!scores || !sel) {
    free(scores), free(sel);
    return MER_ORACLE_ERR_BUFFER_TOO_SMALL;
  }
  gate_scores(g, x, scores);
  for (size_t e = 0; e < E; e++) {
    sel[e].id = (uint32_t)e;
    sel[e].sel = scores[e] + (g->correction_bias ? g->correction_bias[e] : 0.0f);
    if (!g->correction_bias) sel[e].sel = scores[e];
  }
  size_t n_group, group_size;
  if (group_filter_shape(g, &n_group, &group_size)) {
    sel_entry *gs = (sel_entry *)malloc(sizeof(sel_entry) * n_group);
    for (size_t gi = 0; gi < n_group; gi++) {
      float top1 = -INFINITY, top2 = -INFINITY;
      for (size_t i = 0; i < group_size; i++) {
        float s = sel[gi * group_size + i].sel;
        if (s > top1) {
          top2 = top1;
          top1 = s;
        } else if (s > top2) {
          top2 = s;
        }
      }
      gs[gi].id = (uint32_t)gi;
      gs[gi].sel = top1 + (isfinite(top2) ? top2 : 0.0f);
    }
    qsort(gs, n_group, sizeof(sel_entry), sel_cmp);
    for (size_t e = 0; e < E; e++) {
      int keep = 0;
      for (size_t p = 0; p < g->topk_group && p < n_group; p++) keep |= gs[p].id == e / group_size;
      if (!keep) sel[e].sel = -INFINITY;
    }
    free(gs);
  }
  qsort(sel, E, sizeof(sel_entry), sel_cmp);
  size_t n = 0;
  for (size_t i = 0; i < E && n < g->top_k; i++)
    if (isfinite(sel[i].sel)) {
      experts[n] = sel[i].id;
      weights[n] = scores[sel[i].id];
      n++;
    }
  finish_weights(g, weights, n);
  if (n_selected) *n_selected = n;
  free(scores), free(sel);
  return MER_ORACLE_OK;
}

/* ------------------------------------------------------------- combine */

/* inference.rs:4472-4491; engine.rs:5575-5581 skips zero weights. */
void mer_oracle_combine(const float *outputs, const float *scores, size_t k, size_t d, float *out,
                        int skip_zero) {
  for (size_t i = 0; i < d; i++) out[i] = 0.0f;
  for (size_t s = 0; s < k; s++) {
    if (skip_zero && scores[s] == 0.0f) continue;
    for (size_t i = 0; i < d; i++) out[i] += scores[s] * outputs[s * d + i];
  }
}

/* ------------------------------------------- the steps either side of the MoE block */

/* RmsNorm::forward_inplace, transformer.rs:62-74: sequential sum of squares, scale = 1 / sqrt(mean + eps),
 * y = (x * scale) * weight (two roundings, in that order). */
void mer_oracle_rmsnorm(const float *x, const float *weight, size_t n, float eps, float *y) {
  float sq_sum = 0.0f;
  for (size_t i = 0; i < n; i++) sq_sum += x[i] * x[i];
  float mean_sq = sq_sum / (float)n;
  float scale = 1.0f / sqrtf(mean_sq + eps);
  for (size_t i = 0; i < n; i++) y[i] = x[i] * scale * weight[i];
}

/* SharedExpert::forward, transformer.rs:2224-2231: sigmoid of the sequential dot gate_inp . x. */
float mer_oracle_shared_gate_scale(const float *gate_inp, const float *x, size_t n) {
  float logit = 0.0f;
  for (size_t i = 0; i < n; i++) logit += gate_inp[i] * x[i];
  return 1.0f / (1.0f + expf(-logit));
}

/* add_residual_into, transformer.rs:2006-2011 */
void mer_oracle_add_residual(const float *a, const float *b, size_t n, float *out) {
  for (size_t i = 0; i < n; i++) out[i] = a[i] + b[i];
}

/* engine.rs:1651-1673 */
int mer_oracle_accumulate_ordered_f16(const uint16_t *outputs, size_t outputs_len,
                                      const float *weights, size_t n_weights, size_t d_model,
                                      float *out) {
  if (outputs_len != n_weights * d_model) return 0;
  for (size_t i = 0; i < d_model; i++) out[i] = 0.0f;
  for (size_t s = 0; s < n_weights; s++) {
    if (weights[s] == 0.0f) continue;
    for (size_t i = 0; i < d_model; i++)
      out[i] += weights[s] * mer_oracle_f16_to_f32(outputs[s * d_model + i]);
  }
  return 1;
}

/* ---------------------------------------------------------- generators */

/* inference.rs:3064-3082 */
void mer_oracle_synth_hidden_state(uint64_t token_idx, size_t d_model, uint64_t seed, float *out) {
  uint64_t s = token_idx * 0x9E3779B97F4A7C15ull + seed * 0xBF58476D1CE4E5B9ull;
  for (size_t i = 0; i < d_model; i++) {
    s += 0x9E3779B97F4A7C15ull;
    uint64_t z = s;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    uint32_t u = (uint32_t)(z >> 40);
    out[i] = (float)u / (float)(1u << 23) - 1.0f;
  }
}

/* inference.rs:5905-5926 */
void mer_oracle_randomized_q8_expert(size_t d_model, size_t d_ff, uint64_t state, uint8_t *out) {
  size_t weights = d_model * d_ff;
  size_t blocks = (weights + BLK - 1) / BLK;
  for (int projection = 0; projection < 3; projection++) {
    for (size_t block = 0; block < blocks; block++) {
      size_t count = weights - block * BLK < BLK ? weights - block * BLK : BLK;
      float values[BLK];
      memset(values, 0, sizeof values);
      for (size_t i = 0; i < count; i++) {
        state ^= state << 13;
        state ^= state >> 7;
        state ^= state << 17;
        values[i] = ((float)(uint32_t)(state >> 40) / (float)((1u << 24) - 1) - 0.5f) *
                    (0.08f + (float)projection * 0.01f);
      }
      mer_oracle_quant_q8_0_block(values, count, out);
      out += Q8B;
    }
  }
}

/* ------------------------------------------------------- layer forward */

typedef struct {
  int dtype, variant;
  const mer_oracle_gate *gate;
  const uint8_t *const *blobs;
  size_t blob_len;
  const uint8_t *shared;
  const float *x;
  size_t t0, t1, d_ff;
  float limit;
  float *out;
  uint32_t *ids;
  float *w;
  float *gaps;
  int rc;
} layer_job;

static void *layer_worker(void *arg) {
  layer_job *j = (layer_job *)arg;
  const mer_oracle_gate *g = j->gate;
  size_t D = g->d_model, k = g->top_k;
  float *y = (float *)malloc(sizeof(float) * D);
  uint32_t *ids = (uint32_t *)malloc(sizeof(uint32_t) * k);
  float *w = (float *)malloc(sizeof(float) * k);
  for (size_t t = j->t0; t < j->t1 && !j->rc; t++) {
    const float *xt = j->x + t * D;
    float *ot = j->out + t * D;
    size_t n = 0;
    float gap = 0.0f;
    j->rc = mer_oracle_route(g, xt, ids, w, &n, NULL, &gap);
    if (j->rc) break;
    for (size_t s = 0; s < k; s++) {
      if (j->ids) j->ids[t * k + s] = s < n ? ids[s] : UINT32_MAX;
      if (j->w) j->w[t * k + s] = s < n ? w[s] : 0.0f;
    }
    if (j->gaps) j->gaps[t] = gap;
    for (size_t i = 0; i < D; i++) ot[i] = 0.0f;
    /* engine.rs:5575-5581: acc[d] += weight * y[d] in slot order, zero weights skipped */
    for (size_t s = 0; s < n; s++) {
      j->rc = mer_oracle_expert_forward(j->dtype, j->variant, j->blobs[ids[s]], j->blob_len, xt, D,
                                        j->d_ff, j->limit, y, NULL);
      if (j->rc) break;
      if (w[s] != 0.0f)
        for (size_t i = 0; i < D; i++) ot[i] += w[s] * y[i];
    }
    if (!j->rc && j->shared) {
      /* model.rs:2758-2763: the shared expert's output is added after the routed combine */
      j->rc = mer_oracle_expert_forward(j->dtype, j->variant, j->shared, j->blob_len, xt, D, j->d_ff,
                                        j->limit, y, NULL);
      if (!j->rc)
        for (size_t i = 0; i < D; i++) ot[i] += y[i];
    }
  }
  free(y), free(ids), free(w);
  return NULL;
}

int mer_oracle_moe_layer_forward(int dtype, int variant, const mer_oracle_gate *gate,
                                 const uint8_t *const *expert_blobs, size_t blob_len,
                                 const uint8_t *shared_blob, const float *x, size_t n_tokens,
                                 size_t d_ff, float swiglu_limit, float *out, uint32_t *topk_ids,
                                 float *topk_w, float *gaps, int n_threads) {
  if (n_threads < 1) n_threads = 1;
  if ((size_t)n_threads > n_tokens) n_threads = n_tokens ? (int)n_tokens : 1;
  pthread_t *tids = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)n_threads);
  layer_job *jobs = (layer_job *)malloc(sizeof(layer_job) * (size_t)n_threads);
  for (int t = 0; t < n_threads; t++) {
    layer_job *j = &jobs[t];
    j->dtype = dtype, j->variant = variant, j->gate = gate, j->blobs = expert_blobs;
    j->blob_len = blob_len, j->shared = shared_blob, j->x = x, j->d_ff = d_ff;
    j->limit = swiglu_limit, j->out = out, j->ids = topk_ids, j->w = topk_w, j->gaps = gaps;
    j->rc = 0;
    j->t0 = n_tokens * (size_t)t / (size_t)n_threads;
    j->t1 = n_tokens * (size_t)(t + 1) / (size_t)n_threads;
    if (t > 0) pthread_create(&tids[t], NULL, layer_worker, j);
  }
  layer_worker(&jobs[0]);
  int rc = jobs[0].rc;
  for (int t = 1; t < n_threads; t++) {
    pthread_join(tids[t], NULL);
    if (!rc) rc = jobs[t].rc;
  }
  free(tids), free(jobs);
  return rc;
}

/* ----------------------------------------------- production-shaped layer */

static int expert_forward_rows_1t(int dtype, const uint8_t *blob, size_t proj, const float *x, size_t d_model,
                                  size_t d_ff, float limit, float *gated, float *y) {
  mt_job j;
  j.dtype = dtype, j.gate = blob, j.up = blob + proj, j.down = blob + 2 * proj;
  j.x = x, j.gated = gated, j.y = y, j.d_model = d_model, j.d_ff = d_ff, j.limit = limit;
  j.phase = 0, j.row0 = 0, j.row1 = d_ff;
  mt_worker(&j);
  j.phase = 1, j.row1 = d_model;
  mt_worker(&j);
  return 0;
}

typedef struct {
  int dtype;
  const mer_oracle_gate *gate;
  const uint8_t *const *blobs;
  const uint8_t *shared;
  size_t proj, d_ff, t0, t1;
  const float *x;
  float limit;
  float *out;
  int rc;
} prod_job;

static void *prod_worker(void *arg) {
  prod_job *j = (prod_job *)arg;
  const mer_oracle_gate *g = j->gate;
  size_t D = g->d_model, k = g->top_k;
  float *y = (float *)malloc(sizeof(float) * (D + j->d_ff));
  float *gated = y + D;
  uint32_t *ids = (uint32_t *)malloc(sizeof(uint32_t) * k);
  float *w = (float *)malloc(sizeof(float) * k);
  for (size_t t = j->t0; t < j->t1 && !j->rc; t++) {
    const float *xt = j->x + t * D;
    float *ot = j->out + t * D;
    size_t n = 0;
    j->rc = mer_oracle_route(g, xt, ids, w, &n, NULL, NULL);
    for (size_t i = 0; i < D; i++) ot[i] = 0.0f;
    for (size_t s = 0; s < n && !j->rc; s++) {
      expert_forward_rows_1t(j->dtype, j->blobs[ids[s]], j->proj, xt, D, j->d_ff, j->limit, gated, y);
      if (w[s] != 0.0f)
        for (size_t i = 0; i < D; i++) ot[i] += w[s] * y[i];
    }
    if (!j->rc && j->shared) {
      expert_forward_rows_1t(j->dtype, j->shared, j->proj, xt, D, j->d_ff, j->limit, gated, y);
      for (size_t i = 0; i < D; i++) ot[i] += y[i];
    }
  }
  free(y), free(ids), free(w);
  return NULL;
}

int mer_oracle_moe_layer_forward_production(int dtype, const mer_oracle_gate *gate,
                                            const uint8_t *const *expert_blobs, size_t blob_len,
                                            const uint8_t *shared_blob, const float *x, size_t n_tokens,
                                            size_t d_ff, float swiglu_limit, float *out, int n_threads) {
  size_t D = gate->d_model, proj;
  int rc = check_expert_layout(dtype, blob_len, D, d_ff, &proj);
  if (rc) return rc;
  if (D % BLK || d_ff % BLK) return MER_ORACLE_ERR_INVALID_LAYOUT;
  if (n_threads < 1) n_threads = 1;
  if (n_tokens >= (size_t)n_threads) {
    pthread_t *tids = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)n_threads);
    prod_job *jobs = (prod_job *)malloc(sizeof(prod_job) * (size_t)n_threads);
    for (int t = 0; t < n_threads; t++) {
      prod_job *j = &jobs[t];
      j->dtype = dtype, j->gate = gate, j->blobs = expert_blobs, j->shared = shared_blob, j->proj = proj;
      j->d_ff = d_ff, j->x = x, j->limit = swiglu_limit, j->out = out, j->rc = 0;
      j->t0 = n_tokens * (size_t)t / (size_t)n_threads;
      j->t1 = n_tokens * (size_t)(t + 1) / (size_t)n_threads;
      if (t > 0) pthread_create(&tids[t], NULL, prod_worker, j);
    }
    prod_worker(&jobs[0]);
    rc = jobs[0].rc;
    for (int t = 1; t < n_threads; t++) {
      pthread_join(tids[t], NULL);
      if (!rc) rc = jobs[t].rc;
    }
    free(tids), free(jobs);
    return rc;
  }
  size_t k = gate->top_k;
  float *y = (float *)malloc(sizeof(float) * D);
  uint32_t *ids = (uint32_t *)malloc(sizeof(uint32_t) * k);
  float *w = (float *)malloc(sizeof(float) * k);
  for (size_t t = 0; t < n_tokens && !rc; t++) {
    const float *xt = x + t * D;
    float *ot = out + t * D;
    size_t n = 0;
    rc = mer_oracle_route(gate, xt, ids, w, &n, NULL, NULL);
    for (size_t i = 0; i < D; i++) ot[i] = 0.0f;
    for (size_t s = 0; s < n && !rc; s++) {
      int r = mer_oracle_expert_forward_mt(dtype, expert_blobs[ids[s]], blob_len, xt, D, d_ff, swiglu_limit, y, n_threads);
      if (r < 0) rc = -r;
      if (w[s] != 0.0f)
        for (size_t i = 0; i < D; i++) ot[i] += w[s] * y[i];
    }
    if (!rc && shared_blob) {
      int r = mer_oracle_expert_forward_mt(dtype, shared_blob, blob_len, xt, D, d_ff, swiglu_limit, y, n_threads);
      if (r < 0) rc = -r;
      for (size_t i = 0; i < D; i++) ot[i] += y[i];
    }
  }
  free(y), free(ids), free(w);
  return rc;
}
