/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement of the vecops matmul semantic, used only as the checker in
 * tests/, in __graft_entry__.smoke() and as the "port" CPU baseline of
 * bench.py.  Nothing the library ships calls into this file.
 *
 * What it restates (paths are inside the vecops repository):
 *   - C[M,N] = A[M,K] . B[N,K]^T, B always addressed [N,K]
 *       include/vecops/ops/Matmul.h:13-17
 *   - the form the reference's own tests use as their expected value: a naive
 *     triple loop accumulating in the accumulator type
 *       tests/ops/MatmulTest.cpp:82-97
 *       tests/ops/MatmulConversionTestCommon.h:126-141
 *   - memory dtype != compute dtype: load converts to the compute type, the
 *     store converts from the accumulator type
 *       docs/Tensor.md:218-231
 *   - float -> bfloat16 is round-to-nearest-even on the bit pattern, NaN maps
 *     to 0x7fc0
 *       include/vecops/util/BFloat16.h:25-37
 *   - 8-bit products accumulate in int32 and wrap modulo 2^32
 *       include/vecops/vec/WideningDot.h:100-103, tests/ops/MatmulTest.cpp:1025-1055
 *   - per-output-column scale applied to the fp32 accumulator before the
 *     store conversion
 *       tests/ops/MatmulConversionTestCommon.h:664-671
 *
 * Floating-point sums are taken in double and rounded once to float: the
 * reference fixes no summation order (AMX TMUL, AVX-512 lanes and the scalar
 * test loop all differ), so the checker uses the order-free value that every
 * fp32 order approximates, and the tests carry the tolerance.
 *
 * Pinned against the reference itself: oracle/_ref (the reference's own
 * ops::matmul built from its headers) on the fixtures under tests/golden/.
 * One row is the exception - fp16 operands: PARITY UNPINNED for the product
 * (the reference's fp16 tile kernel needs AMX-FP16, absent on the hosts this
 * was built on); its two conversions are pinned, see oracle_matmul_f16_fused.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t bits) {
  uint32_t wide = (uint32_t)bits << 16;
  float out;
  memcpy(&out, &wide, sizeof(out));
  return out;
}

static inline uint16_t f32_to_bf16(float value) {
  if (isnan(value)) return 0x7fc0;
  uint32_t bits;
  memcpy(&bits, &value, sizeof(bits));
  const uint32_t bias = ((bits >> 16) & 1u) + 0x7fffu;
  return (uint16_t)((bits + bias) >> 16);
}

/* exported so that tests can pin the rounding rule on its own */
uint16_t oracle_f32_to_bf16(float value) { return f32_to_bf16(value); }
float oracle_bf16_to_f32(uint16_t bits) { return bf16_to_f32(bits); }

/* fp32 x fp32 -> fp32.  Element strides on every tensor. */
void oracle_matmul_f32(int64_t m, int64_t n, int64_t k, const float* a, int64_t sam, int64_t sak, const float* b,
                       int64_t sbn, int64_t sbk, float* c, int64_t scm, int64_t scn) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      double sum = 0.0;
      for (int64_t kk = 0; kk < k; ++kk) sum += (double)a[i * sam + kk * sak] * (double)b[j * sbn + kk * sbk];
      c[i * scm + j * scn] = (float)sum;
    }
  }
}

/* bf16 x bf16 -> fp32 accumulate -> (optional column scale) -> bf16 or fp32.
 * c_is_bf16 selects the store type. */
void oracle_matmul_bf16(int64_t m, int64_t n, int64_t k, const uint16_t* a, int64_t sam, int64_t sak,
                        const uint16_t* b, int64_t sbn, int64_t sbk, const float* column_scale, void* c, int64_t scm,
                        int64_t scn, int c_is_bf16) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      double sum = 0.0;
      for (int64_t kk = 0; kk < k; ++kk)
        sum += (double)bf16_to_f32(a[i * sam + kk * sak]) * (double)bf16_to_f32(b[j * sbn + kk * sbk]);
      float acc = (float)sum;
      if (column_scale) acc *= column_scale[j];
      if (c_is_bf16) ((uint16_t*)c)[i * scm + j * scn] = f32_to_bf16(acc);
      else ((float*)c)[i * scm + j * scn] = acc;
    }
  }
}

/* 8-bit x 8-bit -> int32, wrapping.  a_signed / b_signed select int8 or uint8. */
void oracle_matmul_i8(int64_t m, int64_t n, int64_t k, const void* a, int64_t sam, int64_t sak, int a_signed,
                      const void* b, int64_t sbn, int64_t sbk, int b_signed, int32_t* c, int64_t scm, int64_t scn) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      uint32_t sum = 0;
      for (int64_t kk = 0; kk < k; ++kk) {
        const int32_t av = a_signed ? (int32_t)((const int8_t*)a)[i * sam + kk * sak]
                                    : (int32_t)((const uint8_t*)a)[i * sam + kk * sak];
        const int32_t bv = b_signed ? (int32_t)((const int8_t*)b)[j * sbn + kk * sbk]
                                    : (int32_t)((const uint8_t*)b)[j * sbn + kk * sbk];
        sum += (uint32_t)av * (uint32_t)bv;
      }
      int32_t out;
      memcpy(&out, &sum, sizeof(out));
      c[i * scm + j * scn] = out;
    }
  }
}

/* Weight-only int8: bf16 activations x int8 weights (widened exactly to the
 * bf16 compute type) -> fp32 accumulate -> column scale -> bf16 or fp32. */
void oracle_matmul_w8(int64_t m, int64_t n, int64_t k, const uint16_t* a, int64_t sam, int64_t sak, const int8_t* w,
                      int64_t swn, int64_t swk, const float* column_scale, void* c, int64_t scm, int64_t scn,
                      int c_is_bf16) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      double sum = 0.0;
      for (int64_t kk = 0; kk < k; ++kk)
        sum += (double)bf16_to_f32(a[i * sam + kk * sak]) * (double)w[j * swn + kk * swk];
      float acc = (float)sum;
      if (column_scale) acc *= column_scale[j];
      if (c_is_bf16) ((uint16_t*)c)[i * scm + j * scn] = f32_to_bf16(acc);
      else ((float*)c)[i * scm + j * scn] = acc;
    }
  }
}

/* Fused forms: the reference's explicit accumulate form COut = transform(CIn + A.B^T) (ops/Matmul.h:519-570) with the
 * transforms its fusion tests compose (tests/ops/MatmulConversionTestCommon.h:623-704 runtime and per-column scale,
 * :705-770 bias as a stride-0 CIn + clamp, :1028-1160 relu / sigmoid / silu): the accumulator input joins the sum, then
 * value * alpha * column_scale[col], then the activation, then the store conversion.
 * act: 0 none, 1 relu, 2 sigmoid, 3 silu, 4 clamp(lo, hi).  cin: f32 (cin_kind 0) or bf16 bits (1); strides may be 0. */
static float oracle_activation(float x, int act, float lo, float hi) {
  switch (act) {
    case 1: return x > 0.f ? x : 0.f;
    case 2: return (float)(1.0 / (1.0 + exp(-(double)x)));
    case 3: return (float)((double)x / (1.0 + exp(-(double)x)));
    case 4: return x < lo ? lo : (x > hi ? hi : x);
    default: return x;
  }
}

void oracle_matmul_bf16_fused(int64_t m, int64_t n, int64_t k, const uint16_t* a, int64_t sam, int64_t sak,
                              const uint16_t* b, int64_t sbn, int64_t sbk, const void* cin, int cin_kind, int64_t cin_sm,
                              int64_t cin_sn, float alpha, const float* column_scale, int act, float lo, float hi, void* c,
                              int64_t scm, int64_t scn, int c_is_bf16) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      double sum = 0.0;
      if (cin) sum = cin_kind == 1 ? (double)bf16_to_f32(((const uint16_t*)cin)[i * cin_sm + j * cin_sn])
                                   : (double)((const float*)cin)[i * cin_sm + j * cin_sn];
      for (int64_t kk = 0; kk < k; ++kk)
        sum += (double)bf16_to_f32(a[i * sam + kk * sak]) * (double)bf16_to_f32(b[j * sbn + kk * sbk]);
      float acc = (float)sum * alpha;
      if (column_scale) acc *= column_scale[j];
      acc = oracle_activation(acc, act, lo, hi);
      if (c_is_bf16) ((uint16_t*)c)[i * scm + j * scn] = f32_to_bf16(acc);
      else ((float*)c)[i * scm + j * scn] = acc;
    }
  }
}

/* fp16 x fp16 -> fp32 accumulate -> transform -> fp16 or fp32: the AMX_F16F32 row of the reference
 * (include/vecops/matmul/details/kernel/amx/Atoms.h:74-77; the accumulate form is the bf16 one above).
 * float16_t is a 16-bit storage wrapper whose widening is exact and whose narrowing is IEEE round to nearest even
 * (include/vecops/util/Float16.h:272-277).  Both conversions below are pinned bit for bit against the reference's
 * own (all 65536 patterns; a sweep of floats through the narrowing).  The product itself is NOT pinned: the
 * reference's fp16 tile kernel needs AMX-FP16, which the hosts this was developed on do not have ("parity unpinned"
 * for this one row; the tests hold the CUDA path to this restatement). */
static inline float f16_to_f32(uint16_t bits) {
  const uint32_t sign = (uint32_t)(bits & 0x8000u) << 16;
  uint32_t exponent = (bits >> 10) & 0x1fu;
  uint32_t mantissa = bits & 0x3ffu;
  uint32_t wide;
  if (exponent == 0x1fu) {
    wide = sign | 0x7f800000u | (mantissa << 13) | (mantissa ? 0x00400000u : 0u); /* a NaN comes out quiet, payload kept */
  } else if (exponent != 0) {
    wide = sign | ((exponent + 112u) << 23) | (mantissa << 13);
  } else if (mantissa == 0) {
    wide = sign;
  } else { /* subnormal: renormalise */
    int shift = 0;
    while ((mantissa & 0x400u) == 0) {
      mantissa <<= 1;
      ++shift;
    }
    mantissa &= 0x3ffu;
    wide = sign | ((uint32_t)(113 - shift) << 23) | (mantissa << 13);
  }
  float out;
  memcpy(&out, &wide, sizeof(out));
  return out;
}

static inline uint16_t f32_to_f16(float value) {
  uint32_t wide;
  memcpy(&wide, &value, sizeof(wide));
  const uint16_t sign = (uint16_t)((wide >> 16) & 0x8000u);
  const uint32_t magnitude = wide & 0x7fffffffu;
  if (magnitude > 0x7f800000u) return (uint16_t)(sign | 0x7e00u | ((magnitude >> 13) & 0x1ffu)); /* quiet NaN, top payload bits kept */
  if (magnitude >= 0x47800000u) return (uint16_t)(sign | 0x7c00u); /* >= 65536 (or inf): infinity; 65520..65536 rounds there below */
  if (magnitude < 0x33000000u) return sign;                        /* < 2^-25: rounds to zero (2^-25 itself ties to even = 0) */
  const int32_t exponent = (int32_t)(magnitude >> 23) - 127;
  uint32_t mantissa = (magnitude & 0x7fffffu) | 0x800000u;          /* 24 significant bits */
  int drop = exponent >= -14 ? 13 : 13 + (-14 - exponent);           /* bits that do not fit */
  uint32_t kept = mantissa >> drop;
  const uint32_t rest = mantissa & ((1u << drop) - 1u);
  const uint32_t half = 1u << (drop - 1);
  if (rest > half || (rest == half && (kept & 1u))) ++kept;
  uint32_t out;
  if (exponent >= -14) out = ((uint32_t)(exponent + 15) << 10) + (kept - 0x400u); /* a carry out of the mantissa bumps the exponent */
  else out = kept;                                                                  /* subnormal; a carry lands on the smallest normal */
  return (uint16_t)(sign | out);
}

uint16_t oracle_f32_to_f16(float value) { return f32_to_f16(value); }
float oracle_f16_to_f32(uint16_t bits) { return f16_to_f32(bits); }
void oracle_f16_widen(const uint16_t* src, float* dst, int64_t count) {
  for (int64_t i = 0; i < count; ++i) dst[i] = f16_to_f32(src[i]);
}
void oracle_f16_narrow(const float* src, uint16_t* dst, int64_t count) {
  for (int64_t i = 0; i < count; ++i) dst[i] = f32_to_f16(src[i]);
}

/* cin: f32 only (or NULL).  act, alpha, column_scale as in the bf16 form. */
void oracle_matmul_f16_fused(int64_t m, int64_t n, int64_t k, const uint16_t* a, int64_t sam, int64_t sak, const uint16_t* b,
                             int64_t sbn, int64_t sbk, const float* cin, int64_t cin_sm, int64_t cin_sn, float alpha,
                             const float* column_scale, int act, float lo, float hi, void* c, int64_t scm, int64_t scn,
                             int c_is_f16) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      double sum = cin ? (double)cin[i * cin_sm + j * cin_sn] : 0.0;
      for (int64_t kk = 0; kk < k; ++kk)
        sum += (double)f16_to_f32(a[i * sam + kk * sak]) * (double)f16_to_f32(b[j * sbn + kk * sbk]);
      float acc = (float)sum * alpha;
      if (column_scale) acc *= column_scale[j];
      acc = oracle_activation(acc, act, lo, hi);
      if (c_is_f16) ((uint16_t*)c)[i * scm + j * scn] = f32_to_f16(acc);
      else ((float*)c)[i * scm + j * scn] = acc;
    }
  }
}

void oracle_matmul_f32_fused(int64_t m, int64_t n, int64_t k, const float* a, int64_t sam, int64_t sak, const float* b,
                             int64_t sbn, int64_t sbk, const float* cin, int64_t cin_sm, int64_t cin_sn, float alpha,
                             const float* column_scale, int act, float lo, float hi, float* c, int64_t scm, int64_t scn) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      double sum = cin ? (double)cin[i * cin_sm + j * cin_sn] : 0.0;
      for (int64_t kk = 0; kk < k; ++kk) sum += (double)a[i * sam + kk * sak] * (double)b[j * sbn + kk * sbk];
      float acc = (float)sum * alpha;
      if (column_scale) acc *= column_scale[j];
      c[i * scm + j * scn] = oracle_activation(acc, act, lo, hi);
    }
  }
}

/* Native integer accumulate: C = CIn + A.B^T in int32, wrapping (check_native_integer_accumulate). */
void oracle_matmul_i8_accumulate(int64_t m, int64_t n, int64_t k, const void* a, int64_t sam, int64_t sak, int a_signed,
                                 const void* b, int64_t sbn, int64_t sbk, int b_signed, const int32_t* cin, int64_t cin_sm,
                                 int64_t cin_sn, int32_t* c, int64_t scm, int64_t scn) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      uint32_t sum = cin ? (uint32_t)cin[i * cin_sm + j * cin_sn] : 0u;
      for (int64_t kk = 0; kk < k; ++kk) {
        const int32_t x = a_signed ? ((const int8_t*)a)[i * sam + kk * sak] : ((const uint8_t*)a)[i * sam + kk * sak];
        const int32_t y = b_signed ? ((const int8_t*)b)[j * sbn + kk * sbk] : ((const uint8_t*)b)[j * sbn + kk * sbk];
        sum += (uint32_t)(x * y);
      }
      c[i * scm + j * scn] = (int32_t)sum;
    }
  }
}

/* The quantised form as the reference ships it (tests/ops/MatmulConversionTestCommon.h:501-618 check_asymmetric_quantized):
 * A quantised on load, value * scale + zero_point converted to the 8-bit compute type by truncation toward zero with
 * saturation (observed by running the reference: 3.51 -> 3, 255.6 -> 255, -0.6 -> 0, 1e9 -> 255); 8-bit B; an int32
 * accumulator input (the correction row -zero_point * sum_k B[n,k]); int32 accumulate, wrapping; then the float output
 * transform on the converted accumulator: activation(float(acc) * alpha * column_scale[n]). */
void oracle_quantize_rows(int64_t m, int64_t k, const float* src, int64_t ssm, int64_t ssk, float scale, float zero_point,
                          void* dst, int64_t dsm, int64_t dsk, int dst_signed) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < k; ++j) {
      float q = truncf(src[i * ssm + j * ssk] * scale + zero_point);
      if (dst_signed) {
        q = q < -128.f ? -128.f : (q > 127.f ? 127.f : q);
        if (q != q) q = 0.f;
        ((int8_t*)dst)[i * dsm + j * dsk] = (int8_t)q;
      } else {
        q = q < 0.f ? 0.f : (q > 255.f ? 255.f : q);
        if (q != q) q = 0.f;
        ((uint8_t*)dst)[i * dsm + j * dsk] = (uint8_t)q;
      }
    }
  }
}

void oracle_matmul_i8_dequant(int64_t m, int64_t n, int64_t k, const void* a, int64_t sam, int64_t sak, int a_signed,
                              const void* b, int64_t sbn, int64_t sbk, int b_signed, const int32_t* cin, int64_t cin_sm,
                              int64_t cin_sn, float alpha, const float* column_scale, int act, float lo, float hi, void* c,
                              int64_t scm, int64_t scn, int c_is_bf16) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      uint32_t sum = cin ? (uint32_t)cin[i * cin_sm + j * cin_sn] : 0u;
      for (int64_t kk = 0; kk < k; ++kk) {
        const int32_t x = a_signed ? ((const int8_t*)a)[i * sam + kk * sak] : ((const uint8_t*)a)[i * sam + kk * sak];
        const int32_t y = b_signed ? ((const int8_t*)b)[j * sbn + kk * sbk] : ((const uint8_t*)b)[j * sbn + kk * sbk];
        sum += (uint32_t)(x * y);
      }
      float acc = (float)(int32_t)sum * alpha;
      if (column_scale) acc *= column_scale[j];
      acc = oracle_activation(acc, act, lo, hi);
      if (c_is_bf16) ((uint16_t*)c)[i * scm + j * scn] = f32_to_bf16(acc);
      else ((float*)c)[i * scm + j * scn] = acc;
    }
  }
}

/* Per-token quantisation (include/vecops/matmul/Quantization.h:76-246; the expected value of
 * tests/ops/MatmulConversionTestCommon.h:1403-1436): q = convert(x * multipliers[row] + zero_point) on load, int32
 * product plus the correction row, then value * row_scales[row] * column_scales[col] in that order. */
void oracle_quantize_rows_per_row(int64_t m, int64_t k, const float* src, int64_t ssm, int64_t ssk, const float* multipliers,
                                  float zero_point, void* dst, int64_t dsm, int64_t dsk, int dst_signed) {
  for (int64_t i = 0; i < m; ++i)
    oracle_quantize_rows(1, k, src + i * ssm, ssm, ssk, multipliers[i], zero_point, (char*)dst + i * dsm, dsm, dsk, dst_signed);
}

void oracle_matmul_i8_dequant_rows(int64_t m, int64_t n, int64_t k, const void* a, int64_t sam, int64_t sak, int a_signed,
                                   const void* b, int64_t sbn, int64_t sbk, int b_signed, const int32_t* cin, int64_t cin_sm,
                                   int64_t cin_sn, const float* row_scale, const float* column_scale, void* c, int64_t scm,
                                   int64_t scn, int c_is_bf16) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      uint32_t sum = cin ? (uint32_t)cin[i * cin_sm + j * cin_sn] : 0u;
      for (int64_t kk = 0; kk < k; ++kk) {
        const int32_t x = a_signed ? ((const int8_t*)a)[i * sam + kk * sak] : ((const uint8_t*)a)[i * sam + kk * sak];
        const int32_t y = b_signed ? ((const int8_t*)b)[j * sbn + kk * sbk] : ((const uint8_t*)b)[j * sbn + kk * sbk];
        sum += (uint32_t)(x * y);
      }
      float acc = (float)(int32_t)sum;
      if (row_scale) acc *= row_scale[i];
      if (column_scale) acc *= column_scale[j];
      if (c_is_bf16) ((uint16_t*)c)[i * scm + j * scn] = f32_to_bf16(acc);
      else ((float*)c)[i * scm + j * scn] = acc;
    }
  }
}

/* How many threads the loops above use (1 when built without OpenMP). */
/* Scaled dot-product attention for one head, the caller one step above matmul
 * (include/vecops/ops/details/attention/SDPA.h:72-84, :305-383; Common.h:200-345):
 *   S = Q.K^T in the accumulator type (bf16 operands, fp32 sums);
 *   s = S * scale + bias;  kept where the query is active, the key is active, the keep mask is non-zero and - causal -
 *       key <= query (top_left) or key <= query + (Lkv - Lq) (bottom_right); everything else is -inf;
 *   p = exp(s - rowmax) / sum, converted to the PROBABILITY type = the matmul atom's operand type (bf16, round to
 *       nearest even); a row with nothing kept is all zero;
 *   O = P.V in fp32, stored as fp32 or bf16.
 * The reference evaluates exp with its fast estimate (relative error <= 1e-3, tests/ops/AttentionTest.cpp:100-130) and
 * its own tests accept 2.5e-2 .. 5e-2 absolute (AttentionTest.cpp:243-247, :284-286); this restatement uses the exact
 * exponential, and the pin against the reference's outputs carries that tolerance.
 * causal: 0 none, 1 top_left, 2 bottom_right.  Masks are bytes, non-zero = keep; any of them and bias may be NULL. */
void oracle_sdpa_bf16(int64_t lq, int64_t lkv, int64_t dqk, int64_t dv, const uint16_t* q, int64_t sq, const uint16_t* k, int64_t sk,
                      const uint16_t* v, int64_t sv, const uint8_t* query_mask, const uint8_t* key_mask, const uint8_t* keep_mask,
                      int64_t keep_sr, const float* bias, int64_t bias_sr, int causal, float scale, void* out, int64_t so, int out_is_bf16) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < lq; ++i) {
    float* s = (float*)malloc((size_t)(lkv > 0 ? lkv : 1) * sizeof(float));
    uint16_t* p = (uint16_t*)malloc((size_t)(lkv > 0 ? lkv : 1) * sizeof(uint16_t));
    const int64_t last_key = causal == 1 ? i : (causal == 2 ? i + (lkv - lq) : lkv - 1);
    const int query_active = query_mask == NULL || query_mask[i] != 0;
    float maximum = -INFINITY;
    int any = 0;
    for (int64_t j = 0; j < lkv; ++j) {
      double sum = 0.0;
      for (int64_t d = 0; d < dqk; ++d) sum += (double)bf16_to_f32(q[i * sq + d]) * (double)bf16_to_f32(k[j * sk + d]);
      float value = (float)sum * scale;
      if (bias) value += bias[i * bias_sr + j];
      const int keep = query_active && j <= last_key && (key_mask == NULL || key_mask[j] != 0) &&
                       (keep_mask == NULL || keep_mask[i * keep_sr + j] != 0);
      s[j] = keep ? value : -INFINITY;
      if (keep) any = 1;
      if (s[j] > maximum) maximum = s[j];
    }
    double total = 0.0;
    if (any && maximum != -INFINITY)
      for (int64_t j = 0; j < lkv; ++j) {
        s[j] = s[j] == -INFINITY ? 0.f : (float)exp((double)s[j] - (double)maximum);
        total += s[j];
      }
    const int valid = any && maximum != -INFINITY && total > 0.0;
    const float reciprocal = valid ? 1.0f / (float)total : 0.f;
    for (int64_t j = 0; j < lkv; ++j) p[j] = valid ? f32_to_bf16(s[j] * reciprocal) : 0;
    for (int64_t d = 0; d < dv; ++d) {
      double sum = 0.0;
      for (int64_t j = 0; j < lkv; ++j) sum += (double)bf16_to_f32(p[j]) * (double)bf16_to_f32(v[j * sv + d]);
      if (out_is_bf16) ((uint16_t*)out)[i * so + d] = f32_to_bf16((float)sum);
      else ((float*)out)[i * so + d] = (float)sum;
    }
    free(s);
    free(p);
  }
}

/* The same attention by the streaming strategy (include/vecops/ops/details/attention/SparseFlashAttention.h:360-545 walked
 * over every key/value block, as ScaledDotProductAttention does for SDPAStrategy::streaming, :993-1010): per query row a
 * running maximum m, a running sum l and an unnormalised fp32 accumulator O; per block of `block` keys
 *   m' = max(m, block maximum);  a block with nothing kept (or m' = -inf) contributes zero probabilities and alpha = 1;
 *   alpha = 0 when m = -inf, exp(m - m') when the block raised the maximum, else 1;
 *   p = exp(s - m'), summed UNROUNDED into l = alpha * l + sum, then rounded to the probability type (bf16);
 *   O = alpha * O + p.V_block;   out = O / l when l > 0, else 0.
 * `chunk_blocks` > 0 restates what a GPU launch does when it cuts a row's keys into chunks of that many blocks handled by
 * different SMs: every chunk runs the recurrence from (m = -inf, l = 0, O = 0) and the chunk states are merged with the same
 * rule, (m, l, O) = (max m_c, sum l_c exp(m_c - m), sum O_c exp(m_c - m)), before the division.  0 = one chunk. */
void oracle_sdpa_bf16_streaming(int64_t lq, int64_t lkv, int64_t dqk, int64_t dv, const uint16_t* q, int64_t sq, const uint16_t* k,
                                int64_t sk, const uint16_t* v, int64_t sv, const uint8_t* query_mask, const uint8_t* key_mask,
                                const uint8_t* keep_mask, int64_t keep_sr, const float* bias, int64_t bias_sr, int causal, float scale,
                                int64_t block, int64_t chunk_blocks, void* out, int64_t so, int out_is_bf16) {
  if (block < 1) block = 128;
  const int64_t blocks = (lkv + block - 1) / block;
  if (chunk_blocks < 1 || chunk_blocks > blocks) chunk_blocks = blocks > 0 ? blocks : 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < lq; ++i) {
    float* s = (float*)malloc((size_t)block * sizeof(float));
    double* acc = (double*)malloc((size_t)(dv > 0 ? dv : 1) * sizeof(double));      /* the chunk in hand */
    double* merged = (double*)calloc((size_t)(dv > 0 ? dv : 1), sizeof(double));   /* chunks merged so far */
    float merged_m = -INFINITY;
    double merged_l = 0.0;
    const int64_t last_key = causal == 1 ? i : (causal == 2 ? i + (lkv - lq) : lkv - 1);
    const int query_active = query_mask == NULL || query_mask[i] != 0;
    for (int64_t first = 0; first < blocks; first += chunk_blocks) {
      float m = -INFINITY;
      double l = 0.0;
      for (int64_t d = 0; d < dv; ++d) acc[d] = 0.0;
      for (int64_t b = first; b < blocks && b < first + chunk_blocks; ++b) {
        const int64_t j0 = b * block, j1 = j0 + block < lkv ? j0 + block : lkv;
        float block_max = -INFINITY;
        for (int64_t j = j0; j < j1; ++j) {
          double sum = 0.0;
          for (int64_t d = 0; d < dqk; ++d) sum += (double)bf16_to_f32(q[i * sq + d]) * (double)bf16_to_f32(k[j * sk + d]);
          float value = (float)sum * scale;
          if (bias) value += bias[i * bias_sr + j];
          const int keep = query_active && j <= last_key && (key_mask == NULL || key_mask[j] != 0) &&
                           (keep_mask == NULL || keep_mask[i * keep_sr + j] != 0);
          s[j - j0] = keep ? value : -INFINITY;
          if (s[j - j0] > block_max) block_max = s[j - j0];
        }
        const float next = m > block_max ? m : block_max;
        if (next == -INFINITY) continue;  /* nothing kept so far: zero probabilities, alpha = 1 */
        const double alpha = m == -INFINITY ? 0.0 : exp((double)m - (double)next);
        double block_sum = 0.0;
        for (int64_t d = 0; d < dv; ++d) acc[d] *= alpha;
        for (int64_t j = j0; j < j1; ++j) {
          const float pj = s[j - j0] == -INFINITY ? 0.f : (float)exp((double)s[j - j0] - (double)next);
          block_sum += pj;
          const double rounded = (double)bf16_to_f32(f32_to_bf16(pj));
          for (int64_t d = 0; d < dv; ++d) acc[d] += rounded * (double)bf16_to_f32(v[j * sv + d]);
        }
        l = alpha * l + block_sum;
        m = next;
      }
      /* merge the chunk into what the earlier chunks left */
      const float top = merged_m > m ? merged_m : m;
      if (top != -INFINITY) {
        const double w_old = merged_m == -INFINITY ? 0.0 : exp((double)merged_m - (double)top);
        const double w_new = m == -INFINITY ? 0.0 : exp((double)m - (double)top);
        merged_l = merged_l * w_old + l * w_new;
        for (int64_t d = 0; d < dv; ++d) merged[d] = merged[d] * w_old + acc[d] * w_new;
        merged_m = top;
      }
    }
    const double reciprocal = merged_l > 0.0 ? 1.0 / merged_l : 0.0;
    for (int64_t d = 0; d < dv; ++d) {
      const float value = (float)(merged[d] * reciprocal);
      if (out_is_bf16) ((uint16_t*)out)[i * so + d] = f32_to_bf16(value);
      else ((float*)out)[i * so + d] = value;
    }
    free(s);
    free(acc);
    free(merged);
  }
}

#ifdef _OPENMP
#include <omp.h>
int oracle_threads(void) { return omp_get_max_threads(); }
#else
int oracle_threads(void) { return 1; }
#endif
