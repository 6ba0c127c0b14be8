// The fused output transform shared by the GEMM kernels:
//     COut[m,n] = convert( activation( (CIn[m,n] + sum_k A[m,k] B[n,k]) * alpha * row_scale[m] * column_scale[n] ) )
// vecops expresses this as the explicit accumulate form COut = transform(CIn + A.B^T) with an output transform composed
// from vec primitives (include/vecops/ops/Matmul.h:519-570; tests/ops/MatmulConversionTestCommon.h:623-704 runtime and
// per-column scale, :705-770 bias as a stride-0 CIn + clamp, :1028-1160 relu / sigmoid / silu).  On the device the
// transforms those tests compose are an enumeration carried in this record.  The per-row factor is the row half of vecops'
// row-by-column dequantisation (include/vecops/matmul/Quantization.h:195-246: value * row_scales[row] * column_scales[col]).
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace vb200 {

enum : int { kCinNone = 0, kCinF32 = 1, kCinBF16 = 2, kCinI32 = 3 };
enum : int { kActNone = 0, kActRelu = 1, kActSigmoid = 2, kActSilu = 3, kActClamp = 4 };

// Passed by value to the kernels.  `active` == 0 means the plain GEMM: kernels skip the transform with one uniform branch.
struct EpilogueArgs {
  const void* cin = nullptr;     // accumulator input, element strides below (0 = broadcast along that axis)
  long long cin_stride_m = 0;
  long long cin_stride_n = 0;
  int cin_kind = kCinNone;
  int activation = kActNone;
  float alpha = 1.f;
  float clamp_lo = 0.f;
  float clamp_hi = 0.f;
  int active = 0;
  const float* row_scale = nullptr;  // optional [M] factor, one per output row
};

// alpha with the row's own factor folded in (alpha is 1 in vecops' row-by-column form, so the product order is value * row * column)
__device__ __forceinline__ float epilogue_row_alpha(const EpilogueArgs& ep, long long row) {
  return ep.row_scale != nullptr ? ep.alpha * __ldg(ep.row_scale + row) : ep.alpha;
}

__device__ __forceinline__ float epilogue_activation(float x, const EpilogueArgs& ep) {
  switch (ep.activation) {
    case kActRelu: return fmaxf(x, 0.f);
    case kActSigmoid: return 1.f / (1.f + __expf(-x));
    case kActSilu: return x / (1.f + __expf(-x));
    case kActClamp: return fminf(fmaxf(x, ep.clamp_lo), ep.clamp_hi);
    default: return x;
  }
}

// `acc` is the fp32 dot product of output element (row, col), both inside the matrix; `column_factor` the column scale
// (1 when there is none).
__device__ __forceinline__ float epilogue_float(float acc, const EpilogueArgs& ep, long long row, long long col, float column_factor) {
  if (ep.cin_kind == kCinF32) {
    acc += __ldg(static_cast<const float*>(ep.cin) + row * ep.cin_stride_m + col * ep.cin_stride_n);
  } else if (ep.cin_kind == kCinBF16) {
    acc += __bfloat162float(static_cast<const __nv_bfloat16*>(ep.cin)[row * ep.cin_stride_m + col * ep.cin_stride_n]);
  }
  return epilogue_activation(acc * epilogue_row_alpha(ep, row) * column_factor, ep);
}

// The same transform over 32 consecutive columns of one row held in registers (`v` = fp32 bit patterns), written as a
// few short loops - one per stage, the activation chosen OUTSIDE its loop - so that the unrolled code stays small: an
// earlier form that inlined the whole per-element transform 64 times per slab ran the tensor-core GEMM 3x slower
// (instruction fetch, not arithmetic).  Elements outside the matrix (row >= M or col >= N) are left alone.
__device__ __forceinline__ void epilogue_float_row32(uint32_t (&v)[32], const EpilogueArgs& ep, const float* __restrict__ column_scale,
                                                     long long row, int col0, int M, int N) {
  if (row >= M) return;
  const int valid = min(32, N - col0);
  const float alpha = epilogue_row_alpha(ep, row);
  if (ep.cin_kind == kCinF32) {
    const float* src = static_cast<const float*>(ep.cin) + row * ep.cin_stride_m + static_cast<long long>(col0) * ep.cin_stride_n;
    if (ep.cin_stride_n == 1 && valid == 32 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
      // contiguous columns: eight 16-byte loads (one address for the whole warp when CIn is a bias row)
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 part = __ldg(reinterpret_cast<const float4*>(src) + q);
        v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) + part.x);
        v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) + part.y);
        v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) + part.z);
        v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) + part.w);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < valid) v[j] = __float_as_uint(__uint_as_float(v[j]) + __ldg(src + j * ep.cin_stride_n));
    }
  } else if (ep.cin_kind == kCinBF16) {
    const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(ep.cin) + row * ep.cin_stride_m + static_cast<long long>(col0) * ep.cin_stride_n;
    if (ep.cin_stride_n == 1 && valid == 32 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 part = __ldg(reinterpret_cast<const uint4*>(src) + q);
        const uint32_t words[4] = {part.x, part.y, part.z, part.w};
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          v[8 * q + 2 * h] = __float_as_uint(__uint_as_float(v[8 * q + 2 * h]) + __uint_as_float(words[h] << 16));
          v[8 * q + 2 * h + 1] = __float_as_uint(__uint_as_float(v[8 * q + 2 * h + 1]) + __uint_as_float(words[h] & 0xffff0000u));
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < valid) v[j] = __float_as_uint(__uint_as_float(v[j]) + __bfloat162float(src[j * ep.cin_stride_n]));
    }
  }
  if (column_scale != nullptr) {
    if (valid == 32 && (reinterpret_cast<uintptr_t>(column_scale + col0) & 15u) == 0) {
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(column_scale + col0) + q);
        v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) * alpha * f.x);
        v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) * alpha * f.y);
        v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) * alpha * f.z);
        v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) * alpha * f.w);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < valid) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha * __ldg(column_scale + col0 + j));
    }
  } else if (alpha != 1.f) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
  }
  switch (ep.activation) {
    case kActRelu:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(fmaxf(__uint_as_float(v[j]), 0.f));
      break;
    case kActSigmoid:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__fdividef(1.f, 1.f + __expf(-__uint_as_float(v[j]))));
      break;
    case kActSilu:
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float x = __uint_as_float(v[j]);
        v[j] = __float_as_uint(__fdividef(x, 1.f + __expf(-x)));
      }
      break;
    case kActClamp:
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(fminf(fmaxf(__uint_as_float(v[j]), ep.clamp_lo), ep.clamp_hi));
      break;
    default:
      break;
  }
}

__device__ __forceinline__ void epilogue_int_row32(uint32_t (&v)[32], const EpilogueArgs& ep, long long row, int col0, int M, int N) {
  if (row >= M || ep.cin_kind != kCinI32) return;
  const int valid = min(32, N - col0);
  const int32_t* src = static_cast<const int32_t*>(ep.cin) + row * ep.cin_stride_m + static_cast<long long>(col0) * ep.cin_stride_n;
  if (ep.cin_stride_n == 1 && valid == 32 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
    // contiguous columns: eight 16-byte loads (one address for the whole warp when CIn is a correction row); thirty-two
    // scalar loads here cost an int8 tile's epilogue more than its MMAs
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int4 part = __ldg(reinterpret_cast<const int4*>(src) + q);
      v[4 * q] += static_cast<uint32_t>(part.x);
      v[4 * q + 1] += static_cast<uint32_t>(part.y);
      v[4 * q + 2] += static_cast<uint32_t>(part.z);
      v[4 * q + 3] += static_cast<uint32_t>(part.w);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) v[j] += static_cast<uint32_t>(__ldg(src + j * ep.cin_stride_n));
  }
}

// int32 accumulators take an int32 accumulator input and nothing else (wrapping add, like the accumulation itself).
__device__ __forceinline__ uint32_t epilogue_int(uint32_t acc, const EpilogueArgs& ep, long long row, long long col) {
  if (ep.cin_kind == kCinI32)
    acc += static_cast<uint32_t>(__ldg(static_cast<const int32_t*>(ep.cin) + row * ep.cin_stride_m + col * ep.cin_stride_n));
  return acc;
}

}  // namespace vb200
