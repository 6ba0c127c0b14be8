// The fused output transform shared by the GEMM kernels:
//     COut[m,n] = convert( activation( (CIn[m,n] + sum_k A[m,k] B[n,k]) * alpha * column_scale[n] ) )
// vecops expresses this as the explicit accumulate form COut = transform(CIn + A.B^T) with an output transform composed
// from vec primitives (include/vecops/ops/Matmul.h:519-570; tests/ops/MatmulConversionTestCommon.h:623-704 runtime and
// per-column scale, :705-770 bias as a stride-0 CIn + clamp, :1028-1160 relu / sigmoid / silu).  On the device the
// transforms those tests compose are an enumeration carried in this record.
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
};

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
  return epilogue_activation(acc * ep.alpha * column_factor, ep);
}

// int32 accumulators take an int32 accumulator input and nothing else (wrapping add, like the accumulation itself).
__device__ __forceinline__ uint32_t epilogue_int(uint32_t acc, const EpilogueArgs& ep, long long row, long long col) {
  if (ep.cin_kind == kCinI32)
    acc += static_cast<uint32_t>(__ldg(static_cast<const int32_t*>(ep.cin) + row * ep.cin_stride_m + col * ep.cin_stride_n));
  return acc;
}

}  // namespace vb200
