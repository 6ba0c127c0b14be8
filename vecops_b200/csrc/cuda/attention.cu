// Scaled dot-product attention for one head, built the way vecops builds it: two products through the matmul
// entry points with a row softmax between them (include/vecops/ops/details/attention/SDPA.h:305-383, the
// "materialized" strategy).  The caller one step above the matmul path - not a fused attention kernel: the score
// matrix makes one round trip through device memory.
//
//   S = Q.K^T            vecops_b200_matmul_run, bf16 x bf16 -> f32            (tcgen05 when the operands allow)
//   P = softmax rows     sdpa_softmax_kernel: scale, bias, masks, causal cut, exp, normalise, round to bf16
//   Vt = pack(V^T)       vecops_b200_matmul_pack: V is [Lkv, Dv]; the product wants B = V^T as K-contiguous rows
//   O = P.Vt^T           vecops_b200_matmul_run, bf16 x bf16 -> f32 | bf16
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "vecops_b200/matmul_cuda.h"

#include "shim_util.h"

using namespace vb200;

namespace {

__device__ __forceinline__ float block_reduce(float value, bool take_max, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, value, offset);
    value = take_max ? fmaxf(value, other) : value + other;
  }
  __syncthreads();  // the previous use of `scratch` is over
  if (lane == 0) scratch[warp] = value;
  __syncthreads();
  float total = scratch[0];
  for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w) total = take_max ? fmaxf(total, scratch[w]) : total + scratch[w];
  return total;
}

// One CTA per score row: decorate (s * scale + bias, -inf where not kept) and take the maximum; exponentiate and sum;
// normalise into the probability type (Common.h:236-345).
//
// kPerThread > 0: rows of up to 256 x kPerThread scores stay in registers between the passes - one 16-byte read of S
// per four scores, one 8-byte write of P.  The kernel is bound by instruction issue, not by memory, so the count is a
// template parameter (no dead slots) and kPlain drops the mask and bias handling when none of them was given.
// kPerThread == 0: rows of any length go through S in place, as the reference does, each thread revisiting only the
// elements it wrote itself (no barrier beyond the two reductions).
constexpr int kSoftmaxThreads = 256;

template <int kPerThread, bool kPlain>
__global__ void __launch_bounds__(kSoftmaxThreads) sdpa_softmax_kernel(float* __restrict__ scores, long long ld_scores,
                                                                       __nv_bfloat16* __restrict__ probabilities, long long ld_probabilities, int lq,
                                                                       int lkv, float scale, const uint8_t* __restrict__ query_mask,
                                                                       const uint8_t* __restrict__ key_mask, const uint8_t* __restrict__ keep_mask,
                                                                       long long keep_sr, long long keep_sc, const float* __restrict__ bias,
                                                                       long long bias_sr, long long bias_sc, int causal) {
  __shared__ float scratch[kSoftmaxThreads / 32];
  const float negative_infinity = -INFINITY;
  for (int row = blockIdx.x; row < lq; row += gridDim.x) {
    float* s = scores + row * ld_scores;
    __nv_bfloat16* p = probabilities + row * ld_probabilities;
    const bool query_active = query_mask == nullptr || query_mask[row] != 0;
    const long long last_key = causal == 1 ? row : (causal == 2 ? static_cast<long long>(row) + (lkv - lq) : lkv - 1);
    // keys [0, limit) survive the query mask, the causal cut and the row's end
    const int limit = !query_active ? 0 : static_cast<int>(last_key + 1 < 0 ? 0 : (last_key + 1 < lkv ? last_key + 1 : lkv));
    auto decorated = [&](int j, float score) {
      float value = __fmul_rn(score, scale);
      if (kPlain || j >= limit) return j < limit ? value : negative_infinity;  // (nothing past `limit` is read: it may lie past the row)
      if (bias != nullptr) value = __fadd_rn(value, bias[row * bias_sr + j * bias_sc]);
      const bool keep = (key_mask == nullptr || key_mask[j] != 0) && (keep_mask == nullptr || keep_mask[row * keep_sr + j * keep_sc] != 0);
      return keep ? value : negative_infinity;
    };
    float held[kPerThread > 0 ? kPerThread : 1];
    float maximum = negative_infinity;
    if constexpr (kPerThread > 0) {
      // 16-byte loads: the row pitch is a multiple of four floats, so a vector that starts inside the row ends inside the pitch
#pragma unroll
      for (int i = 0; i < kPerThread / 4; ++i) {
        const int j = 4 * (threadIdx.x + i * kSoftmaxThreads);
        float4 raw = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < lkv) raw = *reinterpret_cast<const float4*>(s + j);
        const float in[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          held[4 * i + e] = decorated(j + e, in[e]);  // (limit <= Lkv: slots past the row's end are -inf too)
          maximum = fmaxf(maximum, held[4 * i + e]);
        }
      }
    } else {
      for (int j = threadIdx.x; j < lkv; j += kSoftmaxThreads) {
        const float value = decorated(j, s[j]);
        s[j] = value;
        maximum = fmaxf(maximum, value);
      }
    }
    maximum = block_reduce(maximum, true, scratch);
    if (maximum == negative_infinity) {  // nothing kept in this row (uniform across the CTA): all zero
      for (int j = threadIdx.x; j < lkv; j += kSoftmaxThreads) p[j] = __float2bfloat16_rn(0.f);
      continue;
    }
    float sum = 0.f;
    if constexpr (kPerThread > 0) {
#pragma unroll
      for (int i = 0; i < kPerThread; ++i) {
        held[i] = __expf(held[i] - maximum);  // exp(-inf) = 0 for the dropped ones
        sum += held[i];
      }
    } else {
      for (int j = threadIdx.x; j < lkv; j += kSoftmaxThreads) {
        const float e = __expf(s[j] - maximum);
        s[j] = e;
        sum += e;
      }
    }
    sum = block_reduce(sum, false, scratch);
    const float reciprocal = sum > 0.f ? 1.f / sum : 0.f;
    if constexpr (kPerThread > 0) {
      // 8-byte stores; the probability pitch is a multiple of 64 elements, positions past Lkv inside it get zeros
#pragma unroll
      for (int i = 0; i < kPerThread / 4; ++i) {
        const int j = 4 * (threadIdx.x + i * kSoftmaxThreads);
        if (j >= lkv) continue;
        const __nv_bfloat162 lo = __floats2bfloat162_rn(held[4 * i] * reciprocal, held[4 * i + 1] * reciprocal);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(held[4 * i + 2] * reciprocal, held[4 * i + 3] * reciprocal);
        uint2 packed;
        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p + j) = packed;
      }
    } else {
      for (int j = threadIdx.x; j < lkv; j += kSoftmaxThreads) p[j] = __float2bfloat16_rn(s[j] * reciprocal);
    }
  }
}

using SoftmaxKernel = void (*)(float*, long long, __nv_bfloat16*, long long, int, int, float, const uint8_t*, const uint8_t*, const uint8_t*, long long,
                               long long, const float*, long long, long long, int);

template <bool kPlain>
SoftmaxKernel softmax_for(int64_t lkv) {
  if (lkv <= kSoftmaxThreads * 4) return &sdpa_softmax_kernel<4, kPlain>;
  if (lkv <= kSoftmaxThreads * 8) return &sdpa_softmax_kernel<8, kPlain>;
  if (lkv <= kSoftmaxThreads * 16) return &sdpa_softmax_kernel<16, kPlain>;
  if (lkv <= kSoftmaxThreads * 32) return &sdpa_softmax_kernel<32, kPlain>;
  return &sdpa_softmax_kernel<0, kPlain>;
}

uint64_t round_up(uint64_t value, uint64_t to) { return (value + to - 1) / to * to; }

struct Plan {
  int64_t ld_scores, pitch;           // elements
  uint64_t scores_at, probabilities_at, values_at, scratch_at, scratch_bytes, total;
  VecopsB200Matmul qk, pv;
};

int32_t plan_of(const VecopsB200Attention& a, char* base, Plan* out, VecopsError* error) {
  if (a.lq < 0 || a.lkv < 0 || a.dqk < 0 || a.dv < 0 || a.lq >= (INT64_C(1) << 31) || a.lkv >= (INT64_C(1) << 31) - 128)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "sdpa: extent out of range");
  if (a.qkv_dtype != VECOPS_DTYPE_BF16 || (a.out_dtype != VECOPS_DTYPE_F32 && a.out_dtype != VECOPS_DTYPE_BF16))
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "sdpa serves bf16 q, k, v with an f32 or bf16 output");
  if (a.causal > 2) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "sdpa: causal is 0 (none), 1 (top left) or 2 (bottom right)");
  Plan p{};
  p.ld_scores = static_cast<int64_t>(round_up(static_cast<uint64_t>(a.lkv), 4));
  uint64_t packed_bytes = 0;
  int32_t rc = vecops_b200_matmul_packed_layout(VECOPS_DTYPE_BF16, a.dv, a.lkv, &p.pitch, &packed_bytes, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  p.scores_at = 0;
  p.probabilities_at = round_up(static_cast<uint64_t>(a.lq) * p.ld_scores * 4, 256);
  p.values_at = round_up(p.probabilities_at + static_cast<uint64_t>(a.lq) * p.pitch * 2, 256);
  p.scratch_at = round_up(p.values_at + packed_bytes, 256);

  VecopsB200Matmul& qk = p.qk;
  qk.struct_size = sizeof(VecopsB200Matmul);
  qk.kernel = VECOPS_B200_KERNEL_AUTO;
  qk.m = a.lq, qk.n = a.lkv, qk.k = a.dqk;
  qk.a = a.q, qk.a_stride_m = a.q_stride_row, qk.a_stride_k = a.q_stride_col;
  qk.b = a.k, qk.b_stride_n = a.k_stride_row, qk.b_stride_k = a.k_stride_col;
  qk.c = base + p.scores_at, qk.c_stride_m = p.ld_scores, qk.c_stride_n = 1;
  qk.a_dtype = qk.b_dtype = VECOPS_DTYPE_BF16;
  qk.c_dtype = VECOPS_DTYPE_F32;
  qk.device_index = a.device_index;
  qk.stream = a.stream;
  qk.flags = VECOPS_B200_MATMUL_FLAG_ASYNC;

  VecopsB200Matmul& pv = p.pv;
  pv = qk;
  pv.m = a.lq, pv.n = a.dv, pv.k = a.lkv;
  pv.a = base + p.probabilities_at, pv.a_stride_m = p.pitch, pv.a_stride_k = 1;
  pv.b = base + p.values_at, pv.b_stride_n = p.pitch, pv.b_stride_k = 1;
  pv.c = a.out, pv.c_stride_m = a.out_stride_row, pv.c_stride_n = a.out_stride_col;
  pv.c_dtype = a.out_dtype;
  pv.flags = a.flags & VECOPS_B200_MATMUL_FLAG_ASYNC;

  uint64_t need_qk = 0, need_pv = 0;
  if (a.lq > 0 && a.lkv > 0) {
    rc = vecops_b200_matmul_workspace(&qk, &need_qk, error);
    if (rc != VECOPS_STATUS_OK) return rc;
  }
  if (a.lq > 0 && a.dv > 0) {
    rc = vecops_b200_matmul_workspace(&pv, &need_pv, error);
    if (rc != VECOPS_STATUS_OK) return rc;
  }
  p.scratch_bytes = need_qk > need_pv ? need_qk : need_pv;
  p.total = p.scratch_at + p.scratch_bytes;
  qk.workspace = pv.workspace = p.scratch_bytes != 0 ? base + p.scratch_at : nullptr;
  qk.workspace_size = pv.workspace_size = p.scratch_bytes;
  *out = p;
  return VECOPS_STATUS_OK;
}

}  // namespace

extern "C" {

int32_t vecops_b200_sdpa_workspace(const VecopsB200Attention* attention, uint64_t* bytes, VecopsError* error) {
  if (attention == nullptr || attention->struct_size < sizeof(VecopsB200Attention) || bytes == nullptr)
    return set_error(error, VECOPS_STATUS_ABI_MISMATCH, "attention record is null or too small, or no output pointer");
  Plan plan;
  const int32_t rc = plan_of(*attention, nullptr, &plan, error);
  if (rc == VECOPS_STATUS_OK) *bytes = plan.total;
  return rc;
}

static int32_t sdpa_run_one(const VecopsB200Attention& a, VecopsError* error);

int32_t vecops_b200_sdpa_run(const VecopsB200Attention* attention, VecopsError* error) {
  if (attention == nullptr || attention->struct_size < sizeof(VecopsB200Attention))
    return set_error(error, VECOPS_STATUS_ABI_MISMATCH, "attention record is null or too small");
  const DeviceRestore restore;  // the heads below switch to the record's device; the caller gets its own back
  if (attention->heads <= 1) return sdpa_run_one(*attention, error);
  // one head after the other on the stream, sharing the scratch; only the last one synchronises (when the caller wants that)
  for (int64_t h = 0; h < attention->heads; ++h) {
    VecopsB200Attention head = *attention;
    head.heads = 1;
    auto at = [h](const void* base, int64_t stride, size_t elem) -> const void* {
      return base == nullptr ? nullptr : static_cast<const char*>(base) + h * stride * static_cast<int64_t>(elem);
    };
    head.q = at(attention->q, attention->q_stride_head, 2);
    head.k = at(attention->k, attention->k_stride_head, 2);
    head.v = at(attention->v, attention->v_stride_head, 2);
    head.out = const_cast<void*>(at(attention->out, attention->out_stride_head, attention->out_dtype == VECOPS_DTYPE_F32 ? 4 : 2));
    head.query_mask = static_cast<const uint8_t*>(at(attention->query_mask, attention->query_mask_stride_head, 1));
    head.key_mask = static_cast<const uint8_t*>(at(attention->key_mask, attention->key_mask_stride_head, 1));
    head.keep_mask = static_cast<const uint8_t*>(at(attention->keep_mask, attention->keep_stride_head, 1));
    head.bias = static_cast<const float*>(at(attention->bias, attention->bias_stride_head, 4));
    if (h + 1 < attention->heads) head.flags |= VECOPS_B200_MATMUL_FLAG_ASYNC;
    const int32_t rc = sdpa_run_one(head, error);
    if (rc != VECOPS_STATUS_OK) return rc;
  }
  return VECOPS_STATUS_OK;
}

}  // extern "C"

static int32_t sdpa_run_one(const VecopsB200Attention& a, VecopsError* error) {
  Plan plan;
  int32_t rc = plan_of(a, static_cast<char*>(a.workspace), &plan, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  if (a.lq == 0 || a.dv == 0) return VECOPS_STATUS_OK;  // no output element exists
  if (a.out == nullptr || (a.lkv > 0 && a.v == nullptr))  // (q and k are checked by the first product, which knows whether Dqk is 0)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "sdpa: null operand");
  if (a.workspace == nullptr || (reinterpret_cast<uintptr_t>(a.workspace) & 255u) != 0 || a.workspace_size < plan.total)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "sdpa needs %llu bytes of 256-byte aligned device scratch (vecops_b200_sdpa_workspace)",
                     (unsigned long long)plan.total);
  if (vecops_b200_device_count() == 0)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "no usable CUDA device; there is no CPU fallback");
  if (a.device_index >= 0) {
    const cudaError_t status = cudaSetDevice(a.device_index);
    if (status != cudaSuccess) return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "cudaSetDevice(%d): %s", a.device_index, cudaGetErrorString(status));
  }
  cudaStream_t stream = static_cast<cudaStream_t>(a.stream);
  char* base = static_cast<char*>(a.workspace);
  if (a.lkv > 0) {
    rc = vecops_b200_matmul_run(&plan.qk, error);  // S = Q.K^T (zeros when Dqk == 0)
    if (rc != VECOPS_STATUS_OK) return rc;
    const int rows = static_cast<int>(a.lq < 148 * 64 ? a.lq : 148 * 64);
    const bool plain = a.key_mask == nullptr && a.keep_mask == nullptr && a.bias == nullptr;
    const SoftmaxKernel softmax = plain ? softmax_for<true>(a.lkv) : softmax_for<false>(a.lkv);
    softmax<<<rows, kSoftmaxThreads, 0, stream>>>(reinterpret_cast<float*>(base + plan.scores_at), plan.ld_scores,
                                                  reinterpret_cast<__nv_bfloat16*>(base + plan.probabilities_at), plan.pitch, static_cast<int>(a.lq),
                                                  static_cast<int>(a.lkv), a.scale, a.query_mask, a.key_mask, a.keep_mask, a.keep_stride_row,
                                                  a.keep_stride_col, a.bias, a.bias_stride_row, a.bias_stride_col, static_cast<int>(a.causal));
    g_launches.fetch_add(1);
    const cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "sdpa softmax launch: %s", cudaGetErrorString(status));
    VecopsB200Pack pack{};
    pack.struct_size = sizeof(VecopsB200Pack);
    pack.operand = 1;
    pack.rows = a.dv, pack.k = a.lkv;   // B of the second product is V^T: rows run along V's columns
    pack.src = a.v, pack.src_stride_row = a.v_stride_col, pack.src_stride_k = a.v_stride_row;
    pack.src_dtype = pack.dst_dtype = VECOPS_DTYPE_BF16;
    pack.dst = base + plan.values_at;
    pack.dst_size = plan.scratch_at - plan.values_at;
    pack.device_index = a.device_index;
    pack.stream = a.stream;
    rc = vecops_b200_matmul_pack(&pack, error);
    if (rc != VECOPS_STATUS_OK) return rc;
  }
  return vecops_b200_matmul_run(&plan.pv, error);  // O = P.V (zeros when Lkv == 0); synchronises unless the caller asked not to
}
