// Scaled dot-product attention, the caller one step above the matmul path, in vecops' two strategies
// (include/vecops/ops/details/attention/SDPA.h:21-25):
//   * streaming: one kernel over all heads (sdpa_stream.cuh), then - when query blocks were cut into key chunks to fill
//     the SMs - a small kernel that merges the chunks; nothing of size Lq x Lkv exists in device memory.  Taken
//     whenever the operands allow (head dims up to 128, TMA-addressable Q and K; a V that TMA cannot address is
//     re-pitched into scratch first);
//   * materialized, built the way vecops builds it: two products through the matmul entry points with a row softmax
//     between them (SDPA.h:305-383); the score matrix makes one round trip through device memory.  Serves the rest.
//
//   S = Q.K^T            vecops_b200_matmul_run, bf16 x bf16 -> f32            (tcgen05 when the operands allow)
//   P = softmax rows     sdpa_softmax_kernel: scale, bias, masks, causal cut, exp, normalise, round to bf16
//   Vt = pack(V^T)       vecops_b200_matmul_pack: V is [Lkv, Dv]; the product wants B = V^T as K-contiguous rows
//   O = P.Vt^T           vecops_b200_matmul_run, bf16 x bf16 -> f32 | bf16
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>

#include "vecops_b200/matmul_cuda.h"

#include "sdpa_stream.cuh"
#include "shim_device.h"
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


// ---------------------------------------------------------------- streaming strategy

struct StreamPlan {
  int q_blocks = 0, tiles_per_chunk = 1, max_chunks = 1;
  int uniform_chunks = 0;     // chunks per query block when every block has the same number, else 0
  int64_t items_per_head = 0; // work items (query block x chunk) of one head
  // V is read where it lies when TMA can address it; otherwise a re-pitched copy per head (or one, when the heads share
  // V) is made in scratch first: rows of `pitch` elements, zero past Dv
  int value_slabs = 0;
  int64_t pitch = 0;
  uint64_t slab_bytes = 0, partials_at = 0, total = 0;
};

uint32_t strategy_of(const VecopsB200Attention& a) {
  if (a.strategy != VECOPS_B200_SDPA_AUTOMATIC) return a.strategy;
  const char* forced = getenv("VECOPS_B200_SDPA");
  if (forced != nullptr && strcmp(forced, "materialized") == 0) return VECOPS_B200_SDPA_MATERIALIZED;
  if (forced != nullptr && strcmp(forced, "streaming") == 0) return VECOPS_B200_SDPA_STREAMING;
  return VECOPS_B200_SDPA_AUTOMATIC;
}

bool tma_addressable(const void* base, int64_t stride_row, int64_t stride_col, int64_t stride_head, int64_t heads) {
  return stride_col == 1 && stride_row > 0 && stride_row % 8 == 0 && (reinterpret_cast<uintptr_t>(base) & 15u) == 0 &&
         (heads <= 1 || (stride_head >= 0 && stride_head % 8 == 0));
}

// What the streaming kernel can serve; `why` names the first obstacle.
bool stream_applicable(const VecopsB200Attention& a, const char** why) {
  const int64_t heads = a.heads <= 1 ? 1 : a.heads;
  const char* reason = nullptr;
  if (a.qkv_dtype != VECOPS_DTYPE_BF16) reason = "q, k, v must be bf16";
  else if (a.lq < 1 || a.lkv < 1) reason = "no queries or no keys";
  else if (a.dqk < 1 || a.dqk > SdpaStream::kMaxHeadDim || a.dv < 1 || a.dv > SdpaStream::kMaxHeadDim) reason = "head dims must be 1..128";
  else if (heads > 65535 || (a.lq + SdpaStream::kBlockQ - 1) / SdpaStream::kBlockQ > (1 << 20)) reason = "too many heads or query blocks for one grid";
  else if (!tma_addressable(a.q, a.q_stride_row, a.q_stride_col, a.q_stride_head, heads)) reason = "q is not K-contiguous on 16-byte aligned rows";
  else if (!tma_addressable(a.k, a.k_stride_row, a.k_stride_col, a.k_stride_head, heads)) reason = "k is not K-contiguous on 16-byte aligned rows";
  if (why != nullptr) *why = reason;
  return reason == nullptr;
}

int32_t plan_stream(const VecopsB200Attention& a, int sms, uint64_t scratch_limit, StreamPlan* out, VecopsError* error) {
  using G = SdpaStream;
  StreamPlan p;
  const int64_t heads = a.heads <= 1 ? 1 : a.heads;
  p.q_blocks = static_cast<int>((a.lq + G::kBlockQ - 1) / G::kBlockQ);
  if (!tma_addressable(a.v, a.v_stride_row, a.v_stride_col, a.v_stride_head, heads)) {
    p.value_slabs = (heads > 1 && a.v_stride_head != 0) ? static_cast<int>(heads) : 1;
    uint64_t packed_bytes = 0;
    const int32_t rc = vecops_b200_matmul_packed_layout(VECOPS_DTYPE_BF16, a.lkv, a.dv, &p.pitch, &packed_bytes, error);
    if (rc != VECOPS_STATUS_OK) return rc;
    p.slab_bytes = round_up(packed_bytes, 256);
  }
  // 128-key tiles per query block after the causal cut, over all heads
  const int64_t shift = a.causal == 2 ? a.lkv - a.lq : 0;
  auto tiles_of = [&](int b) {
    const int64_t last_row = (b + 1 < p.q_blocks ? static_cast<int64_t>(b + 1) * G::kBlockQ : a.lq) - 1;
    int64_t last_key = a.causal != 0 ? last_row + shift : a.lkv - 1;
    if (last_key > a.lkv - 1) last_key = a.lkv - 1;
    return last_key < 0 ? int64_t{0} : last_key / G::kBlockKv + 1;
  };
  int64_t total_tiles = 0, most = 0;
  for (int b = 0; b < p.q_blocks; ++b) {
    const int64_t tiles = tiles_of(b);
    total_tiles += tiles;
    if (tiles > most) most = tiles;
  }
  total_tiles *= heads;
  // Fill the SMs once: a work item gets about total / SMs tiles; a block is never cut into more than kMaxChunks
  int64_t per_chunk = (total_tiles + sms - 1) / sms;
  if (per_chunk < 1) per_chunk = 1;
  if (per_chunk * G::kMaxChunks < most) per_chunk = (most + G::kMaxChunks - 1) / G::kMaxChunks;
  if (per_chunk > most) per_chunk = most > 0 ? most : 1;
  // VECOPS_B200_SDPA_CHUNK_TILES=n: tiles per work item fixed by hand (tuning aid; tests use it to hold cut and uncut
  // launches to the restatement with the same cut).  Still never more than kMaxChunks chunks per block.
  if (const char* forced = getenv("VECOPS_B200_SDPA_CHUNK_TILES")) {
    const long long asked = atoll(forced);
    if (asked >= 1) per_chunk = asked > most ? (most > 0 ? most : 1) : asked;
    if (per_chunk * G::kMaxChunks < most) per_chunk = (most + G::kMaxChunks - 1) / G::kMaxChunks;
  }
  auto layout = [&](int64_t chunk_tiles) {
    p.tiles_per_chunk = static_cast<int>(chunk_tiles);
    p.max_chunks = most > 0 ? static_cast<int>((most + chunk_tiles - 1) / chunk_tiles) : 1;
    p.items_per_head = 0;
    int64_t fewest = p.max_chunks;
    for (int b = 0; b < p.q_blocks; ++b) {
      const int64_t tiles = tiles_of(b);
      const int64_t chunks = tiles > 0 ? (tiles + chunk_tiles - 1) / chunk_tiles : 1;
      p.items_per_head += chunks;
      if (chunks < fewest) fewest = chunks;
    }
    p.uniform_chunks = fewest == p.max_chunks ? p.max_chunks : 0;
    p.partials_at = p.slab_bytes * p.value_slabs;
    const uint64_t partial_bytes =
        p.max_chunks > 1 ? static_cast<uint64_t>(heads) * p.q_blocks * p.max_chunks * G::kPartialFloats * sizeof(float) : 0;
    p.total = p.partials_at + partial_bytes;
  };
  layout(per_chunk);
  // a caller that brings no scratch, or scratch sized for another SM count, still runs: uncut blocks need no records
  if (p.total > scratch_limit) layout(most > 0 ? most : 1);
  *out = p;
  return VECOPS_STATUS_OK;
}

int32_t sdpa_run_streaming(const VecopsB200Attention& a, VecopsError* error) {
  using G = SdpaStream;
  if (a.out == nullptr || a.q == nullptr || a.k == nullptr || a.v == nullptr)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "sdpa: null operand");
  if (vecops_b200_device_count() == 0)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "no usable CUDA device; there is no CPU fallback");
  int device = a.device_index;
  if (device >= 0) {
    const cudaError_t status = cudaSetDevice(device);
    if (status != cudaSuccess) return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "cudaSetDevice(%d): %s", device, cudaGetErrorString(status));
  } else {
    cudaGetDevice(&device);
  }
  int sms = 0, major = 0;
  uint32_t* status_word = nullptr;
  int32_t rc = shim_device_facts(device, &sms, &major, &status_word, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  if (major != 10) return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "the streaming attention kernel needs an sm_100 device, found sm_%dx", major);
  StreamPlan plan;
  rc = plan_stream(a, sms, a.workspace != nullptr && (reinterpret_cast<uintptr_t>(a.workspace) & 255u) == 0 ? a.workspace_size : 0, &plan, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  if (plan.total != 0 && (a.workspace == nullptr || (reinterpret_cast<uintptr_t>(a.workspace) & 255u) != 0 || a.workspace_size < plan.total))
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "sdpa needs %llu bytes of 256-byte aligned device scratch (vecops_b200_sdpa_workspace)",
                     (unsigned long long)plan.total);
  const int64_t heads = a.heads <= 1 ? 1 : a.heads;
  char* base = static_cast<char*>(a.workspace);
  cudaStream_t stream = static_cast<cudaStream_t>(a.stream);

  for (int slab = 0; slab < plan.value_slabs; ++slab) {
    VecopsB200Pack pack{};
    pack.struct_size = sizeof(VecopsB200Pack);
    pack.operand = 1;
    pack.rows = a.lkv, pack.k = a.dv;
    pack.src = static_cast<const char*>(a.v) + static_cast<int64_t>(slab) * a.v_stride_head * 2;
    pack.src_stride_row = a.v_stride_row, pack.src_stride_k = a.v_stride_col;
    pack.src_dtype = pack.dst_dtype = VECOPS_DTYPE_BF16;
    pack.dst = base + plan.slab_bytes * slab;
    pack.dst_size = plan.slab_bytes;
    pack.device_index = a.device_index;
    pack.stream = a.stream;
    rc = vecops_b200_matmul_pack(&pack, error);
    if (rc != VECOPS_STATUS_OK) return rc;
  }
  CUtensorMap map_q, map_k, map_v;
  auto operand_map = [&](CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t stride_row, int64_t stride_head, bool per_head) {
    const uint64_t dims[3] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows), per_head ? static_cast<uint64_t>(heads) : 1};
    const uint64_t strides[2] = {static_cast<uint64_t>(stride_row) * 2,
                                 per_head ? static_cast<uint64_t>(stride_head) * 2 : static_cast<uint64_t>(stride_row) * 2 * static_cast<uint64_t>(rows)};
    const uint32_t box[3] = {64, 128, 1};
    return shim_encode_map(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ptr, dims, strides, box, error);
  };
  const bool q_per_head = heads > 1 && a.q_stride_head != 0, k_per_head = heads > 1 && a.k_stride_head != 0;
  rc = operand_map(&map_q, a.q, a.lq, a.dqk, a.q_stride_row, a.q_stride_head, q_per_head);
  if (rc != VECOPS_STATUS_OK) return rc;
  rc = operand_map(&map_k, a.k, a.lkv, a.dqk, a.k_stride_row, a.k_stride_head, k_per_head);
  if (rc != VECOPS_STATUS_OK) return rc;
  const bool v_per_head = heads > 1 && a.v_stride_head != 0;
  if (plan.value_slabs > 0) rc = operand_map(&map_v, base, a.lkv, a.dv, plan.pitch, static_cast<int64_t>(plan.slab_bytes / 2), v_per_head);
  else rc = operand_map(&map_v, a.v, a.lkv, a.dv, a.v_stride_row, a.v_stride_head, v_per_head);
  if (rc != VECOPS_STATUS_OK) return rc;

  SdpaStreamParams p{};
  p.lq = static_cast<int>(a.lq), p.lkv = static_cast<int>(a.lkv), p.dqk = static_cast<int>(a.dqk), p.dv = static_cast<int>(a.dv);
  p.causal = static_cast<int>(a.causal);
  p.tiles_per_chunk = plan.tiles_per_chunk;
  p.q_blocks = plan.q_blocks, p.max_chunks = plan.max_chunks, p.uniform_chunks = plan.uniform_chunks;
  p.q_head = q_per_head ? 1 : 0, p.k_head = k_per_head ? 1 : 0, p.v_head = v_per_head ? 1 : 0;
  p.scale = a.scale;
  p.out = a.out, p.out_sr = a.out_stride_row, p.out_sc = a.out_stride_col, p.out_sh = heads > 1 ? a.out_stride_head : 0;
  p.out_bf16 = a.out_dtype == VECOPS_DTYPE_BF16 ? 1 : 0;
  p.query_mask = a.query_mask, p.query_mask_sh = heads > 1 ? a.query_mask_stride_head : 0;
  p.key_mask = a.key_mask, p.key_mask_sh = heads > 1 ? a.key_mask_stride_head : 0;
  p.keep_mask = a.keep_mask, p.keep_sr = a.keep_stride_row, p.keep_sc = a.keep_stride_col, p.keep_sh = heads > 1 ? a.keep_stride_head : 0;
  p.bias = a.bias, p.bias_sr = a.bias_stride_row, p.bias_sc = a.bias_stride_col, p.bias_sh = heads > 1 ? a.bias_stride_head : 0;
  p.partials = reinterpret_cast<float*>(base + plan.partials_at);
  p.status = status_word;
  p.trace = shim_trace();

  const bool plain = a.key_mask == nullptr && a.keep_mask == nullptr && a.bias == nullptr;
  // (the timeline variant is its own instantiation: its bookkeeping costs registers the plain one needs)
  auto kernel = p.trace != nullptr ? (plain ? &sdpa_stream_kernel<true, true> : &sdpa_stream_kernel<false, true>)
                                   : (plain ? &sdpa_stream_kernel<true, false> : &sdpa_stream_kernel<false, false>);
  static std::atomic<bool> raised[4][64];
  const int variant = (plain ? 1 : 0) + (p.trace != nullptr ? 2 : 0);
  if (device < 0 || device >= 64 || !raised[variant][device].load()) {
    const cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G::kSmemBytes);
    if (status != cudaSuccess) return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "cudaFuncSetAttribute(sdpa_stream): %s", cudaGetErrorString(status));
    if (device >= 0 && device < 64) raised[variant][device].store(true);
  }
  const dim3 grid(static_cast<unsigned>(plan.items_per_head), static_cast<unsigned>(heads), 1);
  kernel<<<grid, G::kThreads, G::kSmemBytes, stream>>>(map_q, map_k, map_v, p);
  g_launches.fetch_add(1);
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess) return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "sdpa_stream launch: %s", cudaGetErrorString(status));
  if (plan.max_chunks > 1) {
    // the chunks of the blocks that were cut meet here: launched as a programmatic dependent, so its CTAs are resident
    // when the last work item finishes
    cudaLaunchConfig_t config = {};
    cudaLaunchAttribute attribute[1] = {};
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.gridDim = dim3(static_cast<unsigned>(plan.q_blocks) * 4, static_cast<unsigned>(heads), 1);
    config.blockDim = dim3(kMergeThreads);
    config.stream = stream;
    config.attrs = attribute;
    const char* pdl = getenv("VECOPS_B200_GEMM_PDL");  // =0: an ordinary launch behind the kernel that writes the records
    config.numAttrs = (pdl != nullptr && pdl[0] == '0') ? 0 : 1;
    status = cudaLaunchKernelEx(&config, sdpa_merge_kernel, p);
    g_launches.fetch_add(1);
    if (status != cudaSuccess) return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "sdpa_merge launch: %s", cudaGetErrorString(status));
  }
  if ((a.flags & VECOPS_B200_MATMUL_FLAG_ASYNC) == 0) {
    status = cudaStreamSynchronize(stream);
    if (status != cudaSuccess) return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "cudaStreamSynchronize: %s", cudaGetErrorString(status));
    if (const uint32_t word = shim_take_status(device))
      return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "sdpa_stream on device %d: a bounded device wait ran out (status 0x%x)", device, word);
  }
  return VECOPS_STATUS_OK;
}

}  // namespace

extern "C" {

int32_t vecops_b200_sdpa_workspace(const VecopsB200Attention* attention, uint64_t* bytes, VecopsError* error) {
  if (attention == nullptr || attention->struct_size < sizeof(VecopsB200Attention) || bytes == nullptr)
    return set_error(error, VECOPS_STATUS_ABI_MISMATCH, "attention record is null or too small, or no output pointer");
  const uint32_t strategy = strategy_of(*attention);
  const char* why = nullptr;
  if (strategy > VECOPS_B200_SDPA_STREAMING) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "sdpa: unknown strategy %u", strategy);
  if (strategy != VECOPS_B200_SDPA_MATERIALIZED && stream_applicable(*attention, &why)) {
    // the SM count of the device the record names, or of a B200 when no device can be asked
    int sms = 148, device = attention->device_index;
    if (vecops_b200_device_count() > 0 && (device >= 0 || cudaGetDevice(&device) == cudaSuccess)) {
      int asked = 0;
      if (shim_device_facts(device, &asked, nullptr, nullptr, nullptr) == VECOPS_STATUS_OK && asked > 0) sms = asked;
    }
    StreamPlan stream;
    const int32_t rc = plan_stream(*attention, sms, UINT64_MAX, &stream, error);
    if (rc == VECOPS_STATUS_OK) *bytes = stream.total;
    return rc;
  }
  if (strategy == VECOPS_B200_SDPA_STREAMING) return set_error(error, VECOPS_STATUS_NOT_APPLICABLE, "sdpa: the streaming strategy cannot serve this call: %s", why);
  Plan plan;
  const int32_t rc = plan_of(*attention, nullptr, &plan, error);
  if (rc == VECOPS_STATUS_OK) *bytes = plan.total;
  return rc;
}

static int32_t sdpa_run_one(const VecopsB200Attention& a, VecopsError* error);

int32_t vecops_b200_sdpa_plan(const VecopsB200Attention* attention, uint32_t* strategy, uint32_t* tiles_per_item, VecopsError* error) {
  if (attention == nullptr || attention->struct_size < sizeof(VecopsB200Attention) || strategy == nullptr || tiles_per_item == nullptr)
    return set_error(error, VECOPS_STATUS_ABI_MISMATCH, "attention record is null or too small, or no output pointer");
  const uint32_t asked = strategy_of(*attention);
  if (asked > VECOPS_B200_SDPA_STREAMING) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "sdpa: unknown strategy %u", asked);
  const char* why = nullptr;
  *tiles_per_item = 0;
  if (asked != VECOPS_B200_SDPA_MATERIALIZED && stream_applicable(*attention, &why)) {
    int sms = 148, device = attention->device_index;
    if (vecops_b200_device_count() > 0 && (device >= 0 || cudaGetDevice(&device) == cudaSuccess)) {
      int count = 0;
      if (shim_device_facts(device, &count, nullptr, nullptr, nullptr) == VECOPS_STATUS_OK && count > 0) sms = count;
    }
    StreamPlan stream;
    const int32_t rc = plan_stream(*attention, sms, attention->workspace_size != 0 ? attention->workspace_size : UINT64_MAX, &stream, error);
    if (rc != VECOPS_STATUS_OK) return rc;
    *strategy = VECOPS_B200_SDPA_STREAMING;
    *tiles_per_item = static_cast<uint32_t>(stream.tiles_per_chunk);
    return VECOPS_STATUS_OK;
  }
  if (asked == VECOPS_B200_SDPA_STREAMING)
    return set_error(error, VECOPS_STATUS_NOT_APPLICABLE, "sdpa: the streaming strategy cannot serve this call: %s", why);
  *strategy = VECOPS_B200_SDPA_MATERIALIZED;
  return VECOPS_STATUS_OK;
}

int32_t vecops_b200_sdpa_run(const VecopsB200Attention* attention, VecopsError* error) {
  if (attention == nullptr || attention->struct_size < sizeof(VecopsB200Attention))
    return set_error(error, VECOPS_STATUS_ABI_MISMATCH, "attention record is null or too small");
  const DeviceRestore restore;  // the heads below switch to the record's device; the caller gets its own back
  const uint32_t strategy = strategy_of(*attention);
  if (strategy > VECOPS_B200_SDPA_STREAMING) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "sdpa: unknown strategy %u", strategy);
  if (strategy != VECOPS_B200_SDPA_MATERIALIZED) {
    const char* why = nullptr;
    if (stream_applicable(*attention, &why)) {
      if (attention->out_dtype != VECOPS_DTYPE_F32 && attention->out_dtype != VECOPS_DTYPE_BF16)
        return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "sdpa serves bf16 q, k, v with an f32 or bf16 output");
      if (attention->causal > 2) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "sdpa: causal is 0 (none), 1 (top left) or 2 (bottom right)");
      if (attention->dv == 0) return VECOPS_STATUS_OK;
      return sdpa_run_streaming(*attention, error);  // all heads in one launch
    }
    if (strategy == VECOPS_B200_SDPA_STREAMING)
      return set_error(error, VECOPS_STATUS_NOT_APPLICABLE, "sdpa: the streaming strategy cannot serve this call: %s", why);
  }
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
