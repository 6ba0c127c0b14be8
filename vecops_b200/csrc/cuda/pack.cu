// C ABI of operand preparation: the device counterpart of vecops' ops::matmul_pack and
// ops::matmul_pack_b_compensated (include/vecops/ops/MatmulPack.h:93-131, :28-35).
#include <cuda_runtime.h>
#include <stdint.h>

#include "vecops_b200/matmul_cuda.h"

#include "pack_kernels.cuh"
#include "shim_util.h"

using namespace vb200;

namespace {

size_t pack_elem_size(uint32_t dtype) {
  switch (dtype) {
    case VECOPS_DTYPE_F32: return 4;
    case VECOPS_DTYPE_BF16: case VECOPS_DTYPE_F16: return 2;
    case VECOPS_DTYPE_I8: case VECOPS_DTYPE_U8: return 1;
    default: return 0;
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int32_t launch_status(VecopsError* error, const char* what) {
  g_launches.fetch_add(1);
  const cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "%s: %s", what, cudaGetErrorString(status));
  return VECOPS_STATUS_OK;
}

template <typename TS, typename TD>
int32_t pack_typed(const VecopsB200Pack& p, int64_t pitch, VecopsError* error) {
  const TS* src = static_cast<const TS*>(p.src);
  TD* dst = static_cast<TD*>(p.dst);
  cudaStream_t stream = static_cast<cudaStream_t>(p.stream);
  const int k = static_cast<int>(p.k);
  if (p.src_stride_k == 1 || p.k == 1) {
    const bool vec = aligned16(src) && (p.src_stride_row * sizeof(TS)) % 16 == 0 && p.src_stride_k == 1;
    const long long chunks = p.rows * (pitch / (16 / static_cast<int64_t>(sizeof(TD))));
    const int blocks = static_cast<int>(chunks / 256 + 1 < 148 * 16 ? chunks / 256 + 1 : 148 * 16);
    if (vec) pack_rows_copy_kernel<TS, TD, true><<<blocks, 256, 0, stream>>>(src, p.src_stride_row, dst, pitch, p.rows, k);
    else pack_rows_copy_kernel<TS, TD, false><<<blocks, 256, 0, stream>>>(src, p.src_stride_row, dst, pitch, p.rows, k);
    return launch_status(error, "pack (row copy) launch");
  }
  const dim3 grid(static_cast<unsigned>((pitch + PackTile::kK - 1) / PackTile::kK), static_cast<unsigned>((p.rows + PackTile::kRows - 1) / PackTile::kRows));
  if (grid.y > 65535u) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "pack: more than 65535 x 128 rows");
  const bool vec = p.src_stride_row == 1 && aligned16(src) && (p.src_stride_k * sizeof(TS)) % 16 == 0;
  if (vec) pack_rows_transpose_kernel<TS, TD, true><<<grid, PackTile::kThreads, 0, stream>>>(src, p.src_stride_row, p.src_stride_k, dst, pitch, p.rows, k);
  else pack_rows_transpose_kernel<TS, TD, false><<<grid, PackTile::kThreads, 0, stream>>>(src, p.src_stride_row, p.src_stride_k, dst, pitch, p.rows, k);
  return launch_status(error, "pack (transpose) launch");
}

}  // namespace

extern "C" {

int32_t vecops_b200_matmul_packed_layout(uint32_t dtype, int64_t rows, int64_t k, int64_t* pitch_elements, uint64_t* bytes,
                                         VecopsError* error) {
  const size_t elem = pack_elem_size(dtype);
  if (elem == 0) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "packed_layout: dtype %u has no packed form", dtype);
  if (rows < 0 || k < 0) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "packed_layout: negative extent");
  const int64_t per_line = 128 / static_cast<int64_t>(elem);
  const int64_t pitch = (k + per_line - 1) / per_line * per_line;
  if (pitch_elements != nullptr) *pitch_elements = pitch;
  if (bytes != nullptr) *bytes = static_cast<uint64_t>(rows) * static_cast<uint64_t>(pitch) * elem;
  return VECOPS_STATUS_OK;
}

int32_t vecops_b200_matmul_pack(const VecopsB200Pack* pack, VecopsError* error) {
  if (pack == nullptr || pack->struct_size < sizeof(VecopsB200Pack))
    return set_error(error, VECOPS_STATUS_ABI_MISMATCH, "pack record is null or too small");
  const VecopsB200Pack& p = *pack;
  int64_t pitch = 0;
  uint64_t need = 0;
  int32_t rc = vecops_b200_matmul_packed_layout(p.dst_dtype, p.rows, p.k, &pitch, &need, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  if (pack_elem_size(p.src_dtype) == 0) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "pack: source dtype %u is not served", p.src_dtype);
  if (p.rows == 0 || p.k == 0) return VECOPS_STATUS_OK;  // nothing to write, nothing is read (a zero-K packed layout is empty)
  if (p.src == nullptr || p.dst == nullptr) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "pack: null pointer");
  if (p.dst_size < need)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "pack: destination holds %llu bytes, the packed layout needs %llu",
                     (unsigned long long)p.dst_size, (unsigned long long)need);
  if (!aligned16(p.dst)) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "pack: destination must be 16-byte aligned");
  if (p.src_stride_row < 0 || p.src_stride_k < 0) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "pack: negative source stride");
  if (p.k >= (INT64_C(1) << 31) - 128) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "pack: K out of range");
  {  // the destination may not overlap the source view (the reference rejects aliasing too, tests/ops/MatmulPackTest.cpp:461-487)
    const uintptr_t s0 = reinterpret_cast<uintptr_t>(p.src);
    const uintptr_t s1 = s0 + (static_cast<uint64_t>(p.rows - 1) * p.src_stride_row + static_cast<uint64_t>(p.k - 1) * p.src_stride_k + 1) *
                                  pack_elem_size(p.src_dtype);
    const uintptr_t d0 = reinterpret_cast<uintptr_t>(p.dst), d1 = d0 + need;
    if (s0 < d1 && d0 < s1) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "pack: source and destination overlap");
  }
  if (vecops_b200_device_count() == 0)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "no usable CUDA device; there is no CPU fallback");
  if (p.device_index >= 0) {
    const cudaError_t status = cudaSetDevice(p.device_index);
    if (status != cudaSuccess) return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "cudaSetDevice(%d): %s", p.device_index, cudaGetErrorString(status));
  }
  if (p.src_dtype == p.dst_dtype) {
    switch (pack_elem_size(p.src_dtype)) {
      case 1: return pack_typed<uint8_t, uint8_t>(p, pitch, error);
      case 2: return pack_typed<uint16_t, uint16_t>(p, pitch, error);
      default: return pack_typed<uint32_t, uint32_t>(p, pitch, error);
    }
  }
  if (p.src_dtype == VECOPS_DTYPE_F32 && p.dst_dtype == VECOPS_DTYPE_BF16) return pack_typed<float, __nv_bfloat16>(p, pitch, error);
  if (p.src_dtype == VECOPS_DTYPE_F32 && p.dst_dtype == VECOPS_DTYPE_F16) return pack_typed<float, __half>(p, pitch, error);
  return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "pack: dtype %u -> %u is not served (same type, or f32 narrowed to bf16 / f16)",
                   p.src_dtype, p.dst_dtype);
}

int32_t vecops_b200_matmul_pack_b_compensated(const VecopsB200Pack* pack, int32_t a_zero_point, int32_t* compensation, VecopsError* error) {
  if (pack == nullptr || pack->struct_size < sizeof(VecopsB200Pack))
    return set_error(error, VECOPS_STATUS_ABI_MISMATCH, "pack record is null or too small");
  if (pack->dst_dtype != VECOPS_DTYPE_I8 || pack->src_dtype != VECOPS_DTYPE_I8)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "pack_b_compensated serves a signed 8-bit B (u8 x s8 -> i32 products)");
  if (pack->rows > 0 && compensation == nullptr)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "pack_b_compensated: null compensation row");
  int32_t rc = vecops_b200_matmul_pack(pack, error);
  if (rc != VECOPS_STATUS_OK || pack->rows == 0) return rc;
  if (pack->k == 0) {  // an empty reduction: the row is all zero, and no packed byte exists to sum
    const cudaError_t status = cudaMemsetAsync(compensation, 0, static_cast<size_t>(pack->rows) * sizeof(int32_t), static_cast<cudaStream_t>(pack->stream));
    if (status != cudaSuccess) return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "pack_b_compensated: %s", cudaGetErrorString(status));
    return VECOPS_STATUS_OK;
  }
  int64_t pitch = 0;
  rc = vecops_b200_matmul_packed_layout(pack->dst_dtype, pack->rows, pack->k, &pitch, nullptr, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  // sums over the packed rows (K-contiguous by now); K == 0 leaves an all-zero row, as the reference does
  return vecops_b200_column_correction(pack->dst, pack->dst_dtype, pitch, pack->rows, pack->k, a_zero_point, compensation, pack->stream, error);
}

}  // extern "C"
