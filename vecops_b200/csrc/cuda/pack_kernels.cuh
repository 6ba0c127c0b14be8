// Operand preparation ("pack"): any strided [rows, K] view -> K-contiguous rows on a 128-byte pitch, zero-filled
// past K, optionally narrowing fp32 to a 16-bit compute type on the way.  That layout is what the TMA-fed tensor-core
// kernels want; a [K, N]-stored weight matrix (rows contiguous along N) is transposed here once instead of being read
// through the strided kernel on every product.
//
// Both kernels are bound by HBM: each source element is read once and each destination element written once.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vb200 {

template <typename TD, typename TS>
__device__ __forceinline__ TD pack_convert(TS value) {
  return value;  // same width: a bit copy (uint8_t, uint16_t and uint32_t stand for every 1-, 2- and 4-byte type)
}
template <>
__device__ __forceinline__ __nv_bfloat16 pack_convert<__nv_bfloat16, float>(float value) {
  return __float2bfloat16_rn(value);
}
template <>
__device__ __forceinline__ __half pack_convert<__half, float>(float value) {
  return __float2half_rn(value);
}

template <typename T>
__device__ __forceinline__ T pack_zero() {
  return T(0);
}
template <>
__device__ __forceinline__ __nv_bfloat16 pack_zero<__nv_bfloat16>() {
  return __float2bfloat16_rn(0.f);
}
template <>
__device__ __forceinline__ __half pack_zero<__half>() {
  return __float2half_rn(0.f);
}

// ---------------------------------------------------------------- K-contiguous source: a row copy onto the new pitch
//
// One thread per 16 bytes of destination.  kVec: the source rows can be read in 16-byte pieces too (base and row
// pitch 16-byte aligned); otherwise element loads.  `pitch` counts destination elements and is a multiple of
// 16 / sizeof(TD); elements at k >= K are written as zero.
template <typename TS, typename TD, bool kVec>
__global__ void __launch_bounds__(256) pack_rows_copy_kernel(const TS* __restrict__ src, long long s_row, TD* __restrict__ dst,
                                                             long long pitch, long long rows, int k) {
  constexpr int kOut = 16 / static_cast<int>(sizeof(TD));  // elements per thread
  const long long chunks = pitch / kOut;
  const long long total = rows * chunks;
  for (long long u = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; u < total;
       u += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = u / chunks;
    const int k0 = static_cast<int>(u % chunks) * kOut;
    alignas(16) TD out[kOut];
    const TS* in = src + row * s_row + k0;
    if (kVec && k0 + kOut <= k) {
      constexpr int kLoads = static_cast<int>(sizeof(TS)) * kOut / 16;  // 1, or 2 when narrowing fp32
      alignas(16) TS staged[kOut];
#pragma unroll
      for (int j = 0; j < kLoads; ++j) reinterpret_cast<uint4*>(staged)[j] = __ldg(reinterpret_cast<const uint4*>(in) + j);
#pragma unroll
      for (int j = 0; j < kOut; ++j) out[j] = pack_convert<TD, TS>(staged[j]);
    } else {
#pragma unroll
      for (int j = 0; j < kOut; ++j) out[j] = k0 + j < k ? pack_convert<TD, TS>(in[j]) : pack_zero<TD>();
    }
    *reinterpret_cast<uint4*>(dst + row * pitch + k0) = *reinterpret_cast<const uint4*>(out);
  }
}

// ---------------------------------------------------------------- any other source: transpose through shared memory
//
// A CTA moves a tile of 128 rows x 64 k.  Load phase: threads run along the ROW axis of the source (the contiguous one
// of a [K, N]-stored matrix) - 16 bytes per thread when kVec (s_row == 1, base and k-pitch 16-byte aligned), else
// one element - convert, and scatter into a shared tile held in destination order.  Store phase: 16 bytes per
// thread along k.  The tile's 16-byte pieces are permuted per row (piece ^ f(row)) so that the scatter of one
// source vector - same k, consecutive rows - spreads over the banks.
struct PackTile {
  static constexpr int kRows = 128;
  static constexpr int kK = 64;
  static constexpr int kThreads = 256;
};

template <typename TS, typename TD, bool kVec>
__global__ void __launch_bounds__(PackTile::kThreads) pack_rows_transpose_kernel(const TS* __restrict__ src, long long s_row, long long s_k,
                                                                                 TD* __restrict__ dst, long long pitch, long long rows, int k) {
  using T = PackTile;
  constexpr int kIn = 16 / static_cast<int>(sizeof(TS));    // source elements per vector (along rows)
  constexpr int kOut = 16 / static_cast<int>(sizeof(TD));   // destination elements per 16-byte piece (along k)
  constexpr int kPieces = T::kK / kOut;                     // pieces per tile row: 4 (8-bit), 8 (16-bit), 16 (32-bit)
  __shared__ __align__(16) TD tile[T::kRows * T::kK];

  const long long row0 = static_cast<long long>(blockIdx.y) * T::kRows;
  const int k0 = blockIdx.x * T::kK;

  auto slot = [&](int r, int kk) -> int {  // where element (r, kk) of the tile lives
    const int piece = (kk / kOut) ^ ((r / kIn) % kPieces);
    return r * T::kK + piece * kOut + kk % kOut;
  };

  if constexpr (kVec && sizeof(TS) == 1 && sizeof(TD) == 1) {
    // 8-bit elements: four k-lines at a time, transposed 4x4 in registers (PRMT), so that the scatter writes whole
    // words - (row, k..k+3) - instead of single bytes
    constexpr int kVectorsPerLine = T::kRows / 16;
    for (int item = threadIdx.x; item < kVectorsPerLine * (T::kK / 4); item += T::kThreads) {
      const int rv = item % kVectorsPerLine, kk = (item / kVectorsPerLine) * 4;
      const long long row = row0 + rv * 16;
      uint32_t line[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (k0 + kk + i < k && row + 16 <= rows) {
          const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + row + static_cast<long long>(k0 + kk + i) * s_k));
          line[i][0] = v.x, line[i][1] = v.y, line[i][2] = v.z, line[i][3] = v.w;
        } else {
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const bool inside = k0 + kk + i < k && row + 4 * w + b < rows;
              const uint32_t value = inside ? static_cast<uint32_t>(static_cast<uint8_t>(src[row + 4 * w + b + static_cast<long long>(k0 + kk + i) * s_k])) : 0u;
              word |= value << (8 * b);
            }
            line[i][w] = word;
          }
        }
      }
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t lo01 = __byte_perm(line[0][w], line[1][w], 0x5140), hi01 = __byte_perm(line[0][w], line[1][w], 0x7362);
        const uint32_t lo23 = __byte_perm(line[2][w], line[3][w], 0x5140), hi23 = __byte_perm(line[2][w], line[3][w], 0x7362);
        const uint32_t out[4] = {__byte_perm(lo01, lo23, 0x5410), __byte_perm(lo01, lo23, 0x7632), __byte_perm(hi01, hi23, 0x5410),
                                 __byte_perm(hi01, hi23, 0x7632)};
#pragma unroll
        for (int b = 0; b < 4; ++b) *reinterpret_cast<uint32_t*>(&tile[slot(rv * 16 + 4 * w + b, kk)]) = out[b];
      }
    }
  } else if (kVec) {
    constexpr int kVectorsPerLine = T::kRows / kIn;
    constexpr int kVectors = kVectorsPerLine * T::kK;
    for (int v = threadIdx.x; v < kVectors; v += T::kThreads) {
      const int rv = v % kVectorsPerLine, kk = v / kVectorsPerLine;
      const long long row = row0 + rv * kIn;
      alignas(16) TS staged[kIn];
      if (k0 + kk < k && row + kIn <= rows) {
        *reinterpret_cast<uint4*>(staged) = __ldg(reinterpret_cast<const uint4*>(src + row + static_cast<long long>(k0 + kk) * s_k));
      } else {
#pragma unroll
        for (int j = 0; j < kIn; ++j)
          staged[j] = (k0 + kk < k && row + j < rows) ? src[row + j + static_cast<long long>(k0 + kk) * s_k] : TS(0);
      }
#pragma unroll
      for (int j = 0; j < kIn; ++j) tile[slot(rv * kIn + j, kk)] = pack_convert<TD, TS>(staged[j]);
    }
  } else {
    for (int e = threadIdx.x; e < T::kRows * T::kK; e += T::kThreads) {
      const int r = e % T::kRows, kk = e / T::kRows;
      const bool inside = row0 + r < rows && k0 + kk < k;
      tile[slot(r, kk)] = inside ? pack_convert<TD, TS>(src[(row0 + r) * s_row + static_cast<long long>(k0 + kk) * s_k]) : pack_zero<TD>();
    }
  }
  __syncthreads();
  for (int p = threadIdx.x; p < T::kRows * kPieces; p += T::kThreads) {
    const int r = p / kPieces, piece = p % kPieces;
    if (row0 + r >= rows || k0 + piece * kOut >= pitch) continue;
    const int physical = piece ^ ((r / kIn) % kPieces);
    *reinterpret_cast<uint4*>(dst + (row0 + r) * pitch + k0 + piece * kOut) =
        *reinterpret_cast<const uint4*>(&tile[r * T::kK + physical * kOut]);
  }
}

}  // namespace vb200
