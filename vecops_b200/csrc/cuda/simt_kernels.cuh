// CUDA-core kernels: the strided any-dtype GEMM that serves ragged and
// unaligned problems, and the tiled FP32 FMA GEMM.
#pragma once

#include "epilogue.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vb200 {

// ------------------------------------------------------------------ element conversion

template <typename Acc, typename T>
__device__ __forceinline__ Acc load_as(const T* p) {
  return static_cast<Acc>(*p);
}
template <>
__device__ __forceinline__ float load_as<float, __nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
// 8-bit operands widen to 32-bit and accumulate modulo 2^32 (the vecops
// int32 accumulator wraps: include/vecops/vec/WideningDot.h:100-103).
template <>
__device__ __forceinline__ float load_as<float, __half>(const __half* p) {
  return __half2float(*p);
}
template <>
__device__ __forceinline__ uint32_t load_as<uint32_t, int8_t>(const int8_t* p) {
  return static_cast<uint32_t>(static_cast<int32_t>(*p));
}
template <>
__device__ __forceinline__ uint32_t load_as<uint32_t, uint8_t>(const uint8_t* p) {
  return static_cast<uint32_t>(*p);
}

template <typename Out, typename Acc>
__device__ __forceinline__ void store_from(Out* p, Acc v) {
  *p = static_cast<Out>(v);
}
template <>
__device__ __forceinline__ void store_from<__nv_bfloat16, float>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ void store_from<__half, float>(__half* p, float v) {
  *p = __float2half_rn(v);
}
template <>
__device__ __forceinline__ void store_from<int32_t, uint32_t>(int32_t* p, uint32_t v) {
  *p = static_cast<int32_t>(v);
}

// ------------------------------------------------------------------ strided any-dtype GEMM

// C[m,n] = convert( (sum_k A[m,k] * B[n,k]) * scale[n] ), arbitrary element
// strides on all three tensors.  32x32 output tile, 32-deep k-blocks staged in
// shared memory in accumulator type, 4 outputs per thread.
template <typename TA, typename TB, typename TC, typename Acc>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(const TA* __restrict__ a, long long sam, long long sak, const TB* __restrict__ b, long long sbn,
                    long long sbk, TC* __restrict__ c, long long scm, long long scn, int M, int N, int K,
                    const float* __restrict__ column_scale, EpilogueArgs ep) {
  constexpr int T = 32;
  __shared__ Acc as[T][T + 1];
  __shared__ Acc bs[T][T + 1];
  const int tx = threadIdx.x & 31;
  const int ty = threadIdx.x >> 5;  // 0..7
  const int m0 = blockIdx.y * T;
  const int n0 = blockIdx.x * T;
  Acc acc[4] = {Acc(0), Acc(0), Acc(0), Acc(0)};
  for (int k0 = 0; k0 < K; k0 += T) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = ty + 8 * j;
      const int kk = k0 + tx;
      const int m = m0 + r;
      const int n = n0 + r;
      as[r][tx] = (m < M && kk < K) ? load_as<Acc, TA>(a + m * sam + kk * sak) : Acc(0);
      bs[r][tx] = (n < N && kk < K) ? load_as<Acc, TB>(b + n * sbn + kk * sbk) : Acc(0);
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < T; ++kk) {
      const Acc bv = bs[tx][kk];
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] += as[ty + 8 * j][kk] * bv;
    }
    __syncthreads();
  }
  const int n = n0 + tx;
  if (n >= N) return;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int m = m0 + ty + 8 * j;
    if (m >= M) continue;
    Acc v = acc[j];
    if constexpr (std::is_same<Acc, float>::value) {
      const float factor = column_scale != nullptr ? column_scale[n] : 1.f;
      if (ep.active) v = epilogue_float(v, ep, m, n, factor);
      else v *= factor;
    } else if constexpr (std::is_same<Acc, uint32_t>::value) {
      if (ep.active) v = epilogue_int(v, ep, m, n);
      if constexpr (!std::is_same<TC, int32_t>::value) {
        // the dequantising form: the int32 accumulator, converted, takes the float transform
        const float factor = column_scale != nullptr ? column_scale[n] : 1.f;
        store_from<TC, float>(c + m * scm + n * scn, epilogue_float(static_cast<float>(static_cast<int32_t>(v)), ep, m, n, factor));
        continue;
      }
    }
    store_from<TC, Acc>(c + m * scm + n * scn, v);
  }
}

// ------------------------------------------------------------------ FP32 FMA GEMM

// C[M,N] = A[M,K] . B[N,K]^T in FP32 with FP32 FMA accumulation (no tensor
// cores, so FP32 semantics are kept exactly: every product is an fp32 product
// and every sum an fp32 sum).  64x64 tile, 16-deep k-blocks, 4x4 outputs per
// thread.  A must be k-contiguous; B is either k-contiguous ([N,K] rows) or
// n-contiguous (a row-major [K,N] matrix viewed as [N,K]).
struct GemmF32 {
  static constexpr int kTile = 64;
  static constexpr int kDepth = 16;
  static constexpr int kPad = 4;
};

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ a, long long lda, const float* __restrict__ b, long long sbn,
                long long sbk, float* __restrict__ c, long long ldc, int M, int N, int K, EpilogueArgs ep) {
  using G = GemmF32;
  __shared__ __align__(16) float as[2][G::kDepth][G::kTile + G::kPad];
  __shared__ __align__(16) float bs[2][G::kDepth][G::kTile + G::kPad];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * G::kTile;
  const int n0 = blockIdx.x * G::kTile;
  const int tx = tid & 15;   // 4 columns each
  const int ty = tid >> 4;   // 4 rows each
  const bool b_k_contig = (sbk == 1);

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  float ra[4], rb[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // A: 16 consecutive k per row, 16 rows per pass
      const int kk = tid & 15, r = (tid >> 4) + 16 * j;
      const int m = m0 + r, k = k0 + kk;
      ra[j] = (m < M && k < K) ? __ldg(a + static_cast<long long>(m) * lda + k) : 0.f;
      if (b_k_contig) {
        const int n = n0 + r;
        rb[j] = (n < N && k < K) ? __ldg(b + static_cast<long long>(n) * sbn + k) : 0.f;
      } else {
        // B n-contiguous: 64 consecutive n per k, 4 k per pass
        const int nn = tid & 63, kq = (tid >> 6) + 4 * j;
        const int n = n0 + nn, k2 = k0 + kq;
        rb[j] = (n < N && k2 < K) ? __ldg(b + static_cast<long long>(n) * sbn + static_cast<long long>(k2) * sbk) : 0.f;
      }
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kk = tid & 15, r = (tid >> 4) + 16 * j;
      as[buf][kk][r] = ra[j];
      if (b_k_contig) {
        bs[buf][kk][r] = rb[j];
      } else {
        const int nn = tid & 63, kq = (tid >> 6) + 4 * j;
        bs[buf][kq][nn] = rb[j];
      }
    }
  };

  const int num_kb = (K + G::kDepth - 1) / G::kDepth;
  if (num_kb > 0) {
    fetch(0);
    stash(0);
  }
  __syncthreads();
  for (int kb = 0; kb < num_kb; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < num_kb) fetch((kb + 1) * G::kDepth);
#pragma unroll
    for (int kk = 0; kk < G::kDepth; ++kk) {
      const float4 av = *reinterpret_cast<const float4*>(&as[buf][kk][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&bs[buf][kk][tx * 4]);
      const float avs[4] = {av.x, av.y, av.z, av.w};
      const float bvs[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(avs[i], bvs[j], acc[i][j]);
    }
    if (kb + 1 < num_kb) stash(buf ^ 1);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
    float* dst = c + static_cast<long long>(m) * ldc + n0 + tx * 4;
    const int n = n0 + tx * 4;
    if (ep.active) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n + j < N) acc[i][j] = epilogue_float(acc[i][j], ep, m, n + j, 1.f);
    }
    if (n + 3 < N && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
      *reinterpret_cast<float4*>(dst) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n + j < N) dst[j] = acc[i][j];
    }
  }
}

// The same product for shapes made of whole tiles with 16-byte aligned rows (C1 is one): a 64 x 64 x 16 tile per CTA of
// 64 threads, 8 x 8 outputs per thread held as four 4 x 4 quadrants 32 rows / columns apart (so that a warp's 16-byte
// shared-memory reads fall on consecutive words), 16-byte global loads prefetched into registers one k-tile ahead, two
// shared buffers, one barrier per k-tile.  64 independent accumulators per thread keep the FMA pipe busy from a single
// warp per scheduler, which is all a 1024^3 problem gives 148 SMs.  Every product and sum is still an fp32 FMA.
// kBKContig: B rows are K-contiguous ([N,K] storage); otherwise N-contiguous ([K,N] storage, C1's layout).
// kSplit > 1: the kernel is launched as thread-block clusters of kSplit CTAs along z, CTA r of a cluster sums the r-th
// part of K; the others park their sums in their own shared memory and CTA 0 reads them through distributed shared
// memory, adds them in rank order (the same order every run) and stores.  That multiplies the resident warps of a
// problem too small to fill the SMs with 64 x 64 tiles.
template <bool kBKContig, int kRowsPerThread, int kSplit>
__global__ void __launch_bounds__(512 / kRowsPerThread)
gemm_f32_tile8_kernel(const float* __restrict__ a, long long lda, const float* __restrict__ b, long long ldb, float* __restrict__ c,
                      long long ldc, int K, EpilogueArgs ep) {
  // kRowsPerThread 8: 64 threads, 8 x 8 outputs each (rows 4ty.. and 32+4ty..); 4: 128 threads, 4 x 8 outputs each (rows 4ty..)
  constexpr int kTile = 64, kDepth = 16, kPitch = kTile + 4, kThreads = 512 / kRowsPerThread;
  constexpr int kLoads = 256 / kThreads;  // 16-byte pieces of each operand tile per thread
  __shared__ __align__(16) float staging[2 * 2 * kDepth * kPitch];  // as[2][16][68] then bs[2][16][68]; 4096 sums fit for the exchange
  float (*as)[kDepth][kPitch] = reinterpret_cast<float (*)[kDepth][kPitch]>(staging);
  float (*bs)[kDepth][kPitch] = reinterpret_cast<float (*)[kDepth][kPitch]>(staging + 2 * kDepth * kPitch);
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
  const int tx = tid & 7, ty = tid >> 3;
  const int rank = kSplit > 1 ? static_cast<int>(cluster_cta_rank()) : 0;
  const int k_begin = rank * (K / kSplit);  // K is a multiple of 16 * kSplit

  float acc[kRowsPerThread][8];
#pragma unroll
  for (int i = 0; i < kRowsPerThread; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  float4 ra[kLoads], rb[kLoads];
  // A (and a K-contiguous B): a thread owns row (t mod 64) of the tile and kLoads of its four 16-byte pieces along k
  const int row = tid & 63, first_piece = (tid >> 6) * kLoads;
  const float* a_row = a + static_cast<long long>(m0 + row) * lda + 4 * first_piece;
  const float* b_row = kBKContig ? b + static_cast<long long>(n0 + row) * ldb + 4 * first_piece : b + n0 + 4 * (tid & 15);
  auto fetch = [&](int k0) {
#pragma unroll
    for (int q = 0; q < kLoads; ++q) {
      ra[q] = __ldg(reinterpret_cast<const float4*>(a_row + k0 + 4 * q));
      if (kBKContig) rb[q] = __ldg(reinterpret_cast<const float4*>(b_row + k0 + 4 * q));
      else rb[q] = __ldg(reinterpret_cast<const float4*>(b_row + static_cast<long long>(k0 + (tid >> 4) + (kThreads / 16) * q) * ldb));
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int q = 0; q < kLoads; ++q) {
      const int k4 = 4 * (first_piece + q);
      as[buf][k4 + 0][row] = ra[q].x, as[buf][k4 + 1][row] = ra[q].y, as[buf][k4 + 2][row] = ra[q].z, as[buf][k4 + 3][row] = ra[q].w;
      if (kBKContig) {
        bs[buf][k4 + 0][row] = rb[q].x, bs[buf][k4 + 1][row] = rb[q].y, bs[buf][k4 + 2][row] = rb[q].z, bs[buf][k4 + 3][row] = rb[q].w;
      } else {
        *reinterpret_cast<float4*>(&bs[buf][(tid >> 4) + (kThreads / 16) * q][4 * (tid & 15)]) = rb[q];
      }
    }
  };

  const int num_kb = K / kSplit / kDepth;
  if (num_kb > 0) {
    fetch(k_begin);
    stash(0);
  }
  __syncthreads();
  for (int kb = 0; kb < num_kb; ++kb) {
    const int buf = kb & 1;
    if (kb + 1 < num_kb) fetch(k_begin + (kb + 1) * kDepth);
#pragma unroll
    for (int kk = 0; kk < kDepth; ++kk) {
      float av[kRowsPerThread];
      const float4 a_lo = *reinterpret_cast<const float4*>(&as[buf][kk][4 * ty]);
      av[0] = a_lo.x, av[1] = a_lo.y, av[2] = a_lo.z, av[3] = a_lo.w;
      if constexpr (kRowsPerThread == 8) {
        const float4 a_hi = *reinterpret_cast<const float4*>(&as[buf][kk][32 + 4 * ty]);
        av[4] = a_hi.x, av[5] = a_hi.y, av[6] = a_hi.z, av[7] = a_hi.w;
      }
      const float4 b_lo = *reinterpret_cast<const float4*>(&bs[buf][kk][4 * tx]);
      const float4 b_hi = *reinterpret_cast<const float4*>(&bs[buf][kk][32 + 4 * tx]);
      const float bv[8] = {b_lo.x, b_lo.y, b_lo.z, b_lo.w, b_hi.x, b_hi.y, b_hi.z, b_hi.w};
#pragma unroll
      for (int i = 0; i < kRowsPerThread; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (kb + 1 < num_kb) stash(buf ^ 1);
    __syncthreads();
  }
  if constexpr (kSplit > 1) {
    // (the loop's last barrier is behind every thread: the operand tiles are dead, the buffer is free)
    if (rank != 0) {
#pragma unroll
      for (int i = 0; i < kRowsPerThread; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) staging[(i * 8 + j) * kThreads + tid] = acc[i][j];
    }
    cluster_sync_all();  // the parked sums are visible cluster-wide
    if (rank == 0) {
      const uint32_t mine = static_cast<uint32_t>(__cvta_generic_to_shared(staging));
      for (int r = 1; r < kSplit; ++r) {
        const uint32_t theirs = map_to_cta(mine, static_cast<uint32_t>(r));
#pragma unroll
        for (int i = 0; i < kRowsPerThread; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] += ld_shared_cluster_f32(theirs + 4u * static_cast<uint32_t>((i * 8 + j) * kThreads + tid));
      }
    }
    cluster_sync_all();  // nobody leaves while CTA 0 may still read its shared memory
    if (rank != 0) return;
  }
#pragma unroll
  for (int i = 0; i < kRowsPerThread; ++i) {
    const int m = m0 + (i < 4 ? 4 * ty + i : 32 + 4 * ty + i - 4);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int n = n0 + 32 * half + 4 * tx;
      float out[4] = {acc[i][4 * half], acc[i][4 * half + 1], acc[i][4 * half + 2], acc[i][4 * half + 3]};
      if (ep.active) {
#pragma unroll
        for (int j = 0; j < 4; ++j) out[j] = epilogue_float(out[j], ep, m, n + j, 1.f);
      }
      *reinterpret_cast<float4*>(c + static_cast<long long>(m) * ldc + n) = make_float4(out[0], out[1], out[2], out[3]);
    }
  }
}

// ------------------------------------------------------------------ fp32 product on the tensor cores: operand split
//
// An fp32 value x is the sum of two tf32 values to within 2^-22 of itself: hi = tf32(x) (round to nearest, 10 mantissa
// bits) and lo = tf32(x - hi).  With both operands split, a.b = a_hi.b_hi + a_lo.b_hi + a_hi.b_lo up to a term of 2^-22,
// and each of the three products is exact in the tensor core's fp32 accumulator.  The three are run as ONE product over
// a K three times as long: this kernel writes each operand's rows once as [ hi | lo ], each half Kp wide (K rounded up
// to the 32 words of a k-block, zero past K), and the GEMM's producer walks k' over the three terms - A's halves in the
// order hi, lo, hi against B's hi, hi, lo - so that what is summed is the fp32 product.  Any element strides: a 32 x 32 tile goes through shared memory so
// that both the reads (along whichever axis is contiguous) and the writes (along K) are coalesced.
__device__ __forceinline__ float round_to_tf32(float x) {
  uint32_t bits;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(x));
  return __uint_as_float(bits);
}

// One launch splits both operands: blocks [0, a_blocks) take A's 32 x 32 tiles, the rest B's.
struct SplitOperand {
  const float* src;
  long long stride_row, stride_k;
  float* dst;
  int rows;
};

// One CTA takes kSplitTiles consecutive 32 x 32 tiles along k of one 32-row block and has all their loads in flight
// before the first store: with one tile per CTA the launch was two waves of CTAs each waiting out one DRAM latency.
constexpr int kSplitTiles = 4;

__global__ void __launch_bounds__(256)
f32_split3_kernel(SplitOperand a, SplitOperand b, int a_blocks, int K, int Kp) {
  __shared__ float tile[kSplitTiles][32][33];
  const bool is_b = static_cast<int>(blockIdx.x) >= a_blocks;
  const SplitOperand o = is_b ? b : a;
  const int block = is_b ? blockIdx.x - a_blocks : blockIdx.x;
  const int k_tiles = Kp / 32;
  const int k_groups = (k_tiles + kSplitTiles - 1) / kSplitTiles;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int r0 = (block / k_groups) * 32, kt0 = (block % k_groups) * kSplitTiles;
  const bool k_contiguous = o.stride_k == 1 || o.stride_row != 1;
  float v[kSplitTiles][4];
#pragma unroll
  for (int t = 0; t < kSplitTiles; ++t) {
    const int k0 = (kt0 + t) * 32;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = r0 + (k_contiguous ? ty + 8 * j : tx), k = k0 + (k_contiguous ? tx : ty + 8 * j);
      v[t][j] = (r < o.rows && k < K) ? __ldg(o.src + static_cast<long long>(r) * o.stride_row + static_cast<long long>(k) * o.stride_k) : 0.f;
    }
  }
#pragma unroll
  for (int t = 0; t < kSplitTiles; ++t) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (k_contiguous) tile[t][ty + 8 * j][tx] = v[t][j];
      else tile[t][tx][ty + 8 * j] = v[t][j];
    }
  }
  __syncthreads();
#pragma unroll
  for (int t = 0; t < kSplitTiles; ++t) {
    const int k0 = (kt0 + t) * 32;
    if (k0 >= Kp) break;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = r0 + ty + 8 * j;
      if (r >= o.rows) continue;
      const float x = tile[t][ty + 8 * j][tx];
      const float hi = round_to_tf32(x);
      const float lo = round_to_tf32(x - hi);
      float* row = o.dst + static_cast<long long>(r) * (2ll * Kp) + k0 + tx;  // [hi | lo], each Kp wide
      row[0] = hi;
      row[Kp] = lo;
    }
  }
}

// ------------------------------------------------------------------ quantise-on-load helpers

// dst[m,k] = convert(src[m,k] * scale + zero_point): truncation toward zero, saturating to the 8-bit range, as vecops
// converts an fp32 memory element to an 8-bit compute element (tests/ops/MatmulConversionTestCommon.h:549-556 quantize_a;
// the conversion rule was observed by running the reference: 3.51 -> 3, 255.6 -> 255, -0.6 -> 0).
template <typename TS, bool kSigned>
__global__ void quantize_rows_kernel(const TS* __restrict__ src, long long ssm, long long ssk, uint8_t* __restrict__ dst,
                                     long long dsm, long long rows, long long cols, float scale, float zero_point,
                                     const float* __restrict__ multipliers) {
  // `multipliers` (may be null): one factor per row in place of `scale` - vecops' per-row asymmetric quantisation,
  // q = x * multipliers[row] + zero_point (include/vecops/matmul/Quantization.h:76-140)
  const long long total = rows * cols;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long m = i / cols, k = i % cols;
    const float factor = multipliers != nullptr ? __ldg(multipliers + m) : scale;
    float q = truncf(load_as<float, TS>(src + m * ssm + k * ssk) * factor + zero_point);
    if (!(q == q)) q = 0.f;
    if (kSigned) dst[m * dsm + k] = static_cast<uint8_t>(static_cast<int8_t>(fminf(fmaxf(q, -128.f), 127.f)));
    else dst[m * dsm + k] = static_cast<uint8_t>(fminf(fmaxf(q, 0.f), 255.f));
  }
}

// The common case of the above - fp32 rows, K-contiguous, whole 16-byte groups - four elements per thread.
template <bool kSigned>
__global__ void quantize_rows_f32x4_kernel(const float* __restrict__ src, long long ssm, uint8_t* __restrict__ dst, long long dsm,
                                           long long rows, long long groups_per_row, float scale, float zero_point,
                                           const float* __restrict__ multipliers) {
  const long long total = rows * groups_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long m = i / groups_per_row, g = i % groups_per_row;
    if (multipliers != nullptr) scale = __ldg(multipliers + m);
    const float4 x = __ldg(reinterpret_cast<const float4*>(src + m * ssm) + g);
    const float in[4] = {x.x, x.y, x.z, x.w};
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float q = truncf(in[j] * scale + zero_point);
      if (!(q == q)) q = 0.f;
      const uint32_t byte = kSigned ? static_cast<uint32_t>(static_cast<uint8_t>(static_cast<int8_t>(fminf(fmaxf(q, -128.f), 127.f))))
                                    : static_cast<uint32_t>(static_cast<uint8_t>(fminf(fmaxf(q, 0.f), 255.f)));
      packed |= byte << (8 * j);
    }
    reinterpret_cast<uint32_t*>(dst + m * dsm)[g] = packed;
  }
}

// Rows whose length is a multiple of 16 floats: sixteen elements per thread - four independent 16-byte loads in flight,
// one 16-byte store - which is what brings this pass to the memory system's pace.
template <bool kSigned>
__global__ void quantize_rows_f32x16_kernel(const float* __restrict__ src, long long ssm, uint8_t* __restrict__ dst, long long dsm,
                                            long long rows, long long groups_per_row, float scale, float zero_point,
                                            const float* __restrict__ multipliers) {
  const long long total = rows * groups_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long m = i / groups_per_row, g = i % groups_per_row;
    if (multipliers != nullptr) scale = __ldg(multipliers + m);
    const float4* in = reinterpret_cast<const float4*>(src + m * ssm) + 4 * g;
    float4 x[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) x[q] = __ldg(in + q);
    uint32_t packed[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float values[4] = {x[q].x, x[q].y, x[q].z, x[q].w};
      uint32_t word = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = truncf(values[j] * scale + zero_point);
        if (!(v == v)) v = 0.f;
        const uint32_t byte = kSigned ? static_cast<uint32_t>(static_cast<uint8_t>(static_cast<int8_t>(fminf(fmaxf(v, -128.f), 127.f))))
                                      : static_cast<uint32_t>(static_cast<uint8_t>(fminf(fmaxf(v, 0.f), 255.f)));
        word |= byte << (8 * j);
      }
      packed[q] = word;
    }
    reinterpret_cast<uint4*>(dst + m * dsm)[g] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

// out[n] = -zero_point * sum_k B[n,k]: the accumulator-input row that removes the activations' zero point from an
// asymmetric 8-bit product (MatmulConversionTestCommon.h:529-541; ops/MatmulPack.h:28-35 matmul_pack_b_compensated).
// One warp per row of B.
template <typename TB>
__global__ void column_correction_kernel(const TB* __restrict__ b, long long sbn, int N, int K, int zero_point, int32_t* __restrict__ out) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= N) return;
  const TB* row = b + static_cast<long long>(warp) * sbn;
  int sum = 0;
  if (K % 16 == 0 && (reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
    // 16 bytes per lane and step, summed four at a time by a dot product with ones
    const uint4* words = reinterpret_cast<const uint4*>(row);
    for (int q = lane; q < K / 16; q += 32) {
      const uint4 v = __ldg(words + q);
      const uint32_t part[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        sum = sizeof(TB) == 1 && static_cast<TB>(-1) < 0 ? __dp4a(static_cast<int>(part[j]), 0x01010101, sum)
                                                          : static_cast<int>(__dp4a(part[j], 0x01010101u, static_cast<unsigned>(sum)));
    }
  } else {
    for (int k = lane; k < K; k += 32) sum += static_cast<int>(row[k]);
  }
  for (int offset = 16; offset > 0; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
  if (lane == 0) out[warp] = -zero_point * sum;
}

// ------------------------------------------------------------------ fills and slab placement

__global__ void fill_zero_kernel(uint8_t* __restrict__ c, long long row_pitch_bytes, long long col_pitch_bytes,
                                 int elem_bytes, long long M, long long N) {
  const long long total = M * N;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint8_t* p = c + (i / N) * row_pitch_bytes + (i % N) * col_pitch_bytes;
    for (int e = 0; e < elem_bytes; ++e) p[e] = 0;
  }
}

// dst[r, col0 + j] = src[r, j] in 16-byte units (caller guarantees alignment).
__global__ void place_columns_kernel(uint4* __restrict__ dst, long long dst_pitch16, long long col0_16,
                                     const uint4* __restrict__ src, long long src_pitch16, long long rows,
                                     long long cols16) {
  const long long total = rows * cols16;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols16, j = i % cols16;
    dst[r * dst_pitch16 + col0_16 + j] = src[r * src_pitch16 + j];
  }
}

// Up to eight destinations of one push, passed by value.
struct PushTargets {
  uint4* dst[8];
  int count;
};

// Columns [col0, col0 + cols) of src[rows, pitch] go to the same position of every destination: each 16-byte piece is
// read once and stored `count` times.  A CTA takes whole rows; four pieces per thread are in flight before the first
// store leaves.  Only stores reach the destinations.
//
// Sized to run BESIDE a tensor-core GEMM that fills the SMs: that kernel's CTA leaves 1.7 KB of an SM's shared memory
// (every CTA reserves 1 KB even when it declares none) and 2560 registers in two of the SM's four register
// partitions, so exactly one CTA of 256 threads at no more than 40 registers fits next to it - hence 256 threads,
// 32 registers, and a grid of at most one CTA per SM.
__global__ void __launch_bounds__(256, 8) push_columns_kernel(const uint4* __restrict__ src, PushTargets targets, long long pitch16,
                                                              long long col0_16, int rows, int cols16) {
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const long long row_at = r * pitch16 + col0_16;
    const uint4* from = src + row_at;
    for (int j0 = threadIdx.x; j0 < cols16; j0 += 4 * 256) {
      uint4 piece[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (j0 + u * 256 < cols16) piece[u] = __ldcs(from + j0 + u * 256);
      for (int d = 0; d < targets.count; ++d) {
        uint4* to = targets.dst[d] + row_at;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (j0 + u * 256 < cols16) to[j0 + u * 256] = piece[u];
      }
    }
  }
}

}  // namespace vb200
