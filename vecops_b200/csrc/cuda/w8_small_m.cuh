// Weight-only int8 dequant-GEMM for decode shapes (small M):
//     C[m,n] = convert( (sum_k f32(A[m,k]) * f32(W[n,k])) * scale[n] )
// A bf16 [M,K], W int8 [N,K] (K-contiguous), scale f32 [N], C bf16 or f32.
//
// The kernel is bound by the single pass over W (N*K bytes from HBM).  Each
// warp owns 16 weight rows and a quarter of K; a thread streams its rows with
// 128-bit non-allocating loads (32 bytes per row per step, a full 128-byte line
// per row per quad), widens int8 -> bf16 in registers (exact: |w| <= 128 fits
// bf16's 8 significant bits) and feeds mma.sync.m16n8k16 with the weights as
// the 16-row operand and up to 8 activation rows as the 8-column operand, so
// products and sums are fp32 and no CUDA-core FMA is spent per weight.  The
// reduction index K may be visited in any order as long as both operands
// agree: thread t of a quad feeds its own 4 consecutive k per step into the
// fragment slots {2t, 2t+1, 2t+8, 2t+9} of both A and B.  The four K-quarters
// of a row tile meet in shared memory (split-K inside the CTA: no global
// scratch, fixed summation order).
//
// Algorithmic traffic per launch: N*K + 4*N + 2*M*K + sizeof(C)*M*N bytes.
#pragma once

#include "epilogue.cuh"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vb200 {

struct W8SmallM {
  static constexpr int kRowsPerCta = 32;   // two 16-row tiles
  static constexpr int kKSplit = 4;        // warps sharing one row tile
  static constexpr int kThreads = 256;
  static constexpr int kChunkK = 128;      // k per warp step
};

__device__ __forceinline__ uint4 ldg_stream_128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Four int8 in one word -> two bf16x2 words {w0,w1}, {w2,w3}, exactly.
// Flip the sign bit (w + 128 as unsigned), drop each byte into the mantissa of
// 2^23 with PRMT, subtract 2^23 + 128 in fp32, then pack pairs to bf16.
__device__ __forceinline__ void dequant4(uint32_t packed, uint32_t& lo, uint32_t& hi) {
  const uint32_t biased = packed ^ 0x80808080u;
  const float kMagic = 8388736.f;  // 2^23 + 128
  const float f0 = __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7540)) - kMagic;
  const float f1 = __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7541)) - kMagic;
  const float f2 = __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7542)) - kMagic;
  const float f3 = __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7543)) - kMagic;
  __nv_bfloat162 p0 = __floats2bfloat162_rn(f0, f1);
  __nv_bfloat162 p1 = __floats2bfloat162_rn(f2, f3);
  lo = *reinterpret_cast<uint32_t*>(&p0);
  hi = *reinterpret_cast<uint32_t*>(&p1);
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// kMTiles: activation rows handled per CTA in groups of 8 (1, 2 or 4).
// Requirements checked on the host: K % 32 == 0, W rows 16-byte aligned
// (ldw % 16 == 0), A rows 16-byte aligned (lda % 8 == 0), both K-contiguous.
template <int kMTiles, typename OutT>
__global__ void __launch_bounds__(W8SmallM::kThreads)
w8_small_m_kernel(const __nv_bfloat16* __restrict__ a, long long lda, const int8_t* __restrict__ w, long long ldw,
                  const float* __restrict__ scale, OutT* __restrict__ c, long long ldc, int M, int N, int K, EpilogueArgs ep) {
  using G = W8SmallM;
  __shared__ float red[2][G::kKSplit][kMTiles][32][4];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;  // fragment row
  const int t = lane & 3;   // thread in quad
  const int row_tile = warp >> 2;
  const int kq = warp & 3;
  const int m_base = blockIdx.y * (8 * kMTiles);
  const int n_tile0 = blockIdx.x * G::kRowsPerCta + row_tile * 16;

  // clamp rows so that every load stays inside W; out-of-range rows are dropped at the store
  const int n_lo = min(n_tile0 + g, N - 1);
  const int n_hi = min(n_tile0 + g + 8, N - 1);
  const int8_t* w_lo = w + static_cast<long long>(n_lo) * ldw + 32 * t;
  const int8_t* w_hi = w + static_cast<long long>(n_hi) * ldw + 32 * t;
  const __nv_bfloat16* a_row[kMTiles];
  bool a_valid[kMTiles];
#pragma unroll
  for (int j = 0; j < kMTiles; ++j) {
    const int m = m_base + 8 * j + g;
    a_valid[j] = m < M;
    a_row[j] = a + static_cast<long long>(a_valid[j] ? m : 0) * lda + 32 * t;
  }

  float acc[kMTiles][4];
#pragma unroll
  for (int j = 0; j < kMTiles; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

  const int num_chunks = (K + G::kChunkK - 1) / G::kChunkK;

  uint4 wl[2], wh[2];        // 32 weights of row g and of row g+8
  uint4 av[kMTiles][4];      // 32 activations (bf16) per m-tile
  auto fetch = [&](int chunk, uint4 (&l)[2], uint4 (&h)[2], uint4 (&x)[kMTiles][4]) {
    const int k = chunk * G::kChunkK;
    const bool in_k = k + 32 * t < K;  // K % 32 == 0: a thread's 32-k unit is all in or all out
    if (in_k) {
      l[0] = ldg_stream_128(w_lo + k);
      l[1] = ldg_stream_128(w_lo + k + 16);
      h[0] = ldg_stream_128(w_hi + k);
      h[1] = ldg_stream_128(w_hi + k + 16);
    } else {
      l[0] = l[1] = h[0] = h[1] = make_uint4(0x0, 0x0, 0x0, 0x0);
    }
#pragma unroll
    for (int j = 0; j < kMTiles; ++j) {
      if (in_k && a_valid[j]) {
        const uint4* p = reinterpret_cast<const uint4*>(a_row[j] + k);
#pragma unroll
        for (int q = 0; q < 4; ++q) x[j][q] = __ldg(p + q);
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) x[j][q] = make_uint4(0, 0, 0, 0);
      }
    }
  };

  int chunk = kq;
  if (chunk < num_chunks) fetch(chunk, wl, wh, av);
  for (; chunk < num_chunks; chunk += G::kKSplit) {
    uint4 nl[2], nh[2], nx[kMTiles][4];
    const int next = chunk + G::kKSplit;
    if (next < num_chunks) fetch(next, nl, nh, nx);

    const uint32_t lo_words[8] = {wl[0].x, wl[0].y, wl[0].z, wl[0].w, wl[1].x, wl[1].y, wl[1].z, wl[1].w};
    const uint32_t hi_words[8] = {wh[0].x, wh[0].y, wh[0].z, wh[0].w, wh[1].x, wh[1].y, wh[1].z, wh[1].w};
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      uint32_t a0, a1, a2, a3;
      dequant4(lo_words[s], a0, a2);  // row g:   k+0,1 | k+2,3
      dequant4(hi_words[s], a1, a3);  // row g+8: k+0,1 | k+2,3
#pragma unroll
      for (int j = 0; j < kMTiles; ++j) {
        const uint4 x = av[j][s >> 1];
        const uint32_t b0 = (s & 1) ? x.z : x.x;
        const uint32_t b1 = (s & 1) ? x.w : x.y;
        mma_bf16_16816(acc[j], a0, a1, a2, a3, b0, b1);
      }
    }
    if (next < num_chunks) {
      wl[0] = nl[0]; wl[1] = nl[1]; wh[0] = nh[0]; wh[1] = nh[1];
#pragma unroll
      for (int j = 0; j < kMTiles; ++j)
#pragma unroll
        for (int q = 0; q < 4; ++q) av[j][q] = nx[j][q];
    }
  }

  // split-K reduction across the four warps of this row tile, in fixed order
#pragma unroll
  for (int j = 0; j < kMTiles; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) red[row_tile][kq][j][lane][e] = acc[j][e];
  __syncthreads();
  if (kq != 0) return;

  float s_lo = 1.f, s_hi = 1.f;
  const int n_out_lo = n_tile0 + g, n_out_hi = n_tile0 + g + 8;
  if (scale != nullptr) {
    if (n_out_lo < N) s_lo = __ldg(scale + n_out_lo);
    if (n_out_hi < N) s_hi = __ldg(scale + n_out_hi);
  }
#pragma unroll
  for (int j = 0; j < kMTiles; ++j) {
    float sum[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      sum[e] = red[row_tile][0][j][lane][e];
#pragma unroll
      for (int q = 1; q < G::kKSplit; ++q) sum[e] += red[row_tile][q][j][lane][e];
    }
    // fragment: sum[0], sum[1] = (n = g,   m = 2t, 2t+1); sum[2], sum[3] = (n = g+8, m = 2t, 2t+1)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int m = m_base + 8 * j + 2 * t + (e & 1);
      const int n = (e < 2) ? n_out_lo : n_out_hi;
      if (m < M && n < N) {
        const float factor = (e < 2) ? s_lo : s_hi;
        const float v = ep.active ? epilogue_float(sum[e], ep, m, n, factor) : sum[e] * factor;
        if constexpr (sizeof(OutT) == 2) c[static_cast<long long>(m) * ldc + n] = __float2bfloat16_rn(v);
        else c[static_cast<long long>(m) * ldc + n] = v;
      }
    }
  }
}

}  // namespace vb200
