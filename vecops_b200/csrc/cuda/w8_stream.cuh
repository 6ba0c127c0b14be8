// Weight-only int8 dequant-GEMM for decode shapes, streaming form (M <= 16,
// K <= 4096, K % 128 == 0):
//     C[m,n] = convert( (sum_k f32(A[m,k]) * f32(W[n,k])) * scale[n] )
//
// How the bytes move:
//   * one persistent CTA per SM; work items are 16-row tiles of W (16 x K bytes,
//     contiguous rows), taken round-robin;
//   * a producer warp streams items into a 3-stage shared-memory ring with
//     cp.async.bulk (one bulk copy per row, completion counted in bytes on an
//     mbarrier), so ~190 KB per SM are in flight without holding registers;
//   * 16 consumer warps split K: warp w owns the 128-wide k-chunks w, w+16.
//     Its activation fragments for those chunks are loaded ONCE into registers
//     at kernel start and reused for every item, so the inner loop touches
//     shared memory only for weights;
//   * per item the 16 partial 16x(8*MT) fragments meet in shared memory and are
//     summed in fixed warp order (deterministic), scaled, converted and stored.
//     The hand-over uses two mbarriers (partials written / partials consumed),
//     so only the few warps that do the summing ever wait.
//
// How the arithmetic is done.  The kernel is HBM-bound only if widening a
// weight costs about one instruction, so the widening goes int8 -> fp16 (two
// weights per PRMT + one HSUB2: 0x6400|u is 1024+u in fp16, minus 1152 gives the
// signed value exactly) and mma.sync.m16n8k16 runs in fp16 x fp16 -> fp32.
// Weights are exact in fp16.  Activations are bf16; each activation row is
// multiplied by a power of two that brings its largest magnitude to 2^14 and
// then converted to fp16, which is exact for every element within 2^31 of the
// row maximum (bf16 carries 8 significant bits, fp16 carries 11, and fp16
// subnormals reach 2^-24); smaller elements lose low bits that lie below what
// an fp32 accumulator resolves next to the row maximum anyway.  Products are
// exact in fp32, sums are fp32, and the power of two is divided out of the
// accumulator before the column scale.  Rows whose maximum is zero, subnormal,
// infinite or NaN are left unscaled.
//
// Smem rows are padded to K + 64 bytes: with a thread reading 16 bytes at
// 16*t of its row, the 8 rows of a fragment then fall on disjoint banks.
//
// Algorithmic traffic per launch: N*K + 4*N + 2*M*K + sizeof(C)*M*N bytes.
#pragma once

#include <cuda_fp16.h>

#include "epilogue.cuh"
#include "gemm_tcgen05.cuh"  // status codes, report_status
#include "ptx.cuh"

namespace vb200 {

struct W8Stream {
  static constexpr int kConsumerWarps = 16;
  static constexpr int kThreads = 32 * (1 + kConsumerWarps);
  static constexpr int kStages = 3;
  static constexpr int kRows = 16;
  static constexpr int kChunkK = 128;
  static constexpr int kMaxK = 4096;
  static constexpr int kRowPad = 64;
  static constexpr int kSideBytes = 16 * 16 * 4 /* row maxima */ + 16 * 4 /* inverse row scales */ + 128 /* barriers */;
  __host__ __device__ static constexpr int stage_bytes(int K) { return kRows * (K + kRowPad); }
  __host__ __device__ static constexpr int red_bytes(int m_tiles) { return kConsumerWarps * m_tiles * 32 * 4 * 4; }
  __host__ __device__ static constexpr int smem_bytes(int K, int m_tiles) {
    return kStages * stage_bytes(K) + red_bytes(m_tiles) + kSideBytes + 128;
  }
};

__device__ __forceinline__ void bulk_copy_g2s(uint32_t smem_dst, const void* gmem_src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
               "l"(gmem_src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// Four int8 in one word -> two fp16x2 words {w0,w1}, {w2,w3}, exactly.
__device__ __forceinline__ void dequant4_f16(uint32_t packed, uint32_t& lo, uint32_t& hi) {
  const uint32_t biased = packed ^ 0x80808080u;                 // w + 128 as unsigned bytes
  uint32_t p0 = __byte_perm(biased, 0x64646464u, 0x4140);       // {1024 + u0, 1024 + u1}
  uint32_t p1 = __byte_perm(biased, 0x64646464u, 0x4342);       // {1024 + u2, 1024 + u3}
  const uint32_t kBias = 0x64806480u;                           // {1152, 1152}
  asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(p0), "r"(kBias));
  asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(p1), "r"(kBias));
}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// kMTiles: 1 (M <= 8) or 2 (M <= 16).  kChunks: k-chunks per warp, 1 (K <= 2048) or 2 (K <= 4096).
template <int kMTiles, int kChunks, typename OutT>
__global__ void __launch_bounds__(W8Stream::kThreads, 1)
w8_stream_kernel(const __nv_bfloat16* __restrict__ a, long long lda, const int8_t* __restrict__ w, long long ldw,
                 const float* __restrict__ scale, OutT* __restrict__ c, long long ldc, int M, int N, int K, EpilogueArgs ep,
                 uint32_t* __restrict__ status) {
  using G = W8Stream;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 127u) & ~127u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int pitch = K + G::kRowPad;
  const int stage_bytes = G::kRows * pitch;
  const int side_offset = G::kStages * stage_bytes + G::red_bytes(kMTiles);
  float* red = reinterpret_cast<float*>(smem_gen + G::kStages * stage_bytes);
  uint32_t* row_max = reinterpret_cast<uint32_t*>(smem_gen + side_offset);          // [16 warps][16 rows]
  float* inv_row_scale = reinterpret_cast<float*>(smem_gen + side_offset + 1024);   // [16 rows]
  uint8_t* bar_gen = smem_gen + side_offset + 1024 + 64;
  const uint32_t bar_base = smem_base + side_offset + 1024 + 64;
  const uint32_t full_bar = bar_base;                       // W stage landed            (producer -> consumers)
  const uint32_t empty_bar = bar_base + 8 * G::kStages;     // W stage consumed          (consumers -> producer)
  const uint32_t red_full_bar = bar_base + 16 * G::kStages; // all partial sums written  (consumers -> summing warps)
  const uint32_t red_free_bar = red_full_bar + 8;           // partial sums consumed     (summing warps -> consumers)
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bar_gen + 16 * G::kStages + 16);
  constexpr int kSumWarps = 4 * kMTiles;                    // 128 sums per m-tile, one per thread

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_items = (N + G::kRows - 1) / G::kRows;

  if (threadIdx.x == 0) {
    for (int s = 0; s < G::kStages; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, G::kConsumerWarps);
    }
    mbar_init(red_full_bar, G::kConsumerWarps);
    mbar_init(red_free_bar, kSumWarps);
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == G::kConsumerWarps) {
    // ---------------------------------------------------------------- producer warp
    int stage = 0;
    uint32_t phase = 0;
    for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
      if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag)) {
        if (lane == 0) {
          report_status(status, kStatusW8Wait);
          *abort_flag = 1;
        }
        break;
      }
      const int row0 = item * G::kRows;
      const int rows = min(G::kRows, N - row0);
      if (lane == 0) mbar_arrive_expect_tx(full_bar + 8 * stage, static_cast<uint32_t>(rows) * K);
      __syncwarp();
      if (lane < rows)
        bulk_copy_g2s(smem_base + stage * stage_bytes + lane * pitch, w + static_cast<long long>(row0 + lane) * ldw,
                      static_cast<uint32_t>(K), full_bar + 8 * stage);
      if (++stage == G::kStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
  } else {
    // ---------------------------------------------------------------- consumer warps
    const int g = lane >> 2;
    const int t = lane & 3;

    // Activation fragments of this warp's k-chunks: bf16 from global, kept in registers as fp16.
    uint4 act[kMTiles][kChunks][4];
    uint32_t local_max[kMTiles];
#pragma unroll
    for (int j = 0; j < kMTiles; ++j) {
      local_max[j] = 0;
      const int m = 8 * j + g;
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch) {
        const int k0 = (warp + G::kConsumerWarps * ch) * G::kChunkK;
        const bool valid = m < M && k0 < K;
        const __nv_bfloat16* src = a + static_cast<long long>(valid ? m : 0) * lda + (valid ? k0 : 0) + 16 * t;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          // q = 0,1: k0 + 16t + [0,16);  q = 2,3: k0 + 64 + 16t + [0,16)   (8 bf16 per 16-byte load)
          const uint4 v = valid ? __ldg(reinterpret_cast<const uint4*>(src + (q >> 1) * 64) + (q & 1)) : make_uint4(0, 0, 0, 0);
          act[j][ch][q] = v;
          const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            local_max[j] = max(local_max[j], words[i] & 0x7fffu);
            local_max[j] = max(local_max[j], (words[i] >> 16) & 0x7fffu);
          }
        }
      }
      // the four threads of a quad hold the same row
      local_max[j] = max(local_max[j], __shfl_xor_sync(0xffffffffu, local_max[j], 1));
      local_max[j] = max(local_max[j], __shfl_xor_sync(0xffffffffu, local_max[j], 2));
      if (t == 0) row_max[warp * 16 + 8 * j + g] = local_max[j];
    }
    if (kMTiles == 1 && t == 0) row_max[warp * 16 + 8 + g] = 0;
    // consumer-only barrier; every consumer warp reaches it exactly once, before any bounded wait
    asm volatile("bar.sync 1, %0;" ::"n"(G::kConsumerWarps * 32) : "memory");

    float row_scale[kMTiles];
#pragma unroll
    for (int j = 0; j < kMTiles; ++j) {
      const int m = 8 * j + g;
      uint32_t biggest = 0;
#pragma unroll
      for (int q = 0; q < G::kConsumerWarps; ++q) biggest = max(biggest, row_max[q * 16 + m]);
      const int exponent = static_cast<int>(biggest >> 7);  // biased exponent of the largest |a| in the row
      int shift = (exponent == 0 || exponent == 255) ? 0 : (127 + 14) - exponent;
      shift = min(shift, 120);
      row_scale[j] = __uint_as_float(static_cast<uint32_t>(shift + 127) << 23);
      if (warp == 0 && t == 0) inv_row_scale[m] = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t words[4] = {act[j][ch][q].x, act[j][ch][q].y, act[j][ch][q].z, act[j][ch][q].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float lo = __uint_as_float(words[i] << 16) * row_scale[j];
            const float hi = __uint_as_float(words[i] & 0xffff0000u) * row_scale[j];
            const __half2 h = __floats2half2_rn(lo, hi);
            words[i] = *reinterpret_cast<const uint32_t*>(&h);
          }
          act[j][ch][q] = make_uint4(words[0], words[1], words[2], words[3]);
        }
    }

    int stage = 0;
    uint32_t phase = 0, red_phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
      float acc[kMTiles][4];
#pragma unroll
      for (int j = 0; j < kMTiles; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

      if (ok && !mbar_wait(full_bar + 8 * stage, phase, abort_flag)) {
        if (lane == 0) {
          report_status(status, kStatusW8Wait);
          *abort_flag = 1;
        }
        ok = false;
      }
      if (!ok) break;
      const uint32_t tile = smem_base + stage * stage_bytes;
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch) {
        const int k0 = (warp + G::kConsumerWarps * ch) * G::kChunkK;
        if (k0 < K) {
          const uint32_t lo = tile + g * pitch + k0 + 16 * t;
          const uint32_t hi = lo + 8 * pitch;
          const uint4 wl[2] = {lds128(lo), lds128(lo + 64)};
          const uint4 wh[2] = {lds128(hi), lds128(hi + 64)};
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const uint32_t lw[4] = {wl[half].x, wl[half].y, wl[half].z, wl[half].w};
            const uint32_t hw[4] = {wh[half].x, wh[half].y, wh[half].z, wh[half].w};
#pragma unroll
            for (int s = 0; s < 4; ++s) {
              uint32_t a0, a1, a2, a3;
              dequant4_f16(lw[s], a0, a2);  // row g:   k+0,1 | k+2,3
              dequant4_f16(hw[s], a1, a3);  // row g+8: k+0,1 | k+2,3
#pragma unroll
              for (int j = 0; j < kMTiles; ++j) {
                const uint4 x = act[j][ch][2 * half + (s >> 1)];
                const uint32_t b0 = (s & 1) ? x.z : x.x;
                const uint32_t b1 = (s & 1) ? x.w : x.y;
                mma_f16_16816(acc[j], a0, a1, a2, a3, b0, b1);
              }
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar + 8 * stage);
      if (++stage == G::kStages) {
        stage = 0;
        phase ^= 1u;
      }

      // hand the 16 K-slices of this item to the summing warps
      if (!mbar_wait(red_free_bar, red_phase ^ 1u, abort_flag)) {  // previous item's partials have been read
        if (lane == 0) {
          report_status(status, kStatusW8Wait);
          *abort_flag = 1;
        }
        break;
      }
#pragma unroll
      for (int j = 0; j < kMTiles; ++j)
        *reinterpret_cast<float4*>(&red[((warp * kMTiles + j) * 32 + lane) * 4]) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
      __syncwarp();
      if (lane == 0) mbar_arrive(red_full_bar);
      if (warp < kSumWarps) {
        if (!mbar_wait(red_full_bar, red_phase, abort_flag)) {
          if (lane == 0) {
            report_status(status, kStatusW8Wait);
            *abort_flag = 1;
          }
          break;
        }
        const int tid = threadIdx.x;  // 0 .. 128*kMTiles-1
        const int j = tid >> 7;
        const int slot = tid & 127;  // = lane * 4 + e of the fragment
        float sum = 0.f;
#pragma unroll
        for (int q = 0; q < G::kConsumerWarps; ++q) sum += red[(q * kMTiles + j) * 128 + slot];
        __syncwarp();
        if (lane == 0) mbar_arrive(red_free_bar);
        const int fl = slot >> 2, e = slot & 3;
        const int fg = fl >> 2, ft = fl & 3;
        const int m = 8 * j + 2 * ft + (e & 1);
        const int n = item * G::kRows + fg + ((e & 2) ? 8 : 0);
        if (m < M && n < N) {
          const float factor = scale != nullptr ? __ldg(scale + n) : 1.f;
          // (the fused form's accumulator input joins the sum once the power of two of the row is divided out)
          const float v = ep.active ? epilogue_float(sum * inv_row_scale[m], ep, m, n, factor) : sum * inv_row_scale[m] * factor;
          if constexpr (sizeof(OutT) == 2) c[static_cast<long long>(m) * ldc + n] = __float2bfloat16_rn(v);
          else c[static_cast<long long>(m) * ldc + n] = v;
        }
      }
      red_phase ^= 1u;
    }
  }

  __syncthreads();
  if (*abort_flag != 0) {
    // a wait ran out: let bulk copies still in flight land before shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
}

}  // namespace vb200
