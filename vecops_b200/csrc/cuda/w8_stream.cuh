// Weight-only int8 dequant-GEMM for decode shapes, streaming form (M <= 16,
// K <= 4096, K % 128 == 0):
//     C[m,n] = convert( (sum_k f32(A[m,k]) * f32(W[n,k])) * scale[n] )
//
// How the bytes move:
//   * one persistent CTA per SM owns a contiguous range of W's rows, N / gridDim of them to within one row, so every
//     SM streams the same number of bytes; it walks the range in items of 16 rows (up to 8 activation rows) or 8 rows
//     (9 to 16 activation rows), K bytes per row, rows contiguous;
//   * a producer warp streams items into a shared-memory ring with cp.async.bulk (one bulk copy per row, completion
//     counted in bytes on an mbarrier): three 16-row or six 8-row stages at K = 4096, ~195 KB per SM in flight
//     without holding registers;
//   * 16 consumer warps split K: warp w owns the 128-wide k-chunks w, w+16.  Its activation fragments for those
//     chunks are loaded ONCE into registers at kernel start and reused for every item, so the inner loop touches
//     shared memory only for weights.  Up to 8 activation rows the weights are the A operand of mma.m16n8k16 (sixteen
//     rows of W = the m of the instruction) and the activations its B operand; from 9 to 16 activation rows the
//     weights are its B operand (eight rows of W = its n) and the activations its A operand;
//   * per item each consumer warp leaves its 16 x 8 partial fragment in a ring of two reduction buffers and goes
//     on to the next item; a summing warp of its own adds the sixteen fragments in fixed warp order (deterministic),
//     scales, converts and stores.  A consumer waits for a sum only when it is two items ahead of the summing warp.
// The kernel is launched as a programmatic dependent: its set-up runs while the previous kernel of the stream drains.
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
  static constexpr int kThreads = 32 * (kConsumerWarps + 2);  // + the producer warp and the summing warp
  // Weight rows per item.  Up to 8 activation rows the weights are the m16 operand of mma.m16n8k16 (16 rows of W per
  // instruction, the activations its n8): half as many instructions per byte of W as the other way round, and
  // mma.sync is slow enough on this part (one per ~30 cycles per scheduler) to be what bounds the kernel otherwise.
  // From 9 to 16 activation rows they are its n8 operand (8 rows of W, the activations its m16).
  __host__ __device__ static constexpr int rows(bool rows16) { return rows16 ? 8 : 16; }
  static constexpr int kChunkK = 128;
  static constexpr int kMaxK = 4096;
  static constexpr int kRowPad = 64;
  static constexpr int kMaxStages = 8;
  static constexpr int kRedStages = 2;
  static constexpr int kRedBytes = kConsumerWarps * 32 * 16;  // 8 KB: one 16 x 8 fp32 fragment (four floats per lane) per consumer warp
  static constexpr int kSideBytes = 16 * 16 * 4 /* row maxima */ + 16 * 4 /* inverse row scales */ + 320 /* barriers */;
  __host__ __device__ static constexpr int stage_bytes(int K, bool rows16) { return rows(rows16) * (K + kRowPad); }
  __host__ __device__ static constexpr int stages(int K, bool rows16) {
    const int fit = (227 * 1024 - 256 - kRedStages * kRedBytes - kSideBytes) / stage_bytes(K, rows16);
    return fit < kMaxStages ? fit : kMaxStages;
  }
  __host__ __device__ static constexpr int smem_bytes(int K, bool rows16) {
    return stages(K, rows16) * stage_bytes(K, rows16) + kRedStages * kRedBytes + kSideBytes + 128;
  }
};
static_assert(W8Stream::stages(W8Stream::kMaxK, false) >= 3 && W8Stream::stages(W8Stream::kMaxK, true) >= 3, "the weight ring must hold enough bytes in flight");

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

// kChunks: k-chunks per warp, 1 (K <= 2048) or 2 (K <= 4096).  kRows16: activation rows 8..15 exist (M > 8).
template <int kChunks, bool kRows16, typename OutT>
__global__ void __launch_bounds__(W8Stream::kThreads, 1)
w8_stream_kernel(const __nv_bfloat16* __restrict__ a, long long lda, const int8_t* __restrict__ w, long long ldw,
                 const float* __restrict__ scale, OutT* __restrict__ c, long long ldc, int M, int N, int K, EpilogueArgs ep,
                 uint32_t* __restrict__ status, unsigned long long* __restrict__ trace) {
  using G = W8Stream;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 127u) & ~127u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  constexpr int kRows = G::rows(kRows16);  // weight rows per item
  const int pitch = K + G::kRowPad;
  const int stage_bytes = kRows * pitch;
  const int stages = G::stages(K, kRows16);
  const int red_offset = stages * stage_bytes;
  const int side_offset = red_offset + G::kRedStages * G::kRedBytes;
  uint32_t* row_max = reinterpret_cast<uint32_t*>(smem_gen + side_offset);          // [16 warps][16 rows]
  float* inv_row_scale = reinterpret_cast<float*>(smem_gen + side_offset + 1024);   // [16 rows]
  uint8_t* bar_gen = smem_gen + side_offset + 1024 + 64;
  const uint32_t bar_base = smem_base + side_offset + 1024 + 64;
  const uint32_t full_bar = bar_base;                                // W stage landed                (producer -> consumers)
  const uint32_t empty_bar = full_bar + 8 * G::kMaxStages;           // W stage consumed              (consumers -> producer)
  const uint32_t red_full_bar = empty_bar + 8 * G::kMaxStages;       // all partial fragments written (consumers -> summing warp)
  const uint32_t red_free_bar = red_full_bar + 8 * G::kRedStages;    // partial fragments summed      (summing warp -> consumers)
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bar_gen + 16 * G::kMaxStages + 16 * G::kRedStages);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // optional timeline for tuning: 16 slots per CTA (nanosecond stamps and per-role wait cycles), written only when a trace buffer is given
  auto stamp = [&](int slot) {
    if (trace != nullptr) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      trace[blockIdx.x * 16 + slot] = now;
    }
  };
  if (threadIdx.x == 0) stamp(0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < G::kMaxStages; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, G::kConsumerWarps);
    }
    for (int r = 0; r < G::kRedStages; ++r) {
      mbar_init(red_full_bar + 8 * r, G::kConsumerWarps);
      mbar_init(red_free_bar + 8 * r, 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  // this CTA's rows of W: an equal share to within one row
  const int row_begin = static_cast<int>(static_cast<long long>(N) * blockIdx.x / gridDim.x);
  const int row_end = static_cast<int>(static_cast<long long>(N) * (blockIdx.x + 1) / gridDim.x);
  const int num_items = (row_end - row_begin + kRows - 1) / kRows;
  // Everything above touched only this CTA's shared memory and may run while the previous kernel of the stream drains;
  // everything below reads or writes global memory and waits for it.  One thing is done before the wait: the rows that
  // will fill the ring first are asked into L2.  That is a hint, not a read - nothing is consumed, and should the
  // previous kernel still be writing those rows the copies below, issued after the wait, see its data - but HBM is idle
  // while the previous kernel drains its last stages, and the first copies of this one then find their bytes in L2.
  grid_launch_dependents();
  if (warp == G::kConsumerWarps) {
    for (int item = 0; item < stages && item < num_items; ++item) {
      const int row = row_begin + item * kRows + lane;
      if (lane < kRows && row < row_end) prefetch_l2_bulk(w + static_cast<long long>(row) * ldw, static_cast<uint32_t>(K));
    }
  }
  grid_dependency_wait();

  auto give_up = [&]() {
    if (lane == 0) {
      report_status(status, kStatusW8Wait);
      *abort_flag = 1;
    }
  };

  if (warp == G::kConsumerWarps) {
    // ---------------------------------------------------------------- producer warp
    int stage = 0;
    uint32_t phase = 0;
    long long waited = 0;
    if (lane == 0) stamp(1);
    for (int item = 0; item < num_items; ++item) {
      const long long t0 = trace != nullptr ? clock64() : 0;
      if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag)) {
        give_up();
        break;
      }
      if (trace != nullptr) waited += clock64() - t0;
      const int row0 = row_begin + item * kRows;
      const int rows = min(kRows, row_end - row0);
      if (lane == 0) mbar_arrive_expect_tx(full_bar + 8 * stage, static_cast<uint32_t>(rows) * K);
      __syncwarp();
      if (lane < rows)
        bulk_copy_g2s(smem_base + stage * stage_bytes + lane * pitch, w + static_cast<long long>(row0 + lane) * ldw,
                      static_cast<uint32_t>(K), full_bar + 8 * stage);
      if (++stage == stages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    if (lane == 0 && trace != nullptr) {
      trace[blockIdx.x * 16 + 8] = static_cast<unsigned long long>(waited);
      stamp(2);
    }
  } else if (warp == G::kConsumerWarps + 1) {
    // ---------------------------------------------------------------- summing warp
    // lane l holds, like every consumer lane, the fragment entries (m = g, n = 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)
    const int g = lane >> 2, t = lane & 3;
    long long waited = 0;
    for (int item = 0; item < num_items; ++item) {
      const int rb = item % G::kRedStages;
      const long long t0 = trace != nullptr ? clock64() : 0;
      if (!mbar_wait(red_full_bar + 8 * rb, static_cast<uint32_t>(item / G::kRedStages) & 1u, abort_flag)) {
        give_up();
        break;
      }
      if (trace != nullptr) waited += clock64() - t0;
      if (item == 0 && lane == 0) stamp(6);
      const uint32_t red = smem_base + red_offset + rb * G::kRedBytes + lane * 16;
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int q = 0; q < G::kConsumerWarps; ++q) {
        const uint4 v = lds128(red + q * 512);
        sum.x += __uint_as_float(v.x);
        sum.y += __uint_as_float(v.y);
        sum.z += __uint_as_float(v.z);
        sum.w += __uint_as_float(v.w);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(red_free_bar + 8 * rb);
      // fragment entries of this lane: (i = g, j = 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1), where the 16-row index i is the
      // activation row m and the 8-column index j the weight row when the activations are the m16 operand (kRows16),
      // and the other way round when the weights are
      const float sums[2][2] = {{sum.x, sum.y}, {sum.z, sum.w}};
      const int item_row0 = row_begin + item * kRows;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float out[2];
        bool valid[2];
        int ms[2], ns[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          ms[i] = kRows16 ? g + 8 * half : 2 * t + i;
          ns[i] = kRows16 ? item_row0 + 2 * t + i : item_row0 + g + 8 * half;
          valid[i] = ms[i] < M && ns[i] < row_end;
          const float factor = (valid[i] && scale != nullptr) ? __ldg(scale + ns[i]) : 1.f;
          // (the fused form's accumulator input joins the sum once the power of two of the row is divided out)
          const float base = sums[half][i] * inv_row_scale[ms[i] & 15];
          out[i] = !valid[i] ? 0.f : ep.active ? epilogue_float(base, ep, ms[i], ns[i], factor) : base * factor;
        }
        if constexpr (kRows16) {
          // two neighbouring columns of one output row
          OutT* dst = c + static_cast<long long>(ms[0]) * ldc + ns[0];
          if constexpr (sizeof(OutT) == 2) {
            if (valid[0] && valid[1] && (reinterpret_cast<uintptr_t>(dst) & 3u) == 0) {
              *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(out[0], out[1]);
              continue;
            }
          }
          if (valid[0]) dst[0] = static_cast<OutT>(out[0]);
          if (valid[1]) dst[1] = static_cast<OutT>(out[1]);
        } else {
          // one column of two neighbouring output rows
#pragma unroll
          for (int i = 0; i < 2; ++i)
            if (valid[i]) c[static_cast<long long>(ms[i]) * ldc + ns[i]] = static_cast<OutT>(out[i]);
        }
      }
    }
    if (lane == 0 && trace != nullptr) {
      trace[blockIdx.x * 16 + 9] = static_cast<unsigned long long>(waited);
      stamp(7);
    }
  } else {
    // ---------------------------------------------------------------- consumer warps
    const int g = lane >> 2;
    const int t = lane & 3;
    constexpr int kRowHalves = kRows16 ? 2 : 1;

    // Activation fragments of this warp's k-chunks: bf16 from global, kept in registers as fp16.  For the 64 k of
    // group gq of chunk ch, this lane holds A[g + 8*rh][k0 + 64*gq + 16*t + 0..15] as two 16-byte halves.
    uint4 act[kChunks][2][kRowHalves][2];
    uint32_t local_max[kRowHalves];
#pragma unroll
    for (int rh = 0; rh < kRowHalves; ++rh) {
      local_max[rh] = 0;
      const int m = g + 8 * rh;
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch) {
        const int k0 = (warp + G::kConsumerWarps * ch) * G::kChunkK;
        const bool valid = m < M && k0 < K;
        const __nv_bfloat16* src = a + static_cast<long long>(valid ? m : 0) * lda + (valid ? k0 : 0) + 16 * t;
#pragma unroll
        for (int gq = 0; gq < 2; ++gq)
#pragma unroll
          for (int hv = 0; hv < 2; ++hv) {
            const uint4 v = valid ? __ldg(reinterpret_cast<const uint4*>(src + 64 * gq) + hv) : make_uint4(0, 0, 0, 0);
            act[ch][gq][rh][hv] = v;
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              local_max[rh] = max(local_max[rh], words[i] & 0x7fffu);
              local_max[rh] = max(local_max[rh], (words[i] >> 16) & 0x7fffu);
            }
          }
      }
      // the four threads of a quad hold the same row
      local_max[rh] = max(local_max[rh], __shfl_xor_sync(0xffffffffu, local_max[rh], 1));
      local_max[rh] = max(local_max[rh], __shfl_xor_sync(0xffffffffu, local_max[rh], 2));
      if (t == 0) row_max[warp * 16 + 8 * rh + g] = local_max[rh];
    }
    if (!kRows16 && t == 0) row_max[warp * 16 + 8 + g] = 0;
    // consumer-only barrier; every consumer warp reaches it exactly once, before any bounded wait
    asm volatile("bar.sync 1, %0;" ::"n"(G::kConsumerWarps * 32) : "memory");

#pragma unroll
    for (int rh = 0; rh < kRowHalves; ++rh) {
      const int m = g + 8 * rh;
      uint32_t biggest = 0;
#pragma unroll
      for (int q = 0; q < G::kConsumerWarps; ++q) biggest = max(biggest, row_max[q * 16 + m]);
      const int exponent = static_cast<int>(biggest >> 7);  // biased exponent of the largest |a| in the row
      int shift = (exponent == 0 || exponent == 255) ? 0 : (127 + 14) - exponent;
      shift = min(shift, 120);
      const float row_scale = __uint_as_float(static_cast<uint32_t>(shift + 127) << 23);
      if (warp == 0 && t == 0) inv_row_scale[m] = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch)
#pragma unroll
        for (int gq = 0; gq < 2; ++gq)
#pragma unroll
          for (int hv = 0; hv < 2; ++hv) {
            uint4& v = act[ch][gq][rh][hv];
            uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float lo = __uint_as_float(words[i] << 16) * row_scale;
              const float hi = __uint_as_float(words[i] & 0xffff0000u) * row_scale;
              const __half2 h = __floats2half2_rn(lo, hi);
              words[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
            v = make_uint4(words[0], words[1], words[2], words[3]);
          }
    }
    if (!kRows16 && warp == 0 && t == 0) inv_row_scale[8 + g] = 1.f;

    int stage = 0;
    uint32_t phase = 0;
    const bool tracing = trace != nullptr && warp == 0 && lane == 0;
    long long waited_full = 0, waited_red = 0;
    if (tracing) stamp(3);  // activations in registers
    const long long loop_start = tracing ? clock64() : 0;
    for (int item = 0; item < num_items; ++item) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const long long t0 = tracing ? clock64() : 0;
      if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag)) {
        give_up();
        break;
      }
      if (tracing) {
        waited_full += clock64() - t0;
        if (item == 0) stamp(4);  // first stage landed
      }
      const uint32_t tile = smem_base + stage * stage_bytes + g * pitch + 16 * t;  // this lane's weight row g (and g + 8 when the weights are the m16 operand)
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch) {
        const int k0 = (warp + G::kConsumerWarps * ch) * G::kChunkK;
        if (k0 < K) {
          // One instruction per word of a 16-byte load: its four weights are the k pairs (2t, 2t+1) and (2t+8, 2t+9) of
          // the fragment, and the activations of the same four k are taken for the other operand - any pairing of k
          // works as long as both operands use it.
          if constexpr (kRows16) {
            const uint4 wv[2] = {lds128(tile + k0), lds128(tile + k0 + 64)};
#pragma unroll
            for (int gq = 0; gq < 2; ++gq) {
              const uint32_t words[4] = {wv[gq].x, wv[gq].y, wv[gq].z, wv[gq].w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t b0, b1;
                dequant4_f16(words[j], b0, b1);
                const uint4 x0 = act[ch][gq][0][j >> 1], x1 = act[ch][gq][kRowHalves - 1][j >> 1];
                mma_f16_16816(acc, (j & 1) ? x0.z : x0.x, (j & 1) ? x1.z : x1.x, (j & 1) ? x0.w : x0.y, (j & 1) ? x1.w : x1.y, b0, b1);
              }
            }
          } else {
            const uint4 wl[2] = {lds128(tile + k0), lds128(tile + k0 + 64)};
            const uint4 wh[2] = {lds128(tile + 8 * pitch + k0), lds128(tile + 8 * pitch + k0 + 64)};
#pragma unroll
            for (int gq = 0; gq < 2; ++gq) {
              const uint32_t lw[4] = {wl[gq].x, wl[gq].y, wl[gq].z, wl[gq].w};
              const uint32_t hw[4] = {wh[gq].x, wh[gq].y, wh[gq].z, wh[gq].w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t a0, a1, a2, a3;
                dequant4_f16(lw[j], a0, a2);  // weight row g
                dequant4_f16(hw[j], a1, a3);  // weight row g + 8
                const uint4 x = act[ch][gq][0][j >> 1];  // activation row g: the n of the fragment
                mma_f16_16816(acc, a0, a1, a2, a3, (j & 1) ? x.z : x.x, (j & 1) ? x.w : x.y);
              }
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar + 8 * stage);
      if (++stage == stages) {
        stage = 0;
        phase ^= 1u;
      }
      // leave the fragment for the summing warp and go on
      const int rb = item % G::kRedStages;
      const long long t1 = tracing ? clock64() : 0;
      if (!mbar_wait(red_free_bar + 8 * rb, (static_cast<uint32_t>(item / G::kRedStages) & 1u) ^ 1u, abort_flag)) {
        give_up();
        break;
      }
      if (tracing) waited_red += clock64() - t1;
      const uint32_t red = smem_base + red_offset + rb * G::kRedBytes + (warp * 32 + lane) * 16;
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(red), "f"(acc[0]), "f"(acc[1]), "f"(acc[2]), "f"(acc[3]) : "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(red_full_bar + 8 * rb);
    }
    if (tracing) {
      trace[blockIdx.x * 16 + 10] = static_cast<unsigned long long>(waited_full);
      trace[blockIdx.x * 16 + 11] = static_cast<unsigned long long>(waited_red);
      trace[blockIdx.x * 16 + 12] = static_cast<unsigned long long>(clock64() - loop_start);
      stamp(5);
    }
  }

  __syncthreads();
  if (threadIdx.x == 0) stamp(15);
  if (*abort_flag != 0) {
    // a wait ran out: let bulk copies still in flight land before shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
}

}  // namespace vb200
