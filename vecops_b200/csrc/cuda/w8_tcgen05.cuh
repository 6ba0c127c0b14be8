// Weight-only int8 dequant-GEMM on the 5th-generation tensor cores (M <= 128):
//     C[m,n] = convert( (sum_k f32(A[m,k]) * f32(W[n,k])) * scale[n] )
// A bf16 [M,K], W int8 [N,K] K-contiguous, scale f32 [N], C bf16 or f32 [M,N].
//
// The product is computed transposed, D[n,m] = W[n,:] . A[m,:], so that the
// 128 rows of a weight tile fill the tensor core's M dimension and the few
// activation rows are its N dimension (vecops' SwapAB idea, ops/Matmul.h:76-83):
//   * A-operand: the weight tile, widened int8 -> bf16 (exact: |w| <= 128 needs 8 significant bits) by sixteen
//     CUDA-core warps and written with tcgen05.st straight into TENSOR MEMORY - the widened weights never touch
//     shared memory;
//   * B-operand: the activation tile, bf16 exactly as the caller stores it, TMA-loaded with the 128-byte swizzle
//     (rows past M are zero-filled by TMA);
//   * tcgen05.mma kind::f16 with A = bf16 from TMEM and B = bf16 from shared memory, fp32 accumulators in TMEM.
//     Every product is exact in fp32, as with the reference's AMX tdpbf16ps on a bf16-converted weight.
//   An older operand form remains selectable (and is what the static-scratch entry point uses): weights widened to
//   fp16 (one instruction less per weight) against an fp16 copy of the activations that w8_prepare_activations_kernel
//   makes once per launch - each bf16 row multiplied by the power of two that brings its largest magnitude to 2^14,
//   exact for every element within 2^31 of the row maximum, the power of two divided out of the accumulator.  It
//   costs a second launch, which is why it is no longer the default.  (Mixed formats, A = f16 with B = bf16, are
//   not an option: that instruction descriptor raises an illegal-instruction error on this part.)
//
// Work is cut stream-K style: the (128-row tile) x (128-wide k-block) units are
// laid out tile-major and each of the <= 148 persistent CTAs takes an equal
// contiguous range, so HBM traffic is balanced to one unit.  A CTA whose range
// STARTS inside a tile writes that tile's fp32 partial sums to DEVICE SCRATCH
// (caller-provided workspace) right after its first segment - early in its
// life - and raises a flag; the CTA whose range holds the tile's first k-block
// reaches the tile last, adds the partials in fixed order, applies the column
// scale once, converts and stores (vecops' split-K rule: the output transform
// runs once, at the end, kernel/AccumulatorRoute.h:22-56).  Flags carry a
// 64-bit nonce and count their readers down to it, so the scratch needs no
// clearing between launches and a captured launch can be replayed.  Waits on
// flags are bounded.
//
// Warps: 0 TMA producer | 1 MMA issuer + TMEM owner | 4-7 epilogue | 8-23 widening (two groups, alternate units).
//
// CTA pairs (kPair): the thread that issues tcgen05 work, not HBM, sets the pace of the single-CTA form (about 70
// cycles per MMA, eight MMAs per 16 KB of weights).  Two CTAs of a cluster therefore share 256-row weight tiles: each
// streams and widens its own 128 rows into its own TMEM and holds half of the activation rows in shared memory, and
// the leader issues ONE tcgen05.mma.cta_group::2 (M = 256) where the single form needs two - half the issue work per
// byte of weights.  Barriers follow the dense GEMM's pair form: both CTAs' activation loads count on the leader's
// `act_full`, both CTAs' widening warps arrive on the leader's `a_full`, the leader's commits arrive on `a_empty`,
// `act_empty` and `d_full` of both CTAs, both epilogues arrive on the leader's `d_empty`.  Stream-K ranges are per
// pair; each CTA exchanges partial sums with the CTA of the same rank in the neighbouring pairs.
//
// Algorithmic traffic per launch: N*K + 4*N + 2*M*K + sizeof(C)*M*N bytes.
#pragma once

#include "gemm_tcgen05.cuh"
#include "ptx.cuh"
#include "w8_stream.cuh"  // dequant4_f16, lds128

namespace vb200 {

struct W8Tc {
  static constexpr int kTileN = 128;        // weight rows per tile (UMMA M)
  static constexpr int kBlockK = 128;       // k per unit
  static constexpr int kMaxM = 128;         // activation rows (UMMA N, padded to 16)
  static constexpr int kRawBatch = 4;       // weight tiles requested together: 512 contiguous bytes per row, kind to DRAM pages
  static constexpr int kRawStages = 8;      // int8 weight tiles in flight (two batches)
  static constexpr int kRawBytes = kTileN * kBlockK;
  static constexpr int kMaxActStages = 6;
  static constexpr int kMaxAStages = 6;     // widened weight tiles in TMEM (as many as the accumulators leave room for)
  static constexpr int kAColumns = kBlockK / 2;  // two fp16 per 32-bit TMEM column
  // TMEM: two accumulators of d_columns each, then the ring of widened weight tiles
  __host__ __device__ static constexpr int d_columns(int mpad) { return mpad <= 32 ? 32 : mpad <= 64 ? 64 : 128; }
  __host__ __device__ static constexpr int a_stages(int mpad) {
    const int fit = (512 - 2 * d_columns(mpad)) / (kBlockK / 2);
    return fit < kMaxAStages ? fit : kMaxAStages;
  }
  // k-blocks per activation stage: few activation rows make small k-blocks, and one barrier round trip per
  // k-block costs the MMA thread more than the MMAs themselves
  __host__ __device__ static constexpr int act_kblocks(int mpad) { return mpad <= 16 ? 4 : mpad <= 32 ? 2 : 1; }
  static constexpr int kTmemColumns = 512;  // D0 | D1 | A ring
  static constexpr int kDequantWarps = 8;    // per group: 4 lane quarters x 2 k-halves of one unit
  static constexpr int kDequantGroups = 2;   // groups take alternate units: widening one unit has a long latency
  static constexpr int kThreads = 32 * (8 + kDequantWarps * kDequantGroups);
  static constexpr int kTailParts = 1 + 2 * kDequantGroups;  // warps per lane quarter that share a final combine
  static constexpr int kMaxGrid = 160;      // scratch is sized for this many CTAs
  __host__ __device__ static constexpr int m_padded(int m) { return (m + 15) & ~15; }
  __host__ __device__ static constexpr int act_stage_bytes(int mpad) { return act_kblocks(mpad) * 2 * mpad * 128; }
  // as many activation stages as fit beside the weight ring (32 KB each at M = 128, 4 KB at M <= 16)
  __host__ __device__ static constexpr int act_stages(int mpad) {
    const int fit = (200 * 1024 - kRawStages * kRawBytes) / act_stage_bytes(mpad);
    return fit < kMaxActStages ? fit : kMaxActStages;
  }
  __host__ __device__ static constexpr int smem_bytes(int mpad) {
    return kRawStages * kRawBytes + act_stages(mpad) * act_stage_bytes(mpad) + 512 + kMaxM * 4 + 1024;
  }
  // scratch: per CTA one [mpad][128] fp32 partial tile | four 64-bit flags per CTA (one per 32-row quarter) |
  //          128 inverse row scales (f32) | the fp16 activations [M][k_pitch]
  __host__ __device__ static constexpr unsigned long long partial_bytes(int mpad) { return 4ull * mpad * kTileN; }
  __host__ __device__ static constexpr unsigned long long flags_offset(int mpad) { return kMaxGrid * partial_bytes(mpad); }
  __host__ __device__ static constexpr unsigned long long scales_offset(int mpad) { return flags_offset(mpad) + kMaxGrid * 4 * 8ull; }
  __host__ __device__ static constexpr unsigned long long act_offset(int mpad) { return scales_offset(mpad) + kMaxM * 4ull; }
  __host__ __device__ static constexpr long long act_pitch(long long k) { return (k + 7) & ~7ll; }  // elements; 16-byte rows for TMA
  __host__ __device__ static constexpr unsigned long long scratch_bytes(int m, long long k) {
    return act_offset(m_padded(m)) + 2ull * m * act_pitch(k);
  }
};

// D[tmem] (+)= A[tmem] . B[smem]
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same for a CTA pair: each CTA's 128 rows of A come from its own TMEM, each holds half of B's rows.
__device__ __forceinline__ void umma_f16_ts_pair(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void st_release_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Four int8 in one word -> two bf16x2 words {w0,w1}, {w2,w3}, exactly (|w| <= 128 needs 8 significant bits).  0x43xx
// with bit 7 clear is 128 + (x & 127); the same word reduced to 0x4300 | (x & 128) is 128 or 256: their difference is
// the two's-complement value.
__device__ __forceinline__ void dequant4_bf16(uint32_t packed, uint32_t& lo, uint32_t& hi) {
  const uint32_t p0 = __byte_perm(packed, 0x43434343u, 0x4140);
  const uint32_t p1 = __byte_perm(packed, 0x43434343u, 0x4342);
  const uint32_t x0 = p0 & 0xff7fff7fu, c0 = p0 & 0xff80ff80u;
  const uint32_t x1 = p1 & 0xff7fff7fu, c1 = p1 & 0xff80ff80u;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(x0), "r"(c0));
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(x1), "r"(c1));
}

// One CTA per activation row: largest |a|, power-of-two scale, fp16 copy, inverse scale.  The row is read once,
// 16 bytes per thread per step with every load issued before the first use, and converted from registers.
// Needs 16-byte aligned rows (lda % 8 == 0, checked by the dispatch rules).
struct W8Prepare {
  static constexpr int kThreads = 512;
  static constexpr int kMaxVectors = 4;  // 16-byte loads per thread: rows up to 512 * 4 * 8 = 16384 elements in one pass
};

// (static: this header is included by more than one translation unit)
static __global__ void __launch_bounds__(W8Prepare::kThreads)
w8_prepare_activations_kernel(const __nv_bfloat16* __restrict__ a, long long lda, __half* __restrict__ out, long long pitch,
                              float* __restrict__ inv_scale, int K) {
  using P = W8Prepare;
  __shared__ uint32_t warp_max[P::kThreads / 32];
  __shared__ float row_scale;
  const int m = blockIdx.x;
  const uint4* row = reinterpret_cast<const uint4*>(a + static_cast<long long>(m) * lda);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(m) * pitch);
  const int vectors = static_cast<int>(pitch / 8);  // pitch is K rounded up to 8 elements
  uint32_t biggest = 0;
  for (int base = 0; base < vectors; base += P::kThreads * P::kMaxVectors) {
    uint4 v[P::kMaxVectors];
#pragma unroll
    for (int i = 0; i < P::kMaxVectors; ++i) {
      const int index = base + i * P::kThreads + threadIdx.x;
      v[i] = index < vectors ? __ldg(row + index) : make_uint4(0, 0, 0, 0);
      // elements past K inside the last vector belong to the caller's row padding: mask them out
      if (index < vectors && index * 8 + 8 > K) {
        uint32_t* words = reinterpret_cast<uint32_t*>(&v[i]);
        for (int e = 0; e < 8; ++e)
          if (index * 8 + e >= K) words[e >> 1] &= (e & 1) ? 0x0000ffffu : 0xffff0000u;
      }
      const uint32_t words[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) biggest = max(biggest, max(words[j] & 0x7fffu, (words[j] >> 16) & 0x7fffu));
    }
    if (vectors > P::kThreads * P::kMaxVectors) {
      // longer rows: this pass only gathers the maximum; the conversion below re-reads
      continue;
    }
    for (int offset = 16; offset > 0; offset >>= 1) biggest = max(biggest, __shfl_xor_sync(0xffffffffu, biggest, offset));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = biggest;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 1; i < P::kThreads / 32; ++i) biggest = max(biggest, warp_max[i]);
      const int exponent = static_cast<int>(biggest >> 7);  // biased exponent of the row's largest magnitude
      int shift = (exponent == 0 || exponent == 255) ? 0 : (127 + 14) - exponent;
      shift = min(shift, 120);
      row_scale = __uint_as_float(static_cast<uint32_t>(shift + 127) << 23);
      inv_scale[m] = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
    }
    __syncthreads();
    const float scale = row_scale;
#pragma unroll
    for (int i = 0; i < P::kMaxVectors; ++i) {
      const int index = i * P::kThreads + threadIdx.x;
      if (index >= vectors) continue;
      uint32_t words[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2 h = __floats2half2_rn(__uint_as_float(words[j] << 16) * scale, __uint_as_float(words[j] & 0xffff0000u) * scale);
        words[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
      dst[index] = make_uint4(words[0], words[1], words[2], words[3]);
    }
    return;
  }
  // rows longer than one pass holds in registers: maximum first, then a second sweep
  for (int offset = 16; offset > 0; offset >>= 1) biggest = max(biggest, __shfl_xor_sync(0xffffffffu, biggest, offset));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = biggest;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < P::kThreads / 32; ++i) biggest = max(biggest, warp_max[i]);
    const int exponent = static_cast<int>(biggest >> 7);
    int shift = (exponent == 0 || exponent == 255) ? 0 : (127 + 14) - exponent;
    shift = min(shift, 120);
    row_scale = __uint_as_float(static_cast<uint32_t>(shift + 127) << 23);
    inv_scale[m] = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);
  }
  __syncthreads();
  const float scale = row_scale;
  for (int index = threadIdx.x; index < vectors; index += P::kThreads) {
    const uint4 v = __ldg(row + index);
    uint32_t words[4] = {v.x, v.y, v.z, v.w};
    for (int e = 0; e < 8; ++e)
      if (index * 8 + e >= K) words[e >> 1] &= (e & 1) ? 0x0000ffffu : 0xffff0000u;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 h = __floats2half2_rn(__uint_as_float(words[j] << 16) * scale, __uint_as_float(words[j] & 0xffff0000u) * scale);
      words[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    dst[index] = make_uint4(words[0], words[1], words[2], words[3]);
  }
}

struct W8TcSegment {
  int tile;       // weight tile (128 rows)
  int kb_begin;   // first k-block of this CTA inside the tile
  int kb_end;     // one past the last
  bool owner;     // this CTA processes the tile's first k-block and stores the tile
  bool has_contributors;  // owner, but the tile's later k-blocks belong to the following CTAs' ranges
};

__device__ __forceinline__ long long w8tc_range_begin(long long total_units, int grid, int cta) {
  return total_units * cta / grid;
}

// Segment `index` of CTA `cta` (false when past the end of its range).
__device__ __forceinline__ bool w8tc_segment(long long total_units, int grid, int cta, int kblocks, int index,
                                             W8TcSegment& seg) {
  const long long begin = w8tc_range_begin(total_units, grid, cta);
  const long long end = w8tc_range_begin(total_units, grid, cta + 1);
  long long u = begin;
  for (int i = 0;; ++i) {
    if (u >= end) return false;
    const int tile = static_cast<int>(u / kblocks);
    const long long tile_end = static_cast<long long>(tile + 1) * kblocks;
    const long long stop = tile_end < end ? tile_end : end;
    if (i == index) {
      seg.tile = tile;
      seg.kb_begin = static_cast<int>(u - static_cast<long long>(tile) * kblocks);
      seg.kb_end = static_cast<int>(stop - static_cast<long long>(tile) * kblocks);
      seg.owner = seg.kb_begin == 0;
      seg.has_contributors = seg.owner && stop != tile_end;
      return true;
    }
    u = stop;
  }
}

template <typename OutT, bool kPair>
__global__ void __launch_bounds__(W8Tc::kThreads, 1)
w8_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_a,
                  const float* __restrict__ scale, OutT* __restrict__ c, long long ldc, int M, int N, int K, int mpad,
                  float* __restrict__ partials, unsigned long long* __restrict__ flags,
                  const float* __restrict__ inv_row_scale, unsigned long long nonce, uint32_t idesc, EpilogueArgs ep,
                  uint32_t* __restrict__ status, unsigned long long* __restrict__ trace) {
  using G = W8Tc;
  // Two operand formats, chosen by the launcher through `inv_row_scale`: null = the activations are the caller's bf16
  // rows and the weights are widened to bf16 (exact both ways, no pre-pass); non-null = the activations are the
  // row-scaled fp16 copy w8_prepare_activations_kernel made and the weights are widened to fp16.
  const bool bf16_operands = inv_row_scale == nullptr;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  constexpr int kTileRows = kPair ? 2 * G::kTileN : G::kTileN;  // weight rows a worker (CTA or pair) covers per tile
  const uint32_t pair_rank = kPair ? cluster_cta_rank() : 0u;
  const int act_rows = kPair ? mpad / 2 : mpad;                  // activation rows this CTA keeps in shared memory
  const int act_kb_bytes = 2 * act_rows * 128;                   // one k-block: two 64-wide swizzle atoms
  const int act_kblocks = G::act_kblocks(mpad);                  // k-blocks per activation stage
  const int act_stage = act_kblocks * act_kb_bytes;
  const int act_stages = G::act_stages(mpad);
  const int a_stages = G::a_stages(mpad);
  const int d_columns = G::d_columns(mpad);
  const uint32_t raw_base = smem_base;
  const uint32_t act_base = smem_base + G::kRawStages * G::kRawBytes;
  const int bar_offset = G::kRawStages * G::kRawBytes + act_stages * act_stage;
  uint8_t* bar_gen = smem_gen + bar_offset;
  const uint32_t bar_base = smem_base + bar_offset;
  uint32_t next_bar = bar_base;
  auto take = [&](int count) { const uint32_t at = next_bar; next_bar += 8 * count; return at; };
  const uint32_t raw_full = take(G::kRawStages), raw_empty = take(G::kRawStages);
  const uint32_t act_full = take(G::kMaxActStages), act_empty = take(G::kMaxActStages);
  const uint32_t a_full = take(G::kMaxAStages), a_empty = take(G::kMaxAStages);
  const uint32_t d_full = take(2), d_empty = take(2);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_gen + (next_bar - bar_base));
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bar_gen + (next_bar - bar_base) + 4);
  float* inv_scale_smem = reinterpret_cast<float*>(bar_gen + 512);  // [kMaxM], filled before the first barrier

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kblocks = (K + G::kBlockK - 1) / G::kBlockK;
  const int tiles = (N + kTileRows - 1) / kTileRows;
  const long long total_units = static_cast<long long>(tiles) * kblocks;
  // `cta` of `grid` counts workers (CTAs, or pairs); scratch slots are per CTA
  const int grid = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int cta = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  auto slot_of = [&](int worker) { return kPair ? 2 * worker + static_cast<int>(pair_rank) : worker; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < G::kRawStages; ++s) {
      mbar_init(raw_full + 8 * s, 1);
      // one "batch consumed" barrier per group of kRawBatch stages (only the first of each group is used)
      mbar_init(raw_empty + 8 * s, G::kDequantWarps * G::kRawBatch);
    }
    for (int s = 0; s < G::kMaxActStages; ++s) {
      mbar_init(act_full + 8 * s, 1);
      mbar_init(act_empty + 8 * s, 1);
    }
    for (int s = 0; s < G::kMaxAStages; ++s) {
      mbar_init(a_full + 8 * s, G::kDequantWarps * (kPair ? 2 : 1));  // the leader's collects both CTAs' widening warps
      mbar_init(a_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(d_full + 8 * s, 1);
      mbar_init(d_empty + 8 * s, 4 * (kPair ? 2 : 1));
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_descriptor(&tma_w);
    tma_prefetch_descriptor(&tma_a);
  }
  if (warp == 1) {
    if constexpr (kPair) {
      tmem_alloc_pair(smem_u32(tmem_slot), G::kTmemColumns);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), G::kTmemColumns);
      tmem_relinquish();
    }
  }
  if (warp == 2) {
    for (int m = lane; m < G::kMaxM; m += 32) inv_scale_smem[m] = m >= M ? 0.f : bf16_operands ? 1.f : __ldg(inv_row_scale + m);
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_a_base = tmem_base + 2 * d_columns;

  // optional timeline (nanoseconds) for tuning: 16 slots per CTA, written only when a trace buffer is given
  auto mark = [&](int slot) {
    if (trace != nullptr) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      trace[blockIdx.x * 16 + slot] = now;
    }
  };
  if (threadIdx.x == 0) mark(0);

  auto give_up = [&](uint32_t code) {
    report_status(status, code);
    *abort_flag = 1;
  };

  // Drain (part of) one accumulator: the owner of a tile adds the following CTAs' partial sums and stores C, any
  // other CTA publishes its partial sums.  Column groups of 16 are dealt round-robin to `parts` cooperating warps
  // per lane quarter (`part` = this warp's turn).  Callable by every warp whose id % 4 is its TMEM lane quarter.
  auto finish = [&](const W8TcSegment& seg, int buf, int part, int parts) -> bool {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // weight row inside the tile = TMEM lane
    const int n = seg.tile * kTileRows + static_cast<int>(pair_rank) * G::kTileN + row;
    const float s = (scale != nullptr && n < N) ? __ldg(scale + n) : 1.f;
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * d_columns;
    // contributors: the CTAs after this one whose ranges begin inside this tile (they published early)
    int last_contributor = cta;
    if (seg.has_contributors) {
      const long long tile_end_unit = static_cast<long long>(seg.tile + 1) * kblocks;
      while (last_contributor + 1 < grid && w8tc_range_begin(total_units, grid, last_contributor + 1) < tile_end_unit) ++last_contributor;
      // a warp only needs its own 32 rows of each partner, published by the partner's warp of the same quarter
      for (int other = cta + 1; other <= last_contributor; ++other)
        if (!wait_flag_window_u64(flags + 4 * slot_of(other) + quarter, nonce, G::kTailParts, abort_flag)) return false;
    }
    for (int col0 = 16 * part; col0 < mpad && col0 < M; col0 += 16 * parts) {
      uint32_t v[16];
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
            "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
          : "r"(taddr + col0)
          : "memory");
      if (seg.owner) {
        // one partner per round trip, its sixteen loads issued before the first is consumed
        float acc[16];
        bool first_pass = true;
        for (int other = cta + 1; other <= last_contributor || first_pass; ++other) {
          float part_sum[16];
          const bool has = other <= last_contributor;
          const float* src = partials + static_cast<long long>(slot_of(other)) * mpad * G::kTileN + col0 * G::kTileN + row;
#pragma unroll
          for (int j = 0; j < 16; ++j) part_sum[j] = (has && col0 + j < M) ? __ldcg(src + j * G::kTileN) : 0.f;
          if (first_pass) {
            tmem_load_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = __uint_as_float(v[j]);
            first_pass = false;
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] += part_sum[j];
        }
        if (n < N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = col0 + j;
            if (m < M) {
              const float out = ep.active ? epilogue_float(acc[j] * inv_scale_smem[m], ep, m, n, s) : acc[j] * inv_scale_smem[m] * s;
              if constexpr (sizeof(OutT) == 2) c[static_cast<long long>(m) * ldc + n] = __float2bfloat16_rn(out);
              else c[static_cast<long long>(m) * ldc + n] = out;
            }
          }
        }
      } else {
        tmem_load_wait();
        float* dst = partials + static_cast<long long>(slot_of(cta)) * mpad * G::kTileN + col0 * G::kTileN + row;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (col0 + j < M) __stcg(dst + j * G::kTileN, __uint_as_float(v[j]));
      }
    }
    if (!seg.owner) {
      // kTailParts warps of the owner read this quarter: the flag counts them down (see ptx.cuh), so that a replay of
      // a captured launch, which carries the same nonce, finds the flag unpublished again
      __threadfence();
      __syncwarp();
      if (lane == 0) st_release_u64(flags + 4 * slot_of(cta) + quarter, nonce + G::kTailParts);
    } else if (seg.has_contributors) {
      __syncwarp();
      if (lane == 0)
        for (int other = cta + 1; other <= last_contributor; ++other) flag_reader_done_u64(flags + 4 * slot_of(other) + quarter);
    }
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one thread)
    // Two independent rings: the int8 weight tiles run as far ahead as their ring allows (they are what HBM
    // latency is hidden behind), the activation tiles follow the MMA.  Neither waits for the other.
    if (lane == 0) {
      const long long begin = w8tc_range_begin(total_units, grid, cta);
      const int my_units = static_cast<int>(w8tc_range_begin(total_units, grid, cta + 1) - begin);
      int raw_issued = 0, act_issued = 0, rs = 0, as = 0;
      uint32_t rphase = 0, aphase = 0;
      const long long started = clock64();
      mark(1);
      while (raw_issued < my_units || act_issued < my_units) {
        bool progress = false;
        if (raw_issued < my_units && mbar_test_wait(raw_empty + 8 * rs, rphase ^ 1u)) {
          // a whole batch of consecutive k-blocks at once
          for (int b = 0; b < G::kRawBatch && raw_issued < my_units; ++b, ++raw_issued) {
            const long long u = begin + raw_issued;
            const int tile = static_cast<int>(u / kblocks), kb = static_cast<int>(u % kblocks);
            mbar_arrive_expect_tx(raw_full + 8 * (rs + b), G::kRawBytes);
            tma_load_2d(raw_base + (rs + b) * G::kRawBytes, &tma_w, raw_full + 8 * (rs + b), kb * G::kBlockK,
                        tile * kTileRows + static_cast<int>(pair_rank) * G::kTileN);
          }
          rs += G::kRawBatch;
          if (rs == G::kRawStages) { rs = 0; rphase ^= 1u; }
          progress = true;
        }
        if (act_issued < my_units && mbar_test_wait(act_empty + 8 * as, aphase ^ 1u)) {
          // one stage = the aligned group of act_kblocks k-blocks that holds this unit's; the units of the group
          // that follow in this CTA's range share it
          const int kb = static_cast<int>((begin + act_issued) % kblocks);
          const int first_kb = kb - kb % act_kblocks;
          const uint32_t act_dst = act_base + as * act_stage;
          const int first_row = kPair ? static_cast<int>(pair_rank) * act_rows : 0;
          uint32_t bar = act_full + 8 * as;
          if constexpr (kPair) {
            // each CTA brings its half of the activation rows; the bytes of both are counted on the leader's barrier
            if (pair_rank == 0) mbar_arrive_expect_tx(act_full + 8 * as, 2u * static_cast<uint32_t>(act_stage));
            bar = map_to_cta(bar, 0);
          } else {
            mbar_arrive_expect_tx(act_full + 8 * as, static_cast<uint32_t>(act_stage));
          }
          for (int j = 0; j < act_kblocks; ++j) {
            const uint32_t dst = act_dst + j * act_kb_bytes;
            const int k0 = (first_kb + j) * G::kBlockK;  // past K: zero-filled by TMA
            if constexpr (kPair) {
              tma_load_2d_pair(dst, &tma_a, bar, k0, first_row);
              tma_load_2d_pair(dst + act_rows * 128, &tma_a, bar, k0 + 64, first_row);
            } else {
              tma_load_2d(dst, &tma_a, bar, k0, first_row);
              tma_load_2d(dst + act_rows * 128, &tma_a, bar, k0 + 64, first_row);
            }
          }
          if (++as == act_stages) { as = 0; aphase ^= 1u; }
          // the rest of the group, which ends with the tile at the latest (may run past my_units: the loop ends)
          act_issued += min(act_kblocks - kb % act_kblocks, kblocks - kb);
          progress = true;
        }
        if (!progress && (*abort_flag != 0 || clock64() - started > 4 * kWaitCycleBudget)) {
          give_up(kStatusProducerWait);
          break;
        }
      }
      mark(2);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (one thread; of a pair, the leader's)
    if (lane == 0 && pair_rank == 0) {
      int as = 0, ai = 0;
      uint32_t aphase = 0, iphase = 0;
      uint32_t dphase[2] = {0, 0};
      W8TcSegment seg;
      bool ok = true;
      bool have_act = false;
      const bool tracing = trace != nullptr;
      long long spent[5] = {0, 0, 0, 0, 0};  // tuning aid: cycles waiting for widened weights | for activations | issuing MMAs | committing; units
      const long long loop_start = tracing ? clock64() : 0;
      for (int si = 0; ok && w8tc_segment(total_units, grid, cta, kblocks, si, seg); ++si) {
        const int buf = si & 1;
        if (!(kPair ? mbar_wait_cluster(d_empty + 8 * buf, dphase[buf] ^ 1u, abort_flag)
                    : mbar_wait(d_empty + 8 * buf, dphase[buf] ^ 1u, abort_flag))) {
          give_up(kStatusMmaWaitTmem);
          break;
        }
        tcgen05_fence_after_sync();
        const uint32_t tmem_d = tmem_base + buf * d_columns;
        for (int kb = seg.kb_begin; kb < seg.kb_end; ++kb) {
          const long long t0 = tracing ? clock64() : 0;
          if (!(kPair ? mbar_wait_cluster(a_full + 8 * ai, iphase, abort_flag) : mbar_wait(a_full + 8 * ai, iphase, abort_flag))) {
            give_up(kStatusMmaWaitFull);
            ok = false;
            break;
          }
          const long long t1 = tracing ? clock64() : 0;
          // one activation stage serves an aligned group of k-blocks (or what of it lies in this CTA's range)
          if (!have_act) {
            if (!mbar_wait(act_full + 8 * as, aphase, abort_flag)) {
              give_up(kStatusMmaWaitFull);
              ok = false;
              break;
            }
            have_act = true;
          }
          tcgen05_fence_after_sync();
          const long long t2 = tracing ? clock64() : 0;
          if (si == 0 && kb == seg.kb_begin) mark(3);
          const uint32_t act_src = act_base + as * act_stage + (kb % act_kblocks) * act_kb_bytes;
          const uint64_t b_lo = umma_smem_desc_sw128(act_src);
          const uint64_t b_hi = umma_smem_desc_sw128(act_src + act_rows * 128);
          const uint32_t a_src = tmem_a_base + ai * G::kAColumns;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint64_t b_desc = (i < 4 ? b_lo : b_hi) + 2 * (i & 3);  // +32 bytes along K per MMA
            if constexpr (kPair) umma_f16_ts_pair(tmem_d, a_src + 8 * i, b_desc, idesc, (kb != seg.kb_begin || i != 0) ? 1u : 0u);
            else umma_f16_ts(tmem_d, a_src + 8 * i, b_desc, idesc, (kb != seg.kb_begin || i != 0) ? 1u : 0u);
          }
          const long long t3 = tracing ? clock64() : 0;
          if constexpr (kPair) umma_commit_pair(a_empty + 8 * ai);
          else umma_commit(a_empty + 8 * ai);
          if ((kb + 1) % act_kblocks == 0 || kb + 1 == kblocks) {
            // the group ends here: its stage goes back to the producer as soon as these MMAs have read it
            if constexpr (kPair) umma_commit_pair(act_empty + 8 * as);
            else umma_commit(act_empty + 8 * as);
            if (++as == act_stages) { as = 0; aphase ^= 1u; }
            have_act = false;
          }
          if (tracing) {
            const long long t4 = clock64();
            spent[0] += t1 - t0;
            spent[1] += t2 - t1;
            spent[2] += t3 - t2;
            spent[3] += t4 - t3;
            ++spent[4];
          }
          if (++ai == a_stages) { ai = 0; iphase ^= 1u; }
        }
        if (!ok) break;
        if constexpr (kPair) umma_commit_pair(d_full + 8 * buf);
        else umma_commit(d_full + 8 * buf);
        dphase[buf] ^= 1u;
      }
      if (tracing) {
        trace[blockIdx.x * 16 + 4] = static_cast<unsigned long long>(spent[0]);
        trace[blockIdx.x * 16 + 5] = static_cast<unsigned long long>(spent[1]);
        trace[blockIdx.x * 16 + 11] = static_cast<unsigned long long>(spent[2]);
        trace[blockIdx.x * 16 + 14] = static_cast<unsigned long long>(spent[3]);
        trace[blockIdx.x * 16 + 15] = static_cast<unsigned long long>(spent[4]);
        trace[blockIdx.x * 16 + 9] = static_cast<unsigned long long>(clock64() - loop_start);
      }
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------ widening warps: int8 smem -> fp16 TMEM
    const int d = (warp - 8) % G::kDequantWarps;
    const int group = (warp - 8) / G::kDequantWarps;
    const int quarter = d & 3;  // = warp & 3: the TMEM lane quarter this warp may touch
    const int half = d >> 2;    // which 64 of the unit's 128 k
    const int row = quarter * 32 + lane;
    // These warps do not care about tiles or segments: they see a plain sequence of units, every other one theirs.
    const int my_units = static_cast<int>(w8tc_range_begin(total_units, grid, cta + 1) - w8tc_range_begin(total_units, grid, cta));
    bool ok = true;
    for (int u = group; ok && u < my_units; u += G::kDequantGroups) {
      const int rs = u % G::kRawStages, ai = u % a_stages;
      const uint32_t rphase = static_cast<uint32_t>(u / G::kRawStages) & 1u;
      const uint32_t iphase = static_cast<uint32_t>(u / a_stages) & 1u;
      if (!mbar_wait(raw_full + 8 * rs, rphase, abort_flag)) {
        if (lane == 0) give_up(kStatusW8Wait);
        ok = false;
        break;
      }
      const uint32_t src = raw_base + rs * G::kRawBytes + row * 128;
      uint4 raw[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) raw[q] = lds128(src + (((4 * half + q) ^ (row & 7)) << 4));
      __syncwarp();
      if (lane == 0) mbar_arrive(raw_empty + 8 * (rs & ~(G::kRawBatch - 1)));  // the batch this stage belongs to
      uint32_t wide[32];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t words[4] = {raw[q].x, raw[q].y, raw[q].z, raw[q].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (bf16_operands) dequant4_bf16(words[j], wide[8 * q + 2 * j], wide[8 * q + 2 * j + 1]);
          else dequant4_f16(words[j], wide[8 * q + 2 * j], wide[8 * q + 2 * j + 1]);
        }
      }
      if (!mbar_wait(a_empty + 8 * ai, iphase ^ 1u, abort_flag)) {
        if (lane == 0) give_up(kStatusW8Wait);
        ok = false;
        break;
      }
      tcgen05_fence_after_sync();
      tmem_store_32x32(tmem_a_base + (static_cast<uint32_t>(quarter * 32) << 16) + ai * G::kAColumns + 32 * half, wide);
      tmem_store_wait();
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kPair) mbar_arrive_cluster(map_to_cta(a_full + 8 * ai, 0));
        else mbar_arrive(a_full + 8 * ai);
      }
    }
    if (warp == 8 && lane == 0) mark(12);
    // A final tile that collects partial sums is latency-bound (L2 round trips per column group): these warps are
    // idle by now and share it with the epilogue warp of their lane quarter.
    if (ok) {
      W8TcSegment last{};
      int segments = 0;
      while (w8tc_segment(total_units, grid, cta, kblocks, segments, last)) ++segments;
      if (segments > 0 && last.has_contributors) {
        const int buf = (segments - 1) & 1;
        const uint32_t parity = static_cast<uint32_t>((segments - 1) >> 1) & 1u;  // how often this buffer was filled before
        if (mbar_wait(d_full + 8 * buf, parity, abort_flag)) {
          tcgen05_fence_after_sync();
          if (!finish(last, buf, 1 + 2 * group + half, G::kTailParts) && lane == 0) give_up(kStatusEpilogueWait);
        } else if (lane == 0) {
          give_up(kStatusEpilogueWait);
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue warps
    uint32_t dphase[2] = {0, 0};
    bool ok = true;
    W8TcSegment seg;
    for (int si = 0; ok && w8tc_segment(total_units, grid, cta, kblocks, si, seg); ++si) {
      const int buf = si & 1;
      if (!mbar_wait(d_full + 8 * buf, dphase[buf], abort_flag)) {
        if (lane == 0) give_up(kStatusEpilogueWait);
        ok = false;
        break;
      }
      dphase[buf] ^= 1u;
      tcgen05_fence_after_sync();
      if (warp == 4 && lane == 0) mark(6 + (si == 0 ? 0 : 1));
      // the widening warps help with a final tile that has partial sums to collect (see below)
      const bool shared_tail = seg.has_contributors;
      if (!finish(seg, buf, 0, shared_tail ? G::kTailParts : 1)) {
        if (lane == 0) give_up(kStatusEpilogueWait);
        ok = false;
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kPair) mbar_arrive_cluster(map_to_cta(d_empty + 8 * buf, 0));
        else mbar_arrive(d_empty + 8 * buf);
      }
      if (warp == 4 && lane == 0 && si == 0) mark(8);
    }
    if (warp == 4 && lane == 0) mark(10);
  }


  // ---------------------------------------------------------------- teardown
  __syncthreads();
  if (threadIdx.x == 0) mark(13);
  if (*abort_flag != 0) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if constexpr (kPair) cluster_sync_all();  // neither CTA leaves while the peer can still touch its barriers or TMEM
  if (warp == 1) {
    tcgen05_fence_after_sync();
    if constexpr (kPair) tmem_dealloc_pair(tmem_base, G::kTmemColumns);
    else tmem_dealloc(tmem_base, G::kTmemColumns);
  }
}

}  // namespace vb200
