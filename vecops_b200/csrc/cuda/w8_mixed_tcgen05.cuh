// Weight-only int8 dequant-GEMM on the 5th-generation tensor cores, weights as the MMA's N operand (M <= 128):
//     C[m,n] = convert( (sum_k f32(A[m,k]) * f32(W[n,k])) * scale[n] )
// A bf16 [M,K], W int8 [N,K] K-contiguous, scale f32 [N], C bf16 or f32 [M,N].
//
// Why this shape.  Measured on B200: a tcgen05.mma costs its issuing SM about 100 cycles however small it is, so
// what bounds a decode-shaped kernel is the NUMBER of MMAs per byte of weights.  With the weights on the M side
// (w8_tcgen05.cuh) one MMA covers 128 rows x 16 k = 2 KB of weights; here they are the N side of a
// 128 x 256 x 16 MMA, 4 KB of weights each, which also is the largest MMA one CTA can issue (128 tensor cycles).
//
//   * int8 weight tiles (256 rows x 128 k = 32 KB) arrive by TMA, 128-byte swizzle, in a ring that holds what HBM
//     latency needs in flight;
//   * sixteen CUDA-core warps widen them int8 -> bf16 (exact: |w| <= 128 needs 8 significant bits) and write
//     them, swizzled, into a second ring of 256 x 64 bf16 tiles in shared memory (one thread per weight row);
//   * the activations are bf16 as the caller stores them - no scaled copy, no pre-pass - TMA-loaded per 128 k;
//     only round_up(M, 8) rows are loaded, the MMA's remaining A rows read whatever follows in shared memory and
//     produce accumulator rows nobody reads;
//   * tcgen05.mma kind::f16 (bf16 x bf16, fp32 accumulate in TMEM): every product is exact, like the AMX
//     tdpbf16ps path of the reference's input<bfloat16_t>(int8 W) conversion.
//
// Work is cut stream-K style over (256-row tile) x (128-wide k-block) units, tile-major, an equal contiguous range
// per persistent CTA.  A CTA whose range STARTS inside a tile publishes that tile's fp32 partial sums to DEVICE
// SCRATCH right after its first segment and raises a nonce-carrying flag; the CTA that holds the tile's first
// k-block reaches the tile last, adds the partials in fixed order, applies the column scale once, converts and
// stores.  Flags carry a per-launch 64-bit nonce: the scratch needs no clearing.  Every wait is bounded.
//
// Warps: 0 TMA producer | 1 MMA issuer + TMEM owner | 2-5 epilogue | 6-21 widening (two groups, one per k half).
//
// Algorithmic traffic per launch: N*K + 4*N + 2*M*K + sizeof(C)*M*N bytes.
#pragma once

#include "gemm_tcgen05.cuh"
#include "ptx.cuh"
#include "w8_tcgen05.cuh"  // W8TcSegment, w8tc_segment, wait_flag, st_release_u64, lds128

namespace vb200 {

struct W8Mix {
  static constexpr int kTileN = 256;       // weight rows per tile (UMMA N)
  static constexpr int kUnitK = 128;       // k per unit: one raw stage, 128 bytes per weight row
  static constexpr int kStepK = 64;        // k per widened stage: one 128-byte swizzle atom of bf16
  static constexpr int kMaxM = 128;        // activation rows (UMMA M is always 128)
  static constexpr int kRawBytes = kTileN * kUnitK;        // 32 KB
  static constexpr int kWideBytes = kTileN * kStepK * 2;   // 32 KB
  static constexpr int kWideStages = 2;    // stage h always holds k half h of a unit
  static constexpr int kActStages = 2;
  static constexpr int kMaxRawStages = 4;
  static constexpr int kWidenWarps = 16;   // two groups of eight: 256 threads = one per weight row
  static constexpr int kThreads = 32 * (6 + kWidenWarps);
  static constexpr int kMaxGrid = 160;     // scratch is sized for this many CTAs
  static constexpr int kBarrierBytes = 512;
  static constexpr int kTailParts = 5;     // warps of one lane quarter that share the last drain: 1 epilogue + 4 widening
  __host__ __device__ static constexpr int act_rows(int m) { return (m + 7) & ~7; }
  __host__ __device__ static constexpr int act_stage_bytes(int m) { return 2 * act_rows(m) * 128; }  // two 64-wide atoms
  __host__ __device__ static constexpr int raw_stages(int m) {
    const int fit = (227 * 1024 - 1024 - kBarrierBytes - kWideStages * kWideBytes - kActStages * act_stage_bytes(m)) / kRawBytes;
    return fit < kMaxRawStages ? fit : kMaxRawStages;
  }
  // layout: activation ring | raw ring | widened ring | barriers   (+ 1 KB alignment slack)
  __host__ __device__ static constexpr int smem_bytes(int m) {
    return kActStages * act_stage_bytes(m) + raw_stages(m) * kRawBytes + kWideStages * kWideBytes + kBarrierBytes + 1024;
  }
  // scratch: per CTA one [256 columns][partial_rows] fp32 partial tile | four 64-bit flags per CTA (one per 32-row quarter)
  __host__ __device__ static constexpr int partial_rows(int m) { return (m + 31) & ~31; }
  __host__ __device__ static constexpr unsigned long long partial_bytes(int m) { return 4ull * kTileN * partial_rows(m); }
  __host__ __device__ static constexpr unsigned long long flags_offset(int m) { return kMaxGrid * partial_bytes(m); }
  __host__ __device__ static constexpr unsigned long long scratch_bytes(int m) { return flags_offset(m) + kMaxGrid * 4 * 8ull; }
};
static_assert(W8Mix::smem_bytes(128) <= 227 * 1024 && W8Mix::smem_bytes(8) <= 227 * 1024, "w8_mixed shared memory budget");
static_assert(W8Mix::raw_stages(128) >= 3, "the raw ring must hold enough weight bytes in flight");

// Four int8 in one word -> two bf16x2 words {w0,w1}, {w2,w3}, exactly.  0x43xx with bit 7 clear is 128 + (x & 127);
// the same word reduced to 0x4300 | (x & 128) is 128 or 256: their difference is the two's-complement value.
__device__ __forceinline__ void dequant4_bf16(uint32_t packed, uint32_t& lo, uint32_t& hi) {
  const uint32_t p0 = __byte_perm(packed, 0x43434343u, 0x4140);
  const uint32_t p1 = __byte_perm(packed, 0x43434343u, 0x4342);
  uint32_t x0 = p0 & 0xff7fff7fu, c0 = p0 & 0xff80ff80u;
  uint32_t x1 = p1 & 0xff7fff7fu, c1 = p1 & 0xff80ff80u;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(x0), "r"(c0));
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(x1), "r"(c1));
}

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

template <typename OutT>
__global__ void __launch_bounds__(W8Mix::kThreads, 1)
w8_mixed_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_a,
                        const float* __restrict__ scale, OutT* __restrict__ c, long long ldc, int M, int N, int K,
                        float* __restrict__ partials, unsigned long long* __restrict__ flags, unsigned long long nonce,
                        uint32_t idesc, uint32_t* __restrict__ status, unsigned long long* __restrict__ trace) {
  using G = W8Mix;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int act_rows = G::act_rows(M);
  const int act_stage = G::act_stage_bytes(M);
  const int raw_stages = G::raw_stages(M);
  // the activation ring comes first: the MMA reads 128 rows of A whatever M is, and what it reads past the loaded
  // rows must still be this CTA's shared memory
  const uint32_t act_base = smem_base;
  const uint32_t raw_base = act_base + G::kActStages * act_stage;
  const uint32_t wide_base = raw_base + raw_stages * G::kRawBytes;
  const int bar_offset = G::kActStages * act_stage + raw_stages * G::kRawBytes + G::kWideStages * G::kWideBytes;
  uint8_t* bar_gen = smem_gen + bar_offset;
  const uint32_t bar_base = smem_base + bar_offset;
  uint32_t next_bar = bar_base;
  auto take = [&](int count) { const uint32_t at = next_bar; next_bar += 8 * count; return at; };
  const uint32_t raw_full = take(G::kMaxRawStages), raw_empty = take(G::kMaxRawStages);
  const uint32_t act_full = take(G::kActStages), act_empty = take(G::kActStages);
  const uint32_t wide_full = take(G::kWideStages), wide_empty = take(G::kWideStages);
  const uint32_t d_full = take(2), d_empty = take(2);
  const uint32_t tail_bar = take(4);  // per lane quarter: the warps sharing the last drain have published
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_gen + (next_bar - bar_base));
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bar_gen + (next_bar - bar_base) + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kblocks = (K + G::kUnitK - 1) / G::kUnitK;
  const int tiles = (N + G::kTileN - 1) / G::kTileN;
  const long long total_units = static_cast<long long>(tiles) * kblocks;
  const int grid = gridDim.x;
  const int cta = blockIdx.x;
  const long long range_begin = w8tc_range_begin(total_units, grid, cta);
  const int my_units = static_cast<int>(w8tc_range_begin(total_units, grid, cta + 1) - range_begin);
  const int partial_rows = G::partial_rows(M);

  if (threadIdx.x == 0) {
    for (int s = 0; s < G::kMaxRawStages; ++s) {
      mbar_init(raw_full + 8 * s, 1);
      mbar_init(raw_empty + 8 * s, G::kWidenWarps);
    }
    for (int s = 0; s < G::kActStages; ++s) {
      mbar_init(act_full + 8 * s, 1);
      mbar_init(act_empty + 8 * s, 1);
    }
    for (int s = 0; s < G::kWideStages; ++s) {
      mbar_init(wide_full + 8 * s, G::kWidenWarps / 2);
      mbar_init(wide_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(d_full + 8 * s, 1);
      mbar_init(d_empty + 8 * s, 4);
    }
    for (int q = 0; q < 4; ++q) mbar_init(tail_bar + 8 * q, G::kTailParts);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_descriptor(&tma_w);
    tma_prefetch_descriptor(&tma_a);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

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

  int num_segments = 0;
  {
    W8TcSegment probe;
    while (w8tc_segment(total_units, grid, cta, kblocks, num_segments, probe)) {
      // the column scales of a tile this CTA will store: into L2 now, they are needed at the very end
      if (probe.owner && scale != nullptr && warp == 2) {
        const int n = probe.tile * G::kTileN + lane * 8;  // 32 lanes x 32 bytes = the tile's 256 scales
        if (n < N) asm volatile("prefetch.global.L2 [%0];" ::"l"(scale + n));
      }
      ++num_segments;
    }
  }

  // Drain (part of) one accumulator.  The owner of a tile adds the partial sums of the CTAs that follow it and
  // stores C; any other CTA writes its partial sums to the scratch (the caller raises the flag).  The tile's 256
  // columns are dealt in groups of 8, round-robin, to `parts` cooperating warps of one lane quarter (`part` = this
  // warp's turn): callable by every warp whose index % 4 is the quarter.  Loads from the scratch are issued for all
  // contributors of a group before the first is used, so a group costs one L2 round trip, not one per contributor.
  auto drain = [&](const W8TcSegment& seg, int buf, int part, int parts) -> bool {
    const int quarter = warp & 3;
    const int m = quarter * 32 + lane;  // activation row = TMEM lane
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * G::kTileN;
    const int n0 = seg.tile * G::kTileN;
    int last_contributor = cta;
    if (seg.owner && seg.has_contributors) {
      const long long tile_end_unit = static_cast<long long>(seg.tile + 1) * kblocks;
      while (last_contributor + 1 < grid && w8tc_range_begin(total_units, grid, last_contributor + 1) < tile_end_unit) ++last_contributor;
      for (int other = cta + 1; other <= last_contributor; ++other)
        if (!wait_flag(flags + 4 * other + quarter, nonce, abort_flag)) return false;
    }
#pragma unroll 1
    for (int group = part; group < G::kTileN / 8; group += parts) {
      const int col0 = n0 + group * 8;
      if (col0 >= N) break;
      uint32_t v[8];
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                   : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                   : "r"(taddr + group * 8)
                   : "memory");
      if (seg.owner) {
        const int valid = min(8, N - col0);
        // every load of the group - the column scales and up to four partners' partial sums - is issued before
        // the first is used (few enough registers that the compiler keeps it so): one round trip per group
        float factor[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) factor[j] = (scale != nullptr && j < valid) ? __ldg(scale + col0 + j) : 1.f;
        float acc[8];
        for (int other = cta + 1; other <= last_contributor || other == cta + 1; other += 4) {
          float p[4][8];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const bool has = other + q <= last_contributor;
            const float* src = partials + (static_cast<size_t>(other + q) * G::kTileN + group * 8) * partial_rows + m;
#pragma unroll
            for (int j = 0; j < 8; ++j) p[q][j] = has ? __ldcg(src + static_cast<size_t>(j) * partial_rows) : 0.f;
          }
          if (other == cta + 1) {
            tmem_load_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = __uint_as_float(v[j]);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = (((acc[j] + p[0][j]) + p[1][j]) + p[2][j]) + p[3][j];
        }
        if (m < M) {
          OutT* dst = c + static_cast<long long>(m) * ldc + col0;
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] *= factor[j];
          const bool vec = valid == 8 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
          if constexpr (sizeof(OutT) == 2) {
            if (vec) {
              *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                          pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (j < valid) dst[j] = __float2bfloat16_rn(acc[j]);
            }
          } else {
            if (vec) {
              reinterpret_cast<float4*>(dst)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
              reinterpret_cast<float4*>(dst)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (j < valid) dst[j] = acc[j];
            }
          }
        }
      } else {
        // partial sums: [column][row], rows contiguous, so a warp writes 128 bytes per column
        tmem_load_wait();
        float* dst = partials + (static_cast<size_t>(cta) * G::kTileN + group * 8) * partial_rows + m;
#pragma unroll
        for (int j = 0; j < 8; ++j) __stcg(dst + static_cast<size_t>(j) * partial_rows, __uint_as_float(v[j]));
      }
    }
    if (!seg.owner) __threadfence();
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one thread)
    // Two independent rings: the weight tiles run as far ahead as their ring allows (they are what HBM latency is
    // hidden behind), the activation tiles follow the MMA.  Neither waits for the other.
    if (lane == 0) {
      int raw_issued = 0, act_issued = 0, rs = 0, as = 0;
      uint32_t rphase = 0, aphase = 0;
      const long long started = clock64();
      while (raw_issued < my_units || act_issued < my_units) {
        bool progress = false;
        if (raw_issued < my_units && mbar_test_wait(raw_empty + 8 * rs, rphase ^ 1u)) {
          const long long u = range_begin + raw_issued;
          const int tile = static_cast<int>(u / kblocks), kb = static_cast<int>(u % kblocks);
          mbar_arrive_expect_tx(raw_full + 8 * rs, G::kRawBytes);
          tma_load_2d(raw_base + rs * G::kRawBytes, &tma_w, raw_full + 8 * rs, kb * G::kUnitK, tile * G::kTileN);
          if (++rs == raw_stages) { rs = 0; rphase ^= 1u; }
          ++raw_issued;
          progress = true;
        }
        if (act_issued < my_units && mbar_test_wait(act_empty + 8 * as, aphase ^ 1u)) {
          const int kb = static_cast<int>((range_begin + act_issued) % kblocks);
          const uint32_t dst = act_base + as * act_stage;
          mbar_arrive_expect_tx(act_full + 8 * as, static_cast<uint32_t>(act_stage));
          tma_load_2d(dst, &tma_a, act_full + 8 * as, kb * G::kUnitK, 0);
          tma_load_2d(dst + act_rows * 128, &tma_a, act_full + 8 * as, kb * G::kUnitK + G::kStepK, 0);
          if (++as == G::kActStages) { as = 0; aphase ^= 1u; }
          ++act_issued;
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
    // ------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      int as = 0, unit = 0;
      uint32_t aphase = 0;
      uint32_t dphase[2] = {0, 0};
      W8TcSegment seg;
      bool ok = true;
      const bool tracing = trace != nullptr;
      long long spent[4] = {0, 0, 0, 0};  // tuning aid: cycles waiting for activations | for widened weights | issuing; units
      const long long loop_start = tracing ? clock64() : 0;
      for (int si = 0; ok && w8tc_segment(total_units, grid, cta, kblocks, si, seg); ++si) {
        const int buf = si & 1;
        if (!mbar_wait(d_empty + 8 * buf, dphase[buf] ^ 1u, abort_flag)) {
          give_up(kStatusMmaWaitTmem);
          break;
        }
        tcgen05_fence_after_sync();
        const uint32_t tmem_d = tmem_base + buf * G::kTileN;
        for (int kb = seg.kb_begin; kb < seg.kb_end; ++kb, ++unit) {
          const long long t0 = tracing ? clock64() : 0;
          if (!mbar_wait(act_full + 8 * as, aphase, abort_flag)) {
            give_up(kStatusMmaWaitFull);
            ok = false;
            break;
          }
          if (tracing) spent[0] += clock64() - t0;
          const uint32_t wphase = static_cast<uint32_t>(unit) & 1u;  // widened stage h is refilled once per unit
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const long long t1 = tracing ? clock64() : 0;
            if (!mbar_wait(wide_full + 8 * h, wphase, abort_flag)) {
              give_up(kStatusMmaWaitFull);
              ok = false;
              break;
            }
            tcgen05_fence_after_sync();
            const long long t2 = tracing ? clock64() : 0;
            if (unit == 0 && h == 0) mark(3);
            const uint64_t a_desc = umma_smem_desc_sw128(act_base + as * act_stage + h * act_rows * 128);
            const uint64_t b_desc = umma_smem_desc_sw128(wide_base + h * G::kWideBytes);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)  // +32 bytes along K inside the swizzle atom = +2 in the address field
              umma_f16(tmem_d, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kb != seg.kb_begin || h != 0 || kk != 0) ? 1u : 0u);
            umma_commit(wide_empty + 8 * h);
            if (tracing) {
              spent[1] += t2 - t1;
              spent[2] += clock64() - t2;
            }
          }
          if (!ok) break;
          umma_commit(act_empty + 8 * as);
          if (tracing) ++spent[3];
          if (++as == G::kActStages) { as = 0; aphase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(d_full + 8 * buf);
        dphase[buf] ^= 1u;
      }
      mark(4);
      if (tracing) {
        trace[blockIdx.x * 16 + 5] = static_cast<unsigned long long>(spent[0]);
        trace[blockIdx.x * 16 + 9] = static_cast<unsigned long long>(spent[1]);
        trace[blockIdx.x * 16 + 11] = static_cast<unsigned long long>(spent[2]);
        trace[blockIdx.x * 16 + 14] = static_cast<unsigned long long>(clock64() - loop_start);
        trace[blockIdx.x * 16 + 15] = static_cast<unsigned long long>(spent[3]);
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------ widening warps: int8 smem -> bf16 smem
    // Group h (eight warps, one thread per weight row) widens k half h of every unit into widened stage h.
    const int h = (warp - 6) >> 3;
    const int row = ((warp - 6) & 7) * 32 + lane;
    const int sw = row & 7;  // the 128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r & 7)
    bool ok = true;
    for (int u = 0; ok && u < my_units; ++u) {
      const int rs = u % raw_stages;
      const uint32_t rphase = static_cast<uint32_t>(u / raw_stages) & 1u;
      if (!mbar_wait(raw_full + 8 * rs, rphase, abort_flag)) {
        if (lane == 0) give_up(kStatusW8Wait);
        ok = false;
        break;
      }
      const uint32_t src = raw_base + rs * G::kRawBytes + row * 128;
      uint4 raw[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) raw[q] = lds128(src + (((4 * h + q) ^ sw) << 4));
      __syncwarp();
      if (lane == 0) mbar_arrive(raw_empty + 8 * rs);
      uint32_t wide[32];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t words[4] = {raw[q].x, raw[q].y, raw[q].z, raw[q].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) dequant4_bf16(words[j], wide[8 * q + 2 * j], wide[8 * q + 2 * j + 1]);
      }
      // the MMAs that read this stage's previous contents (one unit ago) must have finished
      if (!mbar_wait(wide_empty + 8 * h, (static_cast<uint32_t>(u) & 1u) ^ 1u, abort_flag)) {
        if (lane == 0) give_up(kStatusW8Wait);
        ok = false;
        break;
      }
      const uint32_t dst = wide_base + h * G::kWideBytes + row * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) sts128(dst + ((j ^ sw) << 4), wide[4 * j], wide[4 * j + 1], wide[4 * j + 2], wide[4 * j + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(wide_full + 8 * h);
    }
    // The CTA's last segment ends its life: these warps are idle by then and share its drain with the epilogue warp
    // of their lane quarter (L2 round trips per column group are what it costs; five warps take them side by side).
    if (ok && num_segments > 0 && (warp & 3) * 32 < M) {
      W8TcSegment last;
      w8tc_segment(total_units, grid, cta, kblocks, num_segments - 1, last);
      const int buf = (num_segments - 1) & 1;
      const uint32_t parity = static_cast<uint32_t>((num_segments - 1) >> 1) & 1u;  // how often this buffer was filled before
      if (mbar_wait(d_full + 8 * buf, parity, abort_flag)) {
        tcgen05_fence_after_sync();
        const int helper = 1 + ((warp - 6) >> 2);  // 1..4 within the quarter
        if (!drain(last, buf, helper, G::kTailParts) && lane == 0) give_up(kStatusEpilogueWait);
        tcgen05_fence_before_sync();
        __syncwarp();
        if (!last.owner && lane == 0) mbar_arrive(tail_bar + 8 * (warp & 3));
      } else if (lane == 0) {
        give_up(kStatusEpilogueWait);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (2-5)
    const int quarter = warp & 3;
    const bool quarter_used = quarter * 32 < M;
    uint32_t dphase[2] = {0, 0};
    bool ok = true;
    W8TcSegment seg;
    for (int si = 0; ok && si < num_segments; ++si) {
      w8tc_segment(total_units, grid, cta, kblocks, si, seg);
      const int buf = si & 1;
      if (!mbar_wait(d_full + 8 * buf, dphase[buf], abort_flag)) {
        if (lane == 0) give_up(kStatusEpilogueWait);
        ok = false;
        break;
      }
      dphase[buf] ^= 1u;
      tcgen05_fence_after_sync();
      if (warp == 4 && lane == 0) mark(6 + (si == 0 ? 0 : 1));
      if (quarter_used) {
        // the CTA's last segment is drained together with the by then idle widening warps of this lane quarter
        const bool shared = si == num_segments - 1;
        if (!drain(seg, buf, 0, shared ? G::kTailParts : 1)) {
          if (lane == 0) give_up(kStatusEpilogueWait);
          ok = false;
          break;
        }
        if (!seg.owner) {
          // the flag goes up once every warp that shared the drain has its stores behind a fence
          if (shared) {
            __syncwarp();
            if (lane == 0) mbar_arrive(tail_bar + 8 * quarter);
            if (!mbar_wait(tail_bar + 8 * quarter, 0, abort_flag)) {
              if (lane == 0) give_up(kStatusEpilogueWait);
              ok = false;
              break;
            }
          }
          __syncwarp();
          if (lane == 0) st_release_u64(flags + 4 * cta + quarter, nonce);
        }
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(d_empty + 8 * buf);
      if (warp == 4 && lane == 0 && si == 0) mark(8);
    }
    if (warp == 4 && lane == 0) mark(10);
  }

  // ---------------------------------------------------------------- teardown
  __syncthreads();
  if (*abort_flag != 0) {
    // A wait ran out: give copies and MMAs still in flight time to land before shared memory and TMEM go back.
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace vb200
