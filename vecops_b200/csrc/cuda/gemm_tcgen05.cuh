// Dense GEMM C[M,N] = A[M,K] . B[N,K]^T on the 5th-generation tensor cores.
//
// One persistent CTA per SM walks 128x256 output tiles.  Roles:
//   warp 0    TMA producer: A (128 x 128 B) and B (256 x 128 B) k-blocks into a
//             4-stage shared-memory ring, 128-byte swizzle, mbarrier full/empty
//   warp 1    owns TMEM (512 columns = two 128x256 fp32/int32 accumulators) and
//             issues tcgen05.mma from one thread; tcgen05.commit releases smem
//             stages and publishes finished accumulators
//   warps 2-5 epilogue: tcgen05.ld their TMEM lane quarter, convert, and either
//             stage 32-row x 128-byte slabs in swizzled smem for TMA stores or
//             store straight to global (ragged / unaligned C)
// The second accumulator lets the epilogue of tile i overlap the main loop of
// tile i+1.  kind::f16 (bf16 in, fp32 accumulate) and kind::i8 (8-bit in, int32
// accumulate) share this file; the operand formats arrive in the instruction
// descriptor.
//
// Fused all-gather: the TMA-store epilogue can send every finished slab to up to
// eight destinations - the C matrices of all GPUs of a column-sharded GEMM, reached
// through peer pointers over NVLink - at a column offset, so the gather of the
// output overlaps the main loop tile by tile and needs no staging pass.  Where the
// result is bound to an NVSwitch multicast object the epilogue instead writes each
// slab ONCE, with multimem.st, and the switch delivers it to every GPU.  (Only
// stores cross GPUs; every load stays local.)
//
// Tail splitting: when the tile count leaves the last wave mostly empty (512 tiles
// on 148 SMs = 3.46 waves), the tail tiles are cut along K into S slices (S a power
// of two) so that the last wave keeps S times as many SMs busy for 1/S of the time.
// The S CTAs of a tile exchange fp32 (int32) partial accumulators through DEVICE
// SCRATCH: each publishes the columns it does not own and raises a flag that carries
// the launch's 64-bit nonce and counts its readers down, then adds the others'
// partials to the columns it owns and stores those.  The last reader leaves the flag
// at the bare nonce, so a captured launch can be replayed.  Fixed summation order,
// so results are reproducible.  Without scratch S = 1.
//
// CTA pairs (kPair): two CTAs of a cluster, on the two SMs of one TPC, share a 256x256 tile.  Each loads its 128 rows
// of A and its 128 of the 256 rows of B (half the shared-memory fill and L2 traffic per SM of the single-CTA form) into
// a 6-stage ring; the leader's MMA thread issues tcgen05.mma.cta_group::2 (M = 256), which reads both CTAs' shared
// memory and writes each CTA's 128 rows of D into that CTA's TMEM; both CTAs run the epilogue on their own rows.
// Barriers: both CTAs' loads count bytes on the leader's `full`; the leader's commits arrive on `empty` and
// `tmem_full` of both CTAs; both epilogues arrive on the leader's `tmem_empty`.  Loads go to one CTA each.
//
// Weight-only form (kW8): B is int8 in memory and bf16 in the product - vecops' input<bfloat16_t>(int8 W) - while A
// stays the caller's bf16 activations.  256-row x 128-k units of W arrive by TMA as bytes; eight more warps widen
// them (exactly: |w| <= 128 needs 8 significant bits) into the same 128-byte-swizzled K-major bf16 tiles the dense form
// gets from TMA, one 64-k block at a time, and the MMA issuer runs the dense form's 128x256x16 MMAs on them: 4 KB of
// weights per MMA, the most one CTA's instruction covers.  Everything downstream - accumulators, the K-slice exchange,
// the fused output transform, the stores - is the dense form's.  Decode shapes have few tiles (N / 256), so every tile is
// cut along K over the idle SMs and each CTA runs exactly ONE (tile, K slice): the grid is tiles x slices, not persistent,
// which lets the epilogue's staging buffers lie over the drained weight ring.
//
// Algorithmic traffic per launch: (M*K + N*K) * sizeof(in) + M*N * sizeof(out).
#pragma once

#include <cuda_fp16.h>
#include <type_traits>

#include "epilogue.cuh"
#include "ptx.cuh"

namespace vb200 {

struct GemmTc {
  static constexpr int kBlockM = 128;
  static constexpr int kBlockN = 256;
  static constexpr int kBlockKBytes = 128;  // one swizzle atom along K
  static constexpr int kStages = 4;
  static constexpr int kABytes = kBlockM * kBlockKBytes;
  static constexpr int kBBytes = kBlockN * kBlockKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiWarps = 4;
  static constexpr int kEpiBufBytes = 32 * 128;  // 32 rows x 128 bytes
  static constexpr int kEpiBytes = kEpiWarps * 2 * kEpiBufBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarrierBytes + 1024;  // + alignment slack
  static constexpr int kThreads = 32 * (2 + kEpiWarps);
  static constexpr int kTmemColumns = 512;
  static constexpr long long kGroupBytes = 32ll << 20;  // raster: row-tiles holding this much of A share each sweep over N
  // Tail split: a slice owns whole 128-byte output slabs, so the split cannot exceed the slabs of a tile row.
  static constexpr int kMinSliceKb = 4;  // k-blocks a slice must keep for the split to pay
  __host__ __device__ static constexpr int max_split(size_t out_elem) { return out_elem == 2 ? 4 : 8; }
  // scratch: `slices` partial accumulators of kBlockM x kBlockN 32-bit words, then 4 flags (one per row quarter) per slice
  __host__ __device__ static constexpr unsigned long long split_flags_offset(long long slices) {
    return static_cast<unsigned long long>(slices) * kBlockM * kBlockN * 4;
  }
  __host__ __device__ static constexpr unsigned long long split_scratch_bytes(long long slices) {
    return split_flags_offset(slices) + static_cast<unsigned long long>(slices) * 4 * 8;
  }
};

// The CTA-pair form: per-CTA constants (a CTA still owns 128 rows x 256 columns of accumulators).
struct GemmPair : GemmTc {
  static constexpr int kStages = 6;
  static constexpr int kBRows = kBlockN / 2;  // rows of B this CTA feeds to the pair MMA
  static constexpr int kBBytes = kBRows * kBlockKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarrierBytes + 1024;
};
// The weight-only form: per-CTA constants.  Shared memory: activation ring | int8 weight ring | widened weight ring |
// barriers; the epilogue's staging buffers lie over the start of the int8 ring (free by then: one work item per CTA).
struct GemmW8 : GemmTc {
  static constexpr int kUnitK = 128;                  // k per unit: one TMA box of W (256 rows x 128 bytes)
  static constexpr int kStages = 4;                   // activation 64-k atoms in flight (16 KB each: the MMA's 128 rows)
  static constexpr int kRawStages = 3;                // int8 weight units in flight
  static constexpr int kRawBytes = kBlockN * kUnitK;  // 32 KB
  static constexpr int kWideStages = 2;               // widened 64-k blocks: one being multiplied, one being written
  static constexpr int kWideBytes = kBBytes;          // 32 KB
  static constexpr int kConvertWarps = 8;
  static constexpr int kThreads = 32 * (2 + kEpiWarps + kConvertWarps);
  static constexpr int kRawOffset = kStages * kABytes;
  static constexpr int kWideOffset = kRawOffset + kRawStages * kRawBytes;
  static constexpr int kRingBytes = kWideOffset + kWideStages * kWideBytes;
  static constexpr int kSmemBytes = kRingBytes + kBarrierBytes + 1024;
  static constexpr int kExtraBarrierOffset = 128;     // raw_full[3] raw_empty[3] wide_full[2] wide_empty[2] inside the barrier block
  static constexpr int kMinSliceUnits = 4;            // units a K slice must keep for the cut to pay
};
static_assert(GemmPair::kSmemBytes <= 227 * 1024 && GemmTc::kSmemBytes <= 227 * 1024 && GemmW8::kSmemBytes <= 227 * 1024, "shared memory budget");
static_assert(GemmW8::kEpiBytes <= GemmW8::kRawStages * GemmW8::kRawBytes, "the epilogue staging buffers lie over the int8 weight ring");

// Destinations of the TMA-store epilogue: map[0] is the local C, the rest are peers' C matrices.
struct GemmStoreMaps {
  static constexpr int kMax = 8;
  CUtensorMap map[kMax];
};

// Device status codes ORed into the status word by a wait that ran out.
enum : uint32_t {
  kStatusProducerWait = 1u << 0,
  kStatusMmaWaitFull = 1u << 1,
  kStatusMmaWaitTmem = 1u << 2,
  kStatusEpilogueWait = 1u << 3,
  kStatusW8Wait = 1u << 4,
};

// The status word lives in pinned host memory mapped into the device: a plain
// system-scope store is enough, it only ever happens when a wait ran out.
__device__ __forceinline__ void report_status(uint32_t* status, uint32_t code) {
  *reinterpret_cast<volatile uint32_t*>(status) = code;
  __threadfence_system();
}

// Raster: `group_m` row-tiles share each sweep over N, so that one wave of tiles re-reads few rows of A and B.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int per_group = group_m * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int group_rows = min(tiles_m - first_m, group_m);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % group_rows;
  tn = in_group / group_rows;
}

// What a CTA works on in its i-th round.
struct GemmItem {
  int tile;
  int kb_begin, kb_end;
  int slice;    // which K slice of a split tail tile (0 when the tile is whole)
  int slices;   // 1 = whole tile
  int tail_index;  // index of the tile among the split tail tiles
};

// The whole tiles go round-robin over the workers (`cta` of `grid`: CTAs, or CTA pairs).  The tail tiles - those
// left after the last full round - follow as whole tiles when `split` == 1.  When they are split, worker w takes slice
// (w % split) of tail tile (w / split) and takes it FIRST: the exchange of partial sums and the wait for the other
// slices then hide under the main loop of the worker's next tile instead of ending the kernel.
__device__ __forceinline__ bool gemm_item(int round, int num_tiles, int num_kb, int split, int cta, int grid, GemmItem& item) {
  const int full_rounds = num_tiles / grid;
  const int first_tail = full_rounds * grid;
  const int tail = num_tiles - first_tail;
  item.slice = 0;
  item.slices = 1;
  item.tail_index = 0;
  item.kb_begin = 0;
  item.kb_end = num_kb;
  if (split > 1 && cta < tail * split) {
    if (round == 0) {
      item.tail_index = cta / split;
      item.tile = first_tail + item.tail_index;
      item.slice = cta % split;
      item.slices = split;
      item.kb_begin = static_cast<int>(static_cast<long long>(num_kb) * item.slice / split);
      item.kb_end = static_cast<int>(static_cast<long long>(num_kb) * (item.slice + 1) / split);
      return true;
    }
    --round;
  }
  if (round < full_rounds) {
    item.tile = cta + round * grid;
    return true;
  }
  if (round == full_rounds && split <= 1 && cta < tail) {
    item.tile = first_tail + cta;
    return true;
  }
  return false;
}

// Host and device agree on the split: the largest power of two S with tail * S <= grid, S <= max_split,
// and at least kMinSliceKb k-blocks left per slice.
__host__ __device__ inline int gemm_tail_split(long long num_tiles, int grid, int num_kb, int max_split) {
  const long long tail = num_tiles % grid;
  if (tail == 0 || num_tiles < grid) return 1;
  int split = 1;
  while (split * 2 <= max_split && tail * (split * 2) <= grid && split * 2 * GemmTc::kMinSliceKb <= num_kb) split *= 2;
  return split;
}

// Two fp32 values -> one word of two 16-bit outputs of type OutT (bf16 or fp16), round to nearest even.
template <typename OutT>
__device__ __forceinline__ uint32_t pack_out16x2(float lo, float hi);

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <>
__device__ __forceinline__ uint32_t pack_out16x2<__nv_bfloat16>(float lo, float hi) {
  return pack_bf16x2(lo, hi);
}
template <>
__device__ __forceinline__ uint32_t pack_out16x2<__half>(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Four int8 in one word -> two bf16x2 words {w0,w1}, {w2,w3}, exactly (|w| <= 128 needs 8 significant bits).  0x43xx
// with bit 7 clear is 128 + (x & 127); the same word reduced to 0x4300 | (x & 128) is 128 or 256: their difference is
// the two's-complement value.
__device__ __forceinline__ void widen4_bf16(uint32_t packed, uint32_t& lo, uint32_t& hi) {
  const uint32_t p0 = __byte_perm(packed, 0x43434343u, 0x4140);
  const uint32_t p1 = __byte_perm(packed, 0x43434343u, 0x4342);
  const uint32_t x0 = p0 & 0xff7fff7fu, c0 = p0 & 0xff80ff80u;
  const uint32_t x1 = p1 & 0xff7fff7fu, c1 = p1 & 0xff80ff80u;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(x0), "r"(c0));
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(x1), "r"(c1));
}

// OutT: __nv_bfloat16, __half or float for kind::f16 (bf16 or fp16 operands, chosen by the instruction descriptor), int32_t for kind::i8.
// kTf32: the operands are fp32 words multiplied as tf32 (kind::tf32, single CTAs only) - the building block of the split fp32 product.
template <bool kInt8, typename OutT, bool kPair, bool kW8 = false, bool kTf32 = false>
__global__ void __launch_bounds__(kW8 ? GemmW8::kThreads : GemmTc::kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const __grid_constant__ GemmStoreMaps tma_c, int num_dest, int c_col_offset, OutT* __restrict__ c,
                    long long ldc, int M, int N, int K, const float* __restrict__ column_scale, uint32_t idesc,
                    int use_tma_store, int raster_group, int split, uint32_t* __restrict__ partials, unsigned long long* __restrict__ flags,
                    unsigned long long nonce, EpilogueArgs ep, uint32_t* __restrict__ status,
                    unsigned long long* __restrict__ trace) {
  static_assert(!kW8 || (!kInt8 && !kPair), "the weight-only form is a single-CTA 16-bit product");
  using G = typename std::conditional<kW8, GemmW8, typename std::conditional<kPair, GemmPair, GemmTc>::type>::type;
  static_assert(!kTf32 || (!kInt8 && !kPair && !kW8 && std::is_same<OutT, float>::value), "the tf32 form is a single-CTA fp32 product");
  constexpr int kElemBytes = kInt8 ? 1 : kTf32 ? 4 : 2;
  // elements of K per step of the main loop: one 128-byte swizzle atom, or - weight-only form - one unit of two
  constexpr int kBlockK = kW8 ? GemmW8::kUnitK : G::kBlockKBytes / kElemBytes;
  constexpr int kRingBytes = kW8 ? GemmW8::kRingBytes : G::kStages * G::kStageBytes;
  constexpr int kMaxRounds = kW8 ? 1 : 0x7fffffff;  // the weight-only form runs one work item per CTA
  constexpr int kTileM = kPair ? 2 * G::kBlockM : G::kBlockM;  // rows of the tile a worker (CTA or pair) owns
  const uint32_t pair_rank = kPair ? cluster_cta_rank() : 0u;
  const int worker = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int workers = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  constexpr int kOutCols = 128 / static_cast<int>(sizeof(OutT));  // columns per 128-byte slab row

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t epi_base = smem_base + (kW8 ? GemmW8::kRawOffset : kRingBytes);
  constexpr int kBarrierOffset = kW8 ? kRingBytes : kRingBytes + G::kEpiBytes;
  uint8_t* bar_gen = smem_gen + kBarrierOffset;
  const uint32_t bar_base = smem_base + kBarrierOffset;
  // barrier block: full[stages] empty[stages] tmem_full[2] tmem_empty[2] | tmem slot | abort flag
  const uint32_t full_bar = bar_base;
  const uint32_t empty_bar = bar_base + 8 * G::kStages;
  const uint32_t tmem_full_bar = bar_base + 16 * G::kStages;
  const uint32_t tmem_empty_bar = tmem_full_bar + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_gen + 16 * G::kStages + 32);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bar_gen + 16 * G::kStages + 36);
  // weight-only form: int8 unit landed / consumed, widened block written / multiplied
  const uint32_t raw_full_bar = bar_base + GemmW8::kExtraBarrierOffset;
  const uint32_t raw_empty_bar = raw_full_bar + 8 * GemmW8::kRawStages;
  const uint32_t wide_full_bar = raw_empty_bar + 8 * GemmW8::kRawStages;
  const uint32_t wide_empty_bar = wide_full_bar + 8 * GemmW8::kWideStages;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // optional timeline (nanoseconds) for tuning: 16 slots per CTA, written only when a trace buffer is given
  auto mark = [&](int slot) {
    if (trace != nullptr && slot < 16) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      trace[blockIdx.x * 16 + slot] = now;
    }
  };
  if (threadIdx.x == 0) {
    mark(0);
    if (trace != nullptr) trace[blockIdx.x * 16 + 13] = static_cast<unsigned long long>(clock64());  // SM cycle counter at start
  }

  const int tiles_m = (M + kTileM - 1) / kTileM;
  const int tiles_n = (N + G::kBlockN - 1) / G::kBlockN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + kBlockK - 1) / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < G::kStages; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar + 8 * a, 1);
      mbar_init(tmem_empty_bar + 8 * a, G::kEpiWarps * 32 * (kPair ? 2 : 1));  // the leader's collects both epilogues
    }
    if constexpr (kW8) {
      for (int s = 0; s < GemmW8::kRawStages; ++s) {
        mbar_init(raw_full_bar + 8 * s, 1);
        mbar_init(raw_empty_bar + 8 * s, GemmW8::kConvertWarps);
      }
      for (int s = 0; s < GemmW8::kWideStages; ++s) {
        mbar_init(wide_full_bar + 8 * s, GemmW8::kConvertWarps);
        mbar_init(wide_empty_bar + 8 * s, 1);
      }
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_descriptor(&tma_a);
    tma_prefetch_descriptor(&tma_b);
    if (use_tma_store == 1) tma_prefetch_descriptor(&tma_c.map[0]);
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
  tcgen05_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Back-to-back launches: everything above touched only this CTA's own shared and tensor memory, so it may run while
  // the previous kernel of the stream drains; everything below reads or writes global memory and waits for it.  The
  // next kernel's set-up may likewise overlap this kernel's last tiles.
  grid_launch_dependents();
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      GemmItem item;
      if constexpr (kW8) {
        // Two independent rings, neither waiting for the other: the int8 weight units run as far ahead as their ring
        // allows (they are what HBM latency hides behind), the activation atoms (64 k each, from L2) follow the MMA.
        if (gemm_item(0, num_tiles, num_kb, split, worker, workers, item)) {
          int tm, tn;
          tile_coords(item.tile, tiles_m, tiles_n, raster_group, tm, tn);
          const int units = item.kb_end - item.kb_begin;
          const int atoms = 2 * units;
          int raw_issued = 0, act_issued = 0, rs = 0;
          uint32_t rphase = 0;
          const long long started = clock64();
          while (raw_issued < units || act_issued < atoms) {
            bool progress = false;
            if (raw_issued < units && mbar_test_wait(raw_empty_bar + 8 * rs, rphase ^ 1u)) {
              mbar_arrive_expect_tx(raw_full_bar + 8 * rs, GemmW8::kRawBytes);
              tma_load_2d(smem_base + GemmW8::kRawOffset + rs * GemmW8::kRawBytes, &tma_b, raw_full_bar + 8 * rs,
                          (item.kb_begin + raw_issued) * GemmW8::kUnitK, tn * G::kBlockN);
              if (++rs == GemmW8::kRawStages) { rs = 0; rphase ^= 1u; }
              ++raw_issued;
              progress = true;
            }
            if (act_issued < atoms && mbar_test_wait(empty_bar + 8 * stage, phase ^ 1u)) {
              mbar_arrive_expect_tx(full_bar + 8 * stage, G::kABytes);
              tma_load_2d(smem_base + stage * G::kABytes, &tma_a, full_bar + 8 * stage,
                          item.kb_begin * GemmW8::kUnitK + act_issued * 64, tm * G::kBlockM);  // past K: zero-filled by TMA
              if (++stage == G::kStages) { stage = 0; phase ^= 1u; }
              ++act_issued;
              progress = true;
            }
            if (!progress && (*abort_flag != 0 || clock64() - started > 4 * kWaitCycleBudget)) {
              report_status(status, kStatusProducerWait);
              *abort_flag = 1;
              break;
            }
          }
        }
      } else
      for (int round = 0; ok && gemm_item(round, num_tiles, num_kb, split, worker, workers, item); ++round) {
        int tm, tn;
        tile_coords(item.tile, tiles_m, tiles_n, raster_group, tm, tn);
        for (int kb = item.kb_begin; kb < item.kb_end; ++kb) {
          if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag)) {
            report_status(status, kStatusProducerWait);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * G::kStageBytes;
          const uint32_t b_dst = a_dst + G::kABytes;
          if constexpr (kPair) {
            // both CTAs' bytes are counted on the leader's barrier; the leader announces the sum
            const uint32_t leader_full = map_to_cta(full_bar + 8 * stage, 0);
            if (pair_rank == 0) mbar_arrive_expect_tx(full_bar + 8 * stage, 2 * G::kStageBytes);
            tma_load_2d_pair(a_dst, &tma_a, leader_full, kb * kBlockK, tm * kTileM + static_cast<int>(pair_rank) * G::kBlockM);
            tma_load_2d_pair(b_dst, &tma_b, leader_full, kb * kBlockK, tn * G::kBlockN + static_cast<int>(pair_rank) * GemmPair::kBRows);
          } else {
            mbar_arrive_expect_tx(full_bar + 8 * stage, G::kStageBytes);
            int a_k = kb * kBlockK, b_k = kb * kBlockK;
            if constexpr (kTf32) {
              // the split fp32 product: k runs over three terms, a_hi.b_hi, a_lo.b_hi, a_hi.b_lo, of operands stored
              // as [hi | lo]
              const int term_kb = num_kb / 3, term = kb / term_kb, within = (kb - term * term_kb) * kBlockK;
              a_k = (term == 1 ? term_kb * kBlockK : 0) + within;
              b_k = (term == 2 ? term_kb * kBlockK : 0) + within;
            }
            tma_load_2d(a_dst, &tma_a, full_bar + 8 * stage, a_k, tm * G::kBlockM);
            tma_load_2d(b_dst, &tma_b, full_bar + 8 * stage, b_k, tn * G::kBlockN);
          }
          if (++stage == G::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && pair_rank == 0) {  // of a pair, only the leader issues
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      int tile_index = 0;
      GemmItem item;
      for (int round = 0; ok && round < kMaxRounds && gemm_item(round, num_tiles, num_kb, split, worker, workers, item); ++round, ++tile_index) {
        mark(1 + 2 * tile_index);  // MMA issuer reaches tile i
        if (!(kPair ? mbar_wait_cluster(tmem_empty_bar + 8 * acc, acc_phase ^ 1u, abort_flag)
                    : mbar_wait(tmem_empty_bar + 8 * acc, acc_phase ^ 1u, abort_flag))) {
          report_status(status, kStatusMmaWaitTmem);
          *abort_flag = 1;
          break;
        }
        tcgen05_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * G::kBlockN;
        if constexpr (kW8) {
          // per 64-k atom: the activation atom from its ring against the widened block of the same k
          int ws = 0;
          uint32_t wphase = 0;
          for (int atom = 2 * item.kb_begin; ok && atom < 2 * item.kb_end; ++atom) {
            if (!mbar_wait(wide_full_bar + 8 * ws, wphase, abort_flag) || !mbar_wait(full_bar + 8 * stage, phase, abort_flag)) {
              report_status(status, kStatusMmaWaitFull);
              *abort_flag = 1;
              ok = false;
              break;
            }
            tcgen05_fence_after_sync();
            const uint64_t a_desc = umma_smem_desc_sw128(smem_base + stage * G::kABytes);
            const uint64_t b_desc = umma_smem_desc_sw128(smem_base + GemmW8::kWideOffset + ws * GemmW8::kWideBytes);
#pragma unroll
            for (int kk = 0; kk < G::kBlockKBytes / 32; ++kk)
              umma_f16(tmem_d, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (atom != 2 * item.kb_begin || kk != 0) ? 1u : 0u);
            umma_commit(wide_empty_bar + 8 * ws);
            umma_commit(empty_bar + 8 * stage);
            if (++ws == GemmW8::kWideStages) { ws = 0; wphase ^= 1u; }
            if (++stage == G::kStages) { stage = 0; phase ^= 1u; }
          }
        } else
        for (int kb = item.kb_begin; kb < item.kb_end; ++kb) {
          if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag)) {
            report_status(status, kStatusMmaWaitFull);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tcgen05_fence_after_sync();
          const uint32_t a_src = smem_base + stage * G::kStageBytes;
          const uint64_t a_desc = umma_smem_desc_sw128(a_src);
          const uint64_t b_desc = umma_smem_desc_sw128(a_src + G::kABytes);
#pragma unroll
          for (int kk = 0; kk < G::kBlockKBytes / 32; ++kk) {
            // +32 bytes along K inside the swizzle atom = +2 in the address field
            const uint32_t accumulate = (kb != item.kb_begin || kk != 0) ? 1u : 0u;
            if constexpr (kPair) {
              if (kInt8) umma_i8_pair(tmem_d, a_desc + 2 * kk, b_desc + 2 * kk, idesc, accumulate);
              else umma_f16_pair(tmem_d, a_desc + 2 * kk, b_desc + 2 * kk, idesc, accumulate);
            } else {
              if (kInt8) umma_i8(tmem_d, a_desc + 2 * kk, b_desc + 2 * kk, idesc, accumulate);
              else if (kTf32) umma_tf32(tmem_d, a_desc + 2 * kk, b_desc + 2 * kk, idesc, accumulate);
              else umma_f16(tmem_d, a_desc + 2 * kk, b_desc + 2 * kk, idesc, accumulate);
            }
          }
          if constexpr (kPair) umma_commit_pair(empty_bar + 8 * stage);
          else umma_commit(empty_bar + 8 * stage);
          if (++stage == G::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if constexpr (kPair) umma_commit_pair(tmem_full_bar + 8 * acc);
        else umma_commit(tmem_full_bar + 8 * acc);
        mark(2 + 2 * tile_index);  // all MMAs of tile i issued
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (kW8 && warp >= 2 + G::kEpiWarps) {
    // ------------------------------------------------------------ widening warps (weight-only form)
    // A unit is 256 rows x 128 int8 under the 128-byte swizzle; each of its two 64-k halves becomes one 256 x 64 bf16
    // block under the same swizzle.  A thread takes 8 weights (8 bytes in, 16 bytes out) per step.  Lane l: piece
    // e = l % 8 of its row's 64-byte half, row (l / 8) of four; a warp-wide load covers rows {r, r+4, r+1, r+5} of an
    // 8-row block so that each half-warp's 128 bytes fall on all 32 banks (rows r and r+4 swizzle into opposite
    // halves of the 128-byte line), and each quarter-warp stores one whole 128-byte row.
    GemmItem item;
    if (gemm_item(0, num_tiles, num_kb, split, worker, workers, item)) {
      const int cw = warp - (2 + G::kEpiWarps);
      const int e = lane & 7, rsel = lane >> 3;
      const int units = item.kb_end - item.kb_begin;
      bool ok = true;
      int ws = 0;
      uint32_t wphase = 0;
      for (int u = 0; ok && u < units; ++u) {
        const int rs = u % GemmW8::kRawStages;
        const uint32_t rphase = static_cast<uint32_t>(u / GemmW8::kRawStages) & 1u;
        if (!mbar_wait(raw_full_bar + 8 * rs, rphase, abort_flag)) {
          if (lane == 0) {
            report_status(status, kStatusW8Wait);
            *abort_flag = 1;
          }
          break;
        }
        const uint32_t raw = smem_base + GemmW8::kRawOffset + rs * GemmW8::kRawBytes + cw * 4 * 1024;  // this warp's four 8-row blocks
        for (int half = 0; half < 2; ++half) {
          if (!mbar_wait(wide_empty_bar + 8 * ws, wphase ^ 1u, abort_flag)) {
            if (lane == 0) {
              report_status(status, kStatusW8Wait);
              *abort_flag = 1;
            }
            ok = false;
            break;
          }
          const uint32_t wide = smem_base + GemmW8::kWideOffset + ws * GemmW8::kWideBytes + cw * 4 * 1024;
          uint2 in[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rib = (rsel >> 1) + 4 * (rsel & 1) + 2 * (i & 1);  // row inside the 8-row block = row % 8
            const uint32_t src = raw + (i >> 1) * 1024 + rib * 128 + (((4 * half + (e >> 1)) ^ rib) << 4) + (e & 1) * 8;
            asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(in[i].x), "=r"(in[i].y) : "r"(src));
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rib = (rsel >> 1) + 4 * (rsel & 1) + 2 * (i & 1);
            uint32_t out[4];
            widen4_bf16(in[i].x, out[0], out[1]);
            widen4_bf16(in[i].y, out[2], out[3]);
            const uint32_t dst = wide + (i >> 1) * 1024 + rib * 128 + ((e ^ rib) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]) : "memory");
          }
          fence_proxy_async_smem();  // the tensor core reads these stores through the async proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(wide_full_bar + 8 * ws);
          if (++ws == GemmW8::kWideStages) { ws = 0; wphase ^= 1u; }
        }
        __syncwarp();
        if (ok && lane == 0) mbar_arrive(raw_empty_bar + 8 * rs);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32) belong to this warp
    const int epi_warp = warp - 2;
    const uint32_t my_buf = epi_base + epi_warp * 2 * G::kEpiBufBytes;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf_sel = 0;
    GemmItem item;
    bool epilogue_ok = true;
    for (int round = 0; epilogue_ok && round < kMaxRounds && gemm_item(round, num_tiles, num_kb, split, worker, workers, item); ++round) {
      int tm, tn;
      tile_coords(item.tile, tiles_m, tiles_n, raster_group, tm, tn);
      if (!mbar_wait(tmem_full_bar + 8 * acc, acc_phase, abort_flag)) {
        report_status(status, kStatusEpilogueWait);
        *abort_flag = 1;
        break;
      }
      tcgen05_fence_after_sync();
      const bool timeline = round == 0 && item.slices > 1 && warp == 2 && lane == 0;  // the exchange of a launch whose only round is split
      if (timeline) mark(3);
      const int row0 = tm * kTileM + static_cast<int>(pair_rank) * G::kBlockM + quarter * 32;
      const int row = row0 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * G::kBlockN;
      constexpr int kSlabs = G::kBlockN / kOutCols;
      int slab_begin = 0, slab_end = kSlabs;
      // partial accumulators of one split tile: [slice][column][row] 32-bit words, rows contiguous: the 32 lanes of a
      // warp write (and read) one column's 128 contiguous bytes per instruction.  (The transposed layout - a thread's 32
      // columns contiguous, 16-byte accesses - was measured: every instruction then touches 32 lines, and the exchange
      // took twice as long.)
      const size_t tile_words = static_cast<size_t>(G::kBlockN) * G::kBlockM;
      uint32_t* my_partial = nullptr;
      // scratch slot of slice `s` of this tile (of this CTA's half of it, for a pair)
      auto slot_of = [&](int s) {
        const size_t slot = static_cast<size_t>(item.tail_index) * item.slices + s;
        return kPair ? slot * 2 + pair_rank : slot;
      };
      if (item.slices > 1) {
        // this slice stores the columns [slab_begin, slab_end); the rest of its accumulator goes to the owners
        slab_begin = kSlabs * item.slice / item.slices;
        slab_end = kSlabs * (item.slice + 1) / item.slices;
        my_partial = partials + slot_of(item.slice) * tile_words + quarter * 32 + lane;
        auto goes_out = [&](int chunk) {  // warp-uniform: the chunk belongs to another slice's columns
          const int owner_slab = chunk * 32 / kOutCols;
          return owner_slab < slab_begin || owner_slab >= slab_end;
        };
        auto store_chunk = [&](int chunk, const uint32_t (&v)[32]) {
#pragma unroll
          for (int j = 0; j < 32; ++j) __stcg(my_partial + static_cast<size_t>(chunk * 32 + j) * G::kBlockM, v[j]);
        };
        // two chunks per tensor-memory wait: the second read-back overlaps the first chunk's stores
        for (int chunk = 0; chunk < G::kBlockN / 32; chunk += 2) {
          const bool first = goes_out(chunk), second = goes_out(chunk + 1);
          if (!first && !second) continue;
          uint32_t v0[32], v1[32];
          if (first) tmem_load_32x32(taddr + chunk * 32, v0);
          if (second) tmem_load_32x32(taddr + (chunk + 1) * 32, v1);
          tmem_load_wait();
          if (row < M) {  // rows past M are never stored
            if (first) store_chunk(chunk, v0);
            if (second) store_chunk(chunk + 1, v1);
          }
        }
        __threadfence();
        __syncwarp();
        if (timeline) mark(4);
        // every other slice reads this slice's partial sums: the flag counts those readers down (see ptx.cuh)
        const unsigned readers = static_cast<unsigned>(item.slices - 1);
        if (lane == 0) st_release_gpu_u64(flags + slot_of(item.slice) * 4 + quarter, nonce + readers);
        // lane s polls slice s's flag: all the flags are waited for at once, not one round trip after the other
        const bool polls = lane < item.slices && lane != item.slice;
        const bool seen = !polls || wait_flag_window_u64(flags + slot_of(lane) * 4 + quarter, nonce, readers, abort_flag);
        if (!__all_sync(0xffffffffu, seen)) {
          report_status(status, kStatusEpilogueWait);
          *abort_flag = 1;
          epilogue_ok = false;
        }
        if (!epilogue_ok) break;
        if (timeline) mark(5);
      }
      // adds the other slices' partial sums of 32 columns starting at `first_col` (column inside the tile)
      auto add_partials = [&](uint32_t (&v)[32], int first_col) {
        for (int other = 0; other < item.slices; ++other) {
          if (other == item.slice) continue;
          const uint32_t* src = partials + slot_of(other) * tile_words +
                                static_cast<size_t>(first_col) * G::kBlockM + quarter * 32 + lane;
          uint32_t part[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) part[j] = row < M ? __ldcg(src + static_cast<size_t>(j) * G::kBlockM) : 0u;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if constexpr (kInt8) v[j] += part[j];
            else v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(part[j]));
          }
        }
      };
      // accumulators of 32 consecutive columns of this thread's row -> what gets stored (still as 32-bit patterns):
      // int32 accumulators take their int32 accumulator input; when the output is floating point they are then converted
      // and run through the float transform (the dequantising form); fp32 accumulators take the float transform or, for
      // the plain GEMM, just the column scale
      auto transform32 = [&](uint32_t (&v)[32], int first_col) {
        if constexpr (kInt8) {
          if (ep.active) epilogue_int_row32(v, ep, row, first_col, M, N);
          if constexpr (!std::is_same<OutT, int32_t>::value) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(static_cast<float>(static_cast<int32_t>(v[j])));
            if (ep.active || column_scale != nullptr) epilogue_float_row32(v, ep, column_scale, row, first_col, M, N);
          }
        } else {
          if (ep.active) {
            epilogue_float_row32(v, ep, column_scale, row, first_col, M, N);
          } else if (column_scale != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float s = (first_col + j < N) ? __ldg(column_scale + first_col + j) : 0.f;
              v[j] = __float_as_uint(__uint_as_float(v[j]) * s);
            }
          }
        }
      };
#pragma unroll 1
      for (int slab = slab_begin; slab < slab_end; ++slab) {
        const int col0 = tn * G::kBlockN + slab * kOutCols;
        if (col0 >= N) break;  // uniform across the warp
        uint32_t words[32];    // 128 bytes of converted output for this thread's row
        if constexpr (sizeof(OutT) == 4) {
          tmem_load_32x32(taddr + slab * 32, words);
          tmem_load_wait();
          if (item.slices > 1) add_partials(words, slab * 32);
          transform32(words, col0);
        } else {
          uint32_t v0[32], v1[32];
          tmem_load_32x32(taddr + slab * 64, v0);
          tmem_load_32x32(taddr + slab * 64 + 32, v1);
          tmem_load_wait();
          if (item.slices > 1) {
            add_partials(v0, slab * 64);
            add_partials(v1, slab * 64 + 32);
          }
          transform32(v0, col0);
          transform32(v1, col0 + 32);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            words[j] = pack_out16x2<OutT>(__uint_as_float(v0[2 * j]), __uint_as_float(v0[2 * j + 1]));
            words[16 + j] = pack_out16x2<OutT>(__uint_as_float(v1[2 * j]), __uint_as_float(v1[2 * j + 1]));
          }
        }
        if (use_tma_store == 2) {
          // Multicast gather: stage the 32-row x 128-byte slab as for a TMA store, then read it back four rows at a
          // time - eight lanes per row, 16 bytes per lane, 128 contiguous bytes per row on the wire - and store to the
          // multicast address of the full result.  (`c` is that address, `ldc` the full result's pitch.)
          const uint32_t buf = my_buf + buf_sel * G::kEpiBufBytes;
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t dst = buf + lane * 128 + ((j ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(words[4 * j]),
                         "r"(words[4 * j + 1]), "r"(words[4 * j + 2]), "r"(words[4 * j + 3])
                         : "memory");
          }
          __syncwarp();
          const int chunk = lane & 7;
          const int chunk_col = col0 + chunk * (16 / static_cast<int>(sizeof(OutT)));
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + (lane >> 3);
            uint4 piece;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(piece.x), "=r"(piece.y), "=r"(piece.z), "=r"(piece.w)
                         : "r"(buf + r * 128 + ((chunk ^ (r & 7)) << 4)));
            if (row0 + r < M && chunk_col < N)
              multimem_st_v4(c + static_cast<long long>(row0 + r) * ldc + c_col_offset + chunk_col, piece);
          }
          buf_sel ^= 1;
        } else if (use_tma_store) {
          const uint32_t buf = my_buf + buf_sel * G::kEpiBufBytes;
          // the store issued two slabs ago from this buffer must have read it
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t dst = buf + lane * 128 + ((j ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(words[4 * j]),
                         "r"(words[4 * j + 1]), "r"(words[4 * j + 2]), "r"(words[4 * j + 3])
                         : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            // one bulk group per slab, however many destinations read the staging buffer
            for (int d = 0; d < num_dest; ++d) tma_store_2d(&tma_c.map[d], buf, c_col_offset + col0, row0);
            tma_store_commit();
          }
          buf_sel ^= 1;
        } else if (row < M) {
          OutT* dst = c + static_cast<long long>(row) * ldc + col0;
          const int valid = min(kOutCols, N - col0);
          const bool vec = valid == kOutCols && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
          if (vec) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              reinterpret_cast<uint4*>(dst)[j] =
                  make_uint4(words[4 * j], words[4 * j + 1], words[4 * j + 2], words[4 * j + 3]);
          } else {
            // ragged or unaligned edge: element stores, indices kept static so
            // that `words` stays in registers
#pragma unroll
            for (int j = 0; j < kOutCols; ++j) {
              if (j < valid) {
                if constexpr (sizeof(OutT) == 4) {
                  reinterpret_cast<uint32_t*>(dst)[j] = words[j];
                } else {
                  reinterpret_cast<uint16_t*>(dst)[j] = static_cast<uint16_t>(words[j >> 1] >> (16 * (j & 1)));
                }
              }
            }
          }
        }
      }
      if (item.slices > 1) {
        // this warp has read all it needs of the other slices' partial sums
        if (timeline) mark(6);
        __syncwarp();
        if (lane == 0)
          for (int other = 0; other < item.slices; ++other)
            if (other != item.slice) flag_reader_done_u64(flags + slot_of(other) * 4 + quarter);
      }
      tcgen05_fence_before_sync();
      if constexpr (kPair) mbar_arrive_cluster(map_to_cta(tmem_empty_bar + 8 * acc, 0));
      else mbar_arrive(tmem_empty_bar + 8 * acc);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (use_tma_store == 1 && lane == 0) tma_store_wait_all<0>();
    if (warp == 2 && lane == 0) {
      mark(15);
      if (trace != nullptr) trace[blockIdx.x * 16 + 14] = static_cast<unsigned long long>(clock64());  // ... and at the end
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncthreads();
  if (*abort_flag != 0) {
    // A wait ran out: give copies and MMAs still in flight time to land
    // before shared memory and TMEM go back to the SM.
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
