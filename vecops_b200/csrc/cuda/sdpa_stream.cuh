// Scaled dot-product attention, streaming strategy: one kernel, no score matrix in device memory.
//
// vecops' streaming strategy (include/vecops/ops/details/attention/SparseFlashAttention.h:360-545 driven over every
// key/value block, :993-1010) walks the keys block by block with a running row maximum m, a running row sum l and an
// unnormalised output accumulator O:
//     s = (Q.K_j^T) * scale + bias, -inf where a mask or the causal cut drops the pair
//     m' = max(m, max_j s)        p = exp(s - m') rounded to the matmul operand type (bf16)      alpha = exp(m - m')
//     l = alpha * l + sum p (unrounded)          O = alpha * O + p.V_j          out = O / l (0 where nothing was kept)
// This kernel is that recurrence on the tensor cores of one SM per work item:
//   * a work item is one block of 128 query rows of one head against a chunk of consecutive 128-key tiles; a query
//     block whose keys are cut into several chunks (few query blocks, many SMs) leaves each chunk's (O, m, l) in device
//     scratch, and sdpa_merge_kernel, launched behind this one, merges them by the same rule on all SMs at once;
//   * warp 0 streams K tiles and V tiles through TMA into two-stage rings; Q is loaded once.  V is used as it lies in
//     memory, [key][head dim]: the second product takes it as an N-major operand, nothing is transposed;
//   * warp 1 issues tcgen05.mma: S_j = Q.K_j^T into one of two 128x128 fp32 accumulators in tensor memory, and
//     O += P_j.V_j into a third.  S_{j+1} is issued before P_j is needed, so it overlaps the softmax of tile j;
//     the K ring and the V ring are released separately (K after the scores, V after the product);
//   * sixteen softmax warps, four threads per query row (row = tensor-memory lane; each takes 32 of the tile's 128 keys and
//     32 of the output columns): they read S_j once into registers, agree on the row maximum through shared memory and
//     write P_j as bf16 into shared memory in the 128-byte-swizzled K-major layout the MMA reads.  O accumulates in
//     tensor memory over all tiles; a warp multiplies its rows of O by alpha there (load, scale, store) only when one of
//     them got a new maximum - alpha = 1 changes nothing - which for typical scores is the first few tiles.  Scores
//     are kept in units of log2(e), so a probability is one subtraction and one ex2.
// Every wait is bounded; a wait that runs out reports a status code and the CTA tears down normally.
#pragma once

#include <cuda_bf16.h>
#include <math.h>

#include <type_traits>

#include "gemm_tcgen05.cuh"  // status codes, report_status
#include "ptx.cuh"

namespace vb200 {

struct SdpaStream {
  static constexpr int kBlockQ = 128;
  static constexpr int kBlockKv = 128;
  static constexpr int kMaxHeadDim = 128;
  static constexpr int kAtomBytes = 128 * 128;  // 128 rows x 128 bytes: 64 bf16 along K under the 128-byte swizzle
  static constexpr int kStages = 2;
  static constexpr int kQOffset = 0;
  static constexpr int kQBytes = 2 * kAtomBytes;
  static constexpr int kKOffset = kQOffset + kQBytes;
  static constexpr int kKBytes = 2 * kAtomBytes;  // 128 keys x 128 head dims
  static constexpr int kVOffset = kKOffset + kStages * kKBytes;
  static constexpr int kVBytes = 2 * kAtomBytes;  // 128 keys x 128 head dims, as V lies in memory: two boxes of 64 head dims
  static constexpr int kPOffset = kVOffset + kStages * kVBytes;
  static constexpr int kPBytes = 2 * kAtomBytes;  // 128 query rows x 128 keys, one buffer: free again when the product that read it is
  static constexpr int kBarrierOffset = kPOffset + kPBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSplit = 4;  // threads per query row
  static constexpr int kExchangeOffset = kBarrierOffset + kBarrierBytes;  // row maxima of the row's threads: [tile parity][part][row] f32
  static constexpr int kExchangeBytes = 2 * kSplit * kBlockQ * 4;
  static constexpr int kAlignSlack = 1024;  // what the 1024-byte alignment of the operand rings may cost
  static constexpr int kSmemBytes = kExchangeOffset + kExchangeBytes + kAlignSlack;
  static constexpr int kSoftmaxWarps = 4 * kSplit;
  static constexpr int kThreads = 32 * (2 + kSoftmaxWarps);
  static constexpr int kTmemColumns = 512;  // S at columns 0 and 128, O at 256 (allocations are powers of two)
  static constexpr int kPartialFloats = kBlockQ * kMaxHeadDim + 2 * kBlockQ;  // O, then m, then l
  static constexpr int kMaxChunks = 32;  // chunks a query block's keys are cut into at most (the grid's x extent)
};
static_assert(SdpaStream::kSmemBytes <= 227 * 1024, "shared memory budget");

struct SdpaStreamParams {
  int lq, lkv, dqk, dv;
  int causal;           // 0 none, 1 top left, 2 bottom right
  int tiles_per_chunk;  // 128-key tiles per work item
  int q_blocks;         // blocks of 128 query rows per head
  int max_chunks;       // chunks of the query block with the most keys (the stride of the partial records)
  int uniform_chunks;   // chunks per query block when all blocks have the same number, else 0
  int q_head, k_head, v_head;  // 1 when the operand has one slab per head, 0 when all heads share it
  float scale;
  void* out;
  long long out_sr, out_sc, out_sh;
  int out_bf16;
  const uint8_t* query_mask;
  long long query_mask_sh;
  const uint8_t* key_mask;
  long long key_mask_sh;
  const uint8_t* keep_mask;
  long long keep_sr, keep_sc, keep_sh;
  const float* bias;
  long long bias_sr, bias_sc, bias_sh;
  float* partials;               // [head][query block][chunk] records of kPartialFloats, when any block is cut
  uint32_t* status;
  unsigned long long* trace;     // optional timeline for tuning, 16 words per work item (null: none)
};

__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// kPlain: no key mask, no two-dimensional keep mask, no bias (the query mask and the causal cut cost nothing).
template <bool kPlain, bool kTrace = false>
__global__ void __launch_bounds__(SdpaStream::kThreads, 1)
sdpa_stream_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const SdpaStreamParams p) {
  using G = SdpaStream;
  // ---------------------------------------------------------------- which work item
  // The grid's x extent counts the work items of one head, query blocks with the most keys first, a block's chunks next
  // to each other; y counts the heads.  Every CTA is a work item: with one CTA per SM an idle CTA would cost a slot.
  const int head = blockIdx.y;
  const long long shift = p.causal == 2 ? static_cast<long long>(p.lkv) - p.lq : 0;
  auto tiles_of = [&](int block) {  // 128-key tiles the causal cut leaves to query block `block`
    const int first_row = block * G::kBlockQ;
    const int block_rows = min(G::kBlockQ, p.lq - first_row);
    const long long last_key = p.causal != 0 ? min(static_cast<long long>(p.lkv) - 1, first_row + block_rows - 1 + shift) : p.lkv - 1;
    return last_key < 0 ? 0 : static_cast<int>(last_key / G::kBlockKv) + 1;
  };
  auto chunks_of = [&](int tiles) { return max(1, (tiles + p.tiles_per_chunk - 1) / p.tiles_per_chunk); };
  int qb, chunk;
  if (p.uniform_chunks > 0) {  // every block is cut the same way (no causal cut, or no block is cut at all)
    qb = p.q_blocks - 1 - static_cast<int>(blockIdx.x) / p.uniform_chunks;
    chunk = static_cast<int>(blockIdx.x) % p.uniform_chunks;
  } else {
    int remaining = blockIdx.x;
    for (qb = p.q_blocks - 1; qb >= 0; --qb) {
      const int n = chunks_of(tiles_of(qb));
      if (remaining < n) break;
      remaining -= n;
    }
    chunk = remaining;
  }
  if (qb < 0) return;  // (the host sized the grid from the same arithmetic: not reached)
  const int r0 = qb * G::kBlockQ;
  const int tiles_total = tiles_of(qb);
  const int n_chunks = chunks_of(tiles_total);
  const int tile_begin = chunk * p.tiles_per_chunk;
  const int ntiles = max(0, min(tiles_total, tile_begin + p.tiles_per_chunk) - tile_begin);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + G::kBarrierOffset;
  const uint32_t q_full = bar_base;
  const uint32_t k_full = bar_base + 8;     // [2] K tile landed                   (TMA -> MMA)
  const uint32_t k_empty = bar_base + 24;   // [2] the scores that read it done    (MMA -> TMA)
  const uint32_t v_full = bar_base + 40;    // [2] V^T tile landed                 (TMA -> MMA)
  const uint32_t v_empty = bar_base + 56;   // [2] the product that read it done   (MMA -> TMA)
  const uint32_t s_full = bar_base + 72;    // [2] S_j in tensor memory            (MMA -> softmax)
  const uint32_t s_free = bar_base + 88;    // [2] S_j in the softmax registers    (softmax -> MMA)
  const uint32_t pv_done = bar_base + 104;  //     O += P_j.V_j done, P_j read      (MMA -> softmax)
  const uint32_t p_full = bar_base + 112;   //     P_j in shared memory, O rescaled (softmax -> MMA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + G::kBarrierOffset + 160);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + G::kBarrierOffset + 164);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // optional timeline: nanosecond stamps (slots 0-6, 15) and cycle sums of one softmax thread (slots 7-14)
  unsigned long long* trace = !kTrace || p.trace == nullptr ? nullptr : p.trace + (static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * 16;
  auto stamp = [&](int slot) {
    if (trace != nullptr) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      trace[slot] = now;
    }
  };
  if (threadIdx.x == 0) stamp(0);
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full + 8 * s, 1);
      mbar_init(k_empty + 8 * s, 1);
      mbar_init(v_full + 8 * s, 1);
      mbar_init(v_empty + 8 * s, 1);
      mbar_init(s_full + 8 * s, 1);
      mbar_init(s_free + 8 * s, G::kSoftmaxWarps);
    }
    mbar_init(pv_done, 1);
    mbar_init(p_full, G::kSoftmaxWarps);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_descriptor(&map_q);
    tma_prefetch_descriptor(&map_k);
    tma_prefetch_descriptor(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), G::kTmemColumns);
    tmem_relinquish();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  grid_launch_dependents();
  grid_dependency_wait();
  if (threadIdx.x == 0) stamp(1);

  auto give_up = [&](uint32_t code) {
    report_status(p.status, code);
    *abort_flag = 1;
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && ntiles > 0) {
      mbar_arrive_expect_tx(q_full, G::kQBytes);
      tma_load_3d(smem_base + G::kQOffset, &map_q, q_full, 0, r0, head * p.q_head);
      tma_load_3d(smem_base + G::kQOffset + G::kAtomBytes, &map_q, q_full, 64, r0, head * p.q_head);  // past Dqk: zero-filled
      // two rings, neither waiting for the other: a K stage is free as soon as its scores are done, long before the
      // product of the same tile frees the V stage
      int k_issued = 0, v_issued = 0;
      const long long started = clock64();
      while (k_issued < ntiles || v_issued < ntiles) {
        bool progress = false;
        if (k_issued < ntiles && mbar_test_wait(k_empty + 8 * (k_issued & 1), (static_cast<uint32_t>(k_issued >> 1) & 1u) ^ 1u)) {
          const int s = k_issued & 1;
          const int key0 = (tile_begin + k_issued) * G::kBlockKv;
          mbar_arrive_expect_tx(k_full + 8 * s, G::kKBytes);
          tma_load_3d(smem_base + G::kKOffset + s * G::kKBytes, &map_k, k_full + 8 * s, 0, key0, head * p.k_head);
          tma_load_3d(smem_base + G::kKOffset + s * G::kKBytes + G::kAtomBytes, &map_k, k_full + 8 * s, 64, key0, head * p.k_head);
          ++k_issued;
          progress = true;
        }
        if (v_issued < ntiles && mbar_test_wait(v_empty + 8 * (v_issued & 1), (static_cast<uint32_t>(v_issued >> 1) & 1u) ^ 1u)) {
          const int s = v_issued & 1;
          const int key0 = (tile_begin + v_issued) * G::kBlockKv;
          mbar_arrive_expect_tx(v_full + 8 * s, G::kVBytes);
          tma_load_3d(smem_base + G::kVOffset + s * G::kVBytes, &map_v, v_full + 8 * s, 0, key0, head * p.v_head);
          tma_load_3d(smem_base + G::kVOffset + s * G::kVBytes + G::kAtomBytes, &map_v, v_full + 8 * s, 64, key0, head * p.v_head);  // past Dv: zero-filled
          ++v_issued;
          progress = true;
        }
        if (!progress) {
          if (*abort_flag != 0 || clock64() - started > 8 * kWaitCycleBudget) {  // (the whole item, not one wait)
            give_up(kStatusProducerWait);
            break;
          }
          __nanosleep(64);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && ntiles > 0) {
      constexpr uint32_t idesc = umma_instr_desc(kUmmaAccF32, kUmmaBF16, kUmmaBF16, 128, 128);
      constexpr uint32_t idesc_pv = umma_instr_desc(kUmmaAccF32, kUmmaBF16, kUmmaBF16, 128, 128, true);  // B = V, N-major
      const int q_steps = (p.dqk + 15) / 16;  // 16 head dims per instruction; what lies past Dqk is zero in both operands
      bool ok = true;
      // S_i = Q . K_i^T into S[i % 2]
      auto issue_scores = [&](int i) {
        const int s = i & 1;
        const uint32_t parity = static_cast<uint32_t>(i >> 1) & 1u;
        if (!mbar_wait(k_full + 8 * s, parity, abort_flag) || !mbar_wait(s_free + 8 * s, parity ^ 1u, abort_flag)) {
          give_up(kStatusMmaWaitFull);
          return false;
        }
        tcgen05_fence_after_sync();
        for (int ks = 0; ks < q_steps; ++ks) {
          const uint64_t a_desc = umma_smem_desc_sw128(smem_base + G::kQOffset + (ks >> 2) * G::kAtomBytes) + 2 * (ks & 3);
          const uint64_t b_desc = umma_smem_desc_sw128(smem_base + G::kKOffset + s * G::kKBytes + (ks >> 2) * G::kAtomBytes) + 2 * (ks & 3);
          umma_f16(tmem_base + s * 128, a_desc, b_desc, idesc, ks > 0 ? 1u : 0u);
        }
        umma_commit(s_full + 8 * s);
        umma_commit(k_empty + 8 * s);
        return true;
      };
      if (!mbar_wait(q_full, 0, abort_flag)) {
        give_up(kStatusMmaWaitFull);
        ok = false;
      }
      ok = ok && issue_scores(0);
      for (int i = 0; ok && i < ntiles; ++i) {
        if (i + 1 < ntiles && !issue_scores(i + 1)) break;
        const int s = i & 1;
        const uint32_t parity = static_cast<uint32_t>(i >> 1) & 1u;
        if (!mbar_wait(p_full, static_cast<uint32_t>(i) & 1u, abort_flag) || !mbar_wait(v_full + 8 * s, parity, abort_flag)) {
          give_up(kStatusMmaWaitTmem);
          break;
        }
        tcgen05_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < G::kBlockKv / 16; ++ks) {
          const uint64_t a_desc = umma_smem_desc_sw128(smem_base + G::kPOffset + (ks >> 2) * G::kAtomBytes) + 2 * (ks & 3);
          // V as it lies in memory, [key][head dim]: the N-major operand.  16 keys per instruction = 16 rows of 128 bytes.
          const uint64_t b_desc = umma_smem_desc_sw128_mn(smem_base + G::kVOffset + s * G::kVBytes + ks * 16 * 128, G::kAtomBytes, 1024);
          umma_f16(tmem_base + 256, a_desc, b_desc, idesc_pv, (i > 0 || ks > 0) ? 1u : 0u);  // O accumulates over the tiles
        }
        umma_commit(pv_done);
        umma_commit(v_empty + 8 * s);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps: four threads per query row
    // The warps w, w + 4, w + 8, w + 12 read the same quarter of the tensor-memory lanes (a warp's lanes are fixed by its
    // index modulo 4); of a row's 128 scores, 128 probabilities and 128 output columns each takes 32.  The four meet once
    // per tile, to agree on the row maximum, through shared memory and a 128-thread barrier; each keeps the row sum of its
    // own part and the parts are added at the end (the recurrence is linear in l).  Sixteen warps, four per scheduler,
    // are what hides the latency of the tensor-memory loads behind the other warps' arithmetic.
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;
    const int row_local = quarter * 32 + lane;
    const int row = r0 + row_local;
    const bool row_valid = row < p.lq;
    const uint8_t* query_mask = p.query_mask == nullptr ? nullptr : p.query_mask + head * p.query_mask_sh;
    const uint8_t* key_mask = kPlain || p.key_mask == nullptr ? nullptr : p.key_mask + head * p.key_mask_sh;
    const uint8_t* keep_row = kPlain || p.keep_mask == nullptr ? nullptr : p.keep_mask + head * p.keep_sh + row * p.keep_sr;
    const float* bias_row = kPlain || p.bias == nullptr ? nullptr : p.bias + head * p.bias_sh + row * p.bias_sr;
    const bool query_active = row_valid && (query_mask == nullptr || query_mask[row] != 0);
    const long long row_last_key = p.causal != 0 ? row + shift : static_cast<long long>(p.lkv) - 1;
    // keys [0, limit) survive the query mask, the causal cut and the end of the keys
    const int limit = !query_active ? 0 : static_cast<int>(row_last_key + 1 < 0 ? 0 : (row_last_key + 1 < p.lkv ? row_last_key + 1 : p.lkv));
    const float negative_infinity = -INFINITY;
    constexpr float kLog2e = 1.4426950408889634f;
    const float scale_log2 = p.scale * kLog2e;
    // A score in units of log2(e): exp(s - m) is ex2 of a difference of these.  `cut`: the tile reaches past `limit`.
    auto decorated = [&](int j, float score, bool cut) {
      if (cut && j >= limit) return negative_infinity;
      if constexpr (kPlain) {
        return score * scale_log2;
      } else {
        float value = __fmul_rn(score, p.scale);
        if (bias_row != nullptr) value = __fadd_rn(value, bias_row[j * p.bias_sc]);
        const bool keep = (key_mask == nullptr || key_mask[j] != 0) && (keep_row == nullptr || keep_row[j * p.keep_sc] != 0);
        return keep ? value * kLog2e : negative_infinity;
      }
    };
    constexpr int kCols = G::kBlockKv / G::kSplit;  // scores, probabilities and output columns per thread
    static_assert(kCols == 32, "one 32-column tensor-memory load per thread and tile");
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + part * kCols;
    // this thread's 32 keys inside P: atom = 64 keys, then four 16-byte pieces of the row, swizzled by the row
    const uint32_t p_row = smem_base + G::kPOffset + (part >> 1) * G::kAtomBytes + (row_local >> 3) * 1024 + (row_local & 7) * 128;
    float* row_max_of = reinterpret_cast<float*>(smem_gen + G::kExchangeOffset);  // [tile parity][part][row]
    float m = negative_infinity, l = 0.f;
    bool ok = true;
    const bool tracing = kTrace && trace != nullptr && warp == 2 && lane == 0;
    long long spent[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    long long mark = 0;
    auto lap = [&](int what) {  // cycles since the previous lap go to `what`
      if constexpr (!kTrace) return;
      if (tracing) {
        const long long now = clock64();
        spent[what] += now - mark;
        mark = now;
      }
    };
    auto fail = [&](uint32_t code) {
      if (lane == 0) give_up(code);
      ok = false;
    };
    const uint32_t o_base = lane_base + 256;  // this thread's 32 columns of O in tensor memory
    // The product of tile j is in O and P is free again.  (Warp-wide: tensor-memory accesses follow.)
    auto product_done = [&](int j) {
      if (!__all_sync(0xffffffffu, mbar_wait(pv_done, static_cast<uint32_t>(j) & 1u, abort_flag))) {
        fail(kStatusEpilogueWait);
        return;
      }
      tcgen05_fence_after_sync();
    };
    if (tracing) mark = clock64();
    for (int i = 0; i < ntiles; ++i) {
      lap(7);  // adding the product, loop bookkeeping
      // (a thread whose wait ran out keeps walking the tiles without touching anything: its partners meet it at every barrier)
      const int s = i & 1;
      const int key0 = (tile_begin + i) * G::kBlockKv + part * kCols;  // first key of this thread's part of the tile
      // One decision per WARP: what follows holds warp-wide tensor-memory loads (.sync.aligned), which every lane of
      // the warp must reach together - a per-lane choice would split the warp on the diagonal tiles of a causal cut.
      const bool cut = __any_sync(0xffffffffu, key0 + kCols > limit);
      if (ok && !__all_sync(0xffffffffu, mbar_wait(s_full + 8 * s, static_cast<uint32_t>(i >> 1) & 1u, abort_flag))) fail(kStatusEpilogueWait);
      // this part of the row of S into registers, once; the accumulator goes back to the tensor core at once
      float t[kCols];
      float part_max = negative_infinity;
      lap(0);  // waiting for the scores
      if (i == 0 && tracing) stamp(2);
      if (ok) {
        tcgen05_fence_after_sync();
        uint32_t v[kCols];
        tmem_load_32x32(lane_base + s * 128, v);
        tmem_load_wait();
        lap(1);  // reading them
        tcgen05_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free + 8 * s);
        if (cut) {
#pragma unroll
          for (int e = 0; e < kCols; ++e) t[e] = decorated(key0 + e, __uint_as_float(v[e]), true);
        } else {
#pragma unroll
          for (int e = 0; e < kCols; ++e) t[e] = decorated(key0 + e, __uint_as_float(v[e]), false);
        }
#pragma unroll
        for (int e = 0; e < kCols; ++e) part_max = fmaxf(part_max, t[e]);
      }
      lap(2);  // scaling, masking, maximum
      float* exchange = row_max_of + (i & 1) * G::kSplit * G::kBlockQ;
      exchange[part * G::kBlockQ + row_local] = part_max;
      asm volatile("bar.sync %0, %1;" ::"r"(2 + quarter), "n"(32 * G::kSplit) : "memory");
      float tile_max = part_max;
#pragma unroll
      for (int other = 1; other < G::kSplit; ++other) tile_max = fmaxf(tile_max, exchange[((part + other) % G::kSplit) * G::kBlockQ + row_local]);
      lap(3);  // meeting the other parts of the row
      const float m_new = fmaxf(m, tile_max);
      // nothing kept so far: every p is 0 and alpha is 1 (the reference's "block not valid" branch)
      const float m_use = m_new == negative_infinity ? 0.f : m_new;
      const float alpha = m_new == negative_infinity ? 1.f : exp2_approx(m - m_new);  // m = -inf: 0
      if (ok && i > 0) {
        // The product of the tile before this one has to be done before P is written again - and before O is rescaled,
        // which happens only when some row of this warp got a new maximum (alpha = 1 leaves O as it is, exactly); with
        // typical scores the maximum settles after a few tiles and most tiles skip this.
        product_done(i - 1);
        lap(5);  // waiting for the product
        if (ok && __any_sync(0xffffffffu, alpha != 1.f)) {
          uint32_t v[kCols];
          tmem_load_32x32(o_base, v);
          tmem_load_wait();
#pragma unroll
          for (int e = 0; e < kCols; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
          tmem_store_32x32(o_base, v);
          tmem_store_wait();
          tcgen05_fence_before_sync();  // ... before the arrival below lets the next product accumulate into it
          lap(6);  // rescaling O
        }
      }
      if (ok) {
        // p = exp(s - m'), summed unrounded, stored as bf16 where the MMA reads its A operand
        float sum = 0.f;
#pragma unroll
        for (int piece = 0; piece < kCols / 8; ++piece) {
          uint32_t packed[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float p0 = exp2_approx(t[piece * 8 + 2 * e] - m_use);
            const float p1 = exp2_approx(t[piece * 8 + 2 * e + 1] - m_use);
            sum += p0 + p1;
            const __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
            packed[e] = *reinterpret_cast<const uint32_t*>(&pair);
          }
          const uint32_t dst = p_row + ((((part & 1) * 4 + piece) ^ (row_local & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3]) : "memory");
        }
        l = fmaf(l, alpha, sum);
        fence_proxy_async_smem();  // the tensor core reads P through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
        lap(4);  // exponentials, probabilities to shared memory
      }
      m = m_new;
    }
    if (tracing) stamp(3);
    // O leaves tensor memory once, at the end
    float o[kCols];
#pragma unroll
    for (int d = 0; d < kCols; ++d) o[d] = 0.f;
    if (ok && ntiles > 0) {
      product_done(ntiles - 1);
      if (ok) {
        uint32_t v[kCols];
        tmem_load_32x32(o_base, v);
        tmem_load_wait();
#pragma unroll
        for (int e = 0; e < kCols; ++e) o[e] = __uint_as_float(v[e]);
      }
    }
    if (tracing) {
      lap(7);
      stamp(4);
      for (int w = 0; w < 8; ++w) trace[7 + w] = static_cast<unsigned long long>(spent[w]);
      trace[6] = static_cast<unsigned long long>(ntiles);
    }
    // the row sum: this part's plus the other parts' (through the exchange buffer the last tile did not use)
    {
      float* exchange = row_max_of + (ntiles & 1) * G::kSplit * G::kBlockQ;
      exchange[part * G::kBlockQ + row_local] = l;
      asm volatile("bar.sync %0, %1;" ::"r"(2 + quarter), "n"(32 * G::kSplit) : "memory");
#pragma unroll
      for (int other = 1; other < G::kSplit; ++other) l += exchange[((part + other) % G::kSplit) * G::kBlockQ + row_local];
    }

    // ---------------------------------------------------------------- a chunk's state to scratch, or the block's result
    const size_t block_index = static_cast<size_t>(head) * p.q_blocks + qb;
    // every softmax thread gets here whatever happened above
    asm volatile("bar.sync 1, %0;" ::"n"(G::kSoftmaxWarps * 32) : "memory");
    ok = *abort_flag == 0;
    const bool store = ok && n_chunks == 1;
    if (ok && n_chunks > 1) {
      // (O, m, l) of this chunk for sdpa_merge_kernel: O as [column][row], so that the 32 rows of a warp lie side by side
      float* mine = p.partials + (block_index * p.max_chunks + chunk) * G::kPartialFloats;
#pragma unroll
      for (int d = 0; d < kCols; ++d) __stcg(mine + (part * kCols + d) * G::kBlockQ + row_local, o[d]);
      if (part == 0) {
        __stcg(mine + G::kBlockQ * G::kMaxHeadDim + row_local, m);
        __stcg(mine + G::kBlockQ * G::kMaxHeadDim + G::kBlockQ + row_local, l);
      }
    }
    if (store) {  // (uniform over the softmax warps)
      // A block that was not cut: normalise and store.  Through shared memory - the K and V rings are idle by now, every
      // product that read them is done - so that a warp stores whole rows, lanes side by side along the columns.
      constexpr int kPitch = G::kMaxHeadDim + 1;
      static_assert(G::kBlockQ * kPitch * 4 <= G::kStages * (G::kKBytes + G::kVBytes), "the output tile lies over the K and V rings");
      float* tile = reinterpret_cast<float*>(smem_gen + G::kKOffset);
      const float reciprocal = l > 0.f ? 1.f / l : 0.f;  // nothing kept in the row: zeros
#pragma unroll
      for (int d = 0; d < kCols; ++d) tile[row_local * kPitch + part * kCols + d] = o[d] * reciprocal;
      asm volatile("bar.sync 1, %0;" ::"n"(G::kSoftmaxWarps * 32) : "memory");
      const int rows_here = min(G::kBlockQ, p.lq - r0);
      const int d = lane * 4;
      for (int r = warp - 2; r < rows_here; r += G::kSoftmaxWarps) {
        char* out_row = static_cast<char*>(p.out) + (head * p.out_sh + static_cast<long long>(r0 + r) * p.out_sr) * (p.out_bf16 ? 2 : 4);
        const float* src = tile + r * kPitch + d;
        const bool wide = p.out_sc == 1 && (reinterpret_cast<uintptr_t>(out_row) & 15u) == 0 && (p.dv & 3) == 0;
        if (wide && d < p.dv) {
          if (p.out_bf16) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(src[0], src[1]), hi = __floats2bfloat162_rn(src[2], src[3]);
            *reinterpret_cast<uint2*>(out_row + d * 2) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
          } else {
            *reinterpret_cast<float4*>(out_row + d * 4) = make_float4(src[0], src[1], src[2], src[3]);
          }
        } else if (!wide) {
          for (int e = 0; e < 4; ++e) {
            if (d + e < p.dv) {
              if (p.out_bf16) reinterpret_cast<__nv_bfloat16*>(out_row)[(d + e) * p.out_sc] = __float2bfloat16_rn(src[e]);
              else reinterpret_cast<float*>(out_row)[(d + e) * p.out_sc] = src[e];
            }
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  if (warp == 2 && lane == 0) stamp(5);
  __syncthreads();
  if (threadIdx.x == 0) stamp(15);
  if (*abort_flag != 0) {
    // a wait ran out: give copies and MMAs still in flight time to land before shared and tensor memory go back
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_base, G::kTmemColumns);
  }
}

// Merges the chunk states of every query block that was cut: (m, l, O) = (max m_c, sum l_c 2^(m_c - m), sum O_c 2^(m_c - m)),
// out = O / l.  One CTA per 32 rows of a query block, sixteen warps of 8 output columns each; reads are coalesced (the
// records keep O as [column][row]) and the loads of eight chunks are in flight together - the kernel is nothing but
// memory latency, so what counts is how many round trips it takes.  Blocks that were not cut were stored by
// sdpa_stream_kernel itself.
constexpr int kMergeThreads = 512;
__global__ void __launch_bounds__(kMergeThreads) sdpa_merge_kernel(const SdpaStreamParams p) {
  using G = SdpaStream;
  const int head = blockIdx.y;
  const int qb = static_cast<int>(blockIdx.x >> 2);
  const int lane = threadIdx.x & 31, part = threadIdx.x >> 5;
  const int first_row_local = static_cast<int>(blockIdx.x & 3) * 32;  // (signed: the row arithmetic below goes below zero past Lq)
  const int row_local = first_row_local + lane;
  const long long shift = p.causal == 2 ? static_cast<long long>(p.lkv) - p.lq : 0;
  const int block_rows = min(G::kBlockQ, p.lq - qb * G::kBlockQ);
  const long long last_key = p.causal != 0 ? min(static_cast<long long>(p.lkv) - 1, qb * G::kBlockQ + block_rows - 1 + shift) : p.lkv - 1;
  const int tiles = last_key < 0 ? 0 : static_cast<int>(last_key / G::kBlockKv) + 1;
  const int n_chunks = max(1, (tiles + p.tiles_per_chunk - 1) / p.tiles_per_chunk);
  grid_dependency_wait();  // (launched as a programmatic dependent of the kernel that writes the records)
  if (n_chunks == 1) return;  // (uniform over the CTA)
  constexpr int kCols = G::kMaxHeadDim / (kMergeThreads / 32);  // 8
  constexpr int kGroup = 8;                                      // chunks whose loads are in flight together
  const size_t block_index = static_cast<size_t>(head) * p.q_blocks + qb;
  const float* first = p.partials + block_index * p.max_chunks * G::kPartialFloats;
  float o[kCols];
#pragma unroll
  for (int d = 0; d < kCols; ++d) o[d] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int c0 = 0; c0 < n_chunks; c0 += kGroup) {
    float m_c[kGroup], l_c[kGroup], o_c[kGroup][kCols];
#pragma unroll
    for (int j = 0; j < kGroup; ++j) {
      const bool there = c0 + j < n_chunks;
      const float* record = first + (there ? c0 + j : c0) * G::kPartialFloats;
      m_c[j] = there ? __ldcg(record + G::kBlockQ * G::kMaxHeadDim + row_local) : -INFINITY;
      l_c[j] = there ? __ldcg(record + G::kBlockQ * G::kMaxHeadDim + G::kBlockQ + row_local) : 0.f;
#pragma unroll
      for (int d = 0; d < kCols; ++d) o_c[j][d] = there ? __ldcg(record + (part * kCols + d) * G::kBlockQ + row_local) : 0.f;
    }
    float m_new = m;
#pragma unroll
    for (int j = 0; j < kGroup; ++j) m_new = fmaxf(m_new, m_c[j]);
    if (m_new == -INFINITY) continue;  // nothing kept so far
    const float keep = m == -INFINITY ? 0.f : exp2_approx(m - m_new);
    l *= keep;
#pragma unroll
    for (int d = 0; d < kCols; ++d) o[d] *= keep;
#pragma unroll
    for (int j = 0; j < kGroup; ++j) {
      const float w = m_c[j] == -INFINITY ? 0.f : exp2_approx(m_c[j] - m_new);
      l = fmaf(l_c[j], w, l);
#pragma unroll
      for (int d = 0; d < kCols; ++d) o[d] = fmaf(o_c[j][d], w, o[d]);
    }
    m = m_new;
  }
  const float reciprocal = l > 0.f ? 1.f / l : 0.f;  // nothing kept in the row: zeros
  // through shared memory, so that a warp stores whole rows: lanes side by side along the columns, full sectors
  __shared__ float tile[32][G::kMaxHeadDim + 1];
#pragma unroll
  for (int d = 0; d < kCols; ++d) tile[lane][part * kCols + d] = o[d] * reciprocal;
  __syncthreads();
  const int rows_here = min(32, p.lq - (qb * G::kBlockQ + first_row_local));
  for (int r = part; r < rows_here; r += kMergeThreads / 32) {
    const long long out_index = head * p.out_sh + static_cast<long long>(qb * G::kBlockQ + first_row_local + r) * p.out_sr;
    char* out_row = static_cast<char*>(p.out) + out_index * (p.out_bf16 ? 2 : 4);
    const int d = lane * 4;
    const bool wide = p.out_sc == 1 && (reinterpret_cast<uintptr_t>(out_row) & 15u) == 0 && (p.dv & 3) == 0;
    if (wide && d < p.dv) {
      if (p.out_bf16) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(tile[r][d], tile[r][d + 1]), hi = __floats2bfloat162_rn(tile[r][d + 2], tile[r][d + 3]);
        *reinterpret_cast<uint2*>(out_row + d * 2) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
      } else {
        *reinterpret_cast<float4*>(out_row + d * 4) = make_float4(tile[r][d], tile[r][d + 1], tile[r][d + 2], tile[r][d + 3]);
      }
    } else if (!wide) {
      for (int e = 0; e < 4; ++e) {
        if (d + e < p.dv) {
          if (p.out_bf16) reinterpret_cast<__nv_bfloat16*>(out_row)[(d + e) * p.out_sc] = __float2bfloat16_rn(tile[r][d + e]);
          else reinterpret_cast<float*>(out_row)[(d + e) * p.out_sc] = tile[r][d + e];
        }
      }
    }
  }
}

}  // namespace vb200
