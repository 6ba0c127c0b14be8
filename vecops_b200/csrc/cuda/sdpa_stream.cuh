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
//     scratch and the LAST chunk to finish - found by a counter, nobody waits - merges them the same way;
//   * warp 0 streams K tiles and V^T tiles (V transposed once by the pack kernel: tcgen05 wants both operands
//     K-contiguous) through TMA into two-stage rings; Q is loaded once;
//   * warp 1 issues tcgen05.mma: S_j = Q.K_j^T into one of two 128x128 fp32 accumulators in tensor memory, and
//     O_j = P_j.V_j into one of two more.  S_{j+1} is issued before P_j is needed, so it overlaps the softmax of tile j;
//   * four softmax warps own one query row per thread (row = tensor-memory lane): they read S_j twice (maximum, then
//     exponentials), write P_j as bf16 into shared memory in the 128-byte-swizzled K-major layout the MMA reads, and add
//     alpha * O + O_j in registers - 128 fp32 per thread - so no accumulator is ever rescaled in tensor memory.
// Every wait is bounded; a wait that runs out reports a status code and the CTA tears down normally.
#pragma once

#include <cuda_bf16.h>
#include <math.h>

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
  static constexpr int kVBytes = 2 * kAtomBytes;  // 128 head dims x 128 keys (V transposed)
  static constexpr int kPOffset = kVOffset + kStages * kVBytes;
  static constexpr int kPBytes = 2 * kAtomBytes;  // 128 query rows x 128 keys
  static constexpr int kBarrierOffset = kPOffset + kStages * kPBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kBarrierOffset + kBarrierBytes + 1024;  // + alignment slack
  static constexpr int kSoftmaxWarps = 4;
  static constexpr int kThreads = 32 * (2 + kSoftmaxWarps);
  static constexpr int kTmemColumns = 512;  // S at columns 0 and 128, O at 256 and 384
  static constexpr int kPartialFloats = kBlockQ * kMaxHeadDim + 2 * kBlockQ;  // O, then m, then l
  static constexpr int kMaxChunks = 32;  // chunks a query block's keys are cut into at most (the grid's x extent)
};
static_assert(SdpaStream::kSmemBytes <= 227 * 1024, "shared memory budget");

struct SdpaStreamParams {
  int lq, lkv, dqk, dv;
  int causal;           // 0 none, 1 top left, 2 bottom right
  int tiles_per_chunk;  // 128-key tiles per work item
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
  unsigned long long* counters;  // [head][query block] arrival counters
  uint32_t nonce;                // never 0
  uint32_t* status;
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

// Arrival counter in scratch that needs no initialisation: a word holds (nonce << 32 | arrivals).  The first CTA to
// find another launch's state (or memory never written) claims the word with a compare-and-swap on the value it read;
// everyone else adds.  Returns the arrivals before this one, or 0xffffffff when the word keeps changing under it
// (two launches overlapping on one scratch): the attempts are bounded.  The CTA that arrives last puts the word back
// to zero - no launch's nonce - so a replay of a captured launch, which carries the same nonce, counts from zero again.
__device__ __forceinline__ uint32_t sdpa_arrive(unsigned long long* word, uint32_t nonce) {
  for (int attempt = 0; attempt < 16; ++attempt) {
    const unsigned long long seen = *reinterpret_cast<volatile unsigned long long*>(word);
    if (static_cast<uint32_t>(seen >> 32) == nonce) {
      const unsigned long long before = atomicAdd(word, 1ull);
      if (static_cast<uint32_t>(before >> 32) == nonce) return static_cast<uint32_t>(before);
    } else if (atomicCAS(word, seen, (static_cast<unsigned long long>(nonce) << 32) | 1ull) == seen) {
      return 0;
    }
  }
  return 0xffffffffu;
}

// kPlain: no key mask, no two-dimensional keep mask, no bias (the query mask and the causal cut cost nothing).
template <bool kPlain>
__global__ void __launch_bounds__(SdpaStream::kThreads, 1)
sdpa_stream_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_vt, const SdpaStreamParams p) {
  using G = SdpaStream;
  // ---------------------------------------------------------------- which work item
  const int chunk = blockIdx.x;
  const int qb = static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);  // long causal blocks first
  const int head = blockIdx.z;
  const int r0 = qb * G::kBlockQ;
  const int rows = min(G::kBlockQ, p.lq - r0);
  const long long shift = p.causal == 2 ? static_cast<long long>(p.lkv) - p.lq : 0;
  const long long block_last_key = p.causal != 0 ? min(static_cast<long long>(p.lkv) - 1, r0 + rows - 1 + shift) : p.lkv - 1;
  const int tiles_total = block_last_key < 0 ? 0 : static_cast<int>(block_last_key / G::kBlockKv) + 1;
  const int n_chunks = max(1, (tiles_total + p.tiles_per_chunk - 1) / p.tiles_per_chunk);
  if (chunk >= n_chunks) return;  // the grid is sized for the block with the most keys
  const int tile_begin = chunk * p.tiles_per_chunk;
  const int ntiles = max(0, min(tiles_total, tile_begin + p.tiles_per_chunk) - tile_begin);

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + G::kBarrierOffset;
  const uint32_t q_full = bar_base;
  const uint32_t k_full = bar_base + 8;     // [2] K tile landed        (TMA -> MMA)
  const uint32_t v_full = bar_base + 24;    // [2] V^T tile landed      (TMA -> MMA)
  const uint32_t kv_empty = bar_base + 40;  // [2] both products of the stage done (MMA -> TMA)
  const uint32_t s_full = bar_base + 56;    // [2] S_j in tensor memory (MMA -> softmax)
  const uint32_t s_free = bar_base + 72;    // [2] S_j read twice       (softmax -> MMA)
  const uint32_t p_full = bar_base + 88;    // [2] P_j in shared memory (softmax -> MMA)
  const uint32_t o_full = bar_base + 104;   // [2] O_j in tensor memory, P_j and the V stage read (MMA -> softmax)
  const uint32_t o_free = bar_base + 120;   // [2] O_j added            (softmax -> MMA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + G::kBarrierOffset + 144);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + G::kBarrierOffset + 148);
  volatile uint32_t* last_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + G::kBarrierOffset + 152);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full + 8 * s, 1);
      mbar_init(v_full + 8 * s, 1);
      mbar_init(kv_empty + 8 * s, 1);
      mbar_init(s_full + 8 * s, 1);
      mbar_init(s_free + 8 * s, G::kSoftmaxWarps);
      mbar_init(p_full + 8 * s, G::kSoftmaxWarps);
      mbar_init(o_full + 8 * s, 1);
      mbar_init(o_free + 8 * s, G::kSoftmaxWarps);
    }
    *abort_flag = 0;
    *last_flag = 0;
    mbar_fence_init();
    tma_prefetch_descriptor(&map_q);
    tma_prefetch_descriptor(&map_k);
    tma_prefetch_descriptor(&map_vt);
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
      for (int i = 0; i < ntiles; ++i) {
        const int s = i & 1;
        const uint32_t parity = static_cast<uint32_t>(i >> 1) & 1u;
        if (!mbar_wait(kv_empty + 8 * s, parity ^ 1u, abort_flag)) {
          give_up(kStatusProducerWait);
          break;
        }
        const int key0 = (tile_begin + i) * G::kBlockKv;
        mbar_arrive_expect_tx(k_full + 8 * s, G::kKBytes);
        tma_load_3d(smem_base + G::kKOffset + s * G::kKBytes, &map_k, k_full + 8 * s, 0, key0, head * p.k_head);
        tma_load_3d(smem_base + G::kKOffset + s * G::kKBytes + G::kAtomBytes, &map_k, k_full + 8 * s, 64, key0, head * p.k_head);
        mbar_arrive_expect_tx(v_full + 8 * s, G::kVBytes);
        tma_load_3d(smem_base + G::kVOffset + s * G::kVBytes, &map_vt, v_full + 8 * s, key0, 0, head * p.v_head);
        tma_load_3d(smem_base + G::kVOffset + s * G::kVBytes + G::kAtomBytes, &map_vt, v_full + 8 * s, key0 + 64, 0, head * p.v_head);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && ntiles > 0) {
      constexpr uint32_t idesc = umma_instr_desc(kUmmaAccF32, kUmmaBF16, kUmmaBF16, 128, 128);
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
        if (!mbar_wait(p_full + 8 * s, parity, abort_flag) || !mbar_wait(o_free + 8 * s, parity ^ 1u, abort_flag) ||
            !mbar_wait(v_full + 8 * s, parity, abort_flag)) {
          give_up(kStatusMmaWaitTmem);
          break;
        }
        tcgen05_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < G::kBlockKv / 16; ++ks) {
          const uint64_t a_desc = umma_smem_desc_sw128(smem_base + G::kPOffset + s * G::kPBytes + (ks >> 2) * G::kAtomBytes) + 2 * (ks & 3);
          const uint64_t b_desc = umma_smem_desc_sw128(smem_base + G::kVOffset + s * G::kVBytes + (ks >> 2) * G::kAtomBytes) + 2 * (ks & 3);
          umma_f16(tmem_base + 256 + s * 128, a_desc, b_desc, idesc, ks > 0 ? 1u : 0u);
        }
        umma_commit(o_full + 8 * s);
        umma_commit(kv_empty + 8 * s);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps: one query row per thread
    const int quarter = warp & 3;  // the tensor-memory lanes a warp may read are fixed by its index
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
    auto decorated = [&](int j, float score) {
      float value = __fmul_rn(score, p.scale);
      if (j >= limit) return negative_infinity;
      if constexpr (!kPlain) {
        if (bias_row != nullptr) value = __fadd_rn(value, bias_row[j * p.bias_sc]);
        const bool keep = (key_mask == nullptr || key_mask[j] != 0) && (keep_row == nullptr || keep_row[j * p.keep_sc] != 0);
        if (!keep) return negative_infinity;
      }
      return value;
    };
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t p_row = (row_local >> 3) * 1024 + (row_local & 7) * 128;  // this row inside a swizzled atom
    float o[G::kMaxHeadDim];
#pragma unroll
    for (int d = 0; d < G::kMaxHeadDim; ++d) o[d] = 0.f;
    float m = negative_infinity, l = 0.f, alpha_pending = 1.f;
    bool ok = true;
    // O = alpha * O + O_j, the product of tile j read from tensor memory
    auto take_product = [&](int j, float alpha) {
      const int s = j & 1;
      if (!mbar_wait(o_full + 8 * s, static_cast<uint32_t>(j >> 1) & 1u, abort_flag)) {
        if (lane == 0) give_up(kStatusEpilogueWait);
        return false;
      }
      tcgen05_fence_after_sync();
#pragma unroll
      for (int c = 0; c < G::kMaxHeadDim / 32; ++c) {
        uint32_t v[32];
        tmem_load_32x32(lane_base + 256 + s * 128 + c * 32, v);
        tmem_load_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[c * 32 + e] = fmaf(o[c * 32 + e], alpha, __uint_as_float(v[e]));
      }
      tcgen05_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free + 8 * s);
      return true;
    };
    for (int i = 0; ok && i < ntiles; ++i) {
      const int s = i & 1;
      const int key0 = (tile_begin + i) * G::kBlockKv;
      if (!mbar_wait(s_full + 8 * s, static_cast<uint32_t>(i >> 1) & 1u, abort_flag)) {
        if (lane == 0) give_up(kStatusEpilogueWait);
        ok = false;
        break;
      }
      tcgen05_fence_after_sync();
      // first reading: the tile's row maximum
      float tile_max = negative_infinity;
#pragma unroll
      for (int c = 0; c < G::kBlockKv / 32; ++c) {
        uint32_t v[32];
        tmem_load_32x32(lane_base + s * 128 + c * 32, v);
        tmem_load_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) tile_max = fmaxf(tile_max, decorated(key0 + c * 32 + e, __uint_as_float(v[e])));
      }
      const float m_new = fmaxf(m, tile_max);
      // nothing kept so far: every p is 0 and alpha is 1 (the reference's "block not valid" branch)
      const float m_use = m_new == negative_infinity ? 0.f : m_new;
      const float alpha = m_new == negative_infinity ? 1.f : exp2_approx((m - m_new) * kLog2e);  // m = -inf: 0
      // second reading: p = exp(s - m'), summed unrounded, stored as bf16 where the MMA reads its A operand
      float sum = 0.f;
      const uint32_t p_base = smem_base + G::kPOffset + s * G::kPBytes + p_row;
#pragma unroll
      for (int c = 0; c < G::kBlockKv / 32; ++c) {
        uint32_t v[32];
        tmem_load_32x32(lane_base + s * 128 + c * 32, v);
        tmem_load_wait();
        uint32_t packed[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const float p0 = exp2_approx((decorated(key0 + c * 32 + e, __uint_as_float(v[e])) - m_use) * kLog2e);
          const float p1 = exp2_approx((decorated(key0 + c * 32 + e + 1, __uint_as_float(v[e + 1])) - m_use) * kLog2e);
          sum += p0 + p1;
          const __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
          packed[e >> 1] = *reinterpret_cast<const uint32_t*>(&pair);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int piece = c * 4 + q;  // 16-byte piece (8 keys) of the row: atom = piece / 8, position inside it swizzled by the row
          const uint32_t dst = p_base + (piece >> 3) * G::kAtomBytes + (((piece & 7) ^ (row_local & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[4 * q]), "r"(packed[4 * q + 1]), "r"(packed[4 * q + 2]),
                       "r"(packed[4 * q + 3])
                       : "memory");
        }
      }
      l = fmaf(l, alpha, sum);
      tcgen05_fence_before_sync();
      fence_proxy_async_smem();  // the tensor core reads P through the async proxy
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(s_free + 8 * s);
        mbar_arrive(p_full + 8 * s);
      }
      // the product of the tile before this one, issued while this tile's scores were turned into probabilities
      if (i > 0) ok = take_product(i - 1, alpha_pending);
      alpha_pending = alpha;
      m = m_new;
    }
    if (ok && ntiles > 0) ok = take_product(ntiles - 1, alpha_pending);

    // ---------------------------------------------------------------- merge the chunks of this query block, store
    const size_t block_index = static_cast<size_t>(head) * gridDim.y + qb;
    // every softmax thread gets here whatever happened above; what they do next must not differ between them
    asm volatile("bar.sync 1, %0;" ::"n"(G::kSoftmaxWarps * 32) : "memory");
    ok = *abort_flag == 0;
    bool store = ok;
    if (ok && n_chunks > 1) {
      float* mine = p.partials + (block_index * gridDim.x + chunk) * G::kPartialFloats;
      float4* mine_o = reinterpret_cast<float4*>(mine + static_cast<size_t>(row_local) * G::kMaxHeadDim);
#pragma unroll
      for (int d = 0; d < G::kMaxHeadDim; d += 4) __stcg(mine_o + d / 4, make_float4(o[d], o[d + 1], o[d + 2], o[d + 3]));
      __stcg(mine + G::kBlockQ * G::kMaxHeadDim + row_local, m);
      __stcg(mine + G::kBlockQ * G::kMaxHeadDim + G::kBlockQ + row_local, l);
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(G::kSoftmaxWarps * 32) : "memory");
      if (warp == 2 && lane == 0) {
        const uint32_t before = sdpa_arrive(p.counters + block_index, p.nonce);
        if (before == 0xffffffffu) report_status(p.status, kStatusEpilogueWait);
        *last_flag = before == static_cast<uint32_t>(n_chunks - 1) ? 1u : 0u;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(G::kSoftmaxWarps * 32) : "memory");
      store = *last_flag != 0;
      if (store) {
        __threadfence();
        const float* first = p.partials + block_index * gridDim.x * G::kPartialFloats;
        float m_all = m;
        for (int c = 0; c < n_chunks; ++c)
          if (c != chunk) m_all = fmaxf(m_all, __ldcg(first + c * G::kPartialFloats + G::kBlockQ * G::kMaxHeadDim + row_local));
        const float w_mine = m == negative_infinity ? 0.f : exp2_approx((m - m_all) * kLog2e);
        l *= w_mine;
#pragma unroll
        for (int d = 0; d < G::kMaxHeadDim; ++d) o[d] *= w_mine;
        for (int c = 0; c < n_chunks; ++c) {
          if (c == chunk) continue;
          const float* other = first + c * G::kPartialFloats;
          const float m_c = __ldcg(other + G::kBlockQ * G::kMaxHeadDim + row_local);
          const float l_c = __ldcg(other + G::kBlockQ * G::kMaxHeadDim + G::kBlockQ + row_local);
          const float w = m_c == negative_infinity ? 0.f : exp2_approx((m_c - m_all) * kLog2e);
          l = fmaf(l_c, w, l);
          const float4* other_o = reinterpret_cast<const float4*>(other + static_cast<size_t>(row_local) * G::kMaxHeadDim);
#pragma unroll
          for (int d = 0; d < G::kMaxHeadDim; d += 4) {
            const float4 v = __ldcg(other_o + d / 4);
            o[d] = fmaf(v.x, w, o[d]);
            o[d + 1] = fmaf(v.y, w, o[d + 1]);
            o[d + 2] = fmaf(v.z, w, o[d + 2]);
            o[d + 3] = fmaf(v.w, w, o[d + 3]);
          }
        }
        if (warp == 2 && lane == 0) atomicExch(p.counters + block_index, 0ull);  // a replay counts from zero again
      }
    }
    if (store && row_valid) {
      const float reciprocal = l > 0.f ? 1.f / l : 0.f;  // nothing kept in the row: zeros
      char* out_row = static_cast<char*>(p.out) + (head * p.out_sh + row * p.out_sr) * (p.out_bf16 ? 2 : 4);
      const bool wide = p.out_sc == 1 && (reinterpret_cast<uintptr_t>(out_row) & 15u) == 0 && (p.dv & 7) == 0;
      if (wide && p.out_bf16) {
#pragma unroll
        for (int d = 0; d < G::kMaxHeadDim; d += 8) {
          if (d < p.dv) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_bfloat162 pair = __floats2bfloat162_rn(o[d + 2 * e] * reciprocal, o[d + 2 * e + 1] * reciprocal);
              w[e] = *reinterpret_cast<const uint32_t*>(&pair);
            }
            *reinterpret_cast<uint4*>(out_row + d * 2) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      } else if (wide) {
#pragma unroll
        for (int d = 0; d < G::kMaxHeadDim; d += 4)
          if (d < p.dv)
            *reinterpret_cast<float4*>(out_row + d * 4) = make_float4(o[d] * reciprocal, o[d + 1] * reciprocal, o[d + 2] * reciprocal, o[d + 3] * reciprocal);
      } else {
#pragma unroll
        for (int d = 0; d < G::kMaxHeadDim; ++d) {
          if (d < p.dv) {
            if (p.out_bf16) reinterpret_cast<__nv_bfloat16*>(out_row)[d * p.out_sc] = __float2bfloat16_rn(o[d] * reciprocal);
            else reinterpret_cast<float*>(out_row)[d * p.out_sc] = o[d] * reciprocal;
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncthreads();
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

}  // namespace vb200
