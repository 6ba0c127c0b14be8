// Inline-PTX building blocks for the sm_100a kernels: mbarrier, TMA
// (cp.async.bulk.tensor), tcgen05 (alloc / mma / commit / ld) and the UMMA
// shared-memory and instruction descriptors.
//
// Every wait is bounded.  A wait that runs out returns false; the caller
// records where it gave up in the device status word, raises the CTA-wide
// abort flag and falls through to the kernel's teardown (which still frees
// TMEM).  Nothing here traps, asserts or spins without a limit.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vb200 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  // Make the initialised barriers visible to the async proxy (TMA, tcgen05.commit).
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// The same probe with cluster-scope acquire: for barriers that threads of the peer CTA arrive on.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Non-blocking probe of phase `parity` (try_wait may suspend the thread for a while before giving up;
// a loop that watches several barriers must not).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Cycle budget of one wait (about a second at B200 clocks).  A healthy wait
// lasts microseconds; the budget only matters when a pipeline is wedged.
constexpr long long kWaitCycleBudget = 2000000000LL;

// Bounded wait on phase `parity`.  `abort_flag` is a CTA-shared word that any
// role raises when it gives up, so that the other roles stop waiting too.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 0x3ffu) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - start > kWaitCycleBudget) return false;
    }
  }
  return true;
}

__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long start = clock64();
  uint32_t polls = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++polls & 0x3ffu) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - start > kWaitCycleBudget) return false;
    }
  }
  return true;
}

// ---------------------------------------------------------------- CTA pairs (clusters of two)

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}

// Address of this CTA's shared-memory location `smem_addr` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t mapped;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(mapped) : "r"(smem_addr), "r"(rank));
  return mapped;
}

// Every thread of every CTA of the cluster must call this (it cannot be bounded; callers reach it only
// through paths whose own waits are bounded).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Read one float from another CTA's shared memory (`cluster_addr` from map_to_cta).
__device__ __forceinline__ float ld_shared_cluster_f32(uint32_t cluster_addr) {
  float value;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(value) : "r"(cluster_addr) : "memory");
  return value;
}

// Arrive on a barrier that may live in the peer CTA (`cluster_addr` from map_to_cta).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// ---------------------------------------------------------------- flags between CTAs (global memory)

__device__ __forceinline__ void st_release_gpu_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Flags that count their readers down, so that a launch leaves them as it found them.
//
// A producer publishes `base + readers`; each of the `readers` waits until the flag lies in (base, base + readers],
// reads what the flag guards, and takes one off.  When the last reader is done the flag holds `base` again, which is
// "not published" for the next launch that carries the same base - a replay of a captured CUDA graph, whose kernel
// arguments (the base among them) are frozen at capture.  Scratch that was never initialised is harmless as long as
// `base` is a fresh 64-bit random number: garbage falls inside a window of a few values with negligible probability.
__device__ __forceinline__ bool wait_flag_window_u64(const unsigned long long* flag, unsigned long long base, unsigned readers,
                                                     volatile uint32_t* abort_flag) {
  const long long start = clock64();
  for (;;) {
    unsigned long long seen;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(seen) : "l"(flag) : "memory");
    if (seen - base - 1ull < static_cast<unsigned long long>(readers)) return true;
    __nanosleep(100);
    if (*abort_flag != 0 || clock64() - start > kWaitCycleBudget) return false;
  }
}

// One reader is done with what `flag` guards.
__device__ __forceinline__ void flag_reader_done_u64(unsigned long long* flag) {
  asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(flag), "l"(~0ull) : "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch

// Tell the launch machinery that the next kernel in the stream - if it was launched as a programmatic dependent -
// may start being placed on SMs as they free up.  No effect otherwise.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Wait until every kernel this one programmatically depends on has finished and its writes are visible.  Returns at
// once when the kernel was launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---------------------------------------------------------------- NVSwitch multicast

// 16-byte store to a multicast address: the switch writes it into the memory of every GPU bound to the multicast
// object.  (Multicast addresses take multimem.* instructions only.)
__device__ __forceinline__ void multimem_st_v4(void* multicast_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(multicast_addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// ---------------------------------------------------------------- TMA

// Ask for `bytes` (a multiple of 16) of contiguous global memory at `gmem` (16-byte aligned) to be brought into L2.
// A hint: nothing waits for it and nothing depends on it.
__device__ __forceinline__ void prefetch_l2_bulk(const void* gmem, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gmem), "r"(bytes) : "memory");
}

__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tile load global -> shared, completion counted in bytes on `bar`.
// x is the innermost (contiguous) coordinate and must keep x * elem_size a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int32_t x,
                                            int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// The same load issued by either CTA of a pair: the tile lands in the issuing CTA's shared memory, the bytes are
// counted on `cluster_bar`, a barrier of the pair's leader (address from map_to_cta).  One destination CTA per load.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* map, uint32_t cluster_bar, int32_t x,
                                                 int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}

// 2-D tile store shared -> global (bulk async group).  Out-of-range rows and
// columns are clipped by the tensor map.  x >= 0 and y >= 0 always.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t smem_src, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_src), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

template <int kPending>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}

template <int kPending>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(kPending) : "memory");
}

// Generic-proxy writes to shared memory -> visible to the async proxy (TMA
// store source, tcgen05.mma operands).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- tcgen05

__device__ __forceinline__ void tmem_alloc(uint32_t smem_result_slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result_slot),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}

// CTA-pair forms: one warp of EACH CTA of the pair (same warp index) allocates and frees; the address is the same in both.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result_slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result_slot),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] . B[smem]; one thread issues for the CTA.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// kind::tf32: fp32 words in shared memory, of which the tensor core uses sign, exponent and the top 10 mantissa bits;
// K = 8 per instruction (32 bytes of a K-major row, as for the other kinds).
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Pair forms: issued by one thread of the leader CTA; A is 256 rows (128 per CTA), B is N rows (N/2 per CTA), each CTA
// reading its own shared memory at the descriptor's address and accumulating its 128 rows of D in its own TMEM.
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive once on the barrier at the same shared-memory offset in BOTH CTAs of the pair when every pair MMA issued so
// far has finished.  (An arrival on barriers, not a data transfer: no load is involved.)
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(both)
               : "memory");
}

// Arrive once on `bar` when every tcgen05.mma issued so far by this thread
// has finished reading its operands and writing TMEM.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives
// lane (base_lane + i), columns [col, col + 32).
__device__ __forceinline__ void tmem_load_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// 32 lanes x 64 consecutive 32-bit columns in one instruction.
__device__ __forceinline__ void tmem_load_32x64(uint32_t taddr, uint32_t (&v)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]), "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]), "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]), "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// The store counterpart of tmem_load_32x32: thread i of the warp writes lane (base_lane + i), columns [col, col + 32).
__device__ __forceinline__ void tmem_store_32x32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
      "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
      "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}

__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- descriptors

// UMMA shared-memory descriptor of a K-major operand tile stored as rows of
// 128 bytes with the 128-byte swizzle (what TMA SWIZZLE_128B writes): groups
// of 8 rows are 1024 bytes apart (stride byte offset); the leading byte
// offset is unused for swizzled K-major tiles.  Bits: [0,14) address >> 4,
// [16,30) LBO >> 4, [32,46) SBO >> 4, [46,48) descriptor version (1 on
// sm_100), [61,64) layout (2 = SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  desc |= static_cast<uint64_t>(1) << 16;
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(2) << 61;
  return desc;
}

// The same for an MN-major operand under the 128-byte swizzle: rows of 128 bytes hold 64 consecutive elements along M
// (or N) for one k, eight consecutive k make a 1024-byte swizzle atom.  `k_group_bytes` is the distance between groups
// of eight k (stride byte offset), `mn_group_bytes` the distance between groups of 64 elements along M/N (leading byte
// offset).  This is how a row-major [K, N] tile that TMA loaded as boxes of 64 columns lies in shared memory.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128_mn(uint32_t smem_addr, uint32_t mn_group_bytes, uint32_t k_group_bytes) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  desc |= static_cast<uint64_t>((mn_group_bytes >> 4) & 0x3fffu) << 16;
  desc |= static_cast<uint64_t>((k_group_bytes >> 4) & 0x3fffu) << 32;
  desc |= static_cast<uint64_t>(1) << 46;
  desc |= static_cast<uint64_t>(2) << 61;
  return desc;
}

// Operand element formats of the instruction descriptor.
enum : uint32_t {
  kUmmaF16 = 0,
  kUmmaBF16 = 1,
  kUmmaTF32 = 2,
  kUmmaU8 = 0,
  kUmmaS8 = 1,
  kUmmaAccF16 = 0,
  kUmmaAccF32 = 1,
  kUmmaAccS32 = 2,
};

// UMMA instruction descriptor for dense kind::f16 / kind::tf32 / kind::i8
// with both operands K-major.  Bits: [4,6) accumulator format, [7,10) A
// format, [10,13) B format, 15/16 A/B major (0 = K), [17,23) N >> 3,
// [24,29) M >> 4.
__host__ __device__ constexpr uint32_t umma_instr_desc(uint32_t acc_format, uint32_t a_format, uint32_t b_format,
                                                       uint32_t m, uint32_t n, bool b_mn_major = false) {
  return (acc_format << 4) | (a_format << 7) | (b_format << 10) | (b_mn_major ? (1u << 16) : 0u) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

}  // namespace vb200
