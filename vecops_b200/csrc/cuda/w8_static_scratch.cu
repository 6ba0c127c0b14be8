// vecops_b200_matmul_w8_static_scratch: the tensor-memory weight-only int8 kernel for callers that must not
// allocate.
//
// Who cannot allocate: code that runs where cudaMalloc is forbidden or unaffordable - a decode loop whose memory
// pool is sealed after start-up, an embedding whose allocator must never be re-entered from an operator call, a
// latency budget that cannot absorb an allocation's implicit device synchronisation.  For them the scratch that
// w8_tcgen05 normally receives from the caller (stream-K partial sums, flags, the fp16 copy of the activations)
// lives in a fixed array inside this library instead.
//
// The price, stated plainly:
//   * the array is kStaticScratchBytes (8 MiB) of device memory on EVERY GPU on which this library's device code
//     is loaded, held until the process exits.  The CUDA runtime materialises it when it loads this module on a
//     device - with lazy module loading that is at the latest this entry point's first call there, so that first
//     call belongs in start-up code, where the 8 MiB are still to be had;
//   * problems whose scratch need exceeds it are refused with INVALID_ARGUMENT (nothing is truncated).  The need
//     is 81920 * M_pad + 2 * M * K + 5632 bytes with M_pad = M rounded up to 16: M <= 80 at K = 4096, M <= 96 for
//     any K up to 2048, never more than 96 rows;
//   * all calls on one device share the one array, which keeps the previous call's contents.  Nothing in it has
//     to start at zero (flags carry a fresh 64-bit nonce per launch and are counted back down to it by their
//     readers; the status word is cleared when read), but two calls that overlap on the GPU - different streams,
//     or asynchronous calls not ordered by a stream - race on it and produce garbage.  Serialise them.
//
// Set-up: the first call on a device looks the array's device address up (cudaGetSymbolAddress; the array's name
// in host code is only a host-side stand-in, never a pointer a kernel could use) and raises the kernel's
// shared-memory limit.  That first call should be made before any stream capture begins.
//
// This entry point calls no cudaMalloc, cudaFree, cudaHostAlloc or any other allocating routine.
#include <atomic>
#include <cstring>
#include <mutex>

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include "vecops_b200/matmul_cuda.h"

#include "shim_util.h"
#include "w8_tcgen05.cuh"

namespace vb200 {
namespace {

constexpr unsigned long long kStaticScratchBytes = VECOPS_B200_STATIC_SCRATCH_BYTES;

// The scratch itself and the word a bounded device wait reports into.  Device code could name these directly;
// host code must go through cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ uint32_t g_static_status;

struct PerDevice {
  bool ready = false;
  unsigned char* scratch = nullptr;  // device address of g_static_scratch on this device
  uint32_t* status = nullptr;        // device address of g_static_status on this device
  int sm_count = 0;
  int sm_major = 0;
};

std::mutex g_setup_mutex;
PerDevice g_per_device[64];
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

int32_t cuda_error(VecopsError* error, cudaError_t status, const char* what) {
  return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "%s: %s", what, cudaGetErrorString(status));
}

// Once per device, with that device current.
int32_t set_up(int device, const PerDevice** out, VecopsError* error) {
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  PerDevice& state = g_per_device[device];
  if (!state.ready) {
    void* address = nullptr;
    cudaError_t status = cudaGetSymbolAddress(&address, g_static_scratch);
    if (status != cudaSuccess) return cuda_error(error, status, "cudaGetSymbolAddress(static scratch)");
    state.scratch = static_cast<unsigned char*>(address);
    status = cudaGetSymbolAddress(&address, g_static_status);
    if (status != cudaSuccess) return cuda_error(error, status, "cudaGetSymbolAddress(static status word)");
    state.status = static_cast<uint32_t*>(address);
    status = cudaDeviceGetAttribute(&state.sm_count, cudaDevAttrMultiProcessorCount, device);
    if (status != cudaSuccess) return cuda_error(error, status, "cudaDeviceGetAttribute(SM count)");
    status = cudaDeviceGetAttribute(&state.sm_major, cudaDevAttrComputeCapabilityMajor, device);
    if (status != cudaSuccess) return cuda_error(error, status, "cudaDeviceGetAttribute(compute capability)");
    for (auto kernel : {reinterpret_cast<const void*>(w8_tcgen05_kernel<__nv_bfloat16, false>),
                        reinterpret_cast<const void*>(w8_tcgen05_kernel<float, false>)}) {
      status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
      if (status != cudaSuccess) return cuda_error(error, status, "cudaFuncSetAttribute(max dynamic shared memory)");
    }
    state.ready = true;
  }
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult query;
    cudaError_t status = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query);
    if (status != cudaSuccess || fn == nullptr || query != cudaDriverEntryPointSuccess)
      return set_error(error, VECOPS_STATUS_LOAD_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }
  *out = &state;
  return VECOPS_STATUS_OK;
}

int32_t encode_2d(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, uint64_t dim0, uint64_t dim1, uint64_t pitch_bytes,
                  uint32_t box0, uint32_t box1, VecopsError* error) {
  cuuint64_t dims[2] = {dim0, dim1};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t elem_strides[2] = {1, 1};
  const CUresult rc = g_encode(map, dtype, 2, const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(rc));
  return VECOPS_STATUS_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

uint64_t next_nonce() {
  static std::atomic<uint64_t> counter{0x13198A2E03707344ull};
  uint64_t z = counter.fetch_add(0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z == 0 ? 1 : z;
}

template <typename OutT>
void launch(const VecopsB200Matmul& p, const PerDevice& dev, int mpad, const CUtensorMap& map_w, const CUtensorMap& map_a,
            cudaStream_t stream) {
  using G = W8Tc;
  float* partials = reinterpret_cast<float*>(dev.scratch);
  auto* flags = reinterpret_cast<unsigned long long*>(dev.scratch + G::flags_offset(mpad));
  float* inv_scales = reinterpret_cast<float*>(dev.scratch + G::scales_offset(mpad));
  const long long units = ((p.n + G::kTileN - 1) / G::kTileN) * ((p.k + G::kBlockK - 1) / G::kBlockK);
  long long grid = dev.sm_count < G::kMaxGrid ? dev.sm_count : G::kMaxGrid;
  if (units < grid) grid = units;
  const uint32_t idesc = umma_instr_desc(kUmmaAccF32, kUmmaF16, kUmmaF16, G::kTileN, mpad);
  w8_tcgen05_kernel<OutT, false><<<static_cast<int>(grid), G::kThreads, G::smem_bytes(mpad), stream>>>(
      map_w, map_a, p.column_scale, static_cast<OutT*>(p.c), p.c_stride_m, static_cast<int>(p.m), static_cast<int>(p.n),
      static_cast<int>(p.k), mpad, partials, flags, inv_scales, next_nonce(), idesc, EpilogueArgs(), dev.status, nullptr);
}

}  // namespace
}  // namespace vb200

using namespace vb200;

extern "C" int32_t vecops_b200_matmul_w8_static_scratch(const VecopsB200Matmul* problem, VecopsError* error) {
  using G = W8Tc;
  if (problem == nullptr) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "problem record is null");
  if (problem->struct_size < sizeof(VecopsB200Matmul))
    return set_error(error, VECOPS_STATUS_ABI_MISMATCH, "problem record is %u bytes, this library needs %zu", problem->struct_size,
                     sizeof(VecopsB200Matmul));
  const VecopsB200Matmul& p = *problem;
  const bool out_bf16 = p.c_dtype == VECOPS_DTYPE_BF16;
  if (p.a_dtype != VECOPS_DTYPE_BF16 || p.b_dtype != VECOPS_DTYPE_I8 || !(out_bf16 || p.c_dtype == VECOPS_DTYPE_F32))
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "this entry point serves bf16 activations x int8 weights -> bf16 or f32 only");
  if (p.m < 0 || p.n < 0 || p.k < 0) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "negative extent");
  if (p.m == 0 || p.n == 0) return VECOPS_STATUS_OK;
  if (p.m > G::kMaxM || p.k == 0 || p.k % 8 != 0 || p.a_stride_k != 1 || p.b_stride_k != 1 || p.c_stride_n != 1 || p.a == nullptr ||
      p.b == nullptr || p.c == nullptr || !aligned16(p.a) || !aligned16(p.b) || p.a_stride_m % 8 != 0 || p.b_stride_n % 16 != 0 ||
      p.a_stride_m < p.k || p.b_stride_n < p.k || p.n >= (INT64_C(1) << 31) || p.k >= (INT64_C(1) << 31))
    return set_error(error, VECOPS_STATUS_NOT_APPLICABLE,
                     "needs 1 <= M <= %d, K a positive multiple of 8, K-contiguous 16-byte aligned A and W rows, row-major C", G::kMaxM);
  const unsigned long long need = G::scratch_bytes(static_cast<int>(p.m), p.k);
  if (need > kStaticScratchBytes)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT,
                     "M=%lld K=%lld needs %llu bytes of scratch, the built-in array holds %llu; use vecops_b200_matmul_run with a caller workspace",
                     (long long)p.m, (long long)p.k, need, kStaticScratchBytes);

  int count = 0;
  cudaError_t status = cudaGetDeviceCount(&count);
  if (status != cudaSuccess || count == 0) {
    (void)cudaGetLastError();
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "no usable CUDA device; the B200 matmul path has no CPU fallback");
  }
  int previous = -1;
  cudaGetDevice(&previous);
  const int device = p.device_index >= 0 ? p.device_index : previous;
  if (device < 0 || device >= count || device >= 64) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "no CUDA device %d", device);
  if (previous != device) {
    status = cudaSetDevice(device);
    if (status != cudaSuccess) return cuda_error(error, status, "cudaSetDevice");
  }
  const PerDevice* dev = nullptr;
  int32_t rc = set_up(device, &dev, error);
  if (rc == VECOPS_STATUS_OK && dev->sm_major != 10)
    rc = set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "tcgen05 kernels need an sm_100 device, found sm_%dx", dev->sm_major);

  cudaStream_t stream = static_cast<cudaStream_t>(p.stream);
  if (rc == VECOPS_STATUS_OK) {
    const int mpad = G::m_padded(static_cast<int>(p.m));
    __half* act16 = reinterpret_cast<__half*>(dev->scratch + G::act_offset(mpad));
    float* inv_scales = reinterpret_cast<float*>(dev->scratch + G::scales_offset(mpad));
    const long long act_pitch = G::act_pitch(p.k);
    CUtensorMap map_w, map_a;
    rc = encode_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.b, p.k, p.n, p.b_stride_n, G::kBlockK, G::kTileN, error);
    if (rc == VECOPS_STATUS_OK)
      rc = encode_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, act16, p.k, p.m, act_pitch * 2, 64, mpad, error);
    if (rc == VECOPS_STATUS_OK) {
      w8_prepare_activations_kernel<<<static_cast<int>(p.m), W8Prepare::kThreads, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(p.a), p.a_stride_m, act16, act_pitch, inv_scales, static_cast<int>(p.k));
      if (out_bf16) launch<__nv_bfloat16>(p, *dev, mpad, map_w, map_a, stream);
      else launch<float>(p, *dev, mpad, map_w, map_a, stream);
      g_launches.fetch_add(2);
      status = cudaGetLastError();
      if (status != cudaSuccess) rc = cuda_error(error, status, "kernel launch");
    }
  }
  if (rc == VECOPS_STATUS_OK && (p.flags & VECOPS_B200_MATMUL_FLAG_ASYNC) == 0) {
    // Did a bounded device wait run out?  The status word is read on the call's own stream, behind the kernel, so the
    // read orders against nothing but this call (a blocking copy would go through the legacy stream and serialise
    // against every other blocking stream of the process).
    uint32_t word = 0;
    status = cudaMemcpyAsync(&word, dev->status, sizeof(word), cudaMemcpyDeviceToHost, stream);
    if (status == cudaSuccess) status = cudaStreamSynchronize(stream);
    if (status != cudaSuccess) {
      rc = cuda_error(error, status, "reading the status word behind the kernel");
    } else if (word != 0) {
      cudaMemsetAsync(dev->status, 0, sizeof(word), stream);
      cudaStreamSynchronize(stream);
      rc = set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "w8_tcgen05 (static scratch): a bounded device wait ran out (status 0x%x)", word);
    }
  }
  if (previous >= 0 && previous != device) cudaSetDevice(previous);
  return rc;
}
