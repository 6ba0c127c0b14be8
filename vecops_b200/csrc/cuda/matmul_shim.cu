// Host side of the thin C ABI over the sm_100a matmul kernels: argument
// checks, the shape/dtype dispatch rules, tensor-map construction and the
// launches.  No CPU arithmetic lives here: a problem either runs on the GPU
// or the call fails.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <type_traits>
#include <unordered_map>

#include <cstddef>
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include "vecops_b200/matmul_cuda.h"

#include "gemm_tcgen05.cuh"
#include "simt_kernels.cuh"
#include "w8_small_m.cuh"
#include "w8_stream.cuh"
#include "w8_tcgen05.cuh"
#include "shim_device.h"
#include "shim_util.h"

namespace vb200 {

std::atomic<uint64_t> g_launches{0};

int32_t set_error(VecopsError* error, int32_t code, const char* format, ...) {
  char text[512];
  va_list args;
  va_start(args, format);
  const int wanted = vsnprintf(text, sizeof(text), format, args);
  va_end(args);
  if (error != nullptr && error->struct_size >= sizeof(VecopsError)) {
    error->code = code;
    error->message_required = static_cast<size_t>(wanted < 0 ? 0 : wanted) + 1;
    if (error->message != nullptr && error->message_capacity > 0) {
      snprintf(error->message, error->message_capacity, "%s", text);
    }
  }
  return code;
}

DeviceRestore::DeviceRestore() {
  if (cudaGetDevice(&previous) != cudaSuccess) {
    (void)cudaGetLastError();
    previous = -1;
  }
}

DeviceRestore::~DeviceRestore() {
  int now = -1;
  if (previous >= 0 && cudaGetDevice(&now) == cudaSuccess && now != previous) cudaSetDevice(previous);
}

namespace {

// ------------------------------------------------------------------ device bookkeeping

struct DeviceState {
  bool known = false;
  cudaDeviceProp prop{};
};

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
DeviceState g_devices[kMaxDevices];
// Pinned, mapped host memory, one word per device ordinal: kernels running on device d write word d, and only when a
// bounded wait ran out.  Read-and-clear is an atomic exchange, so concurrent pollers cannot both see one record.
uint32_t* g_status_host = nullptr;

uint32_t* status_word_of(int device) {
  return (g_status_host != nullptr && device >= 0 && device < kMaxDevices) ? g_status_host + device : nullptr;
}

uint32_t take_status_word(int device) {
  uint32_t* word = status_word_of(device);
  return word == nullptr ? 0u : __atomic_exchange_n(word, 0u, __ATOMIC_ACQ_REL);
}
unsigned long long* g_trace = nullptr;  // optional device buffer for kernel timelines (tuning aid), see vecops_b200_debug_set_trace
PFN_cuTensorMapEncodeTiled_v12000 g_encode_tiled = nullptr;

int32_t cuda_fail(VecopsError* error, cudaError_t status, const char* what) {
  return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "%s: %s", what, cudaGetErrorString(status));
}

int32_t device_state(int device, const DeviceState** out, VecopsError* error) {
  if (device < 0 || device >= kMaxDevices) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "device index %d out of range", device);
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& state = g_devices[device];
  if (!state.known) {
    cudaError_t status = cudaGetDeviceProperties(&state.prop, device);
    if (status != cudaSuccess) return cuda_fail(error, status, "cudaGetDeviceProperties");
    state.known = true;
  }
  if (g_status_host == nullptr) {
    void* p = nullptr;
    cudaError_t status = cudaHostAlloc(&p, kMaxDevices * sizeof(uint32_t), cudaHostAllocMapped | cudaHostAllocPortable);
    if (status != cudaSuccess) return cuda_fail(error, status, "cudaHostAlloc(status words)");
    memset(p, 0, kMaxDevices * sizeof(uint32_t));
    g_status_host = static_cast<uint32_t*>(p);
  }
  if (g_encode_tiled == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult query;
    cudaError_t status = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query);
    if (status != cudaSuccess || fn == nullptr || query != cudaDriverEntryPointSuccess)
      return set_error(error, VECOPS_STATUS_LOAD_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
    g_encode_tiled = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }
  *out = &state;
  return VECOPS_STATUS_OK;
}

int32_t current_device(const VecopsB200Matmul& p, int* device, VecopsError* error) {
  int count = 0;
  cudaError_t status = cudaGetDeviceCount(&count);
  if (status != cudaSuccess || count == 0) {
    (void)cudaGetLastError();
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR,
                     "no usable CUDA device (%s); the B200 matmul path has no CPU fallback",
                     status == cudaSuccess ? "device count is 0" : cudaGetErrorString(status));
  }
  if (p.device_index >= 0) {
    if (p.device_index >= count)
      return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "device index %d but only %d devices", p.device_index, count);
    *device = p.device_index;
    return VECOPS_STATUS_OK;
  }
  status = cudaGetDevice(device);
  if (status != cudaSuccess) return cuda_fail(error, status, "cudaGetDevice");
  return VECOPS_STATUS_OK;
}

// ------------------------------------------------------------------ problem classification

enum class Row { Invalid, F32, BF16, I8, W8, QI8, F16 };  // QI8: 8-bit operands, int32 accumulate, floating-point output (dequantising form)

size_t dtype_size(uint32_t dtype) {
  switch (dtype) {
    case VECOPS_DTYPE_I8: case VECOPS_DTYPE_U8: return 1;
    case VECOPS_DTYPE_BF16: case VECOPS_DTYPE_F16: return 2;
    case VECOPS_DTYPE_F32: case VECOPS_DTYPE_I32: return 4;
    default: return 0;
  }
}

Row classify(const VecopsB200Matmul& p) {
  const uint32_t a = p.a_dtype, b = p.b_dtype, c = p.c_dtype;
  const bool a8 = a == VECOPS_DTYPE_I8 || a == VECOPS_DTYPE_U8;
  const bool b8 = b == VECOPS_DTYPE_I8 || b == VECOPS_DTYPE_U8;
  if (a == VECOPS_DTYPE_F32 && b == VECOPS_DTYPE_F32 && c == VECOPS_DTYPE_F32) return Row::F32;
  if (a == VECOPS_DTYPE_BF16 && b == VECOPS_DTYPE_BF16 && (c == VECOPS_DTYPE_BF16 || c == VECOPS_DTYPE_F32)) return Row::BF16;
  if (a == VECOPS_DTYPE_F16 && b == VECOPS_DTYPE_F16 && (c == VECOPS_DTYPE_F16 || c == VECOPS_DTYPE_F32)) return Row::F16;
  if (a8 && b8 && c == VECOPS_DTYPE_I32) return Row::I8;
  if (a8 && b8 && (c == VECOPS_DTYPE_F32 || c == VECOPS_DTYPE_BF16)) return Row::QI8;
  if (a == VECOPS_DTYPE_BF16 && b == VECOPS_DTYPE_I8 && (c == VECOPS_DTYPE_BF16 || c == VECOPS_DTYPE_F32)) return Row::W8;
  return Row::Invalid;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Can the TMA-fed tensor-core kernel address these operands?  Both operands
// K-contiguous, 16-byte aligned bases and row pitches (TMA's rules), and
// extents inside the tensor-map limits.
bool tma_operands_ok(const VecopsB200Matmul& p, size_t elem) {
  return p.a_stride_k == 1 && p.b_stride_k == 1 && p.c_stride_n == 1 && p.k > 0 && aligned16(p.a) && aligned16(p.b) &&
         (p.a_stride_m * static_cast<int64_t>(elem)) % 16 == 0 && (p.b_stride_n * static_cast<int64_t>(elem)) % 16 == 0 &&
         p.a_stride_m >= p.k && p.b_stride_n >= p.k && p.c_stride_m >= p.n && p.m < (INT64_C(1) << 31) &&
         p.n < (INT64_C(1) << 31) && p.k < (INT64_C(1) << 31);
}

// Device counterpart of vecops' small-problem predicate
// (RuntimeDispatch.h:24-27 `area_at_most`): tiny outputs are not worth a
// 128x256 tensor-core tile.
bool area_at_most(int64_t m, int64_t n, int64_t limit) { return m > 0 && n > 0 && n <= limit / m; }

// Tuning aid: VECOPS_B200_W8TC_FORM=tmem runs the weight-only tensor-core id on its older kernel (weights as the MMA's
// M operand, widened into tensor memory, stream-K over caller scratch it cannot do without) instead of the default one
// (weights as the N operand of the dense GEMM's MMAs, widened into shared memory).
bool w8_tmem_form() {
  const char* v = getenv("VECOPS_B200_W8TC_FORM");
  return v != nullptr && strcmp(v, "tmem") == 0;
}

bool applicable(const VecopsB200Matmul& p, Row row, uint32_t kernel) {
  switch (kernel) {
    case VECOPS_B200_KERNEL_GENERIC:
      return true;
    case VECOPS_B200_KERNEL_F32_SIMT:
      return row == Row::F32 && p.a_stride_k == 1 && p.c_stride_n == 1 && (p.b_stride_k == 1 || p.b_stride_n == 1) &&
             p.column_scale == nullptr;
    case VECOPS_B200_KERNEL_F32_TF32X3:
      // any operand strides (the split pre-pass reads them); C row-major; K small enough for the tripled reduction
      return row == Row::F32 && p.c_stride_n == 1 && p.k > 0 && p.k < (INT64_C(1) << 29) && p.m < (INT64_C(1) << 31) &&
             p.n < (INT64_C(1) << 31) && p.c_stride_m >= p.n && p.column_scale == nullptr;
    case VECOPS_B200_KERNEL_BF16_TCGEN05:
      return (row == Row::BF16 || row == Row::F16) && tma_operands_ok(p, 2);  // fp16 rides the same kernel: the formats are in the instruction descriptor
    case VECOPS_B200_KERNEL_I8_TCGEN05:
      return (row == Row::I8 && tma_operands_ok(p, 1) && p.column_scale == nullptr) || (row == Row::QI8 && tma_operands_ok(p, 1));
    case VECOPS_B200_KERNEL_W8_SMALL_M:
      return row == Row::W8 && p.a_stride_k == 1 && p.b_stride_k == 1 && p.k > 0 && p.k % 32 == 0 && aligned16(p.a) &&
             aligned16(p.b) && p.a_stride_m % 8 == 0 && p.b_stride_n % 16 == 0 && p.n < (INT64_C(1) << 31) &&
             p.m < (INT64_C(1) << 31) && p.k < (INT64_C(1) << 31);
    case VECOPS_B200_KERNEL_W8_TCGEN05:
      // (the older form of this kernel, weights widened into tensor memory, serves M <= 128 only)
      return row == Row::W8 && p.m >= 1 && (p.m <= W8Tc::kMaxM || !w8_tmem_form()) && p.a_stride_k == 1 && p.b_stride_k == 1 &&
             p.c_stride_n == 1 && p.k > 0 && p.k % 8 == 0 && aligned16(p.a) && aligned16(p.b) && p.a_stride_m % 8 == 0 &&
             p.b_stride_n % 16 == 0 && p.a_stride_m >= p.k && p.b_stride_n >= p.k && p.m < (INT64_C(1) << 31) &&
             p.n < (INT64_C(1) << 31) && p.k < (INT64_C(1) << 31);
    default:
      return false;
  }
}

const char* const kKernelNames[VECOPS_B200_KERNEL_COUNT_] = {
    "auto", "generic", "f32_simt", "bf16_tcgen05", "i8_tcgen05", "w8_small_m", "w8_tcgen05", "f32_tf32x3"};

uint32_t forced_by_environment() {
  const char* text = getenv("VECOPS_B200_FORCE_KERNEL");
  if (text == nullptr || text[0] == '\0') return VECOPS_B200_KERNEL_AUTO;
  for (uint32_t k = 1; k < VECOPS_B200_KERNEL_COUNT_; ++k)
    if (strcmp(text, kKernelNames[k]) == 0) return k;
  return VECOPS_B200_KERNEL_AUTO;
}

int32_t check_problem(const VecopsB200Matmul* p, Row* row, VecopsError* error) {
  if (p == nullptr) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "problem record is null");
  if (p->struct_size < sizeof(VecopsB200Matmul))
    return set_error(error, VECOPS_STATUS_ABI_MISMATCH, "problem record is %u bytes, this library needs %zu", p->struct_size,
                     sizeof(VecopsB200Matmul));
  if (p->m < 0 || p->n < 0 || p->k < 0) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "negative extent m=%lld n=%lld k=%lld",
                                                          (long long)p->m, (long long)p->n, (long long)p->k);
  *row = classify(*p);
  if (*row == Row::Invalid)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "unsupported dtype combination a=%u b=%u c=%u", p->a_dtype, p->b_dtype,
                     p->c_dtype);
  if (p->column_scale != nullptr && *row == Row::I8)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "column_scale applies to f32 accumulators only");
  if (p->kernel >= VECOPS_B200_KERNEL_COUNT_) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "unknown kernel id %u", p->kernel);
  return VECOPS_STATUS_OK;
}

// `for_query`: the answer for the selection and workspace queries - the kernel the rules prefer, whatever scratch the
// record carries; a launch (for_query = false) takes the preferred kernel only if the scratch it cannot do without is there.
bool tf32x3_worthwhile(const VecopsB200Matmul& p);
uint64_t tf32x3_scratch(const VecopsB200Matmul& p);

int32_t select_kernel(const VecopsB200Matmul& p, Row row, uint32_t* kernel, VecopsError* error, bool for_query = true) {
  uint32_t wanted = p.kernel != VECOPS_B200_KERNEL_AUTO ? p.kernel : forced_by_environment();
  if (wanted != VECOPS_B200_KERNEL_AUTO) {
    if (!applicable(p, row, wanted))
      return set_error(error, VECOPS_STATUS_NOT_APPLICABLE, "kernel '%s' cannot serve this problem (dtypes, strides or alignment)",
                       kKernelNames[wanted]);
    *kernel = wanted;
    return VECOPS_STATUS_OK;
  }
  uint32_t pick = VECOPS_B200_KERNEL_GENERIC;
  const bool tiny = p.m == 0 || p.n == 0 || p.k == 0 || area_at_most(p.m, p.n, 1024);
  switch (row) {
    case Row::F32:
      if (!tiny && applicable(p, row, VECOPS_B200_KERNEL_F32_SIMT)) pick = VECOPS_B200_KERNEL_F32_SIMT;
      // Products big enough to pay for the operand split go to the tensor cores as three tf32 products - when the
      // caller brings the scratch the split operands live in (the query reports it); without it the FMA kernel serves.
      if (!tiny && tf32x3_worthwhile(p) && applicable(p, row, VECOPS_B200_KERNEL_F32_TF32X3) &&
          (for_query || (p.workspace != nullptr && aligned16(p.workspace) && p.workspace_size >= tf32x3_scratch(p))))
        pick = VECOPS_B200_KERNEL_F32_TF32X3;
      break;
    case Row::F16:
    case Row::BF16:
      if (!tiny && applicable(p, row, VECOPS_B200_KERNEL_BF16_TCGEN05)) pick = VECOPS_B200_KERNEL_BF16_TCGEN05;
      break;
    case Row::QI8:
    case Row::I8:
      // int32 accumulators must wrap modulo 2^32 (vecops semantic); the tensor
      // pipe is used where |sum| < 2^31 is guaranteed: K * 2^16 < 2^31.
      if (!tiny && p.k <= 32767 && applicable(p, row, VECOPS_B200_KERNEL_I8_TCGEN05)) pick = VECOPS_B200_KERNEL_I8_TCGEN05;
      break;
    case Row::W8:
      // few activation rows: the streaming CUDA-core form; more: the tensor-core form, which uses the scratch its query
      // reports to cut tiles along K and runs them whole without it - the reference's matmul needs no workspace, so a
      // call that brings none is still served.  (Its older form cannot run without scratch: under that tuning switch a
      // call without it goes to the kernels that need none; a forced kernel id is refused by the launcher.)
      if (p.m > 16 && p.n >= 128 && applicable(p, row, VECOPS_B200_KERNEL_W8_TCGEN05) &&
          (for_query || !w8_tmem_form() ||
           (p.workspace != nullptr && aligned16(p.workspace) && p.workspace_size >= W8Tc::scratch_bytes(static_cast<int>(p.m), p.k))))
        pick = VECOPS_B200_KERNEL_W8_TCGEN05;
      else if (p.m > 0 && p.n >= 16 && applicable(p, row, VECOPS_B200_KERNEL_W8_SMALL_M)) pick = VECOPS_B200_KERNEL_W8_SMALL_M;
      break;
    default:
      break;
  }
  *kernel = pick;
  return VECOPS_STATUS_OK;
}

// ------------------------------------------------------------------ tensor maps

struct MapKey {
  const void* base;
  uint64_t dim0, dim1, pitch;
  uint32_t box0, box1, dtype, swizzle;
  bool operator==(const MapKey& o) const {
    return base == o.base && dim0 == o.dim0 && dim1 == o.dim1 && pitch == o.pitch && box0 == o.box0 && box1 == o.box1 &&
           dtype == o.dtype && swizzle == o.swizzle;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uintptr_t>(k.base);
    auto mix = [&](uint64_t v) { h = (h ^ v) * UINT64_C(0x9E3779B97F4A7C15); h ^= h >> 29; };
    mix(k.dim0); mix(k.dim1); mix(k.pitch); mix(k.box0); mix(k.box1); mix(k.dtype); mix(k.swizzle);
    return static_cast<size_t>(h);
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;

// 2-D row-major tensor [dim1 rows][dim0 contiguous elements], row pitch in bytes.
int32_t make_map_2d(CUtensorMap* out, CUtensorMapDataType dtype, size_t elem, const void* base, uint64_t dim0, uint64_t dim1,
                    uint64_t pitch_bytes, uint32_t box0, uint32_t box1, VecopsError* error) {
  const MapKey key{base, dim0, dim1, pitch_bytes, box0, box1, static_cast<uint32_t>(dtype), 128};
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto found = g_map_cache.find(key);
    if (found != g_map_cache.end()) {
      *out = found->second;
      return VECOPS_STATUS_OK;
    }
  }
  cuuint64_t dims[2] = {dim0, dim1};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t elem_strides[2] = {1, 1};
  (void)elem;
  CUresult result = g_encode_tiled(out, dtype, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (result != CUDA_SUCCESS)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR,
                     "cuTensorMapEncodeTiled failed (%d) for dims=(%llu,%llu) pitch=%llu box=(%u,%u)", static_cast<int>(result),
                     (unsigned long long)dim0, (unsigned long long)dim1, (unsigned long long)pitch_bytes, box0, box1);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_map_cache.size() > 512) g_map_cache.clear();
  g_map_cache.emplace(key, *out);
  return VECOPS_STATUS_OK;
}

bool direct_epilogue_forced() {
  const char* text = getenv("VECOPS_B200_EPILOGUE");
  return text != nullptr && strcmp(text, "direct") == 0;
}

// ------------------------------------------------------------------ launches

template <typename Kernel>
int32_t raise_smem_limit(Kernel kernel, int bytes, VecopsError* error) {
  cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (status != cudaSuccess) return cuda_fail(error, status, "cudaFuncSetAttribute(max dynamic shared memory)");
  return VECOPS_STATUS_OK;
}

uint64_t fresh_nonce(const void* salt);

// The fused output transform of the call in flight on this thread (vecops_b200_matmul_run_fused sets it around the
// ordinary run); the launchers hand it to the kernels that implement it.
thread_local EpilogueArgs tl_epilogue;

// Clusters of two CTAs of `kernel` the current device keeps resident at once; 0 when it cannot run them.
int cluster_capacity(const void* kernel, int threads, size_t smem_bytes) {
  cudaLaunchConfig_t config = {};
  cudaLaunchAttribute cluster = {};
  cluster.id = cudaLaunchAttributeClusterDimension;
  cluster.val.clusterDim.x = 2;
  cluster.val.clusterDim.y = 1;
  cluster.val.clusterDim.z = 1;
  config.gridDim = dim3(2);
  config.blockDim = dim3(threads);
  config.dynamicSmemBytes = smem_bytes;
  config.attrs = &cluster;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) clusters = 0;
  cudaGetLastError();
  return clusters;
}

// Tuning aid: VECOPS_B200_TAIL_SPLIT=0 keeps tail tiles whole.
bool tail_split_forced_off() {
  const char* v = getenv("VECOPS_B200_TAIL_SPLIT");
  return v != nullptr && v[0] == '0';
}

// How a tcgen05 GEMM launch is laid out on `sms` SMs.  Shared by the launcher and the workspace query.
struct Tcgen05Plan {
  bool pair = false;       // CTA pairs on 256x256 tiles, else single CTAs on 128x256 tiles
  long long tiles = 0;
  int workers = 0;         // CTAs, or pairs
  int num_kb = 0;
  int split = 1;           // K slices per tail tile
  long long scratch_slots = 0;  // per-CTA partial accumulators the split needs
};

Tcgen05Plan plan_tcgen05(const VecopsB200Matmul& p, bool int8, size_t out_elem, int sms, int max_pairs, size_t elem_override = 0) {
  using G = GemmTc;
  Tcgen05Plan plan;
  const size_t elem = elem_override != 0 ? elem_override : int8 ? 1 : 2;
  plan.num_kb = static_cast<int>((p.k * elem + G::kBlockKBytes - 1) / G::kBlockKBytes);
  const long long tiles_n = (p.n + G::kBlockN - 1) / G::kBlockN;
  const long long pair_tiles = ((p.m + 2 * G::kBlockM - 1) / (2 * G::kBlockM)) * tiles_n;
  // Pairs halve the operand traffic per SM; they pay once the problem fills every pair with a whole 256-row tile.
  plan.pair = max_pairs > 0 && p.m > G::kBlockM && pair_tiles >= max_pairs;
  const char* force = getenv("VECOPS_B200_GEMM_PAIR");  // tuning aid: 0 = never, 1 = whenever the device can
  if (force != nullptr && force[0] == '0') plan.pair = false;
  if (force != nullptr && force[0] == '1') plan.pair = max_pairs > 0;
  if (plan.pair) {
    plan.tiles = pair_tiles;
    plan.workers = static_cast<int>(pair_tiles < max_pairs ? pair_tiles : max_pairs);
  } else {
    plan.tiles = ((p.m + G::kBlockM - 1) / G::kBlockM) * tiles_n;
    plan.workers = static_cast<int>(plan.tiles < sms ? plan.tiles : sms);
  }
  if (!tail_split_forced_off()) plan.split = gemm_tail_split(plan.tiles, plan.workers, plan.num_kb, G::max_split(out_elem));
  if (plan.split > 1) plan.scratch_slots = (plan.tiles % plan.workers) * plan.split * (plan.pair ? 2 : 1);
  // Fewer tiles than SMs (a skinny product with a long K, such as probabilities x values in attention): every tile is
  // a "tail" tile, cut along K over as many CTAs as the SMs hold - the same exchange, just with no whole round before it.
  if (!plan.pair && plan.split == 1 && plan.tiles < sms && !tail_split_forced_off()) {
    int split = 1;
    while (split * 2 <= G::max_split(out_elem) && plan.tiles * (split * 2) <= sms && split * 2 * G::kMinSliceKb <= plan.num_kb) split *= 2;
    if (split > 1) {
      plan.split = split;
      plan.workers = static_cast<int>(plan.tiles * split);
      plan.scratch_slots = plan.tiles * split;
    }
  }
  return plan;
}

// Where the epilogue's TMA stores go when the output is gathered across GPUs.
struct GatherTargets {
  int count = 0;                 // 0 = plain GEMM into p.c
  void* const* c = nullptr;      // `count` device pointers: each GPU's full C (own included)
  int64_t n_total = 0;           // columns of the full C
  int64_t ldc = 0;               // row pitch of the full C, elements
  int64_t col0 = 0;              // first column of this rank's slab
  bool multicast = false;        // c[0] is the NVSwitch multicast address of the full C: multimem stores, no tensor map
};

// One-time per device: raise the dynamic shared memory limits of both forms of the kernel.
template <bool kInt8, typename OutT>
int32_t prepare_gemm_kernels(int device, VecopsError* error) {
  static std::atomic<bool> raised[64];
  if (device < 0 || device >= 64) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "device ordinal out of range");
  if (raised[device].load()) return VECOPS_STATUS_OK;
  int32_t rc = raise_smem_limit(gemm_tcgen05_kernel<kInt8, OutT, false>, GemmTc::kSmemBytes, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  rc = raise_smem_limit(gemm_tcgen05_kernel<kInt8, OutT, true>, GemmPair::kSmemBytes, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  raised[device].store(true);
  return VECOPS_STATUS_OK;
}

// CTA pairs the device can keep resident at once (0 when it cannot run the pair form).  Asked once per device.
template <bool kInt8, typename OutT>
int pair_capacity(int device) {
  static std::atomic<int> cached[64];
  if (device < 0 || device >= 64) return 0;
  int value = cached[device].load();
  if (value != 0) return value > 0 ? value : 0;
  VecopsError ignored = {};
  ignored.struct_size = sizeof ignored;
  int clusters = 0;
  if (prepare_gemm_kernels<kInt8, OutT>(device, &ignored) == VECOPS_STATUS_OK) {
    cudaLaunchConfig_t config = {};
    cudaLaunchAttribute cluster = {};
    cluster.id = cudaLaunchAttributeClusterDimension;
    cluster.val.clusterDim.x = 2;
    cluster.val.clusterDim.y = 1;
    cluster.val.clusterDim.z = 1;
    config.gridDim = dim3(2);
    config.blockDim = dim3(GemmTc::kThreads);
    config.dynamicSmemBytes = GemmPair::kSmemBytes;
    config.attrs = &cluster;
    config.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tcgen05_kernel<kInt8, OutT, true>, &config) != cudaSuccess) clusters = 0;
    cudaGetLastError();
  }
  cached[device].store(clusters > 0 ? clusters : -1);
  return clusters > 0 ? clusters : 0;
}

template <bool kInt8, typename OutT, bool kTf32 = false>
int32_t launch_tcgen05(const VecopsB200Matmul& p, const DeviceState& dev, cudaStream_t stream, VecopsError* error,
                       const GatherTargets& gather = GatherTargets()) {
  using G = GemmTc;
  if (dev.prop.major != 10)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "tcgen05 kernels need an sm_100 device, found sm_%d%d", dev.prop.major,
                     dev.prop.minor);
  constexpr size_t elem = kInt8 ? 1 : kTf32 ? 4 : 2;
  const bool fp16_in = !kInt8 && !kTf32 && p.a_dtype == VECOPS_DTYPE_F16;
  const CUtensorMapDataType in_type = kInt8     ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                      : kTf32   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                      : fp16_in ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUtensorMapDataType out_type = std::is_same<OutT, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                       : std::is_same<OutT, __half>::value      ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                       : std::is_same<OutT, float>::value       ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                                                : CU_TENSOR_MAP_DATA_TYPE_INT32;
  const uint32_t box_k = G::kBlockKBytes / elem;
  int device = 0;
  cudaGetDevice(&device);
  // (the tf32 form has no CTA-pair variant)
  const Tcgen05Plan plan = plan_tcgen05(p, kInt8, sizeof(OutT), dev.prop.multiProcessorCount, kTf32 ? 0 : pair_capacity<kInt8, OutT>(device), elem);
  CUtensorMap map_a, map_b;
  GemmStoreMaps maps;
  // the split fp32 form walks three terms of k over operands stored as two ([hi | lo]): the maps cover what is stored
  const long long stored_k = kTf32 ? p.k / 3 * 2 : p.k;
  int32_t rc = make_map_2d(&map_a, in_type, elem, p.a, stored_k, p.m, p.a_stride_m * elem, box_k, G::kBlockM, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  rc = make_map_2d(&map_b, in_type, elem, p.b, stored_k, p.n, p.b_stride_n * elem, box_k, plan.pair ? GemmPair::kBRows : G::kBlockN, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  bool tma_store;
  int num_dest = 1;
  int col_offset = 0;
  if (gather.count > 0 && gather.multicast) {
    tma_store = false;
    col_offset = static_cast<int>(gather.col0);
    for (int d = 0; d < GemmStoreMaps::kMax; ++d) maps.map[d] = map_a;  // never dereferenced
  } else if (gather.count > 0) {
    // every destination is a full [M, n_total] matrix; this rank's tiles land at column col0 + ...
    tma_store = true;
    num_dest = gather.count;
    col_offset = static_cast<int>(gather.col0);
    for (int d = 0; d < gather.count; ++d) {
      rc = make_map_2d(&maps.map[d], out_type, sizeof(OutT), gather.c[d], gather.n_total, p.m, gather.ldc * sizeof(OutT),
                       128 / sizeof(OutT), 32, error);
      if (rc != VECOPS_STATUS_OK) return rc;
    }
    for (int d = gather.count; d < GemmStoreMaps::kMax; ++d) maps.map[d] = maps.map[0];
  } else {
    tma_store = !direct_epilogue_forced() && aligned16(p.c) && (p.c_stride_m * sizeof(OutT)) % 16 == 0;
    if (tma_store) {
      rc = make_map_2d(&maps.map[0], out_type, sizeof(OutT), p.c, p.n, p.m, p.c_stride_m * sizeof(OutT), 128 / sizeof(OutT), 32, error);
      if (rc != VECOPS_STATUS_OK) return rc;
    } else {
      maps.map[0] = map_a;  // never dereferenced
    }
    for (int d = 1; d < GemmStoreMaps::kMax; ++d) maps.map[d] = maps.map[0];
  }
  const uint32_t mma_m = plan.pair ? 2 * G::kBlockM : G::kBlockM;
  uint32_t idesc;
  if (kInt8) {
    idesc = umma_instr_desc(kUmmaAccS32, p.a_dtype == VECOPS_DTYPE_I8 ? kUmmaS8 : kUmmaU8,
                            p.b_dtype == VECOPS_DTYPE_I8 ? kUmmaS8 : kUmmaU8, mma_m, G::kBlockN);
  } else {
    const uint32_t format = kTf32 ? kUmmaTF32 : fp16_in ? kUmmaF16 : kUmmaBF16;
    idesc = umma_instr_desc(kUmmaAccF32, format, format, mma_m, G::kBlockN);
  }
  if constexpr (kTf32) {
    static std::atomic<bool> raised[kMaxDevices];
    if (device < 0 || device >= kMaxDevices || !raised[device].load()) {
      rc = raise_smem_limit(gemm_tcgen05_kernel<false, float, false, false, true>, GemmTc::kSmemBytes, error);
      if (rc != VECOPS_STATUS_OK) return rc;
      if (device >= 0 && device < kMaxDevices) raised[device].store(true);
    }
  } else {
    rc = prepare_gemm_kernels<kInt8, OutT>(device, error);
    if (rc != VECOPS_STATUS_OK) return rc;
  }
  // Tail tiles are cut along K when the caller supplied the scratch the slices meet in; without it the tail runs whole.
  int split = plan.split;
  uint32_t* partials = nullptr;
  unsigned long long* flags = nullptr;
  if (split > 1) {
    if (p.workspace == nullptr || !aligned16(p.workspace) || p.workspace_size < G::split_scratch_bytes(plan.scratch_slots)) {
      split = 1;
    } else {
      partials = static_cast<uint32_t*>(p.workspace);
      flags = reinterpret_cast<unsigned long long*>(static_cast<char*>(p.workspace) + G::split_flags_offset(plan.scratch_slots));
    }
  }
  cudaLaunchConfig_t config = {};
  cudaLaunchAttribute attributes[2] = {};
  config.blockDim = dim3(G::kThreads);
  config.stream = stream;
  config.attrs = attributes;
  // programmatic dependent launch: the kernel's set-up may overlap the tail of the previous kernel in the stream; it
  // waits (griddepcontrol.wait) before its first global access.  VECOPS_B200_GEMM_PDL=0 launches the ordinary way.
  const char* pdl = getenv("VECOPS_B200_GEMM_PDL");
  if (pdl == nullptr || pdl[0] != '0') {
    attributes[config.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[config.numAttrs].val.programmaticStreamSerializationAllowed = 1;
    ++config.numAttrs;
  }
  if (plan.pair) {
    config.gridDim = dim3(2 * plan.workers);
    config.dynamicSmemBytes = GemmPair::kSmemBytes;
    attributes[config.numAttrs].id = cudaLaunchAttributeClusterDimension;
    attributes[config.numAttrs].val.clusterDim.x = 2;
    attributes[config.numAttrs].val.clusterDim.y = 1;
    attributes[config.numAttrs].val.clusterDim.z = 1;
    ++config.numAttrs;
  } else {
    config.gridDim = dim3(plan.workers);
    config.dynamicSmemBytes = G::kSmemBytes;
  }
  OutT* c = static_cast<OutT*>(p.c);
  long long ldc = p.c_stride_m;
  int m = static_cast<int>(p.m), n = static_cast<int>(p.n), k = static_cast<int>(p.k);
  const float* scale = std::is_same<OutT, int32_t>::value ? nullptr : p.column_scale;
  int store_flag = tma_store ? 1 : 0;
  if (gather.count > 0 && gather.multicast) {
    c = static_cast<OutT*>(gather.c[0]);
    ldc = gather.ldc;
    store_flag = 2;
  }
  // Row-tiles that share a sweep over N: as many as keep their rows of A (about 32 MB) in L2 while B streams past.
  long long group_tiles = G::kGroupBytes / (static_cast<long long>(mma_m) * p.k * static_cast<long long>(elem));
  int raster_group = static_cast<int>(group_tiles < 4 ? 4 : group_tiles > 32 ? 32 : group_tiles);
  if (const char* v = getenv("VECOPS_B200_GEMM_GROUP")) {  // tuning aid
    const int forced = atoi(v);
    if (forced > 0) raster_group = forced;
  }
  unsigned long long nonce = split > 1 ? fresh_nonce(p.workspace) : 0ull;
  uint32_t* status_word = status_word_of(device);
  unsigned long long* trace = g_trace;
  EpilogueArgs epilogue = tl_epilogue;
  void* args[] = {&map_a, &map_b, &maps, &num_dest, &col_offset, &c, &ldc, &m, &n, &k, &scale, &idesc, &store_flag,
                  &raster_group, &split, &partials, &flags, &nonce, &epilogue, &status_word, &trace};
  const void* entry;
  if constexpr (kTf32) entry = reinterpret_cast<const void*>(gemm_tcgen05_kernel<false, float, false, false, true>);
  else entry = plan.pair ? reinterpret_cast<const void*>(gemm_tcgen05_kernel<kInt8, OutT, true>)
                         : reinterpret_cast<const void*>(gemm_tcgen05_kernel<kInt8, OutT, false>);
  cudaError_t launched = cudaLaunchKernelExC(&config, entry, args);
  if (launched != cudaSuccess) return cuda_fail(error, launched, "launch of the tcgen05 GEMM");
  g_launches.fetch_add(1);
  return VECOPS_STATUS_OK;
}

template <typename TA, typename TB, typename TC, typename Acc>
void launch_generic_typed(const VecopsB200Matmul& p, cudaStream_t stream) {
  dim3 grid(static_cast<unsigned>((p.n + 31) / 32), static_cast<unsigned>((p.m + 31) / 32));
  gemm_generic_kernel<TA, TB, TC, Acc><<<grid, 256, 0, stream>>>(
      static_cast<const TA*>(p.a), p.a_stride_m, p.a_stride_k, static_cast<const TB*>(p.b), p.b_stride_n, p.b_stride_k,
      static_cast<TC*>(p.c), p.c_stride_m, p.c_stride_n, static_cast<int>(p.m), static_cast<int>(p.n), static_cast<int>(p.k),
      p.column_scale, tl_epilogue);
  g_launches.fetch_add(1);
}

int32_t launch_generic(const VecopsB200Matmul& p, Row row, cudaStream_t stream, VecopsError* error) {
  if (p.m >= (INT64_C(1) << 31) || p.n >= (INT64_C(1) << 31) || p.k >= (INT64_C(1) << 31) || (p.m + 31) / 32 > 65535)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "extent too large for the strided kernel");
  using bf16 = __nv_bfloat16;
  const bool c_bf16 = p.c_dtype == VECOPS_DTYPE_BF16;
  switch (row) {
    case Row::F32: launch_generic_typed<float, float, float, float>(p, stream); break;
    case Row::BF16:
      if (c_bf16) launch_generic_typed<bf16, bf16, bf16, float>(p, stream);
      else launch_generic_typed<bf16, bf16, float, float>(p, stream);
      break;
    case Row::F16:
      if (p.c_dtype == VECOPS_DTYPE_F16) launch_generic_typed<__half, __half, __half, float>(p, stream);
      else launch_generic_typed<__half, __half, float, float>(p, stream);
      break;
    case Row::W8:
      if (c_bf16) launch_generic_typed<bf16, int8_t, bf16, float>(p, stream);
      else launch_generic_typed<bf16, int8_t, float, float>(p, stream);
      break;
    case Row::I8: {
      const bool as = p.a_dtype == VECOPS_DTYPE_I8, bs = p.b_dtype == VECOPS_DTYPE_I8;
      if (as && bs) launch_generic_typed<int8_t, int8_t, int32_t, uint32_t>(p, stream);
      else if (as) launch_generic_typed<int8_t, uint8_t, int32_t, uint32_t>(p, stream);
      else if (bs) launch_generic_typed<uint8_t, int8_t, int32_t, uint32_t>(p, stream);
      else launch_generic_typed<uint8_t, uint8_t, int32_t, uint32_t>(p, stream);
      break;
    }
    case Row::QI8: {
      const bool as = p.a_dtype == VECOPS_DTYPE_I8, bs = p.b_dtype == VECOPS_DTYPE_I8;
      if (c_bf16) {
        if (as && bs) launch_generic_typed<int8_t, int8_t, bf16, uint32_t>(p, stream);
        else if (as) launch_generic_typed<int8_t, uint8_t, bf16, uint32_t>(p, stream);
        else if (bs) launch_generic_typed<uint8_t, int8_t, bf16, uint32_t>(p, stream);
        else launch_generic_typed<uint8_t, uint8_t, bf16, uint32_t>(p, stream);
      } else {
        if (as && bs) launch_generic_typed<int8_t, int8_t, float, uint32_t>(p, stream);
        else if (as) launch_generic_typed<int8_t, uint8_t, float, uint32_t>(p, stream);
        else if (bs) launch_generic_typed<uint8_t, int8_t, float, uint32_t>(p, stream);
        else launch_generic_typed<uint8_t, uint8_t, float, uint32_t>(p, stream);
      }
      break;
    }
    default: return set_error(error, VECOPS_STATUS_INTERNAL_ERROR, "unclassified problem reached the strided kernel");
  }
  return VECOPS_STATUS_OK;
}

template <int kMTiles, typename OutT>
void launch_w8_small_typed(const VecopsB200Matmul& p, cudaStream_t stream) {
  using G = W8SmallM;
  dim3 grid(static_cast<unsigned>((p.n + G::kRowsPerCta - 1) / G::kRowsPerCta),
            static_cast<unsigned>((p.m + 8 * kMTiles - 1) / (8 * kMTiles)));
  w8_small_m_kernel<kMTiles, OutT><<<grid, G::kThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(p.a), p.a_stride_m, static_cast<const int8_t*>(p.b), p.b_stride_n, p.column_scale,
      static_cast<OutT*>(p.c), p.c_stride_m, static_cast<int>(p.m), static_cast<int>(p.n), static_cast<int>(p.k), tl_epilogue);
  g_launches.fetch_add(1);
}

template <int kChunks, bool kRows16, typename OutT>
int32_t launch_w8_stream_typed(const VecopsB200Matmul& p, const DeviceState& dev, cudaStream_t stream, VecopsError* error) {
  using G = W8Stream;
  auto kernel = w8_stream_kernel<kChunks, kRows16, OutT>;
  const int smem = G::smem_bytes(static_cast<int>(p.k), kRows16);
  int device = 0;
  cudaGetDevice(&device);
  // the attribute is per kernel instantiation and per device: raised once to the most any K needs
  static std::atomic<bool> raised[kMaxDevices];
  if (device < 0 || device >= kMaxDevices || !raised[device].load()) {
    const int32_t rc = raise_smem_limit(kernel, 227 * 1024, error);
    if (rc != VECOPS_STATUS_OK) return rc;
    if (device >= 0 && device < kMaxDevices) raised[device].store(true);
  }
  // one CTA per SM, each with an equal share of W's rows (to within one row); fewer when there are not 8 rows for each
  const long long items = (p.n + G::rows(kRows16) - 1) / G::rows(kRows16);
  const int grid = static_cast<int>(items < dev.prop.multiProcessorCount ? items : dev.prop.multiProcessorCount);
  cudaLaunchConfig_t config = {};
  cudaLaunchAttribute attributes[1] = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(G::kThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  config.attrs = attributes;
  // programmatic dependent launch: barrier set-up overlaps the previous kernel's tail (VECOPS_B200_GEMM_PDL=0: the ordinary way)
  const char* pdl = getenv("VECOPS_B200_GEMM_PDL");
  if (pdl == nullptr || pdl[0] != '0') {
    attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[0].val.programmaticStreamSerializationAllowed = 1;
    config.numAttrs = 1;
  }
  const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(p.a);
  const int8_t* w = static_cast<const int8_t*>(p.b);
  const float* scale = p.column_scale;
  OutT* c = static_cast<OutT*>(p.c);
  long long lda = p.a_stride_m, ldw = p.b_stride_n, ldc = p.c_stride_m;
  int m = static_cast<int>(p.m), n = static_cast<int>(p.n), k = static_cast<int>(p.k);
  EpilogueArgs epilogue = tl_epilogue;
  uint32_t* status_word = status_word_of(device);
  unsigned long long* trace = g_trace;
  void* args[] = {&a, &lda, &w, &ldw, &scale, &c, &ldc, &m, &n, &k, &epilogue, &status_word, &trace};
  const cudaError_t launched = cudaLaunchKernelExC(&config, reinterpret_cast<const void*>(kernel), args);
  if (launched != cudaSuccess) return cuda_fail(error, launched, "launch of the streaming weight-only kernel");
  g_launches.fetch_add(1);
  return VECOPS_STATUS_OK;
}

// The streaming form serves the decode shapes proper: few activation rows
// (they stay in registers) and a K that fits the shared-memory ring.
bool w8_stream_applicable(const VecopsB200Matmul& p, const DeviceState& dev) {
  const char* path = getenv("VECOPS_B200_W8_PATH");
  if (path != nullptr && strcmp(path, "small") == 0) return false;
  return dev.prop.major >= 9 && p.m <= 16 && p.k % W8Stream::kChunkK == 0 && p.k <= W8Stream::kMaxK &&
         static_cast<size_t>(W8Stream::smem_bytes(static_cast<int>(p.k), p.m > 8)) <= dev.prop.sharedMemPerBlockOptin;
}

int32_t launch_w8_small(const VecopsB200Matmul& p, const DeviceState& dev, cudaStream_t stream, VecopsError* error) {
  if (p.c_stride_n != 1) return set_error(error, VECOPS_STATUS_NOT_APPLICABLE, "w8_small_m needs a row-major C");
  if (w8_stream_applicable(p, dev)) {
    const bool bf16_out = p.c_dtype == VECOPS_DTYPE_BF16;
    const bool rows16 = p.m > 8, one_chunk = p.k <= 2048;
    if (!rows16 && one_chunk)
      return bf16_out ? launch_w8_stream_typed<1, false, __nv_bfloat16>(p, dev, stream, error) : launch_w8_stream_typed<1, false, float>(p, dev, stream, error);
    if (!rows16)
      return bf16_out ? launch_w8_stream_typed<2, false, __nv_bfloat16>(p, dev, stream, error) : launch_w8_stream_typed<2, false, float>(p, dev, stream, error);
    if (one_chunk)
      return bf16_out ? launch_w8_stream_typed<1, true, __nv_bfloat16>(p, dev, stream, error) : launch_w8_stream_typed<1, true, float>(p, dev, stream, error);
    return bf16_out ? launch_w8_stream_typed<2, true, __nv_bfloat16>(p, dev, stream, error) : launch_w8_stream_typed<2, true, float>(p, dev, stream, error);
  }
  if ((p.m + 31) / 32 > 65535) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "M too large for w8_small_m");
  const bool c_bf16 = p.c_dtype == VECOPS_DTYPE_BF16;
  if (p.m <= 8) {
    if (c_bf16) launch_w8_small_typed<1, __nv_bfloat16>(p, stream); else launch_w8_small_typed<1, float>(p, stream);
  } else if (p.m <= 16) {
    if (c_bf16) launch_w8_small_typed<2, __nv_bfloat16>(p, stream); else launch_w8_small_typed<2, float>(p, stream);
  } else {
    if (c_bf16) launch_w8_small_typed<4, __nv_bfloat16>(p, stream); else launch_w8_small_typed<4, float>(p, stream);
  }
  return VECOPS_STATUS_OK;
}

// The weight-only form of the tcgen05 GEMM: one (tile, K slice) per CTA.  Tiles are few for decode shapes (N / 256), so
// each is cut along K into the largest power-of-two number of slices that still fits the SMs in one wave.
struct W8MixedPlan {
  long long tiles = 0;
  int units = 0;   // 128-wide k units
  int split = 1;
  long long scratch_slots = 0;
};

W8MixedPlan plan_w8_mixed(const VecopsB200Matmul& p, size_t out_elem, int sms) {
  using G = GemmW8;
  W8MixedPlan plan;
  plan.tiles = ((p.m + G::kBlockM - 1) / G::kBlockM) * ((p.n + G::kBlockN - 1) / G::kBlockN);
  plan.units = static_cast<int>((p.k + G::kUnitK - 1) / G::kUnitK);
  if (!tail_split_forced_off())
    while (plan.split * 2 <= G::max_split(out_elem) && plan.tiles * (plan.split * 2) <= sms &&
           plan.split * 2 * G::kMinSliceUnits <= plan.units)
      plan.split *= 2;
  if (plan.split > 1) plan.scratch_slots = plan.tiles * plan.split;
  return plan;
}

int sm_count_for_query(const VecopsB200Matmul& p) {
  int sms = 148;  // the part this library is built for, when no device can be asked
  int device = p.device_index;
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) device = -1;
  if (device >= 0) {
    int value = 0;
    if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && value > 0) sms = value;
  }
  cudaGetLastError();  // a host without a GPU is a legal caller of the query
  return sms;
}

uint64_t w8_mixed_scratch(const VecopsB200Matmul& p) {
  if (p.m <= 0 || p.n <= 0 || p.k <= 0) return 0;
  const W8MixedPlan plan = plan_w8_mixed(p, p.c_dtype == VECOPS_DTYPE_F32 ? 4 : 2, sm_count_for_query(p));
  return plan.scratch_slots > 0 ? GemmW8::split_scratch_bytes(plan.scratch_slots) : 0;
}

template <typename OutT>
int32_t launch_w8_mixed(const VecopsB200Matmul& p, const DeviceState& dev, cudaStream_t stream, VecopsError* error) {
  using G = GemmW8;
  if (dev.prop.major != 10)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "tcgen05 kernels need an sm_100 device, found sm_%d%d", dev.prop.major,
                     dev.prop.minor);
  int device = 0;
  cudaGetDevice(&device);
  auto kernel = gemm_tcgen05_kernel<false, OutT, false, true>;
  static std::atomic<bool> raised[kMaxDevices];
  if (device < 0 || device >= kMaxDevices || !raised[device].load()) {
    const int32_t rc = raise_smem_limit(kernel, G::kSmemBytes, error);
    if (rc != VECOPS_STATUS_OK) return rc;
    if (device >= 0 && device < kMaxDevices) raised[device].store(true);
  }
  const W8MixedPlan plan = plan_w8_mixed(p, sizeof(OutT), dev.prop.multiProcessorCount);
  if (plan.tiles * plan.split > 0x7fffffffLL) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "problem too large for w8_tcgen05");
  CUtensorMap map_a, map_w;
  GemmStoreMaps maps;
  int32_t rc = make_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.a, p.k, p.m, p.a_stride_m * 2, 64, G::kBlockM, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  rc = make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.b, p.k, p.n, p.b_stride_n, G::kUnitK, G::kBlockN, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  const CUtensorMapDataType out_type = std::is_same<OutT, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const bool tma_store = !direct_epilogue_forced() && aligned16(p.c) && (p.c_stride_m * sizeof(OutT)) % 16 == 0;
  if (tma_store) {
    rc = make_map_2d(&maps.map[0], out_type, sizeof(OutT), p.c, p.n, p.m, p.c_stride_m * sizeof(OutT), 128 / sizeof(OutT), 32, error);
    if (rc != VECOPS_STATUS_OK) return rc;
  } else {
    maps.map[0] = map_a;  // never dereferenced
  }
  for (int d = 1; d < GemmStoreMaps::kMax; ++d) maps.map[d] = maps.map[0];
  int split = plan.split;
  uint32_t* partials = nullptr;
  unsigned long long* flags = nullptr;
  if (split > 1) {
    if (p.workspace == nullptr || !aligned16(p.workspace) || p.workspace_size < G::split_scratch_bytes(plan.scratch_slots)) {
      split = 1;  // no scratch for the slices to meet in: every tile runs whole, on fewer SMs
    } else {
      partials = static_cast<uint32_t*>(p.workspace);
      flags = reinterpret_cast<unsigned long long*>(static_cast<char*>(p.workspace) + G::split_flags_offset(plan.scratch_slots));
    }
  }
  cudaLaunchConfig_t config = {};
  cudaLaunchAttribute attributes[1] = {};
  config.gridDim = dim3(static_cast<unsigned>(plan.tiles * split));
  config.blockDim = dim3(G::kThreads);
  config.dynamicSmemBytes = G::kSmemBytes;
  config.stream = stream;
  config.attrs = attributes;
  const char* pdl = getenv("VECOPS_B200_GEMM_PDL");
  if (pdl == nullptr || pdl[0] != '0') {
    attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[0].val.programmaticStreamSerializationAllowed = 1;
    config.numAttrs = 1;
  }
  uint32_t idesc = umma_instr_desc(kUmmaAccF32, kUmmaBF16, kUmmaBF16, G::kBlockM, G::kBlockN);
  OutT* c = static_cast<OutT*>(p.c);
  long long ldc = p.c_stride_m;
  int m = static_cast<int>(p.m), n = static_cast<int>(p.n), k = static_cast<int>(p.k);
  const float* scale = p.column_scale;
  int store_flag = tma_store ? 1 : 0, num_dest = 1, col_offset = 0, raster_group = 4;
  unsigned long long nonce = split > 1 ? fresh_nonce(p.workspace) : 0ull;
  uint32_t* status_word = status_word_of(device);
  unsigned long long* trace = g_trace;
  EpilogueArgs epilogue = tl_epilogue;
  void* args[] = {&map_a, &map_w, &maps, &num_dest, &col_offset, &c, &ldc, &m, &n, &k, &scale, &idesc, &store_flag,
                  &raster_group, &split, &partials, &flags, &nonce, &epilogue, &status_word, &trace};
  cudaError_t launched = cudaLaunchKernelExC(&config, reinterpret_cast<const void*>(kernel), args);
  if (launched != cudaSuccess) return cuda_fail(error, launched, "launch of w8_tcgen05");
  g_launches.fetch_add(1);
  return VECOPS_STATUS_OK;
}

// ---- FP32 on the tensor cores: three tf32 products of split operands, run as one product over a tripled K.
// Scratch layout: A' [M, 2 Kp] f32 ([hi | lo]) | B' [N, 2 Kp] f32 | the scratch the inner tcgen05 GEMM's K slices meet in.
struct Tf32x3Plan {
  long long kp = 0;          // K rounded up to the 32 words of a k-block
  uint64_t a_bytes = 0, b_bytes = 0, inner = 0;
  VecopsB200Matmul inner_problem{};
};

uint64_t align256(uint64_t v) { return (v + 255u) & ~uint64_t{255}; }

Tf32x3Plan plan_tf32x3(const VecopsB200Matmul& p, int sms) {
  Tf32x3Plan plan;
  plan.kp = (p.k + 31) & ~INT64_C(31);
  // each operand is stored once as [hi | lo], 2 * kp wide; the GEMM walks 3 * kp of k and its producer picks the term
  plan.a_bytes = align256(static_cast<uint64_t>(p.m) * 2 * plan.kp * 4);
  plan.b_bytes = align256(static_cast<uint64_t>(p.n) * 2 * plan.kp * 4);
  VecopsB200Matmul q = p;
  q.k = 3 * plan.kp;
  q.a_stride_m = q.b_stride_n = 2 * plan.kp;
  q.a_stride_k = q.b_stride_k = 1;
  plan.inner_problem = q;
  const Tcgen05Plan inner = plan_tcgen05(q, false, 4, sms, 0, 4);
  plan.inner = inner.scratch_slots > 0 ? GemmTc::split_scratch_bytes(inner.scratch_slots) : 0;
  return plan;
}

uint64_t tf32x3_scratch(const VecopsB200Matmul& p) {
  if (p.m <= 0 || p.n <= 0 || p.k <= 0) return 0;
  const Tf32x3Plan plan = plan_tf32x3(p, sm_count_for_query(p));
  return plan.a_bytes + plan.b_bytes + plan.inner;
}

// The split costs two more launches and reads and writes both operands once: it pays from a few hundred MFLOP up.
bool tf32x3_worthwhile(const VecopsB200Matmul& p) {
  const char* v = getenv("VECOPS_B200_F32_TF32X3");  // tuning aid: 0 = never, 1 = whenever it applies
  if (v != nullptr && v[0] == '0') return false;
  if (v != nullptr && v[0] == '1') return true;
  // (up to K = 8192: the tensor core's fp32 accumulation is coarser than a chain of FMAs, and the relative error of the
  // product, about 2e-6 at K = 1024 and 4e-6 at K = 4096, must stay inside the fp32 bar of 1e-5)
  return p.m >= 256 && p.n >= 256 && p.k >= 256 && p.k <= 8192;
}

int32_t launch_f32_tf32x3(const VecopsB200Matmul& p, const DeviceState& dev, cudaStream_t stream, VecopsError* error) {
  Tf32x3Plan plan = plan_tf32x3(p, dev.prop.multiProcessorCount);
  const uint64_t need = plan.a_bytes + plan.b_bytes + plan.inner;
  if (p.workspace == nullptr || !aligned16(p.workspace) || p.workspace_size < need)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "f32_tf32x3 needs %llu bytes of 16-byte aligned device workspace, %llu were supplied",
                     (unsigned long long)need, (unsigned long long)p.workspace_size);
  char* base = static_cast<char*>(p.workspace);
  float* a_split = reinterpret_cast<float*>(base);
  float* b_split = reinterpret_cast<float*>(base + plan.a_bytes);
  const int kp = static_cast<int>(plan.kp), k = static_cast<int>(p.k);
  const long long k_groups = (kp / 32 + kSplitTiles - 1) / kSplitTiles;
  const long long a_blocks = k_groups * ((p.m + 31) / 32), b_blocks = k_groups * ((p.n + 31) / 32);
  if (a_blocks + b_blocks > 0x7fffffffLL) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "extent too large for f32_tf32x3");
  const SplitOperand split_a{static_cast<const float*>(p.a), p.a_stride_m, p.a_stride_k, a_split, static_cast<int>(p.m)};
  const SplitOperand split_b{static_cast<const float*>(p.b), p.b_stride_n, p.b_stride_k, b_split, static_cast<int>(p.n)};
  f32_split3_kernel<<<static_cast<unsigned>(a_blocks + b_blocks), 256, 0, stream>>>(split_a, split_b, static_cast<int>(a_blocks), k, kp);
  g_launches.fetch_add(1);
  VecopsB200Matmul q = plan.inner_problem;
  q.a = a_split;
  q.b = b_split;
  q.workspace = plan.inner != 0 ? base + plan.a_bytes + plan.b_bytes : nullptr;
  q.workspace_size = plan.inner;
  return launch_tcgen05<false, float, true>(q, dev, stream, error);
}

// Scratch for the K slices of the tail tiles.  The grid is one CTA per SM; the SM count comes from the device the
// problem names when one is usable, else from the part this library is built for (148).
uint64_t tcgen05_tail_scratch(const VecopsB200Matmul& p, bool int8) {
  using G = GemmTc;
  if (p.m <= 0 || p.n <= 0 || p.k <= 0) return 0;
  int sms = 148;
  int device = p.device_index;
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) device = -1;
  if (device >= 0) {
    int value = 0;
    if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && value > 0) sms = value;
  }
  cudaGetLastError();  // a host without a GPU is a legal caller of the query
  const size_t out = (int8 || p.c_dtype == VECOPS_DTYPE_F32) ? 4 : 2;
  // The launcher may find fewer resident pairs than sms / 2 and then lays the work out differently; the answer covers
  // both layouts (a launch whose scratch is too small for its layout runs its tail whole).
  const Tcgen05Plan paired = plan_tcgen05(p, int8, out, sms, sms / 2);
  const Tcgen05Plan single = plan_tcgen05(p, int8, out, sms, 0);
  const long long slots = paired.scratch_slots > single.scratch_slots ? paired.scratch_slots : single.scratch_slots;
  return slots > 0 ? G::split_scratch_bytes(slots) : 0;
}

uint64_t fresh_nonce(const void* salt) {
  static std::atomic<uint64_t> counter{0x243F6A8885A308D3ull};
  uint64_t z = counter.fetch_add(0x9E3779B97F4A7C15ull) ^ reinterpret_cast<uintptr_t>(salt);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z == 0 ? 1 : z;
}

template <typename OutT>
int32_t launch_w8_tcgen05_typed(const VecopsB200Matmul& p, const DeviceState& dev, cudaStream_t stream, VecopsError* error) {
  using G = W8Tc;
  if (dev.prop.major != 10)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "tcgen05 kernels need an sm_100 device, found sm_%d%d", dev.prop.major,
                     dev.prop.minor);
  const int mpad = G::m_padded(static_cast<int>(p.m));
  const uint64_t need = G::scratch_bytes(static_cast<int>(p.m), p.k);
  if (p.workspace == nullptr || p.workspace_size < need)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "w8_tcgen05 needs %llu bytes of device workspace, %llu were supplied",
                     (unsigned long long)need, (unsigned long long)p.workspace_size);
  if (!aligned16(p.workspace)) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "workspace must be 16-byte aligned");
  CUtensorMap map_w, map_a;
  int32_t rc = make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.b, p.k, p.n, p.b_stride_n, G::kBlockK, G::kTileN, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  char* scratch = static_cast<char*>(p.workspace);
  float* partials = reinterpret_cast<float*>(scratch);
  auto* flags = reinterpret_cast<unsigned long long*>(scratch + G::flags_offset(mpad));
  float* inv_scales = reinterpret_cast<float*>(scratch + G::scales_offset(mpad));
  __half* act16 = reinterpret_cast<__half*>(scratch + G::act_offset(mpad));
  const long long act_pitch = G::act_pitch(p.k);
  // CTA pairs: 256-row weight tiles, one MMA for both CTAs.
  auto pair_kernel = w8_tcgen05_kernel<OutT, true>;
  auto single_kernel = w8_tcgen05_kernel<OutT, false>;
  static_assert(G::smem_bytes(G::kMaxM) <= 227 * 1024 && G::smem_bytes(16) <= 227 * 1024, "w8_tcgen05 shared memory budget");
  int device = 0;
  cudaGetDevice(&device);
  static std::atomic<bool> raised[64];
  if (device < 0 || device >= 64 || !raised[device].load()) {
    rc = raise_smem_limit(single_kernel, 227 * 1024, error);
    if (rc != VECOPS_STATUS_OK) return rc;
    rc = raise_smem_limit(pair_kernel, 227 * 1024, error);
    if (rc != VECOPS_STATUS_OK) return rc;
    if (device >= 0 && device < 64) raised[device].store(true);
  }
  static std::atomic<int> pair_cache[64];
  int pairs = device >= 0 && device < 64 ? pair_cache[device].load() : -1;
  if (pairs == 0) {
    pairs = cluster_capacity(reinterpret_cast<const void*>(pair_kernel), G::kThreads, G::smem_bytes(G::kMaxM));
    if (device >= 0 && device < 64) pair_cache[device].store(pairs > 0 ? pairs : -1);
  }
  if (pairs < 0) pairs = 0;
  if (pairs > G::kMaxGrid / 2) pairs = G::kMaxGrid / 2;
  // Measured slower than single CTAs (36 vs 41 us at M = 128): each issuing thread still runs the same number of
  // MMAs, and every hand-off crosses SMs.  Kept as an option for tuning (VECOPS_B200_W8TC_PAIR=1).
  bool pair = false;
  if (const char* v = getenv("VECOPS_B200_W8TC_PAIR")) pair = v[0] == '1' && pairs > 0;
  // Operands: bf16 x bf16 - the activations as the caller stores them, the weights widened to bf16, both exact - unless
  // VECOPS_B200_W8TC_FP16=1 asks for the older form (a row-scaled fp16 copy of the activations made by a pre-pass kernel,
  // weights widened to fp16: one instruction less per weight, one launch more).
  const char* fp16_form = getenv("VECOPS_B200_W8TC_FP16");
  const bool bf16_operands = !(fp16_form != nullptr && fp16_form[0] == '1');
  if (bf16_operands) {
    rc = make_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.a, p.k, p.m, p.a_stride_m * 2, 64, pair ? mpad / 2 : mpad, error);
    if (rc != VECOPS_STATUS_OK) return rc;
    inv_scales = nullptr;
  } else {
    rc = make_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, act16, p.k, p.m, act_pitch * 2, 64, pair ? mpad / 2 : mpad, error);
    if (rc != VECOPS_STATUS_OK) return rc;
    w8_prepare_activations_kernel<<<static_cast<int>(p.m), W8Prepare::kThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(p.a), p.a_stride_m, act16, act_pitch, inv_scales, static_cast<int>(p.k));
    g_launches.fetch_add(1);
  }
  const int tile_rows = pair ? 2 * G::kTileN : G::kTileN;
  const long long units = ((p.n + tile_rows - 1) / tile_rows) * ((p.k + G::kBlockK - 1) / G::kBlockK);
  long long workers = pair ? pairs : (dev.prop.multiProcessorCount < G::kMaxGrid ? dev.prop.multiProcessorCount : G::kMaxGrid);
  if (units < workers) workers = units;
  // A = the widened weights (from tensor memory), B = the activations, same 16-bit format, fp32 accumulate
  const uint32_t format = bf16_operands ? kUmmaBF16 : kUmmaF16;
  uint32_t idesc = umma_instr_desc(kUmmaAccF32, format, format, tile_rows, mpad);
  cudaLaunchConfig_t config = {};
  cudaLaunchAttribute cluster = {};
  config.blockDim = dim3(G::kThreads);
  config.dynamicSmemBytes = G::smem_bytes(mpad);
  config.stream = stream;
  config.gridDim = dim3(static_cast<unsigned>(pair ? 2 * workers : workers));
  if (pair) {
    cluster.id = cudaLaunchAttributeClusterDimension;
    cluster.val.clusterDim.x = 2;
    cluster.val.clusterDim.y = 1;
    cluster.val.clusterDim.z = 1;
    config.attrs = &cluster;
    config.numAttrs = 1;
  }
  const float* scale = p.column_scale;
  OutT* c = static_cast<OutT*>(p.c);
  long long ldc = p.c_stride_m;
  int m = static_cast<int>(p.m), n = static_cast<int>(p.n), k = static_cast<int>(p.k), mpad_arg = mpad;
  const float* inv = inv_scales;
  unsigned long long nonce = fresh_nonce(p.workspace);
  uint32_t* status_word = status_word_of(device);
  unsigned long long* trace = g_trace;
  EpilogueArgs epilogue = tl_epilogue;
  void* args[] = {&map_w, &map_a, &scale, &c, &ldc, &m, &n, &k, &mpad_arg, &partials, &flags, &inv, &nonce, &idesc, &epilogue, &status_word, &trace};
  cudaError_t launched = cudaLaunchKernelExC(&config, pair ? reinterpret_cast<const void*>(pair_kernel) : reinterpret_cast<const void*>(single_kernel), args);
  if (launched != cudaSuccess) return cuda_fail(error, launched, "launch of w8_tcgen05");
  g_launches.fetch_add(1);
  return VECOPS_STATUS_OK;
}

int32_t launch_f32(const VecopsB200Matmul& p, cudaStream_t stream, VecopsError* error) {
  if ((p.m + 63) / 64 > 65535) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "M too large for f32_simt");
  dim3 grid(static_cast<unsigned>((p.n + 63) / 64), static_cast<unsigned>((p.m + 63) / 64));
  // whole tiles and 16-byte aligned rows: the 8 x 8-per-thread form (VECOPS_B200_F32_TILE8=0 keeps the general kernel)
  const char* tile8_switch = getenv("VECOPS_B200_F32_TILE8");
  const bool b_k_contig = p.b_stride_k == 1, b_n_contig = p.b_stride_n == 1;
  const int64_t ldb = b_k_contig ? p.b_stride_n : p.b_stride_k;
  const bool tile8 = !(tile8_switch != nullptr && tile8_switch[0] == '0') && p.m % 64 == 0 && p.n % 64 == 0 && p.k % 16 == 0 && p.k > 0 &&
                     p.a_stride_k == 1 && p.c_stride_n == 1 && (b_k_contig || b_n_contig) && p.a_stride_m % 4 == 0 && ldb % 4 == 0 &&
                     p.c_stride_m % 4 == 0 && aligned16(p.a) && aligned16(p.b) && aligned16(p.c);
  if (tile8) {
    // 8 x 8 outputs per thread (64 threads); VECOPS_B200_F32_TILE8=4 selects 4 x 8 per thread (128 threads), measured 10 % slower
    // at 1024^3 (88 vs 80 us; the general kernel 92 us)
    const bool eight = !(tile8_switch != nullptr && tile8_switch[0] == '4');
    const float* pa = static_cast<const float*>(p.a);
    const float* pb = static_cast<const float*>(p.b);
    float* pc = static_cast<float*>(p.c);
    const long long lda = p.a_stride_m, ldb_arg = ldb, ldc = p.c_stride_m;
    int k = static_cast<int>(p.k);
    EpilogueArgs epilogue = tl_epilogue;
    // Too few tiles for the SMs: clusters of 2 or 4 CTAs share a tile along K (VECOPS_B200_F32_SPLIT=1|2|4 forces the count)
    int device = 0, sms = 148;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const long long tiles = static_cast<long long>(grid.x) * grid.y;
    int split = 1;
    if (eight) {
      // measured at 1024^3 on one box: whole 94 us, pairs 72 us, clusters of four 107 us (three serial remote reads per sum
      // and four CTAs to co-schedule cost more than the extra warps give) - so pairs, and four only when forced
      if (tiles * 2 <= 8LL * sms && p.k % 32 == 0 && p.k >= 128) split = 2;
      if (const char* forced = getenv("VECOPS_B200_F32_SPLIT")) {
        const int want = atoi(forced);
        if ((want == 1 || want == 2 || want == 4) && p.k % (16 * want) == 0) split = want;
      }
    }
    if (!eight) {
      if (b_k_contig) gemm_f32_tile8_kernel<true, 4, 1><<<grid, 128, 0, stream>>>(pa, lda, pb, ldb_arg, pc, ldc, k, epilogue);
      else gemm_f32_tile8_kernel<false, 4, 1><<<grid, 128, 0, stream>>>(pa, lda, pb, ldb_arg, pc, ldc, k, epilogue);
    } else {
      const void* kernel = nullptr;
      if (split == 4) kernel = b_k_contig ? reinterpret_cast<const void*>(gemm_f32_tile8_kernel<true, 8, 4>) : reinterpret_cast<const void*>(gemm_f32_tile8_kernel<false, 8, 4>);
      else if (split == 2) kernel = b_k_contig ? reinterpret_cast<const void*>(gemm_f32_tile8_kernel<true, 8, 2>) : reinterpret_cast<const void*>(gemm_f32_tile8_kernel<false, 8, 2>);
      else kernel = b_k_contig ? reinterpret_cast<const void*>(gemm_f32_tile8_kernel<true, 8, 1>) : reinterpret_cast<const void*>(gemm_f32_tile8_kernel<false, 8, 1>);
      cudaLaunchConfig_t config{};
      config.gridDim = dim3(grid.x, grid.y, static_cast<unsigned>(split));
      config.blockDim = dim3(64, 1, 1);
      config.dynamicSmemBytes = 0;
      config.stream = stream;
      cudaLaunchAttribute attribute{};
      attribute.id = cudaLaunchAttributeClusterDimension;
      attribute.val.clusterDim.x = 1;
      attribute.val.clusterDim.y = 1;
      attribute.val.clusterDim.z = static_cast<unsigned>(split);
      config.attrs = &attribute;
      config.numAttrs = split > 1 ? 1 : 0;
      void* args[] = {&pa, const_cast<long long*>(&lda), &pb, const_cast<long long*>(&ldb_arg), &pc, const_cast<long long*>(&ldc), &k, &epilogue};
      const cudaError_t launched = cudaLaunchKernelExC(&config, kernel, args);
      if (launched != cudaSuccess) return cuda_fail(error, launched, "launch of f32_simt (whole-tile form)");
    }
    g_launches.fetch_add(1);
    return VECOPS_STATUS_OK;
  }
  gemm_f32_kernel<<<grid, 256, 0, stream>>>(static_cast<const float*>(p.a), p.a_stride_m, static_cast<const float*>(p.b), p.b_stride_n,
                                            p.b_stride_k, static_cast<float*>(p.c), p.c_stride_m, static_cast<int>(p.m),
                                            static_cast<int>(p.n), static_cast<int>(p.k), tl_epilogue);
  g_launches.fetch_add(1);
  return VECOPS_STATUS_OK;
}

}  // namespace

int32_t shim_encode_map(CUtensorMap* out, CUtensorMapDataType dtype, uint32_t rank, const void* base, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box, VecopsError* error) {
  if (rank < 2 || rank > 3) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "tensor map rank %u not served", rank);
  if (g_encode_tiled == nullptr) return set_error(error, VECOPS_STATUS_LOAD_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t d[3] = {dims[0], dims[1], rank > 2 ? dims[2] : 1};
  cuuint64_t s[2] = {strides_bytes[0], rank > 2 ? strides_bytes[1] : 0};
  cuuint32_t b[3] = {box[0], box[1], rank > 2 ? box[2] : 1};
  cuuint32_t e[3] = {1, 1, 1};
  const CUresult result = g_encode_tiled(out, dtype, rank, const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (result != CUDA_SUCCESS)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "cuTensorMapEncodeTiled failed (%d) for dims=(%llu,%llu,%llu) strides=(%llu,%llu)",
                     static_cast<int>(result), (unsigned long long)d[0], (unsigned long long)d[1], (unsigned long long)d[2],
                     (unsigned long long)s[0], (unsigned long long)s[1]);
  return VECOPS_STATUS_OK;
}

int32_t shim_device_facts(int device, int* sm_count, int* major, uint32_t** status_word, VecopsError* error) {
  const DeviceState* dev = nullptr;
  const int32_t rc = device_state(device, &dev, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  if (sm_count != nullptr) *sm_count = dev->prop.multiProcessorCount;
  if (major != nullptr) *major = dev->prop.major;
  if (status_word != nullptr) *status_word = status_word_of(device);
  return VECOPS_STATUS_OK;
}

uint64_t shim_nonce(const void* salt) { return fresh_nonce(salt); }

uint32_t shim_take_status(int device) { return take_status_word(device); }

unsigned long long* shim_trace() { return g_trace; }

}  // namespace vb200

using namespace vb200;

extern "C" {

int32_t vecops_b200_matmul_select(const VecopsB200Matmul* problem, uint32_t* kernel, VecopsError* error) {
  Row row;
  int32_t rc = check_problem(problem, &row, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  if (kernel == nullptr) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "kernel output pointer is null");
  return select_kernel(*problem, row, kernel, error);
}

int32_t vecops_b200_matmul_workspace(const VecopsB200Matmul* problem, uint64_t* bytes, VecopsError* error) {
  Row row;
  int32_t rc = check_problem(problem, &row, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  if (bytes == nullptr) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "bytes output pointer is null");
  uint32_t kernel;
  rc = select_kernel(*problem, row, &kernel, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  // Kernels whose CTAs exchange partial sums through device scratch: the stream-K weight-only kernel, and the
  // tcgen05 GEMMs when their last wave is cut along K.  Every other split-K meets in shared memory.
  *bytes = 0;
  if (kernel == VECOPS_B200_KERNEL_W8_TCGEN05) {
    *bytes = w8_tmem_form() ? W8Tc::scratch_bytes(static_cast<int>(problem->m), problem->k) : w8_mixed_scratch(*problem);
  } else if (kernel == VECOPS_B200_KERNEL_F32_TF32X3) {
    *bytes = tf32x3_scratch(*problem);
  } else if (kernel == VECOPS_B200_KERNEL_BF16_TCGEN05 || kernel == VECOPS_B200_KERNEL_I8_TCGEN05) {
    *bytes = tcgen05_tail_scratch(*problem, kernel == VECOPS_B200_KERNEL_I8_TCGEN05);
  }
  return VECOPS_STATUS_OK;
}

int32_t vecops_b200_matmul_run(const VecopsB200Matmul* problem, VecopsError* error) {
  Row row;
  int32_t rc = check_problem(problem, &row, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  const VecopsB200Matmul& p = *problem;
  uint32_t kernel;
  rc = select_kernel(p, row, &kernel, error, false);
  if (rc != VECOPS_STATUS_OK) return rc;
  if (p.m == 0 || p.n == 0) return VECOPS_STATUS_OK;
  if (p.c == nullptr || (p.k > 0 && (p.a == nullptr || p.b == nullptr)))
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "a, b or c is null for a non-empty problem");

  int device = 0;
  rc = current_device(p, &device, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  int previous = -1;
  cudaGetDevice(&previous);
  if (previous != device) {
    cudaError_t status = cudaSetDevice(device);
    if (status != cudaSuccess) return cuda_fail(error, status, "cudaSetDevice");
  }
  const DeviceState* dev = nullptr;
  rc = device_state(device, &dev, error);
  cudaStream_t stream = static_cast<cudaStream_t>(p.stream);

  if (rc == VECOPS_STATUS_OK) {
    if (p.k == 0 && !tl_epilogue.active) {
      // empty reduction: C = 0 (include/vecops/ops/Matmul.h:41-43)
      const size_t esz = dtype_size(p.c_dtype);
      const long long total = p.m * p.n;
      const int blocks = static_cast<int>(total / 256 + 1 < 4096 ? total / 256 + 1 : 4096);
      fill_zero_kernel<<<blocks, 256, 0, stream>>>(static_cast<uint8_t*>(p.c), p.c_stride_m * esz, p.c_stride_n * esz,
                                                   static_cast<int>(esz), p.m, p.n);
      g_launches.fetch_add(1);
    } else {
      switch (kernel) {
        case VECOPS_B200_KERNEL_GENERIC: rc = launch_generic(p, row, stream, error); break;
        case VECOPS_B200_KERNEL_F32_SIMT: rc = launch_f32(p, stream, error); break;
        case VECOPS_B200_KERNEL_F32_TF32X3: rc = launch_f32_tf32x3(p, *dev, stream, error); break;
        case VECOPS_B200_KERNEL_BF16_TCGEN05:
          rc = p.c_dtype == VECOPS_DTYPE_BF16  ? launch_tcgen05<false, __nv_bfloat16>(p, *dev, stream, error)
               : p.c_dtype == VECOPS_DTYPE_F16 ? launch_tcgen05<false, __half>(p, *dev, stream, error)
                                               : launch_tcgen05<false, float>(p, *dev, stream, error);
          break;
        case VECOPS_B200_KERNEL_I8_TCGEN05:
          rc = p.c_dtype == VECOPS_DTYPE_I32    ? launch_tcgen05<true, int32_t>(p, *dev, stream, error)
               : p.c_dtype == VECOPS_DTYPE_BF16 ? launch_tcgen05<true, __nv_bfloat16>(p, *dev, stream, error)
                                                : launch_tcgen05<true, float>(p, *dev, stream, error);
          break;
        case VECOPS_B200_KERNEL_W8_SMALL_M: rc = launch_w8_small(p, *dev, stream, error); break;
        case VECOPS_B200_KERNEL_W8_TCGEN05:
          if (w8_tmem_form())
            rc = p.c_dtype == VECOPS_DTYPE_BF16 ? launch_w8_tcgen05_typed<__nv_bfloat16>(p, *dev, stream, error)
                                                : launch_w8_tcgen05_typed<float>(p, *dev, stream, error);
          else
            rc = p.c_dtype == VECOPS_DTYPE_BF16 ? launch_w8_mixed<__nv_bfloat16>(p, *dev, stream, error)
                                                : launch_w8_mixed<float>(p, *dev, stream, error);
          break;
        default: rc = set_error(error, VECOPS_STATUS_INTERNAL_ERROR, "kernel id %u has no launcher", kernel);
      }
    }
  }
  if (rc == VECOPS_STATUS_OK) {
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) rc = cuda_fail(error, status, "kernel launch");
  }
  if (rc == VECOPS_STATUS_OK && (p.flags & VECOPS_B200_MATMUL_FLAG_ASYNC) == 0) {
    cudaError_t status = cudaStreamSynchronize(stream);
    if (status != cudaSuccess) {
      rc = cuda_fail(error, status, "cudaStreamSynchronize");
    } else if (const uint32_t word = take_status_word(device)) {
      rc = set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "kernel '%s' on device %d: a bounded device wait ran out (status 0x%x)",
                     kKernelNames[kernel], device, word);
    }
  }
  if (previous >= 0 && previous != device) cudaSetDevice(previous);
  return rc;
}

int32_t vecops_b200_matmul_run_fused(const VecopsB200Matmul* problem, const VecopsB200Epilogue* epilogue, VecopsError* error) {
  Row row;
  int32_t rc = check_problem(problem, &row, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  if (epilogue == nullptr) return vecops_b200_matmul_run(problem, error);
  if (epilogue->struct_size < offsetof(VecopsB200Epilogue, row_scale))
    return set_error(error, VECOPS_STATUS_ABI_MISMATCH, "epilogue record is %u bytes, this library needs at least %zu", epilogue->struct_size,
                     offsetof(VecopsB200Epilogue, row_scale));
  const float* row_scale = epilogue->struct_size >= sizeof(VecopsB200Epilogue) ? epilogue->row_scale : nullptr;
  if (epilogue->activation >= VECOPS_B200_ACTIVATION_COUNT_)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "unknown activation %u", epilogue->activation);
  EpilogueArgs args;
  args.activation = static_cast<int>(epilogue->activation);
  args.alpha = epilogue->alpha;
  args.clamp_lo = epilogue->clamp_lo;
  args.clamp_hi = epilogue->clamp_hi;
  if (epilogue->cin != nullptr) {
    args.cin = epilogue->cin;
    args.cin_stride_m = epilogue->cin_stride_m;
    args.cin_stride_n = epilogue->cin_stride_n;
    if (epilogue->cin_stride_m < 0 || epilogue->cin_stride_n < 0)
      return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "accumulator input strides must not be negative");
    if (row == Row::I8 || row == Row::QI8) {
      if (epilogue->cin_dtype != VECOPS_DTYPE_I32)
        return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "int32 accumulators take an int32 accumulator input");
      args.cin_kind = kCinI32;
    } else if (epilogue->cin_dtype == VECOPS_DTYPE_F32) {
      args.cin_kind = kCinF32;
    } else if (epilogue->cin_dtype == VECOPS_DTYPE_BF16) {
      args.cin_kind = kCinBF16;
    } else {
      return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "fp32 accumulators take an f32 or bf16 accumulator input");
    }
  }
  if (row == Row::I8 && (epilogue->alpha != 1.f || epilogue->activation != VECOPS_B200_ACTIVATION_NONE || row_scale != nullptr))
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "int32 accumulators take an accumulator input only: no factor, no activation");
  args.row_scale = row_scale;
  if (epilogue->activation == VECOPS_B200_ACTIVATION_CLAMP && !(epilogue->clamp_lo <= epilogue->clamp_hi))
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "clamp needs clamp_lo <= clamp_hi");
  args.active = (args.cin_kind != kCinNone || args.alpha != 1.f || args.activation != kActNone || args.row_scale != nullptr) ? 1 : 0;
  if (!args.active) return vecops_b200_matmul_run(problem, error);

  // which kernel: the plain problem's choice, unless that kernel does not implement the transform
  VecopsB200Matmul fused = *problem;
  uint32_t kernel;
  rc = select_kernel(fused, row, &kernel, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  // (every kernel implements the transform; `kernel` is only needed for the empty reduction below)
  (void)kernel;
  if (fused.k == 0)  // an empty reduction leaves transform(CIn): the strided kernel computes it with zero trips
    fused.kernel = VECOPS_B200_KERNEL_GENERIC;
  tl_epilogue = args;
  rc = vecops_b200_matmul_run(&fused, error);
  tl_epilogue = EpilogueArgs();
  return rc;
}

int32_t vecops_b200_matmul_run_batched(const VecopsB200Matmul* problem, const VecopsB200Batch* batch, const VecopsB200Epilogue* epilogue,
                                       VecopsError* error) {
  Row row;
  int32_t rc = check_problem(problem, &row, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  if (batch == nullptr || batch->struct_size < sizeof(VecopsB200Batch) || batch->count < 0 || batch->a_stride_b < 0 ||
      batch->b_stride_b < 0 || batch->c_stride_b < 0 || batch->cin_stride_b < 0)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "batch record is null, too small, or has a negative count or stride");
  if (epilogue != nullptr && epilogue->struct_size < sizeof(VecopsB200Epilogue))
    return set_error(error, VECOPS_STATUS_ABI_MISMATCH, "epilogue record is %u bytes, the batched form needs %zu", epilogue->struct_size,
                     sizeof(VecopsB200Epilogue));
  if (batch->count == 0 || problem->m == 0 || problem->n == 0) return VECOPS_STATUS_OK;
  if (batch->count > 1 && batch->c_stride_b == 0)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "the batch entries of C must not share storage");
  const VecopsB200Matmul& p = *problem;
  const bool has_cin = epilogue != nullptr && epilogue->cin != nullptr;
  // shared weights, A / C / CIn stacked densely along the batch axis: one product with M * count rows
  const bool cin_stacks = !has_cin || (epilogue->cin_stride_m == 0 && batch->cin_stride_b == 0) ||
                          (epilogue->cin_stride_m != 0 && batch->cin_stride_b == p.m * epilogue->cin_stride_m);
  if (batch->count == 1 || (batch->b_stride_b == 0 && batch->a_stride_b == p.m * p.a_stride_m && batch->c_stride_b == p.m * p.c_stride_m &&
                            cin_stacks && p.m * batch->count < (INT64_C(1) << 31))) {
    VecopsB200Matmul flat = p;
    flat.m = p.m * batch->count;
    return epilogue != nullptr ? vecops_b200_matmul_run_fused(&flat, epilogue, error) : vecops_b200_matmul_run(&flat, error);
  }
  const size_t a_elem = dtype_size(p.a_dtype), b_elem = dtype_size(p.b_dtype), c_elem = dtype_size(p.c_dtype);
  const size_t cin_elem = has_cin ? dtype_size(epilogue->cin_dtype) : 0;
  if (has_cin && cin_elem == 0) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "unknown accumulator input dtype");
  for (int64_t i = 0; i < batch->count; ++i) {
    VecopsB200Matmul entry = p;
    entry.flags |= VECOPS_B200_MATMUL_FLAG_ASYNC;
    entry.a = p.a == nullptr ? nullptr : static_cast<const char*>(p.a) + i * batch->a_stride_b * static_cast<int64_t>(a_elem);
    entry.b = p.b == nullptr ? nullptr : static_cast<const char*>(p.b) + i * batch->b_stride_b * static_cast<int64_t>(b_elem);
    entry.c = p.c == nullptr ? nullptr : static_cast<char*>(p.c) + i * batch->c_stride_b * static_cast<int64_t>(c_elem);
    if (epilogue != nullptr) {
      VecopsB200Epilogue step = *epilogue;
      if (has_cin) step.cin = static_cast<const char*>(epilogue->cin) + i * batch->cin_stride_b * static_cast<int64_t>(cin_elem);
      // row factors belong to A's rows: entries that share A share them, otherwise entry i owns rows [i*M, (i+1)*M)
      // (vecops' scale index is batch * batch_stride + row with batch_stride = M, 0 for a broadcast A)
      if (step.row_scale != nullptr && batch->a_stride_b != 0) step.row_scale = epilogue->row_scale + i * p.m;
      rc = vecops_b200_matmul_run_fused(&entry, &step, error);
    } else {
      rc = vecops_b200_matmul_run(&entry, error);
    }
    if (rc != VECOPS_STATUS_OK) return rc;
  }
  if ((p.flags & VECOPS_B200_MATMUL_FLAG_ASYNC) == 0) {
    int device = 0;
    rc = current_device(p, &device, error);
    if (rc != VECOPS_STATUS_OK) return rc;
    int previous = -1;
    cudaGetDevice(&previous);
    if (previous != device) cudaSetDevice(device);
    cudaError_t status = cudaStreamSynchronize(static_cast<cudaStream_t>(p.stream));
    if (status != cudaSuccess) {
      rc = cuda_fail(error, status, "cudaStreamSynchronize");
    } else if (const uint32_t word = take_status_word(device)) {
      rc = set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "device %d: a bounded device wait ran out in a batched launch (status 0x%x)", device, word);
    }
    if (previous >= 0 && previous != device) cudaSetDevice(previous);
  }
  return rc;
}

const char* vecops_b200_kernel_name(uint32_t kernel) {
  return kernel < VECOPS_B200_KERNEL_COUNT_ ? kKernelNames[kernel] : nullptr;
}

int32_t vecops_b200_device_count(void) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return count;
}

int32_t vecops_b200_device_info(int32_t device_index, VecopsB200DeviceInfo* info, VecopsError* error) {
  if (info == nullptr || info->struct_size < sizeof(VecopsB200DeviceInfo))
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "device info record is null or too small");
  if (device_index < 0 || device_index >= vecops_b200_device_count())
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "no CUDA device %d", device_index);
  cudaDeviceProp prop;
  cudaError_t status = cudaGetDeviceProperties(&prop, device_index);
  if (status != cudaSuccess) return cuda_fail(error, status, "cudaGetDeviceProperties");
  info->sm_major = prop.major;
  info->sm_minor = prop.minor;
  info->sm_count = prop.multiProcessorCount;
  info->l2_bytes = static_cast<uint64_t>(prop.l2CacheSize);
  info->hbm_bytes = static_cast<uint64_t>(prop.totalGlobalMem);
  info->smem_per_block_optin = static_cast<uint64_t>(prop.sharedMemPerBlockOptin);
  snprintf(info->name, sizeof(info->name), "%.63s", prop.name);
  return VECOPS_STATUS_OK;
}

uint64_t vecops_b200_launch_count(void) { return g_launches.load(); }

// Tuning aid, deliberately not part of the public headers: kernels that support it write a timeline
// (16 x 64-bit nanosecond stamps per CTA) into this device buffer; NULL switches it off.
__attribute__((visibility("default"))) void vecops_b200_debug_set_trace(void* device_buffer) {
  g_trace = static_cast<unsigned long long*>(device_buffer);
}

int32_t vecops_b200_stream_synchronize(void* stream, VecopsError* error) {
  if (vecops_b200_device_count() == 0) return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "no usable CUDA device; there is no CPU fallback");
  const cudaError_t status = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (status != cudaSuccess) return cuda_fail(error, status, "cudaStreamSynchronize");
  return VECOPS_STATUS_OK;
}

int32_t vecops_b200_take_device_status(int32_t device_index, uint32_t* status, VecopsError* error) {
  if (status == nullptr) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "status output pointer is null");
  *status = 0;
  if (device_index < 0 && cudaGetDevice(&device_index) != cudaSuccess) {
    (void)cudaGetLastError();  // no driver, no GPU: nothing can have been recorded
    return VECOPS_STATUS_OK;
  }
  if (device_index >= kMaxDevices) return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "device index %d out of range", device_index);
  *status = take_status_word(device_index);
  return VECOPS_STATUS_OK;
}

int32_t vecops_b200_matmul_allgather_run(const VecopsB200Matmul* problem, const VecopsB200Gather* gather, VecopsError* error) {
  Row row;
  int32_t rc = check_problem(problem, &row, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  const VecopsB200Matmul& p = *problem;
  if (gather == nullptr || gather->struct_size < offsetof(VecopsB200Gather, flags) || gather->world < 1 || gather->world > GemmStoreMaps::kMax ||
      gather->c == nullptr)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "gather record is null, too small, or names more than %d destinations",
                     GemmStoreMaps::kMax);
  if (row != Row::BF16 || !applicable(p, row, VECOPS_B200_KERNEL_BF16_TCGEN05))
    return set_error(error, VECOPS_STATUS_NOT_APPLICABLE, "the fused all-gather serves the bf16 tcgen05 GEMM (K-contiguous, 16-byte aligned operands)");
  const size_t out = dtype_size(p.c_dtype);
  if (gather->col0 < 0 || gather->col0 + p.n > gather->n_total || gather->ldc < gather->n_total || (gather->ldc * out) % 16 != 0 ||
      (gather->col0 * out) % 16 != 0)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "slab [col0, col0+n) must lie inside the full C and start on a 16-byte boundary");
  for (int d = 0; d < gather->world; ++d)
    if (gather->c[d] == nullptr || !aligned16(gather->c[d]))
      return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "destination %d is null or not 16-byte aligned", d);
  const bool has_flags = gather->struct_size >= offsetof(VecopsB200Gather, flags) + sizeof(uint32_t);
  const bool multicast = has_flags && (gather->flags & VECOPS_B200_GATHER_MULTICAST) != 0;
  if (multicast && (gather->world != 1 || (p.n * out) % 16 != 0))
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "a multicast gather takes one destination and a slab of whole 16-byte pieces");
  if (p.m == 0 || p.n == 0) return VECOPS_STATUS_OK;
  if (p.k == 0) return set_error(error, VECOPS_STATUS_NOT_APPLICABLE, "K == 0 has nothing to gather; zero the result instead");

  int device = 0;
  rc = current_device(p, &device, error);
  if (rc != VECOPS_STATUS_OK) return rc;
  int previous = -1;
  cudaGetDevice(&previous);
  if (previous != device) {
    cudaError_t status = cudaSetDevice(device);
    if (status != cudaSuccess) return cuda_fail(error, status, "cudaSetDevice");
  }
  const DeviceState* dev = nullptr;
  rc = device_state(device, &dev, error);
  cudaStream_t stream = static_cast<cudaStream_t>(p.stream);
  if (rc == VECOPS_STATUS_OK) {
    GatherTargets targets;
    targets.count = gather->world;
    targets.c = gather->c;
    targets.n_total = gather->n_total;
    targets.ldc = gather->ldc;
    targets.col0 = gather->col0;
    targets.multicast = multicast;
    rc = p.c_dtype == VECOPS_DTYPE_BF16 ? launch_tcgen05<false, __nv_bfloat16>(p, *dev, stream, error, targets)
                                        : launch_tcgen05<false, float>(p, *dev, stream, error, targets);
  }
  if (rc == VECOPS_STATUS_OK) {
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) rc = cuda_fail(error, status, "kernel launch");
  }
  if (rc == VECOPS_STATUS_OK && (p.flags & VECOPS_B200_MATMUL_FLAG_ASYNC) == 0) {
    cudaError_t status = cudaStreamSynchronize(stream);
    if (status != cudaSuccess) rc = cuda_fail(error, status, "cudaStreamSynchronize");
    else if (const uint32_t word = take_status_word(device))
      rc = set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "fused all-gather GEMM on device %d: a bounded device wait ran out (status 0x%x)", device, word);
  }
  if (previous >= 0 && previous != device) cudaSetDevice(previous);
  return rc;
}

static int32_t quantize_rows_impl(const void* src, uint32_t src_dtype, int64_t src_stride_m, int64_t src_stride_k, void* dst,
                                  uint32_t dst_dtype, int64_t dst_stride_m, int64_t rows, int64_t cols, float scale, float zero_point,
                                  const float* multipliers, void* stream, VecopsError* error) {
  if (rows == 0 || cols == 0) return VECOPS_STATUS_OK;
  if (src == nullptr || dst == nullptr || rows < 0 || cols < 0 || dst_stride_m < cols)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "quantize_rows: null pointer, negative extent or overlapping destination rows");
  if ((src_dtype != VECOPS_DTYPE_F32 && src_dtype != VECOPS_DTYPE_BF16) || (dst_dtype != VECOPS_DTYPE_U8 && dst_dtype != VECOPS_DTYPE_I8))
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "quantize_rows converts f32 or bf16 to u8 or i8");
  if (vecops_b200_device_count() == 0)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "no usable CUDA device; there is no CPU fallback");
  const long long total = rows * cols;
  const int blocks = static_cast<int>(total / 256 + 1 < 148 * 8 ? total / 256 + 1 : 148 * 8);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* out = static_cast<uint8_t*>(dst);
  const bool is_signed = dst_dtype == VECOPS_DTYPE_I8;
  const bool by_four = src_dtype == VECOPS_DTYPE_F32 && src_stride_k == 1 && cols % 4 == 0 && aligned16(src) && src_stride_m % 4 == 0 &&
                       (reinterpret_cast<uintptr_t>(dst) & 3u) == 0 && dst_stride_m % 4 == 0;
  const bool by_sixteen = by_four && cols % 16 == 0 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0 && dst_stride_m % 16 == 0;
  if (by_sixteen) {
    const long long groups = rows * (cols / 16);
    const int grid16 = static_cast<int>(groups / 256 + 1 < 148 * 32 ? groups / 256 + 1 : 148 * 32);
    const float* in = static_cast<const float*>(src);
    if (is_signed) quantize_rows_f32x16_kernel<true><<<grid16, 256, 0, s>>>(in, src_stride_m, out, dst_stride_m, rows, cols / 16, scale, zero_point, multipliers);
    else quantize_rows_f32x16_kernel<false><<<grid16, 256, 0, s>>>(in, src_stride_m, out, dst_stride_m, rows, cols / 16, scale, zero_point, multipliers);
  } else if (by_four) {
    const long long groups = rows * (cols / 4);
    const int grid4 = static_cast<int>(groups / 256 + 1 < 148 * 16 ? groups / 256 + 1 : 148 * 16);
    const float* in = static_cast<const float*>(src);
    if (is_signed) quantize_rows_f32x4_kernel<true><<<grid4, 256, 0, s>>>(in, src_stride_m, out, dst_stride_m, rows, cols / 4, scale, zero_point, multipliers);
    else quantize_rows_f32x4_kernel<false><<<grid4, 256, 0, s>>>(in, src_stride_m, out, dst_stride_m, rows, cols / 4, scale, zero_point, multipliers);
  } else if (src_dtype == VECOPS_DTYPE_F32) {
    const float* in = static_cast<const float*>(src);
    if (is_signed) quantize_rows_kernel<float, true><<<blocks, 256, 0, s>>>(in, src_stride_m, src_stride_k, out, dst_stride_m, rows, cols, scale, zero_point, multipliers);
    else quantize_rows_kernel<float, false><<<blocks, 256, 0, s>>>(in, src_stride_m, src_stride_k, out, dst_stride_m, rows, cols, scale, zero_point, multipliers);
  } else {
    const __nv_bfloat16* in = static_cast<const __nv_bfloat16*>(src);
    if (is_signed) quantize_rows_kernel<__nv_bfloat16, true><<<blocks, 256, 0, s>>>(in, src_stride_m, src_stride_k, out, dst_stride_m, rows, cols, scale, zero_point, multipliers);
    else quantize_rows_kernel<__nv_bfloat16, false><<<blocks, 256, 0, s>>>(in, src_stride_m, src_stride_k, out, dst_stride_m, rows, cols, scale, zero_point, multipliers);
  }
  g_launches.fetch_add(1);
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess) return cuda_fail(error, status, "quantize_rows launch");
  return VECOPS_STATUS_OK;
}

int32_t vecops_b200_quantize_rows(const void* src, uint32_t src_dtype, int64_t src_stride_m, int64_t src_stride_k, void* dst,
                                  uint32_t dst_dtype, int64_t dst_stride_m, int64_t rows, int64_t cols, float scale, float zero_point,
                                  void* stream, VecopsError* error) {
  return quantize_rows_impl(src, src_dtype, src_stride_m, src_stride_k, dst, dst_dtype, dst_stride_m, rows, cols, scale, zero_point, nullptr,
                            stream, error);
}

int32_t vecops_b200_quantize_rows_per_row(const void* src, uint32_t src_dtype, int64_t src_stride_m, int64_t src_stride_k, void* dst,
                                          uint32_t dst_dtype, int64_t dst_stride_m, int64_t rows, int64_t cols, const float* multipliers,
                                          float zero_point, void* stream, VecopsError* error) {
  if (multipliers == nullptr && rows > 0 && cols > 0)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "quantize_rows_per_row: null multipliers");
  return quantize_rows_impl(src, src_dtype, src_stride_m, src_stride_k, dst, dst_dtype, dst_stride_m, rows, cols, 1.f, zero_point, multipliers,
                            stream, error);
}

int32_t vecops_b200_column_correction(const void* b, uint32_t b_dtype, int64_t b_stride_n, int64_t n, int64_t k, int32_t zero_point,
                                      int32_t* out, void* stream, VecopsError* error) {
  if (n == 0) return VECOPS_STATUS_OK;
  if (b == nullptr || out == nullptr || n < 0 || k < 0 || n >= (INT64_C(1) << 31) || k >= (INT64_C(1) << 31))
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "column_correction: null pointer or extent out of range");
  if (b_dtype != VECOPS_DTYPE_I8 && b_dtype != VECOPS_DTYPE_U8)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "column_correction sums the rows of an 8-bit B[N,K]");
  if (vecops_b200_device_count() == 0)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "no usable CUDA device; there is no CPU fallback");
  const int blocks = static_cast<int>((n * 32 + 255) / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (b_dtype == VECOPS_DTYPE_I8)
    column_correction_kernel<int8_t><<<blocks, 256, 0, s>>>(static_cast<const int8_t*>(b), b_stride_n, static_cast<int>(n), static_cast<int>(k), zero_point, out);
  else
    column_correction_kernel<uint8_t><<<blocks, 256, 0, s>>>(static_cast<const uint8_t*>(b), b_stride_n, static_cast<int>(n), static_cast<int>(k), zero_point, out);
  g_launches.fetch_add(1);
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess) return cuda_fail(error, status, "column_correction launch");
  return VECOPS_STATUS_OK;
}

int32_t vecops_b200_place_columns(void* dst, int64_t ldd, int64_t col0, const void* src, int64_t lds, int64_t rows,
                                  int64_t cols, uint32_t elem_size, void* stream, VecopsError* error) {
  if (rows == 0 || cols == 0) return VECOPS_STATUS_OK;
  if (dst == nullptr || src == nullptr || rows < 0 || cols < 0 || elem_size == 0)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "place_columns: null pointer or negative extent");
  if (vecops_b200_device_count() == 0)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "no usable CUDA device; there is no CPU fallback");
  const int64_t e = elem_size;
  if (!aligned16(dst) || !aligned16(src) || (ldd * e) % 16 || (lds * e) % 16 || (col0 * e) % 16 || (cols * e) % 16)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "place_columns needs 16-byte aligned slabs and pitches");
  const long long total = rows * (cols * e / 16);
  const int blocks = static_cast<int>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
  place_columns_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(dst), ldd * e / 16, col0 * e / 16, static_cast<const uint4*>(src), lds * e / 16, rows, cols * e / 16);
  g_launches.fetch_add(1);
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess) return cuda_fail(error, status, "place_columns launch");
  return VECOPS_STATUS_OK;
}

int32_t vecops_b200_push_columns(const void* src, void* const* dst, int32_t count, int64_t ld, int64_t col0, int64_t rows,
                                 int64_t cols, uint32_t elem_size, uint32_t route, void* stream, VecopsError* error) {
  if (rows == 0 || cols == 0 || count == 0) return VECOPS_STATUS_OK;
  if (src == nullptr || dst == nullptr || count < 0 || count > 8 || rows < 0 || cols < 0 || col0 < 0 || elem_size == 0 ||
      col0 + cols > ld)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "push_columns: null pointer, more than 8 destinations or a bad extent");
  if (route != VECOPS_B200_PUSH_KERNEL && route != VECOPS_B200_PUSH_COPY_ENGINE)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "push_columns: unknown route");
  const int64_t e = elem_size;
  bool aligned = aligned16(src) && (ld * e) % 16 == 0 && (col0 * e) % 16 == 0 && (cols * e) % 16 == 0;
  for (int d = 0; d < count; ++d) {
    if (dst[d] == nullptr || dst[d] == src)
      return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "push_columns: a destination is null or is the source itself");
    aligned = aligned && aligned16(dst[d]);
  }
  if (route == VECOPS_B200_PUSH_KERNEL && !aligned)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "push_columns needs 16-byte aligned slabs and pitches");
  if (vecops_b200_device_count() == 0)
    return set_error(error, VECOPS_STATUS_EXECUTION_ERROR, "no usable CUDA device; there is no CPU fallback");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (route == VECOPS_B200_PUSH_COPY_ENGINE) {
    // one strided copy per destination, in the caller's order, on the caller's stream
    for (int d = 0; d < count; ++d) {
      cudaError_t status = cudaMemcpy2DAsync(static_cast<char*>(dst[d]) + col0 * e, static_cast<size_t>(ld * e),
                                             static_cast<const char*>(src) + col0 * e, static_cast<size_t>(ld * e),
                                             static_cast<size_t>(cols * e), static_cast<size_t>(rows), cudaMemcpyDefault, s);
      if (status != cudaSuccess) return cuda_fail(error, status, "push_columns copy");
    }
    return VECOPS_STATUS_OK;
  }
  PushTargets targets{};
  targets.count = count;
  for (int d = 0; d < count; ++d) targets.dst[d] = static_cast<uint4*>(dst[d]);
  // At most one CTA per SM (see the kernel): a second one would keep a GEMM's CTAs off the SM until the push had finished.
  // A kernel without shared memory would also ask for the L1-heavy split of the SM's unified memory, which an SM cannot
  // hold together with the GEMM's split: prefer the shared one.
  static std::atomic<unsigned> configured{0};
  static int sm_count[32] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 32) device = 0;
  if (!(configured.load() & (1u << device))) {
    cudaFuncSetAttribute(push_columns_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaDeviceGetAttribute(&sm_count[device], cudaDevAttrMultiProcessorCount, device);
    configured.fetch_or(1u << device);
  }
  long long limit = sm_count[device] > 0 ? sm_count[device] : 148;
  if (const char* text = std::getenv("VECOPS_B200_PUSH_BLOCKS")) {
    const long long asked = std::atoll(text);
    if (asked >= 1 && asked <= limit) limit = asked;
  }
  if (rows > 0x7fffffff || cols * e / 16 > 0x7fffffff)
    return set_error(error, VECOPS_STATUS_INVALID_ARGUMENT, "push_columns: extent too large");
  const int blocks = static_cast<int>(rows < limit ? rows : limit);
  push_columns_kernel<<<blocks, 256, 0, s>>>(static_cast<const uint4*>(src), targets, ld * e / 16, col0 * e / 16,
                                             static_cast<int>(rows), static_cast<int>(cols * e / 16));
  g_launches.fetch_add(1);
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess) return cuda_fail(error, status, "push_columns launch");
  return VECOPS_STATUS_OK;
}

}  // extern "C"
