// The matmul operator for CUDA devices, assembled from vecops' runtime parts:
//
//   KernelDef "vecops::matmul"  ->  Operator
//       recipes         one CudaMatmulRecipe per sm_100a kernel variant
//       dispatch        MatmulRuntimeDispatch: shape/dtype rules pick the variant
//                       (device counterpart of src/MatmulRuntimeDispatch.cpp:12-32)
//       provider        CudaExecutableProvider: bound recipe -> in-process
//                       descriptor over the prebuilt sm_100a kernel image
//
// vecops itself never wires ops::Matmul into its runtime layer (its matmul is
// a C++ template called directly); this definition is derived from the
// operator's semantic in include/vecops/ops/Matmul.h:13-17 and :530-570.
//
// Positional parameters of the operator:
//   a            [M,K]  dtype TA   input
//   b            [N,K]  dtype TB   input   (a row-major [K,N] matrix = strides (1,N))
//   c            [M,N]  dtype TC   output
//   column_scale [N]    f32        optional input, multiplies the accumulator
// M, N and K are runtime dimensions (they never enter the specialization key,
// so decode-time M may vary freely); TA/TB/TC and the presence of the scale do.
#pragma once

#include <map>
#include <memory>
#include <mutex>
#include <string>

#include "vecops_b200/matmul_cuda.h"
#include "vecops_b200/runtime_mirror/operator.h"

namespace vecops::runtime {

[[nodiscard]] KernelDef matmul_kernel_def();

// Translate the four positional values into the C ABI's problem record.
// `kernel` forces a variant (VECOPS_B200_KERNEL_AUTO = rules decide).
[[nodiscard]] Result<VecopsB200Matmul> matmul_problem_from(std::span<const Value> values, std::uint32_t kernel);

class CudaMatmulRecipe final : public KernelRecipe {
public:
  explicit CudaMatmulRecipe(std::uint32_t kernel);
  [[nodiscard]] std::string_view id() const override { return id_; }
  // NotApplicable when this variant cannot address the call (dtype row, strides, alignment).
  [[nodiscard]] Status match(const KernelCall& call) const override;
  [[nodiscard]] Result<BoundKernelRecipe> bind(const KernelCall& call) const override;
  [[nodiscard]] std::uint32_t kernel() const { return kernel_; }

private:
  std::uint32_t kernel_;
  std::string id_;
  std::shared_ptr<const KernelDef> definition_;
};

// Orders recipes by asking the shape/dtype rules which variant serves the call
// best; the strided kernel is always kept as the last candidate.
class MatmulRuntimeDispatch final : public DispatchPolicy {
public:
  [[nodiscard]] Result<std::vector<std::size_t>> candidates(
      const KernelCall& call, std::span<const std::shared_ptr<const KernelRecipe>> recipes) const override;
};

// Resolves "cuda/sm_100a/<variant>" artifact keys to executables whose
// descriptors live in this library.  Never compiles, never touches files:
// the kernel images were built ahead of time into the library itself.
// Thread-safe; one executable per specialization key is kept and shared.
class CudaExecutableProvider final : public ExecutableProvider {
public:
  [[nodiscard]] Result<std::shared_ptr<Executable>> resolve(const BoundKernelRecipe& recipe) override;
  [[nodiscard]] std::size_t cached() const;

private:
  mutable std::mutex mutex_;
  std::map<std::string, std::shared_ptr<Executable>, std::less<>> cache_;
};

// The assembled operator: every variant's recipe, MatmulRuntimeDispatch, one provider.
[[nodiscard]] std::shared_ptr<Operator> make_matmul_operator();

// ops::matmul_pack, values = {src[R,K], dst[R,P]}, and ops::matmul_pack_b_compensated, values = {src, dst,
// compensation[R], a_zero_point}, as operators; dst a tensor over the packed layout of src
// (include/vecops/ops/MatmulPack.h:93-131, :28-35).
[[nodiscard]] KernelDef matmul_pack_kernel_def();
[[nodiscard]] KernelDef matmul_pack_b_compensated_kernel_def();
[[nodiscard]] std::shared_ptr<Operator> make_matmul_pack_operator(bool compensated = false);

// The callers and data formats either side of the path, as operators (csrc/runtime/caller_operators.cpp):
//   vecops::matmul_batched                a[B,M,K], b[B,N,K], c[B,M,N], column_scale[N]?     (tests/ops/MatmulBatchTest.cpp:96-131)
//   vecops::scaled_dot_product_attention  q[H,Lq,D], k[H,Lkv,D], v[H,Lkv,Dv], out[H,Lq,Dv], scale, causal, key_mask[Lkv]?, bias[H,Lq,Lkv]?
//   vecops::quantize_rows_per_row         src[M,K], multipliers[M], dst[M,K], zero_point     (matmul/Quantization.h:76-140)
[[nodiscard]] std::shared_ptr<Operator> make_matmul_batched_operator();
[[nodiscard]] std::shared_ptr<Operator> make_attention_operator();
[[nodiscard]] std::shared_ptr<Operator> make_quantize_rows_per_row_operator();
// Bridge handles kCallerHandleBase + {0, 1, 2} name the three; null for anything else.
inline constexpr std::uint64_t kCallerHandleBase = 0x6d61746d756c0010ULL;
[[nodiscard]] const Operator* caller_operator_of(std::uint64_t handle);
[[nodiscard]] const KernelDef* caller_kernel_def_of(std::uint64_t handle);

// Static descriptor template of one variant (specialization_key left empty).
[[nodiscard]] const VecopsKernelDescriptorV1* matmul_descriptor_template(std::uint32_t kernel);

}  // namespace vecops::runtime
