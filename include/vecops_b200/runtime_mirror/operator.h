// RESTATED FROM vecops (include/vecops/runtime/Operator.h:34-293), not designed here.  Inside a vecops build this file is not used at all: vecops' own
// runtime takes its place and only the matmul recipe, dispatch policy and executable provider of this library are new
// (csrc/runtime/matmul_operator.cpp).  It exists so that the library builds and is testable standalone, with the
// class names, signatures, checks and status texts a caller of vecops' runtime expects.
//
// Operator = schema + ordered kernel recipes + dispatch policy + executable
// provider.  Mirrors include/vecops/runtime/Operator.h:34-293 and
// src/runtime/Operator.cpp:162-285.
//
// Resolution of one call: normalise (bind against the KernelDef, validate the
// schema) -> ask the DispatchPolicy for candidate recipes -> first recipe whose
// match() and bind() accept the call -> ExecutableProvider::resolve -> check the
// executable's operator name and specialization key -> Executable::invoke.
// NotApplicable (recipe) and NotFound / NotApplicable (provider) fall through
// to the next candidate; every other failure is returned at once.
#pragma once

#include <cstdint>
#include <filesystem>
#include <memory>
#include <span>
#include <string>
#include <string_view>
#include <vector>

#include "vecops_b200/runtime_mirror/executable.h"
#include "vecops_b200/runtime_mirror/kernel_def.h"
#include "vecops_b200/runtime_mirror/schema.h"

namespace vecops::runtime {

struct BoundKernelRecipe {
  std::string recipe_id;
  std::string specialization_key;  // must equal the resolved executable's key
  std::string artifact_key;        // what the provider looks the artifact up by
  // Source-compiled recipes (vecops' JIT path) carry their instantiation here.
  // Prebuilt CUDA recipes leave it null, so no ";$Parallelism" suffix is ever
  // appended to their keys (src/runtime/Operator.cpp:97-99).
  struct SourceInstantiation {
    std::filesystem::path kernel_file;
    std::shared_ptr<const KernelDef> definition;
    BoundKernel binding;
    std::int64_t parallelism = 1;
  };
  std::shared_ptr<const SourceInstantiation> source;
};

[[nodiscard]] BoundKernelRecipe specialize_parallelism(BoundKernelRecipe recipe, std::int64_t parallelism);

// Cheap, side-effect free and thread-safe; never builds or loads anything.
class KernelRecipe {
public:
  virtual ~KernelRecipe() = default;
  [[nodiscard]] virtual std::string_view id() const = 0;
  [[nodiscard]] virtual Status match(const KernelCall& call) const = 0;
  [[nodiscard]] virtual Result<BoundKernelRecipe> bind(const KernelCall& call) const = 0;
};

class DispatchPolicy {
public:
  virtual ~DispatchPolicy() = default;
  // Indices into `recipes`, most preferred first.
  [[nodiscard]] virtual Result<std::vector<std::size_t>> candidates(
      const KernelCall& call, std::span<const std::shared_ptr<const KernelRecipe>> recipes) const = 0;
};

class OrderedDispatchPolicy final : public DispatchPolicy {
public:
  [[nodiscard]] Result<std::vector<std::size_t>> candidates(
      const KernelCall& call, std::span<const std::shared_ptr<const KernelRecipe>> recipes) const override;
};

// The only place allowed to do I/O, load modules or touch the device.
class ExecutableProvider {
public:
  virtual ~ExecutableProvider() = default;
  [[nodiscard]] virtual Result<std::shared_ptr<Executable>> resolve(const BoundKernelRecipe& recipe) = 0;
};

class Operator {
public:
  Operator(OperatorSchema schema, std::vector<std::shared_ptr<const KernelRecipe>> recipes,
           std::shared_ptr<const DispatchPolicy> dispatch_policy, std::shared_ptr<ExecutableProvider> provider);
  Operator(KernelDef definition, std::vector<std::shared_ptr<const KernelRecipe>> recipes,
           std::shared_ptr<const DispatchPolicy> dispatch_policy, std::shared_ptr<ExecutableProvider> provider);

  [[nodiscard]] const OperatorSchema& schema() const { return schema_; }
  [[nodiscard]] Result<std::shared_ptr<Executable>> resolve(const ArgumentMetadata& arguments) const;
  [[nodiscard]] Result<std::shared_ptr<Executable>> resolve(const KernelCall& call,
                                                            const VecopsExecutionContext* context = nullptr) const;
  [[nodiscard]] Status invoke(const ArgumentMetadata& arguments, void* workspace = nullptr,
                              std::uint64_t workspace_size = 0, const VecopsExecutionContext* context = nullptr) const;
  [[nodiscard]] Status invoke(const KernelCall& call, const VecopsExecutionContext* context = nullptr,
                              void* workspace = nullptr, std::uint64_t workspace_size = 0) const;
  [[nodiscard]] Status operator()(const KernelCall& call) const { return invoke(call); }

  template <typename... Values>
  [[nodiscard]] Status invoke_values(Values&&... values) const {
    return invoke(make_arguments(std::forward<Values>(values)...));
  }

private:
  [[nodiscard]] Result<KernelCall> normalize(const KernelCall& call) const;
  [[nodiscard]] Result<std::shared_ptr<Executable>> resolve_normalized(const KernelCall& call,
                                                                       const VecopsExecutionContext* context) const;
  OperatorSchema schema_;
  std::shared_ptr<const KernelDef> kernel_definition_;
  std::vector<std::shared_ptr<const KernelRecipe>> recipes_;
  std::shared_ptr<const DispatchPolicy> dispatch_policy_;
  std::shared_ptr<ExecutableProvider> provider_;
};

// Schema implied by a KernelDef: dtype masks from fixed dtypes, rank, device,
// access flags, optional-ness.  (src/runtime/Operator.cpp:30-62)
[[nodiscard]] OperatorSchema logical_schema(const KernelDef& definition);

}  // namespace vecops::runtime
