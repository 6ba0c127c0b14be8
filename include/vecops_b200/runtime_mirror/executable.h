// RESTATED FROM vecops (include/vecops/runtime/Executable.h:54-168), not designed here.  Inside a vecops build this file is not used at all: vecops' own
// runtime takes its place and only the matmul recipe, dispatch policy and executable provider of this library are new
// (csrc/runtime/matmul_operator.cpp).  It exists so that the library builds and is testable standalone, with the
// class names, signatures, checks and status texts a caller of vecops' runtime expects.
//
// Executable: one loaded kernel specialization, reached only through its
// VecopsKernelDescriptorV1.  Mirrors include/vecops/runtime/Executable.h:36-168
// and src/runtime/Executable.cpp:39-316 (descriptor validation, call
// validation against the descriptor, workspace query, guarded invoke).
//
// Addition for the CUDA artifact: LoadedModule::adopt wraps a descriptor that
// already lives in this process (the B200 kernels are linked into the same
// library as the runtime, so there is nothing to dlopen).  `load` keeps working
// for artifacts shipped as one DSO per specialization.
#pragma once

#include <cstdint>
#include <filesystem>
#include <memory>
#include <string_view>

#include "vecops_b200/kernel_abi.h"
#include "vecops_b200/runtime_mirror/status.h"
#include "vecops_b200/runtime_mirror/values.h"

namespace vecops::runtime {

class LoadedModule {
public:
  ~LoadedModule();
  LoadedModule(const LoadedModule&) = delete;
  LoadedModule& operator=(const LoadedModule&) = delete;

  // dlopen `library_path`, call its vecops_kernel_query_v1 and validate the descriptor.
  static Result<std::shared_ptr<LoadedModule>> load(const std::filesystem::path& library_path);

  // Wrap an in-process descriptor.  `keepalive` owns whatever the descriptor
  // points into (strings, parameter arrays) and is released with the module.
  static Result<std::shared_ptr<LoadedModule>> adopt(const VecopsKernelDescriptorV1* descriptor,
                                                     std::shared_ptr<const void> keepalive);

  [[nodiscard]] const VecopsKernelDescriptorV1& descriptor() const { return *descriptor_; }
  [[nodiscard]] const std::filesystem::path& path() const { return path_; }

private:
  LoadedModule(std::filesystem::path path, void* handle, const VecopsKernelDescriptorV1* descriptor,
               std::shared_ptr<const void> keepalive)
      : path_(std::move(path)), handle_(handle), descriptor_(descriptor), keepalive_(std::move(keepalive)) {}

  std::filesystem::path path_;
  void* handle_ = nullptr;
  const VecopsKernelDescriptorV1* descriptor_ = nullptr;
  std::shared_ptr<const void> keepalive_;
};

class Executable {
public:
  explicit Executable(std::shared_ptr<LoadedModule> module) : module_(std::move(module)) {}

  static Result<std::shared_ptr<Executable>> load(const std::filesystem::path& library_path);

  [[nodiscard]] std::string_view operator_name() const;
  [[nodiscard]] std::string_view specialization_key() const;
  [[nodiscard]] const std::shared_ptr<LoadedModule>& module() const { return module_; }

  // Descriptor-level validation: dtype masks, device, rank, per-axis constraints, access flags.
  [[nodiscard]] Status can_invoke(const ArgumentMetadata& arguments) const;
  // Bytes of caller-provided (device) scratch this call needs.
  [[nodiscard]] Result<std::uint64_t> workspace_size(const ArgumentMetadata& arguments,
                                                     const VecopsExecutionContext* context = nullptr) const;
  // Validate, check the workspace is large enough, then cross the C ABI into `run`.
  [[nodiscard]] Status invoke(const ArgumentMetadata& arguments, void* workspace = nullptr,
                              std::uint64_t workspace_size = 0, const VecopsExecutionContext* context = nullptr) const;
  // Skip validation: for callers that cached a validated signature.
  [[nodiscard]] Status invoke_prevalidated(const VecopsCall& call) const;

private:
  [[nodiscard]] Status invoke_unchecked(const VecopsCall& call) const;
  std::shared_ptr<LoadedModule> module_;
};

}  // namespace vecops::runtime
