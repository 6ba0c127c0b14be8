// RESTATED FROM vecops (src/runtime/Executable.cpp:39-316), not designed here.  Inside a vecops build this file is not used at all: vecops' own
// runtime takes its place and only the matmul recipe, dispatch policy and executable provider of this library are new
// (csrc/runtime/matmul_operator.cpp).  It exists so that the library builds and is testable standalone, with the
// class names, signatures, checks and status texts a caller of vecops' runtime expects.
//
// LoadedModule / Executable.  Behaviour follows src/runtime/Executable.cpp of
// vecops: descriptor validation :39-100, per-call validation against the
// descriptor :102-184, error text recovery :186-197, dlopen loader :208-239,
// workspace query :260-284, guarded invoke :286-316.
#include "vecops_b200/runtime_mirror/executable.h"

#include <dlfcn.h>

#include <array>
#include <cstddef>
#include <limits>
#include <string>

namespace vecops::runtime {
namespace {

constexpr std::size_t kErrorCapacity = 1024;

// Descriptor arrays may use a larger record stride than this runtime knows
// (append-only ABI): step in bytes, read only the v1 prefix.
template <typename T>
const T& at_stride(const T* base, std::uint32_t stride, std::size_t index) {
  return *reinterpret_cast<const T*>(reinterpret_cast<const std::byte*>(base) + static_cast<std::size_t>(stride) * index);
}

Status abi_mismatch(std::string message) { return Status(StatusCode::AbiMismatch, std::move(message)); }
Status invalid(std::string message) { return Status(StatusCode::InvalidArgument, std::move(message)); }

bool dimension_record_ok(const VecopsDimensionConstraint& c) {
  return c.struct_size >= sizeof(VecopsDimensionConstraint) && c.kind <= VECOPS_DIM_DYNAMIC &&
         !(c.kind == VECOPS_DIM_DYNAMIC && c.alignment <= 0);
}

Status validate_descriptor(const VecopsKernelDescriptorV1* d) {
  if (d == nullptr) return abi_mismatch("kernel query returned a null descriptor");
  if (d->struct_size < sizeof(VecopsKernelDescriptorV1)) return abi_mismatch("kernel descriptor is smaller than ABI v1");
  if (d->abi_version_major != VECOPS_KERNEL_ABI_VERSION_MAJOR || d->abi_version_minor > VECOPS_KERNEL_ABI_VERSION_MINOR)
    return abi_mismatch("kernel ABI version is not supported by this runtime");
  if (d->operator_name == nullptr || d->specialization_key == nullptr)
    return abi_mismatch("kernel descriptor has no operator or specialization name");
  if (d->num_parameters != 0 && d->parameters == nullptr) return abi_mismatch("kernel descriptor has no parameter array");
  if (d->num_parameters != 0 &&
      (d->parameter_stride < sizeof(VecopsParameterDescriptor) || d->parameter_stride % alignof(VecopsParameterDescriptor) != 0))
    return abi_mismatch("kernel has an invalid parameter stride");
  if (d->run == nullptr) return abi_mismatch("kernel descriptor has no run entry point");
  if (d->flags != 0) return abi_mismatch("kernel descriptor sets unknown flags");
  for (std::uint32_t i = 0; i < d->num_parameters; ++i) {
    const auto& p = at_stride(d->parameters, d->parameter_stride, i);
    if (p.struct_size < sizeof(VecopsParameterDescriptor) || p.name == nullptr)
      return abi_mismatch("kernel has an invalid parameter descriptor");
    if (p.kind == VECOPS_VALUE_TENSOR) {
      const auto& t = p.constraint.tensor;
      const bool bad_stride = t.rank > 0 && (t.dimension_constraint_stride < sizeof(VecopsDimensionConstraint) ||
                                             t.dimension_constraint_stride % alignof(VecopsDimensionConstraint) != 0);
      if (t.struct_size < sizeof(VecopsTensorParameter) || t.rank < -1 || (t.rank > 0 && t.sizes == nullptr) || bad_stride ||
          (t.rank == -1 && (t.sizes != nullptr || t.strides != nullptr)))
        return abi_mismatch("kernel has an invalid tensor constraint");
      for (std::int32_t axis = 0; axis < t.rank; ++axis) {
        if (!dimension_record_ok(at_stride(t.sizes, t.dimension_constraint_stride, axis)))
          return abi_mismatch("kernel has an invalid size constraint");
        if (t.strides != nullptr && !dimension_record_ok(at_stride(t.strides, t.dimension_constraint_stride, axis)))
          return abi_mismatch("kernel has an invalid stride constraint");
      }
    } else if (p.kind == VECOPS_VALUE_SCALAR) {
      if (p.constraint.scalar.struct_size < sizeof(VecopsScalarParameter)) return abi_mismatch("kernel has an invalid scalar constraint");
    } else {
      return abi_mismatch("kernel parameter has an unknown value kind");
    }
  }
  return Status::success();
}

bool dimension_accepts(const VecopsDimensionConstraint& c, std::int64_t value) {
  if (c.struct_size < sizeof(VecopsDimensionConstraint)) return false;
  switch (c.kind) {
    case VECOPS_DIM_ANY: return true;
    case VECOPS_DIM_CONST: return value == c.value;
    case VECOPS_DIM_DYNAMIC:
      return c.alignment > 0 && value >= c.lower_bound && value <= c.upper_bound && value % c.alignment == 0;
    default: return false;
  }
}

Status validate_call(const ArgumentMetadata& arguments, const VecopsKernelDescriptorV1& d) {
  if (arguments.size() != d.num_parameters) return invalid("argument count does not match the kernel specialization");
  for (std::size_t index = 0; index < arguments.size(); ++index) {
    const Value& value = arguments[index];
    const auto& p = at_stride(d.parameters, d.parameter_stride, index);
    const std::string name(p.name);
    if (std::holds_alternative<std::monostate>(value)) {
      if (p.kind == VECOPS_VALUE_TENSOR && p.constraint.tensor.optional != 0) continue;
      return invalid(name + " is not optional");
    }
    if (p.kind != VECOPS_VALUE_TENSOR) {
      const auto* scalar = std::get_if<Scalar>(&value);
      if (scalar == nullptr || (dtype_bit(scalar->dtype) & p.constraint.scalar.dtype_mask) == 0) return invalid(name + " scalar mismatch");
      continue;
    }
    const auto* tensor = std::get_if<TensorView>(&value);
    if (tensor == nullptr) return invalid(name + " must be a tensor");
    const auto& rule = p.constraint.tensor;
    if ((dtype_bit(tensor->dtype) & rule.dtype_mask) == 0) return invalid(name + " dtype mismatch");
    if ((rule.device_type != 0 && tensor->device_type != rule.device_type) ||
        (rule.device_index >= 0 && tensor->device_index != rule.device_index))
      return invalid(name + " device mismatch");
    if (tensor->sizes.size() != tensor->strides.size() || tensor->sizes.size() > std::numeric_limits<std::uint32_t>::max() ||
        (rule.rank >= 0 && tensor->sizes.size() != static_cast<std::size_t>(rule.rank)))
      return invalid(name + " rank mismatch");
    bool has_elements = true;
    for (const auto size : tensor->sizes) {
      if (size < 0) return invalid(name + " has a negative size");
      if (size == 0) has_elements = false;
    }
    if (has_elements && tensor->data == nullptr) return invalid(name + " has no data");
    const auto access = rule.required_flags & (VECOPS_TENSOR_READ | VECOPS_TENSOR_WRITE);
    if ((tensor->flags & access) != access) return invalid(name + " access mismatch");
    for (std::size_t axis = 0; axis < tensor->sizes.size(); ++axis) {
      if (rule.sizes != nullptr && !dimension_accepts(at_stride(rule.sizes, rule.dimension_constraint_stride, axis), tensor->sizes[axis]))
        return invalid(name + " shape mismatch");
      if (rule.strides != nullptr && !dimension_accepts(at_stride(rule.strides, rule.dimension_constraint_stride, axis), tensor->strides[axis]))
        return invalid(name + " stride mismatch");
    }
  }
  return Status::success();
}

// Turn a callback's return code and the text it left in `error` into a Status.
Status callback_status(std::int32_t rc, const VecopsError& error, std::string_view fallback) {
  if (rc == VECOPS_STATUS_OK) return Status::success();
  std::string message(fallback);
  if (error.message != nullptr && error.message[0] != '\0') message = error.message;
  const bool known = rc >= VECOPS_STATUS_INVALID_ARGUMENT && rc <= VECOPS_STATUS_INTERNAL_ERROR;
  return Status(known ? static_cast<StatusCode>(rc) : StatusCode::ExecutionError, std::move(message));
}

struct ErrorSlot {
  std::array<char, kErrorCapacity> text{};
  VecopsError record{};
  ErrorSlot() {
    record.struct_size = sizeof(VecopsError);
    record.code = VECOPS_STATUS_OK;
    record.message = text.data();
    record.message_capacity = text.size();
    record.message_required = 0;
  }
};

}  // namespace

LoadedModule::~LoadedModule() {
  if (handle_ != nullptr) dlclose(handle_);
}

Result<std::shared_ptr<LoadedModule>> LoadedModule::load(const std::filesystem::path& library_path) {
  dlerror();
  void* handle = dlopen(library_path.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (handle == nullptr) {
    const char* why = dlerror();
    return Status(StatusCode::LoadError,
                  "failed to load " + library_path.string() + ": " + (why == nullptr ? "unknown dynamic-loader error" : why));
  }
  dlerror();
  auto* query = reinterpret_cast<VecopsKernelQueryFnV1>(dlsym(handle, VECOPS_KERNEL_QUERY_SYMBOL_V1));
  const char* symbol_error = dlerror();
  if (symbol_error != nullptr || query == nullptr) {
    std::string message = std::string("kernel artifact does not export ") + VECOPS_KERNEL_QUERY_SYMBOL_V1;
    if (symbol_error != nullptr) message += std::string(": ") + symbol_error;
    dlclose(handle);
    return abi_mismatch(std::move(message));
  }
  const VecopsKernelDescriptorV1* descriptor = query();
  if (auto status = validate_descriptor(descriptor); !status.ok()) {
    dlclose(handle);
    return status;
  }
  return std::shared_ptr<LoadedModule>(new LoadedModule(library_path, handle, descriptor, nullptr));
}

Result<std::shared_ptr<LoadedModule>> LoadedModule::adopt(const VecopsKernelDescriptorV1* descriptor,
                                                          std::shared_ptr<const void> keepalive) {
  if (auto status = validate_descriptor(descriptor); !status.ok()) return status;
  return std::shared_ptr<LoadedModule>(new LoadedModule({}, nullptr, descriptor, std::move(keepalive)));
}

Result<std::shared_ptr<Executable>> Executable::load(const std::filesystem::path& library_path) {
  auto module = LoadedModule::load(library_path);
  if (!module) return module.status();
  return std::make_shared<Executable>(std::move(module).value());
}

std::string_view Executable::operator_name() const { return module_->descriptor().operator_name; }
std::string_view Executable::specialization_key() const { return module_->descriptor().specialization_key; }

Status Executable::can_invoke(const ArgumentMetadata& arguments) const { return validate_call(arguments, module_->descriptor()); }

Result<std::uint64_t> Executable::workspace_size(const ArgumentMetadata& arguments, const VecopsExecutionContext* context) const {
  if (auto status = can_invoke(arguments); !status.ok()) return status;
  const auto query = module_->descriptor().workspace;
  if (query == nullptr) return std::uint64_t{0};
  CallFrame frame(arguments, nullptr, 0, context);
  std::uint64_t bytes = 0;
  ErrorSlot slot;
  const auto rc = query(&frame.abi(), &bytes, &slot.record);
  slot.text.back() = '\0';
  if (auto status = callback_status(rc, slot.record, "kernel workspace query failed"); !status.ok()) return status;
  return bytes;
}

Status Executable::invoke(const ArgumentMetadata& arguments, void* workspace, std::uint64_t workspace_size,
                          const VecopsExecutionContext* context) const {
  auto required = this->workspace_size(arguments, context);
  if (!required) return required.status();
  if (required.value() > workspace_size || (required.value() != 0 && workspace == nullptr))
    return invalid("kernel requires " + std::to_string(required.value()) + " workspace bytes, but " +
                   std::to_string(workspace_size) + " were supplied");
  CallFrame frame(arguments, workspace, workspace_size, context);
  return invoke_unchecked(frame.abi());
}

Status Executable::invoke_unchecked(const VecopsCall& call) const {
  ErrorSlot slot;
  const auto rc = module_->descriptor().run(&call, &slot.record);
  slot.text.back() = '\0';
  return callback_status(rc, slot.record, "kernel execution failed");
}

Status Executable::invoke_prevalidated(const VecopsCall& call) const { return invoke_unchecked(call); }

}  // namespace vecops::runtime
