// RESTATED FROM vecops (src/runtime/Schema.cpp:55-147 and src/runtime/Argument.cpp:37-79), not designed here.  Inside a vecops build this file is not used at all: vecops' own
// runtime takes its place and only the matmul recipe, dispatch policy and executable provider of this library are new
// (csrc/runtime/matmul_operator.cpp).  It exists so that the library builds and is testable standalone, with the
// class names, signatures, checks and status texts a caller of vecops' runtime expects.
//
// OperatorSchema validation and the ABI call frame.  Behaviour follows
// src/runtime/Schema.cpp:55-147 and src/runtime/Argument.cpp:37-79 of vecops.
#include "vecops_b200/runtime_mirror/schema.h"

#include <limits>

namespace vecops::runtime {
namespace {
Status invalid(std::string message) { return Status(StatusCode::InvalidArgument, std::move(message)); }
}  // namespace

CallFrame::CallFrame(const ArgumentMetadata& arguments, void* workspace, std::uint64_t workspace_size,
                     const VecopsExecutionContext* context) {
  values_.reserve(arguments.size());
  for (const auto& value : arguments.values()) {
    VecopsValue record{};
    record.struct_size = sizeof(VecopsValue);
    if (const auto* tensor = std::get_if<TensorView>(&value)) {
      record.kind = VECOPS_VALUE_TENSOR;
      VecopsTensorView& view = record.value.tensor;
      view.struct_size = sizeof(VecopsTensorView);
      view.data = tensor->data;
      view.byte_offset = tensor->byte_offset;
      view.device_type = tensor->device_type;
      view.device_index = tensor->device_index;
      view.dtype = static_cast<std::uint32_t>(tensor->dtype);
      view.rank = static_cast<std::uint32_t>(tensor->sizes.size());
      view.sizes = tensor->sizes.data();      // stays owned by `arguments`
      view.strides = tensor->strides.data();
      view.flags = tensor->flags;
    } else if (const auto* scalar = std::get_if<Scalar>(&value)) {
      record.kind = VECOPS_VALUE_SCALAR;
      record.value.scalar.struct_size = sizeof(VecopsScalar);
      record.value.scalar.dtype = static_cast<std::uint32_t>(scalar->dtype);
      record.value.scalar.value = scalar->value;
    } else {
      record.kind = VECOPS_VALUE_NONE;
    }
    values_.push_back(record);
  }
  call_.struct_size = sizeof(VecopsCall);
  call_.num_values = static_cast<std::uint32_t>(values_.size());
  call_.values = values_.data();
  call_.workspace = workspace;
  call_.workspace_size = workspace_size;
  call_.context = context;
}

Status validate_tensor(const TensorView& tensor, const TensorConstraint& constraint, std::string_view parameter_name) {
  const std::string name(parameter_name);
  if ((dtype_bit(tensor.dtype) & constraint.dtype_mask) == 0) return invalid(name + " has an unsupported dtype");
  if ((constraint.device_type != 0 && tensor.device_type != constraint.device_type) ||
      (constraint.device_index >= 0 && tensor.device_index != constraint.device_index))
    return invalid(name + " is on the wrong device");
  if (tensor.sizes.size() != tensor.strides.size()) return invalid(name + " has different size and stride ranks");
  if (tensor.sizes.size() > std::numeric_limits<std::uint32_t>::max()) return invalid(name + " rank exceeds the ABI limit");
  for (const auto size : tensor.sizes)
    if (size < 0) return invalid(name + " has a negative size");
  if (constraint.rank && tensor.sizes.size() != *constraint.rank) return invalid(name + " has the wrong rank");
  if (!constraint.sizes.empty() && constraint.sizes.size() != tensor.sizes.size())
    return invalid(name + " has no size constraint for its rank");
  if (!constraint.strides.empty() && constraint.strides.size() != tensor.strides.size())
    return invalid(name + " has no stride constraint for its rank");
  for (std::size_t i = 0; i < constraint.sizes.size(); ++i)
    if (!constraint.sizes[i].accepts(tensor.sizes[i])) return invalid(name + " size[" + std::to_string(i) + "] violates schema");
  for (std::size_t i = 0; i < constraint.strides.size(); ++i)
    if (!constraint.strides[i].accepts(tensor.strides[i])) return invalid(name + " stride[" + std::to_string(i) + "] violates schema");
  if ((tensor.flags & constraint.required_flags) != constraint.required_flags)
    return invalid(name + " does not satisfy the required access flags");
  return Status::success();
}

OperatorSchema::OperatorSchema(std::string name, std::vector<ParameterSchema> parameters, RelationValidator relation_validator)
    : name_(std::move(name)), parameters_(std::move(parameters)), relation_validator_(std::move(relation_validator)) {}

Status OperatorSchema::validate(const ArgumentMetadata& arguments) const {
  if (arguments.size() != parameters_.size())
    return invalid(name_ + " expects " + std::to_string(parameters_.size()) + " arguments, got " + std::to_string(arguments.size()));
  for (std::size_t index = 0; index < parameters_.size(); ++index) {
    const ParameterSchema& parameter = parameters_[index];
    const Value& value = arguments[index];
    if (const auto* rule = std::get_if<TensorConstraint>(&parameter.constraint)) {
      if (std::holds_alternative<std::monostate>(value)) {
        if (!rule->optional) return invalid(parameter.name + " is not optional");
        continue;
      }
      const auto* tensor = std::get_if<TensorView>(&value);
      if (tensor == nullptr) return invalid(parameter.name + " must be a tensor");
      if (auto status = validate_tensor(*tensor, *rule, parameter.name); !status.ok()) return status;
    } else {
      const auto* scalar = std::get_if<Scalar>(&value);
      if (scalar == nullptr) return invalid(parameter.name + " must be a scalar");
      if ((dtype_bit(scalar->dtype) & std::get<ScalarConstraint>(parameter.constraint).dtype_mask) == 0)
        return invalid(parameter.name + " has an unsupported scalar dtype");
    }
  }
  return relation_validator_ ? relation_validator_(arguments.values()) : Status::success();
}

}  // namespace vecops::runtime
