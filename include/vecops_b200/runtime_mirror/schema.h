// RESTATED FROM vecops (include/vecops/runtime/Schema.h:35-187), not designed here.  Inside a vecops build this file is not used at all: vecops' own
// runtime takes its place and only the matmul recipe, dispatch policy and executable provider of this library are new
// (csrc/runtime/matmul_operator.cpp).  It exists so that the library builds and is testable standalone, with the
// class names, signatures, checks and status texts a caller of vecops' runtime expects.
//
// OperatorSchema: the framework-neutral signature an Operator validates every
// call against before any recipe sees it.  Mirrors
// include/vecops/runtime/Schema.h:35-187 and src/runtime/Schema.cpp:26-147.
#pragma once

#include <cstdint>
#include <functional>
#include <optional>
#include <span>
#include <string>
#include <string_view>
#include <variant>
#include <vector>

#include "vecops_b200/runtime_mirror/status.h"
#include "vecops_b200/runtime_mirror/values.h"

namespace vecops::runtime {

struct DimensionConstraint {
  enum class Kind { Any, Const, Dynamic };
  Kind kind = Kind::Any;
  std::int64_t value = 0;
  std::int64_t lower_bound = 0;
  std::int64_t upper_bound = INT64_MAX;
  std::int64_t alignment = 1;

  static DimensionConstraint any() { return {}; }
  static DimensionConstraint constant(std::int64_t value) {
    DimensionConstraint c;
    c.kind = Kind::Const;
    c.value = value;
    return c;
  }
  static DimensionConstraint dynamic(std::int64_t lower_bound = 0, std::int64_t upper_bound = INT64_MAX,
                                     std::int64_t alignment = 1) {
    DimensionConstraint c;
    c.kind = Kind::Dynamic;
    c.lower_bound = lower_bound;
    c.upper_bound = upper_bound;
    c.alignment = alignment;
    return c;
  }
  [[nodiscard]] bool accepts(std::int64_t candidate) const {
    switch (kind) {
      case Kind::Any: return true;
      case Kind::Const: return candidate == value;
      case Kind::Dynamic:
        return candidate >= lower_bound && candidate <= upper_bound && alignment > 0 && candidate % alignment == 0;
    }
    return false;
  }
};

struct TensorConstraint {
  std::uint64_t dtype_mask = all_dtypes();
  std::uint32_t device_type = 0;   // 0 = any
  std::int32_t device_index = -1;  // -1 = any
  std::optional<std::uint32_t> rank;
  std::vector<DimensionConstraint> sizes;
  std::vector<DimensionConstraint> strides;
  std::uint64_t required_flags = VECOPS_TENSOR_READ;
  bool optional = false;
};

struct ScalarConstraint {
  std::uint64_t dtype_mask = all_dtypes();
};

struct ParameterSchema {
  std::string name;
  std::variant<TensorConstraint, ScalarConstraint> constraint;
};

class OperatorSchema {
public:
  // Cross-parameter rule run after every parameter passed on its own
  // (for matmul: the K extents of A and B agree, C is [M,N], ...).
  using RelationValidator = std::function<Status(std::span<const Value>)>;

  OperatorSchema(std::string name, std::vector<ParameterSchema> parameters, RelationValidator relation_validator = {});

  [[nodiscard]] const std::string& name() const { return name_; }
  [[nodiscard]] std::span<const ParameterSchema> parameters() const { return parameters_; }
  [[nodiscard]] Status validate(const ArgumentMetadata& arguments) const;

private:
  std::string name_;
  std::vector<ParameterSchema> parameters_;
  RelationValidator relation_validator_;
};

Status validate_tensor(const TensorView& tensor, const TensorConstraint& constraint, std::string_view parameter_name);

}  // namespace vecops::runtime
