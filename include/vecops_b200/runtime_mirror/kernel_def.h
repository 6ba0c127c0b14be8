// RESTATED FROM vecops (include/vecops/runtime/KernelDefinition.h), not designed here.  Inside a vecops build this file is not used at all: vecops' own
// runtime takes its place and only the matmul recipe, dispatch policy and executable provider of this library are new
// (csrc/runtime/matmul_operator.cpp).  It exists so that the library builds and is testable standalone, with the
// class names, signatures, checks and status texts a caller of vecops' runtime expects.
//
// KernelDef / KernelCall / bind_kernel_call: the declarative signature of a
// kernel, a concrete call, and the binding that checks one against the other
// and derives the specialization key.
//
// Mirrors include/vecops/runtime/KernelDefinition.h:23-389 and the binding
// rules of src/runtime/KernelDefinition.cpp:398-534:
//   * named ConstInt / DType symbols are inferred from the first tensor that
//     mentions them and must agree everywhere else;
//   * anonymous Const dimensions, anonymous dtypes and the presence bit of an
//     optional tensor become positional "$i" entries;
//   * Dynamic dimensions (named or not) are checked against alignment/bounds
//     and never enter the key;
//   * key = name;sym=value;...;$0=...;$1=...   (symbols in name order, dtypes
//     spelled i8/u8/i32/f16/bf16/f32/...).
#pragma once

#include <concepts>
#include <cstdint>
#include <map>
#include <optional>
#include <span>
#include <string>
#include <string_view>
#include <variant>
#include <vector>

#include "vecops_b200/runtime_mirror/status.h"
#include "vecops_b200/runtime_mirror/values.h"

namespace vecops::runtime {

using SpecializationValue = std::variant<std::int64_t, DType>;
using SpecializationValues = std::map<std::string, SpecializationValue, std::less<>>;

enum class SpecializationType { ConstInt, DType };

// An integer literal or the name of a ConstInt specialization symbol.
class ConstExpr {
public:
  template <std::integral Integer>
  ConstExpr(Integer value) : value_(static_cast<std::int64_t>(value)) {}
  ConstExpr(std::string symbol) : symbol_(std::move(symbol)) {}
  ConstExpr(const char* symbol) : symbol_(symbol == nullptr ? "" : symbol) {}

  [[nodiscard]] bool is_symbol() const { return symbol_.has_value(); }
  [[nodiscard]] std::int64_t fixed_value() const { return value_; }
  [[nodiscard]] std::string_view symbol() const { return symbol_ ? std::string_view(*symbol_) : std::string_view{}; }

private:
  std::int64_t value_ = 0;
  std::optional<std::string> symbol_;
};

class DimensionDef {
public:
  enum class Kind { Fixed, Symbol, Const, Dynamic };

  template <std::integral Integer>
  DimensionDef(Integer value) : kind_(Kind::Fixed), fixed_value_(static_cast<std::int64_t>(value)) {}
  DimensionDef(std::string symbol) : kind_(Kind::Symbol), symbol_(std::move(symbol)) {}
  DimensionDef(const char* symbol) : DimensionDef(std::string(symbol == nullptr ? "" : symbol)) {}

  static DimensionDef constant() { return DimensionDef(Kind::Const); }
  static DimensionDef dynamic(ConstExpr alignment = 1, ConstExpr lower_bound = INT64_MIN,
                              ConstExpr upper_bound = INT64_MAX);
  static DimensionDef named_dynamic(std::string symbol, ConstExpr alignment = 1, ConstExpr lower_bound = INT64_MIN,
                                    ConstExpr upper_bound = INT64_MAX);
  static DimensionDef any() { return dynamic(); }

  [[nodiscard]] Kind kind() const { return kind_; }
  [[nodiscard]] std::int64_t fixed_value() const { return fixed_value_; }
  [[nodiscard]] std::string_view symbol() const { return symbol_; }
  [[nodiscard]] const ConstExpr& alignment() const { return alignment_; }
  [[nodiscard]] const ConstExpr& lower_bound() const { return lower_bound_; }
  [[nodiscard]] const ConstExpr& upper_bound() const { return upper_bound_; }

private:
  explicit DimensionDef(Kind kind) : kind_(kind) {}
  Kind kind_ = Kind::Dynamic;
  std::int64_t fixed_value_ = 0;
  std::string symbol_;
  ConstExpr alignment_{1};
  ConstExpr lower_bound_{INT64_MIN};
  ConstExpr upper_bound_{INT64_MAX};
};

// Fixed dtype, named DType symbol, or anonymous (positional key entry).
class TensorDTypeDef {
public:
  TensorDTypeDef() = default;
  TensorDTypeDef(DType dtype) : dtype_(dtype) {}
  TensorDTypeDef(std::string symbol) : symbol_(std::move(symbol)) {}
  TensorDTypeDef(const char* symbol) : symbol_(symbol == nullptr ? "" : symbol) {}

  [[nodiscard]] const std::optional<DType>& dtype() const { return dtype_; }
  [[nodiscard]] std::string_view symbol() const { return symbol_; }
  [[nodiscard]] bool anonymous() const { return !dtype_ && symbol_.empty(); }

private:
  std::optional<DType> dtype_;
  std::string symbol_;
};

enum class TensorAccess { Input, Output, InOut };

struct TensorDef {
  std::string name;
  std::vector<DimensionDef> shape;
  std::vector<DimensionDef> strides;
  TensorDTypeDef dtype;
  bool optional = false;
  TensorAccess access = TensorAccess::Input;
  std::uint32_t device_type = VECOPS_DEVICE_CPU;  // a CUDA kernel's definition sets VECOPS_DEVICE_CUDA
  std::int32_t device_index = -1;

  [[nodiscard]] bool readable() const { return access != TensorAccess::Output; }
  [[nodiscard]] bool writable() const { return access != TensorAccess::Input; }
};

struct ValueDef {
  std::string name;
  DType dtype = DType::Invalid;
  std::optional<Scalar> default_value;
};

using KernelParameterDef = std::variant<TensorDef, ValueDef>;

class KernelDef {
public:
  KernelDef(std::string name, std::vector<KernelParameterDef> parameters,
            std::map<std::string, SpecializationType, std::less<>> values = {});

  [[nodiscard]] const std::string& name() const { return name_; }
  [[nodiscard]] std::span<const KernelParameterDef> parameters() const { return parameters_; }
  [[nodiscard]] const std::map<std::string, SpecializationType, std::less<>>& values() const { return values_; }
  [[nodiscard]] Status validate() const;
  [[nodiscard]] std::string canonical() const;

private:
  std::string name_;
  std::vector<KernelParameterDef> parameters_;
  std::map<std::string, SpecializationType, std::less<>> values_;
};

using KernelDefinition = KernelDef;

class KernelCall {
public:
  KernelCall() = default;
  explicit KernelCall(ArgumentMetadata arguments, SpecializationValues values = {})
      : arguments_(std::move(arguments)), values_(std::move(values)) {}

  template <typename... Values>
  static KernelCall from_values(SpecializationValues specialization_values, Values&&... values) {
    return KernelCall(make_arguments(std::forward<Values>(values)...), std::move(specialization_values));
  }

  [[nodiscard]] const ArgumentMetadata& arguments() const { return arguments_; }
  [[nodiscard]] const SpecializationValues& values() const { return values_; }

private:
  ArgumentMetadata arguments_;
  SpecializationValues values_;
};

struct BoundKernel {
  ArgumentMetadata arguments;  // normalised: omitted trailing optionals / defaults filled in
  SpecializationValues values;
  std::vector<SpecializationValue> anonymous_values;
  std::string specialization_key;
};

[[nodiscard]] Result<BoundKernel> bind_kernel_call(const KernelDef& definition, const KernelCall& call);

// Spelling of a dtype inside specialization keys ("bf16", "i8", ...).
[[nodiscard]] std::string dtype_name(DType dtype);

using KernelShapes = KernelCall;

}  // namespace vecops::runtime
