// RESTATED FROM vecops (src/runtime/KernelDefinition.cpp:59-534), not designed here.  Inside a vecops build this file is not used at all: vecops' own
// runtime takes its place and only the matmul recipe, dispatch policy and executable provider of this library are new
// (csrc/runtime/matmul_operator.cpp).  It exists so that the library builds and is testable standalone, with the
// class names, signatures, checks and status texts a caller of vecops' runtime expects.
//
// Binding of a KernelCall against a KernelDef.  Behaviour follows
// src/runtime/KernelDefinition.cpp:59-534 of vecops (dtype spelling :59-91,
// symbol inference :96-118, dimension checks :142-186, definition checks
// :224-330, canonical text :332-396, two-phase bind and key :398-534).
#include "vecops_b200/runtime_mirror/kernel_def.h"

#include <bit>
#include <cctype>
#include <set>
#include <sstream>

namespace vecops::runtime {
namespace {

Status invalid(std::string message) { return Status(StatusCode::InvalidArgument, std::move(message)); }

bool valid_dtype(DType dtype) { return dtype_bit(dtype) != 0; }

bool is_identifier(std::string_view name) {
  if (name.empty() || !(std::isalpha(static_cast<unsigned char>(name[0])) || name[0] == '_')) return false;
  for (const char ch : name)
    if (!(std::isalnum(static_cast<unsigned char>(ch)) || ch == '_')) return false;
  // Symbols become C++ identifiers in vecops' generated sources, so its
  // keywords are refused there; keep the same refusal for the common ones.
  static const std::set<std::string_view> kReserved = {
      "alignas", "alignof", "and", "asm", "auto", "bool", "break", "case", "catch", "char", "class", "concept",
      "const", "constexpr", "continue", "decltype", "default", "delete", "do", "double", "else", "enum",
      "explicit", "export", "extern", "false", "float", "for", "friend", "goto", "if", "inline", "int", "long",
      "namespace", "new", "noexcept", "not", "nullptr", "operator", "or", "private", "protected", "public",
      "register", "reinterpret_cast", "requires", "return", "short", "signed", "sizeof", "static", "struct",
      "switch", "template", "this", "throw", "true", "try", "typedef", "typename", "union", "unsigned", "using",
      "virtual", "void", "volatile", "while"};
  return !kReserved.contains(name);
}

std::string value_text(const SpecializationValue& value) {
  if (const auto* integer = std::get_if<std::int64_t>(&value)) return std::to_string(*integer);
  return dtype_name(std::get<DType>(value));
}

const std::string& parameter_name(const KernelParameterDef& parameter) {
  return std::visit([](const auto& item) -> const std::string& { return item.name; }, parameter);
}

std::string expr_text(const ConstExpr& e) {
  return e.is_symbol() ? "@" + std::string(e.symbol()) : "#" + std::to_string(e.fixed_value());
}

// Record `observed` for the named symbol, or check it against what is known.
Status bind_symbol(const KernelDef& def, SpecializationValues& values, std::string_view name,
                   SpecializationValue observed, const std::string& where) {
  const auto declared = def.values().find(name);
  if (declared == def.values().end())
    return invalid(where + " references undeclared specialization value '" + std::string(name) + "'");
  const bool is_int = std::holds_alternative<std::int64_t>(observed);
  if ((declared->second == SpecializationType::ConstInt) != is_int)
    return invalid("specialization value '" + std::string(name) + "' has the wrong type");
  const auto known = values.find(name);
  if (known == values.end()) {
    values.emplace(std::string(name), observed);
    return Status::success();
  }
  if (known->second != observed)
    return invalid("specialization value '" + std::string(name) + "' is " + value_text(known->second) + ", but " + where +
                   " observed " + value_text(observed));
  return Status::success();
}

Status check_expr_declared(const KernelDef& def, const ConstExpr& e, const std::string& where) {
  if (!e.is_symbol()) return Status::success();
  const auto found = def.values().find(e.symbol());
  if (found == def.values().end() || found->second != SpecializationType::ConstInt)
    return invalid(where + " references undeclared or non-ConstInt symbol '" + std::string(e.symbol()) + "'");
  return Status::success();
}

Result<std::int64_t> evaluate(const ConstExpr& e, const SpecializationValues& values, const std::string& where) {
  if (!e.is_symbol()) return e.fixed_value();
  const auto found = values.find(e.symbol());
  if (found == values.end()) return invalid(where + " requires unresolved symbol '" + std::string(e.symbol()) + "'");
  if (const auto* v = std::get_if<std::int64_t>(&found->second)) return *v;
  return invalid(where + " requires an integer symbol");
}

// Phase one: collect what a dimension teaches us (symbols, anonymous entries,
// named runtime dimensions that must agree across tensors).
Status observe(const KernelDef& def, const DimensionDef& dim, std::int64_t seen, SpecializationValues& values,
               std::vector<SpecializationValue>& anonymous, std::map<std::string, std::int64_t, std::less<>>& runtime_dims,
               const std::string& where) {
  switch (dim.kind()) {
    case DimensionDef::Kind::Symbol:
      return bind_symbol(def, values, dim.symbol(), seen, where);
    case DimensionDef::Kind::Const:
      anonymous.emplace_back(seen);
      return Status::success();
    case DimensionDef::Kind::Dynamic:
      if (!dim.symbol().empty()) {
        const auto [slot, fresh] = runtime_dims.emplace(dim.symbol(), seen);
        if (!fresh && slot->second != seen)
          return invalid("runtime dimension '" + std::string(dim.symbol()) + "' is " + std::to_string(slot->second) +
                         ", but " + where + " observed " + std::to_string(seen));
      }
      return Status::success();
    case DimensionDef::Kind::Fixed:
      return Status::success();
  }
  return Status::success();
}

// Phase two: with every symbol known, check Fixed and Dynamic dimensions.
Status check(const DimensionDef& dim, std::int64_t seen, const SpecializationValues& values, const std::string& where) {
  if (dim.kind() == DimensionDef::Kind::Fixed) {
    if (seen != dim.fixed_value()) return invalid(where + " must equal " + std::to_string(dim.fixed_value()));
    return Status::success();
  }
  if (dim.kind() != DimensionDef::Kind::Dynamic) return Status::success();
  auto alignment = evaluate(dim.alignment(), values, where + " alignment");
  if (!alignment) return alignment.status();
  auto lower = evaluate(dim.lower_bound(), values, where + " lower bound");
  if (!lower) return lower.status();
  auto upper = evaluate(dim.upper_bound(), values, where + " upper bound");
  if (!upper) return upper.status();
  if (alignment.value() <= 0 || !std::has_single_bit(static_cast<std::uint64_t>(alignment.value())))
    return invalid(where + " alignment must be a positive power of two");
  if (lower.value() > upper.value()) return invalid(where + " lower bound exceeds its upper bound");
  if (seen < lower.value() || seen > upper.value() || seen % alignment.value() != 0)
    return invalid(where + " violates Dynamic<" + std::to_string(alignment.value()) + ", " + std::to_string(lower.value()) +
                   ", " + std::to_string(upper.value()) + ">");
  return Status::success();
}

}  // namespace

std::string dtype_name(DType dtype) {
  switch (dtype) {
    case DType::Bool: return "bool";
    case DType::Int8: return "i8";
    case DType::UInt8: return "u8";
    case DType::Int16: return "i16";
    case DType::UInt16: return "u16";
    case DType::Int32: return "i32";
    case DType::UInt32: return "u32";
    case DType::Int64: return "i64";
    case DType::UInt64: return "u64";
    case DType::Float16: return "f16";
    case DType::BFloat16: return "bf16";
    case DType::Float32: return "f32";
    case DType::Float64: return "f64";
    case DType::Invalid: break;
  }
  return "invalid";
}

DimensionDef DimensionDef::dynamic(ConstExpr alignment, ConstExpr lower_bound, ConstExpr upper_bound) {
  DimensionDef d(Kind::Dynamic);
  d.alignment_ = std::move(alignment);
  d.lower_bound_ = std::move(lower_bound);
  d.upper_bound_ = std::move(upper_bound);
  return d;
}

DimensionDef DimensionDef::named_dynamic(std::string symbol, ConstExpr alignment, ConstExpr lower_bound,
                                         ConstExpr upper_bound) {
  DimensionDef d = dynamic(std::move(alignment), std::move(lower_bound), std::move(upper_bound));
  d.symbol_ = std::move(symbol);
  return d;
}

KernelDef::KernelDef(std::string name, std::vector<KernelParameterDef> parameters,
                     std::map<std::string, SpecializationType, std::less<>> values)
    : name_(std::move(name)), parameters_(std::move(parameters)), values_(std::move(values)) {}

Status KernelDef::validate() const {
  if (name_.empty()) return invalid("kernel definition name must not be empty");
  std::set<std::string, std::less<>> seen_names;
  std::map<std::string, std::string, std::less<>> runtime_symbols;
  for (const auto& parameter : parameters_) {
    const std::string& pname = parameter_name(parameter);
    if (pname.empty()) return invalid("kernel parameter names must not be empty");
    if (!seen_names.insert(pname).second) return invalid("duplicate kernel parameter '" + pname + "'");
    if (const auto* scalar = std::get_if<ValueDef>(&parameter)) {
      if (!valid_dtype(scalar->dtype)) return invalid("scalar '" + scalar->name + "' has an invalid dtype");
      if (scalar->default_value && scalar->default_value->dtype != scalar->dtype)
        return invalid("scalar '" + scalar->name + "' default dtype does not match its declaration");
      continue;
    }
    const auto& tensor = std::get<TensorDef>(parameter);
    if (tensor.shape.size() != tensor.strides.size())
      return invalid("tensor '" + tensor.name + "' shape and stride ranks differ");
    if (tensor.optional && tensor.writable()) return invalid("writable tensor '" + tensor.name + "' cannot be optional");
    if (tensor.dtype.dtype() && !valid_dtype(*tensor.dtype.dtype()))
      return invalid("tensor '" + tensor.name + "' has an invalid fixed dtype");
    if (!tensor.dtype.symbol().empty()) {
      const auto found = values_.find(tensor.dtype.symbol());
      if (found == values_.end() || found->second != SpecializationType::DType)
        return invalid("tensor '" + tensor.name + "' references undeclared or non-dtype symbol '" +
                       std::string(tensor.dtype.symbol()) + "'");
    }
    for (const auto* part : {&tensor.shape, &tensor.strides}) {
      const char* label = part == &tensor.shape ? "shape" : "stride";
      for (std::size_t axis = 0; axis < part->size(); ++axis) {
        const DimensionDef& dim = (*part)[axis];
        const std::string where = "tensor '" + tensor.name + "' " + label + "[" + std::to_string(axis) + "]";
        if (dim.kind() == DimensionDef::Kind::Symbol) {
          const auto found = values_.find(dim.symbol());
          if (found == values_.end() || found->second != SpecializationType::ConstInt)
            return invalid(where + " references undeclared or non-ConstInt symbol '" + std::string(dim.symbol()) + "'");
        } else if (dim.kind() == DimensionDef::Kind::Dynamic) {
          for (const auto& [expr, what] : {std::pair{&dim.alignment(), " alignment"}, std::pair{&dim.lower_bound(), " lower bound"},
                                           std::pair{&dim.upper_bound(), " upper bound"}}) {
            if (auto status = check_expr_declared(*this, *expr, where + what); !status.ok()) return status;
          }
          if (!dim.alignment().is_symbol() && !dim.lower_bound().is_symbol() && !dim.upper_bound().is_symbol()) {
            const auto alignment = dim.alignment().fixed_value();
            if (alignment <= 0 || !std::has_single_bit(static_cast<std::uint64_t>(alignment)))
              return invalid(where + " alignment must be a positive power of two");
            if (dim.lower_bound().fixed_value() > dim.upper_bound().fixed_value())
              return invalid(where + " lower bound exceeds its upper bound");
          }
          if (!dim.symbol().empty()) {
            if (!is_identifier(dim.symbol()))
              return invalid(where + " has invalid runtime dimension symbol '" + std::string(dim.symbol()) + "'");
            if (values_.contains(dim.symbol()))
              return invalid(where + " runtime dimension symbol '" + std::string(dim.symbol()) +
                             "' conflicts with a specialization value");
            const std::string declaration =
                expr_text(dim.alignment()) + "," + expr_text(dim.lower_bound()) + "," + expr_text(dim.upper_bound());
            const auto [slot, fresh] = runtime_symbols.emplace(std::string(dim.symbol()), declaration);
            if (!fresh && slot->second != declaration)
              return invalid("runtime dimension symbol '" + std::string(dim.symbol()) + "' has conflicting Dynamic declarations");
          }
        }
      }
    }
  }
  for (const auto& [name, type] : values_) {
    (void)type;
    if (name.empty()) return invalid("specialization value names must not be empty");
    if (!is_identifier(name)) return invalid("specialization value '" + name + "' is not a valid C++ identifier");
  }
  return Status::success();
}

std::string KernelDef::canonical() const {
  auto dimension = [](const DimensionDef& d) -> std::string {
    switch (d.kind()) {
      case DimensionDef::Kind::Fixed: return "F" + std::to_string(d.fixed_value());
      case DimensionDef::Kind::Symbol: return "S" + std::string(d.symbol());
      case DimensionDef::Kind::Const: return "C";
      case DimensionDef::Kind::Dynamic:
        return "D" + (d.symbol().empty() ? std::string{} : "@" + std::string(d.symbol())) + "(" + expr_text(d.alignment()) +
               "," + expr_text(d.lower_bound()) + "," + expr_text(d.upper_bound()) + ")";
    }
    return "?";
  };
  std::ostringstream out;
  out << "name:" << name_;
  for (const auto& [name, type] : values_) out << ";value:" << name << ':' << (type == SpecializationType::ConstInt ? 'i' : 't');
  for (const auto& parameter : parameters_) {
    if (const auto* tensor = std::get_if<TensorDef>(&parameter)) {
      out << ";tensor:" << tensor->name << ":optional=" << tensor->optional << ":access=" << static_cast<int>(tensor->access)
          << ":device=" << tensor->device_type << ':' << tensor->device_index << ":dtype=";
      if (tensor->dtype.dtype()) out << static_cast<std::uint32_t>(*tensor->dtype.dtype());
      else if (!tensor->dtype.symbol().empty()) out << '@' << tensor->dtype.symbol();
      else out << '?';
      out << ":shape=";
      for (const auto& d : tensor->shape) out << dimension(d) << ',';
      out << ":strides=";
      for (const auto& d : tensor->strides) out << dimension(d) << ',';
    } else {
      const auto& scalar = std::get<ValueDef>(parameter);
      out << ";scalar:" << scalar.name << ":dtype=" << static_cast<std::uint32_t>(scalar.dtype) << ":default=";
      if (!scalar.default_value) out << '?';
      else if (scalar.dtype == DType::Float16 || scalar.dtype == DType::BFloat16 || scalar.dtype == DType::Float32 ||
               scalar.dtype == DType::Float64)
        out << std::hexfloat << scalar.default_value->value.f64 << std::defaultfloat;
      else if (scalar.dtype == DType::Int8 || scalar.dtype == DType::Int16 || scalar.dtype == DType::Int32 ||
               scalar.dtype == DType::Int64)
        out << scalar.default_value->value.i64;
      else out << scalar.default_value->value.u64;
    }
  }
  return out.str();
}

Result<BoundKernel> bind_kernel_call(const KernelDef& def, const KernelCall& call) {
  if (auto status = def.validate(); !status.ok()) return status;

  SpecializationValues values = call.values();
  for (const auto& [name, value] : values) {
    const auto declared = def.values().find(name);
    if (declared == def.values().end()) return invalid("unknown specialization value '" + name + "'");
    if ((declared->second == SpecializationType::ConstInt) != std::holds_alternative<std::int64_t>(value))
      return invalid("specialization value '" + name + "' has the wrong type");
    if (const auto* dtype = std::get_if<DType>(&value); dtype && !valid_dtype(*dtype))
      return invalid("specialization value '" + name + "' has an invalid dtype");
  }

  // Positional arguments; omitted trailing optionals and defaulted scalars are filled in.
  std::vector<Value> args(call.arguments().values().begin(), call.arguments().values().end());
  const auto params = def.parameters();
  if (args.size() > params.size()) return invalid("kernel '" + def.name() + "' received too many arguments");
  while (args.size() < params.size()) {
    const auto& parameter = params[args.size()];
    if (const auto* tensor = std::get_if<TensorDef>(&parameter); tensor && tensor->optional) args.emplace_back(std::monostate{});
    else if (const auto* scalar = std::get_if<ValueDef>(&parameter); scalar && scalar->default_value) args.emplace_back(*scalar->default_value);
    else return invalid("kernel '" + def.name() + "' is missing argument '" + parameter_name(parameter) + "'");
  }

  std::vector<SpecializationValue> anonymous;
  std::map<std::string, std::int64_t, std::less<>> runtime_dims;
  for (std::size_t index = 0; index < params.size(); ++index) {
    const auto* tdef = std::get_if<TensorDef>(&params[index]);
    if (tdef == nullptr) continue;
    if (std::holds_alternative<std::monostate>(args[index])) {
      if (!tdef->optional) return invalid("tensor '" + tdef->name + "' is not optional");
      anonymous.emplace_back(std::int64_t{0});
      continue;
    }
    const auto* tensor = std::get_if<TensorView>(&args[index]);
    if (tensor == nullptr) return invalid("parameter '" + tdef->name + "' must be a tensor");
    if (tdef->optional) anonymous.emplace_back(std::int64_t{1});
    if (tensor->sizes.size() != tensor->strides.size() || tensor->sizes.size() != tdef->shape.size())
      return invalid("tensor '" + tdef->name + "' has the wrong rank");
    if (!tdef->dtype.symbol().empty()) {
      if (auto status = bind_symbol(def, values, tdef->dtype.symbol(), tensor->dtype, "tensor '" + tdef->name + "' dtype"); !status.ok())
        return status;
    } else if (tdef->dtype.anonymous()) {
      anonymous.emplace_back(tensor->dtype);
    }
    for (std::size_t axis = 0; axis < tensor->sizes.size(); ++axis) {
      const std::string at = "[" + std::to_string(axis) + "]";
      if (auto status = observe(def, tdef->shape[axis], tensor->sizes[axis], values, anonymous, runtime_dims,
                                "tensor '" + tdef->name + "' shape" + at); !status.ok())
        return status;
      if (auto status = observe(def, tdef->strides[axis], tensor->strides[axis], values, anonymous, runtime_dims,
                                "tensor '" + tdef->name + "' stride" + at); !status.ok())
        return status;
    }
  }
  for (const auto& [name, type] : def.values()) {
    (void)type;
    if (!values.contains(name)) return invalid("specialization value '" + name + "' cannot be inferred and must be supplied");
  }

  for (std::size_t index = 0; index < params.size(); ++index) {
    if (const auto* tdef = std::get_if<TensorDef>(&params[index])) {
      if (std::holds_alternative<std::monostate>(args[index])) continue;
      const auto& tensor = std::get<TensorView>(args[index]);
      if (!valid_dtype(tensor.dtype)) return invalid("tensor '" + tdef->name + "' has an invalid dtype");
      if (tdef->device_type != 0 && tensor.device_type != tdef->device_type)
        return invalid("tensor '" + tdef->name + "' is on the wrong device type");
      if (tdef->device_index >= 0 && tensor.device_index != tdef->device_index)
        return invalid("tensor '" + tdef->name + "' is on the wrong device index");
      const std::uint64_t need = (tdef->readable() ? VECOPS_TENSOR_READ : 0) | (tdef->writable() ? VECOPS_TENSOR_WRITE : 0);
      if ((tensor.flags & need) != need) return invalid("tensor '" + tdef->name + "' has incompatible access flags");
      for (const auto size : tensor.sizes)
        if (size < 0) return invalid("tensor '" + tdef->name + "' has a negative size");
      if (tdef->dtype.dtype() && tensor.dtype != *tdef->dtype.dtype()) return invalid("tensor '" + tdef->name + "' has the wrong dtype");
      for (std::size_t axis = 0; axis < tensor.sizes.size(); ++axis) {
        const std::string at = "[" + std::to_string(axis) + "]";
        if (auto status = check(tdef->shape[axis], tensor.sizes[axis], values, "tensor '" + tdef->name + "' shape" + at); !status.ok())
          return status;
        if (auto status = check(tdef->strides[axis], tensor.strides[axis], values, "tensor '" + tdef->name + "' stride" + at); !status.ok())
          return status;
      }
    } else {
      const auto& sdef = std::get<ValueDef>(params[index]);
      const auto* scalar = std::get_if<Scalar>(&args[index]);
      if (scalar == nullptr) return invalid("parameter '" + sdef.name + "' must be a scalar");
      if (scalar->dtype != sdef.dtype) return invalid("scalar '" + sdef.name + "' has the wrong dtype");
    }
  }

  std::string key = def.name();
  for (const auto& [name, value] : values) key += ";" + name + "=" + value_text(value);
  for (std::size_t index = 0; index < anonymous.size(); ++index) key += ";$" + std::to_string(index) + "=" + value_text(anonymous[index]);
  return BoundKernel{ArgumentMetadata(std::move(args)), std::move(values), std::move(anonymous), std::move(key)};
}

}  // namespace vecops::runtime
