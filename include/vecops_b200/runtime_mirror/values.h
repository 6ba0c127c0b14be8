// RESTATED FROM vecops (include/vecops/runtime/Argument.h:226-370), not designed here.  Inside a vecops build this file is not used at all: vecops' own
// runtime takes its place and only the matmul recipe, dispatch policy and executable provider of this library are new
// (csrc/runtime/matmul_operator.cpp).  It exists so that the library builds and is testable standalone, with the
// class names, signatures, checks and status texts a caller of vecops' runtime expects.
//
// Erased call values: tensors as metadata + address, scalars in the ABI's
// widest lane.  Mirrors include/vecops/runtime/Argument.h:46-475.
//
// TensorView already carries device_type / device_index in vecops
// (Argument.h:226-242); on this path a tensor is CUDA memory: `data` is a
// device pointer and device_type is VECOPS_DEVICE_CUDA.  `device_tensor`
// builds such a view.
#pragma once

#include <concepts>
#include <cstdint>
#include <span>
#include <type_traits>
#include <utility>
#include <variant>
#include <vector>

#include "vecops_b200/call_abi.h"

namespace vecops {

// 16-bit storage wrappers, enough for dtype_of<> and host-side test data.
struct bfloat16_t {
  std::uint16_t bits = 0;
};
struct float16_t {
  std::uint16_t bits = 0;
};

}  // namespace vecops

namespace vecops::runtime {

enum class DType : std::uint32_t {
  Invalid = VECOPS_DTYPE_INVALID,
  Bool = VECOPS_DTYPE_BOOL,
  Int8 = VECOPS_DTYPE_I8,
  UInt8 = VECOPS_DTYPE_U8,
  Int16 = VECOPS_DTYPE_I16,
  UInt16 = VECOPS_DTYPE_U16,
  Int32 = VECOPS_DTYPE_I32,
  UInt32 = VECOPS_DTYPE_U32,
  Int64 = VECOPS_DTYPE_I64,
  UInt64 = VECOPS_DTYPE_U64,
  Float16 = VECOPS_DTYPE_F16,
  BFloat16 = VECOPS_DTYPE_BF16,
  Float32 = VECOPS_DTYPE_F32,
  Float64 = VECOPS_DTYPE_F64,
};

// Bit (dtype - 1) of a dtype mask; 0 for Invalid / out of range.
constexpr std::uint64_t dtype_bit(DType dtype) {
  const auto v = static_cast<std::uint32_t>(dtype);
  return (v < 1 || v > 13) ? 0 : (std::uint64_t{1} << (v - 1));
}
constexpr std::uint64_t all_dtypes() { return (std::uint64_t{1} << 13) - 1; }

template <typename T> inline constexpr DType dtype_of = DType::Invalid;
template <> inline constexpr DType dtype_of<bool> = DType::Bool;
template <> inline constexpr DType dtype_of<std::int8_t> = DType::Int8;
template <> inline constexpr DType dtype_of<std::uint8_t> = DType::UInt8;
template <> inline constexpr DType dtype_of<std::int16_t> = DType::Int16;
template <> inline constexpr DType dtype_of<std::uint16_t> = DType::UInt16;
template <> inline constexpr DType dtype_of<std::int32_t> = DType::Int32;
template <> inline constexpr DType dtype_of<std::uint32_t> = DType::UInt32;
template <> inline constexpr DType dtype_of<std::int64_t> = DType::Int64;
template <> inline constexpr DType dtype_of<std::uint64_t> = DType::UInt64;
template <> inline constexpr DType dtype_of<float16_t> = DType::Float16;
template <> inline constexpr DType dtype_of<bfloat16_t> = DType::BFloat16;
template <> inline constexpr DType dtype_of<float> = DType::Float32;
template <> inline constexpr DType dtype_of<double> = DType::Float64;

struct TensorView {
  void* data = nullptr;
  std::uint64_t byte_offset = 0;
  std::uint32_t device_type = VECOPS_DEVICE_CPU;
  std::int32_t device_index = 0;
  DType dtype = DType::Invalid;
  std::vector<std::int64_t> sizes;
  std::vector<std::int64_t> strides;  // elements
  std::uint64_t flags = VECOPS_TENSOR_READ;

  [[nodiscard]] bool writable() const { return (flags & VECOPS_TENSOR_WRITE) != 0; }
};

// View of CUDA memory: device pointer + device ordinal.
inline TensorView device_tensor(void* device_pointer, DType dtype, std::vector<std::int64_t> sizes,
                                std::vector<std::int64_t> strides, std::int32_t device_index = 0,
                                bool writable = false) {
  TensorView view;
  view.data = device_pointer;
  view.device_type = VECOPS_DEVICE_CUDA;
  view.device_index = device_index;
  view.dtype = dtype;
  view.sizes = std::move(sizes);
  view.strides = std::move(strides);
  view.flags = VECOPS_TENSOR_READ | (writable ? VECOPS_TENSOR_WRITE : 0);
  return view;
}

struct Scalar {
  DType dtype = DType::Invalid;
  VecopsScalarStorage value{};

  static Scalar signed_integer(std::int64_t v, DType dtype = DType::Int64) {
    Scalar s;
    s.dtype = dtype;
    s.value.i64 = v;
    return s;
  }
  static Scalar unsigned_integer(std::uint64_t v, DType dtype = DType::UInt64) {
    Scalar s;
    s.dtype = dtype;
    s.value.u64 = v;
    return s;
  }
  static Scalar floating(double v, DType dtype = DType::Float64) {
    Scalar s;
    s.dtype = dtype;
    s.value.f64 = v;
    return s;
  }
};

using Value = std::variant<std::monostate, TensorView, Scalar>;

class ArgumentMetadata {
public:
  ArgumentMetadata() = default;
  explicit ArgumentMetadata(std::vector<Value> values) : values_(std::move(values)) {}
  [[nodiscard]] std::span<const Value> values() const { return values_; }
  [[nodiscard]] std::span<Value> values() { return values_; }
  [[nodiscard]] std::size_t size() const { return values_.size(); }
  [[nodiscard]] const Value& operator[](std::size_t index) const { return values_[index]; }

private:
  std::vector<Value> values_;
};

// The C-ABI image of an ArgumentMetadata for one workspace query or run.
// Shape/stride arrays stay owned by the metadata, which must outlive the frame.
class CallFrame {
public:
  explicit CallFrame(const ArgumentMetadata& arguments, void* workspace = nullptr, std::uint64_t workspace_size = 0,
                     const VecopsExecutionContext* context = nullptr);
  [[nodiscard]] const VecopsCall& abi() const { return call_; }

private:
  std::vector<VecopsValue> values_;
  VecopsCall call_{};
};

inline Value erase_value(Value v) { return v; }
inline Value erase_value(std::monostate v) { return v; }
inline Value erase_value(TensorView v) { return v; }
inline Value erase_value(Scalar v) { return v; }
inline Value erase_value(bool v) { return Scalar::unsigned_integer(v ? 1 : 0, DType::Bool); }
template <std::signed_integral T>
  requires(dtype_of<std::remove_cv_t<T>> != DType::Invalid)
inline Value erase_value(T v) {
  return Scalar::signed_integer(static_cast<std::int64_t>(v), dtype_of<std::remove_cv_t<T>>);
}
template <std::unsigned_integral T>
  requires(!std::same_as<std::remove_cv_t<T>, bool> && dtype_of<std::remove_cv_t<T>> != DType::Invalid)
inline Value erase_value(T v) {
  return Scalar::unsigned_integer(static_cast<std::uint64_t>(v), dtype_of<std::remove_cv_t<T>>);
}
template <std::floating_point T>
  requires(dtype_of<std::remove_cv_t<T>> != DType::Invalid)
inline Value erase_value(T v) {
  return Scalar::floating(static_cast<double>(v), dtype_of<std::remove_cv_t<T>>);
}

template <typename... Values>
ArgumentMetadata make_arguments(Values&&... values) {
  std::vector<Value> erased;
  erased.reserve(sizeof...(Values));
  (erased.push_back(erase_value(std::forward<Values>(values))), ...);
  return ArgumentMetadata(std::move(erased));
}

}  // namespace vecops::runtime
