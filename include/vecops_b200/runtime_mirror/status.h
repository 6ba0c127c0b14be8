// RESTATED FROM vecops (include/vecops/runtime/Status.h:49-179), not designed here.  Inside a vecops build this file is not used at all: vecops' own
// runtime takes its place and only the matmul recipe, dispatch policy and executable provider of this library are new
// (csrc/runtime/matmul_operator.cpp).  It exists so that the library builds and is testable standalone, with the
// class names, signatures, checks and status texts a caller of vecops' runtime expects.
//
// Status and Result<T>: error transport of the operator runtime.  No exception
// crosses a runtime call; callers branch on code().
//
// Same vocabulary as vecops' include/vecops/runtime/Status.h:23-179 (StatusCode
// values equal the C ABI's VecopsStatusCode).
#pragma once

#include <optional>
#include <string>
#include <utility>

#include "vecops_b200/call_abi.h"

namespace vecops::runtime {

enum class StatusCode : int {
  Ok = VECOPS_STATUS_OK,
  InvalidArgument = VECOPS_STATUS_INVALID_ARGUMENT,
  NotApplicable = VECOPS_STATUS_NOT_APPLICABLE,
  NotFound = VECOPS_STATUS_NOT_FOUND,
  AbiMismatch = VECOPS_STATUS_ABI_MISMATCH,
  LoadError = VECOPS_STATUS_LOAD_ERROR,
  ExecutionError = VECOPS_STATUS_EXECUTION_ERROR,
  InternalError = VECOPS_STATUS_INTERNAL_ERROR,
};

class Status {
public:
  Status() = default;
  Status(StatusCode code, std::string message) : code_(code), message_(std::move(message)) {}

  static Status success() { return {}; }
  [[nodiscard]] bool ok() const { return code_ == StatusCode::Ok; }
  [[nodiscard]] StatusCode code() const { return code_; }
  [[nodiscard]] const std::string& message() const { return message_; }

private:
  StatusCode code_ = StatusCode::Ok;
  std::string message_;
};

// A value, or the status that explains its absence.  Building one from a
// success status is a programming error and is turned into InternalError.
template <typename T>
class Result {
public:
  Result(T value) : value_(std::move(value)) {}
  Result(Status status)
      : status_(status.ok() ? Status(StatusCode::InternalError, "a value-less Result cannot contain success")
                            : std::move(status)) {}

  [[nodiscard]] bool ok() const { return value_.has_value(); }
  [[nodiscard]] explicit operator bool() const { return ok(); }
  [[nodiscard]] const Status& status() const {
    static const Status kSuccess;
    return ok() ? kSuccess : status_;
  }
  [[nodiscard]] T& value() & { return *value_; }
  [[nodiscard]] const T& value() const& { return *value_; }
  [[nodiscard]] T&& value() && { return std::move(*value_); }

private:
  std::optional<T> value_;
  Status status_;
};

template <>
class Result<void> {
public:
  Result() = default;
  Result(Status status) : status_(std::move(status)) {}
  [[nodiscard]] bool ok() const { return status_.ok(); }
  [[nodiscard]] explicit operator bool() const { return ok(); }
  [[nodiscard]] const Status& status() const { return status_; }

private:
  Status status_;
};

}  // namespace vecops::runtime
