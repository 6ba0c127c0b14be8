// Helpers shared by the translation units behind the C ABI.
#pragma once

#include <atomic>
#include <stdint.h>

#include "vecops_b200/call_abi.h"

namespace vb200 {

// Fill `error` (when the caller gave one) with `code` and a printf-style
// message, truncated to the caller's buffer; returns `code`.
int32_t set_error(VecopsError* error, int32_t code, const char* format, ...) __attribute__((format(printf, 3, 4)));

// Puts the calling thread back on the CUDA device it was on when the guard was made (entry points switch to the device
// their record names and must not leave the caller there, error paths included).
struct DeviceRestore {
  int previous = -1;
  DeviceRestore();
  ~DeviceRestore();
  DeviceRestore(const DeviceRestore&) = delete;
  DeviceRestore& operator=(const DeviceRestore&) = delete;
};

// Kernels launched by this library since load.
extern std::atomic<uint64_t> g_launches;

}  // namespace vb200
