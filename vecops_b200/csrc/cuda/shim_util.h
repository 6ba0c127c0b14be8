// Helpers shared by the translation units behind the C ABI.
#pragma once

#include <atomic>
#include <stdint.h>

#include "vecops_b200/call_abi.h"

namespace vb200 {

// Fill `error` (when the caller gave one) with `code` and a printf-style
// message, truncated to the caller's buffer; returns `code`.
int32_t set_error(VecopsError* error, int32_t code, const char* format, ...) __attribute__((format(printf, 3, 4)));

// Kernels launched by this library since load.
extern std::atomic<uint64_t> g_launches;

}  // namespace vb200
