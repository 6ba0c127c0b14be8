// Device-side bookkeeping of the matmul shim that other translation units behind the C ABI use too.
#pragma once

#include <cuda.h>
#include <stdint.h>

#include "shim_util.h"

namespace vb200 {

// Tiled tensor map with the 128-byte swizzle over a tensor of `rank` (2 or 3) dimensions, innermost first:
// dims[rank], strides_bytes[rank - 1] (dimension 0 is contiguous), box[rank].
int32_t shim_encode_map(CUtensorMap* out, CUtensorMapDataType dtype, uint32_t rank, const void* base, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box, VecopsError* error);

// What a launcher needs to know about `device`: SM count, compute capability major, and the pinned status word that
// kernels running there report a bounded wait's failure to.
int32_t shim_device_facts(int device, int* sm_count, int* major, uint32_t** status_word, VecopsError* error);

// A fresh non-zero value per launch for scratch words that must tell this launch's state from stale contents.
uint64_t shim_nonce(const void* salt);

// Reads and clears the device's status word (0 = no bounded wait ran out since the last read).
uint32_t shim_take_status(int device);

// The device buffer kernels write their optional timelines to (a tuning aid; null unless one was registered).
unsigned long long* shim_trace();

}  // namespace vb200
