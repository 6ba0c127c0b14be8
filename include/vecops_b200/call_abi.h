/*
 * vecops call-frame records, restated for the B200 matmul artifact.
 *
 * Every record here is layout-compatible (same field order, widths and enum
 * values) with the vecops C ABI it replaces on this path:
 *   include/vecops/runtime/CallAbi.h:34-51   status codes
 *   include/vecops/runtime/CallAbi.h:53-60   device types (CUDA == 2)
 *   include/vecops/runtime/CallAbi.h:62-91   dtypes
 *   include/vecops/runtime/CallAbi.h:93-107  value kinds, tensor access flags
 *   include/vecops/runtime/CallAbi.h:116-127 VecopsError
 *   include/vecops/runtime/CallAbi.h:137-158 VecopsTensorView
 *   include/vecops/runtime/CallAbi.h:161-197 VecopsScalar / VecopsValue
 *   include/vecops/runtime/CallAbi.h:360-377 VecopsExecutionContext
 *   include/vecops/runtime/CallAbi.h:387-400 VecopsCall
 *
 * Rules inherited from that ABI: the caller sets each `struct_size` to the
 * size of the record it hands over and keeps everything it points at alive
 * until the call returns; nobody on this side owns tensor storage, workspace,
 * stream or user data; shapes and strides count elements, `byte_offset` and
 * workspace sizes count bytes; `data + byte_offset` is logical element zero.
 *
 * A translation unit that already included the vecops header keeps vecops'
 * own definitions: this file then declares nothing.
 */
#ifndef VECOPS_B200_CALL_ABI_H
#define VECOPS_B200_CALL_ABI_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define VECOPS_B200_EXPORT __attribute__((visibility("default")))
#else
#define VECOPS_B200_EXPORT
#endif

#ifndef VECOPS_RUNTIME_CALL_ABI_H /* vecops' own header not seen: define the records */
#define VECOPS_B200_CALL_ABI_OWNS_RECORDS 1

#ifdef __cplusplus
extern "C" {
#endif

typedef enum VecopsStatusCode {
  VECOPS_STATUS_OK = 0,
  VECOPS_STATUS_INVALID_ARGUMENT = 1, /* metadata or values break a contract */
  VECOPS_STATUS_NOT_APPLICABLE = 2,   /* valid call, but this recipe does not serve it */
  VECOPS_STATUS_NOT_FOUND = 3,        /* no recipe / specialization / cubin */
  VECOPS_STATUS_ABI_MISMATCH = 4,     /* version, record size or key disagree */
  VECOPS_STATUS_LOAD_ERROR = 5,       /* loader or symbol lookup failed */
  VECOPS_STATUS_EXECUTION_ERROR = 6,  /* the kernel callback reported a failure */
  VECOPS_STATUS_INTERNAL_ERROR = 7
} VecopsStatusCode;

typedef enum VecopsDeviceType {
  VECOPS_DEVICE_CPU = 1,
  VECOPS_DEVICE_CUDA = 2,
  VECOPS_DEVICE_PRIVATE = 255
} VecopsDeviceType;

typedef enum VecopsDType {
  VECOPS_DTYPE_INVALID = 0,
  VECOPS_DTYPE_BOOL = 1,
  VECOPS_DTYPE_I8 = 2,
  VECOPS_DTYPE_U8 = 3,
  VECOPS_DTYPE_I16 = 4,
  VECOPS_DTYPE_U16 = 5,
  VECOPS_DTYPE_I32 = 6,
  VECOPS_DTYPE_U32 = 7,
  VECOPS_DTYPE_I64 = 8,
  VECOPS_DTYPE_U64 = 9,
  VECOPS_DTYPE_F16 = 10,
  VECOPS_DTYPE_BF16 = 11,
  VECOPS_DTYPE_F32 = 12,
  VECOPS_DTYPE_F64 = 13
} VecopsDType;

typedef enum VecopsValueKind {
  VECOPS_VALUE_NONE = 0,   /* omitted optional tensor */
  VECOPS_VALUE_TENSOR = 1,
  VECOPS_VALUE_SCALAR = 2
} VecopsValueKind;

typedef enum VecopsTensorFlags {
  VECOPS_TENSOR_READ = UINT64_C(1) << 0,
  VECOPS_TENSOR_WRITE = UINT64_C(1) << 1
} VecopsTensorFlags;

/* Diagnostic buffer owned by the caller.  A failing callee writes `code`,
 * the full length it wanted in `message_required` (terminator included) and
 * as much of the text as `message_capacity` allows, always NUL-terminated. */
typedef struct VecopsError {
  uint32_t struct_size;
  int32_t code;
  char* message;
  size_t message_capacity;
  size_t message_required;
} VecopsError;

/* Non-owning tensor metadata.  For a CUDA tensor `data` is a device pointer,
 * `device_type` is VECOPS_DEVICE_CUDA and `device_index` the CUDA ordinal. */
typedef struct VecopsTensorView {
  uint32_t struct_size;
  void* data;
  uint64_t byte_offset;
  uint32_t device_type;
  int32_t device_index;
  uint32_t dtype;
  uint32_t rank;
  const int64_t* sizes;
  const int64_t* strides;
  uint64_t flags;
} VecopsTensorView;

typedef union VecopsScalarStorage {
  int64_t i64;
  uint64_t u64;
  double f64;
} VecopsScalarStorage;

typedef struct VecopsScalar {
  uint32_t struct_size;
  uint32_t dtype;
  VecopsScalarStorage value;
} VecopsScalar;

typedef struct VecopsValue {
  uint32_t struct_size;
  uint32_t kind; /* VecopsValueKind selects the union member */
  union {
    VecopsTensorView tensor;
    VecopsScalar scalar;
  } value;
} VecopsValue;

/* The three trailing extension pointers belong to CPU-side protocols (arena
 * provider, thread pool, allocation observer).  The CUDA artifact never
 * dereferences them; they are kept so that the record has vecops' size. */
struct VecopsWorkspaceArenaProvider;
struct VecopsThreadPoolV1;
struct VecopsAllocationObserverV1;

typedef struct VecopsExecutionContext {
  uint32_t struct_size;
  uint32_t requested_threads;
  void* stream;    /* here: a cudaStream_t, or NULL for the default stream */
  void* user_data;
  uint64_t flags;  /* embedding-defined; see VECOPS_B200_CONTEXT_FLAG_ASYNC */
  const struct VecopsWorkspaceArenaProvider* workspace_provider;
  const struct VecopsThreadPoolV1* thread_pool;
  const struct VecopsAllocationObserverV1* allocation_observer;
} VecopsExecutionContext;

typedef struct VecopsCall {
  uint32_t struct_size;
  uint32_t num_values;
  const VecopsValue* values;
  void* workspace;         /* here: device scratch, sized by the workspace callback */
  uint64_t workspace_size;
  const VecopsExecutionContext* context;
} VecopsCall;

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* VECOPS_RUNTIME_CALL_ABI_H */

/* Bit of VecopsExecutionContext::flags understood by the B200 artifact: the
 * run callback only enqueues on `stream` and returns without synchronising.
 * Without it `run` keeps vecops' synchronous contract (CallAbi.h:15-16). */
#define VECOPS_B200_CONTEXT_FLAG_ASYNC (UINT64_C(1) << 32)

#endif /* VECOPS_B200_CALL_ABI_H */
