/*
 * vecops kernel-descriptor records, restated for the B200 matmul artifact.
 *
 * Layout-compatible with include/vecops/runtime/KernelAbi.h:
 *   :22-27    ABI version 1.1 and the query symbol name
 *   :29-36    dimension constraint kinds
 *   :45-58    VecopsDimensionConstraint
 *   :68-89    VecopsTensorParameter
 *   :92-97    VecopsScalarParameter
 *   :106-121  VecopsParameterDescriptor
 *   :129-131  workspace / run callback types
 *   :141-164  VecopsKernelDescriptorV1
 *
 * A descriptor states, per positional parameter, which dtypes, device, rank,
 * extents and strides one kernel specialization accepts, and carries the two
 * callbacks the runtime drives: `workspace` (bytes of caller-provided scratch;
 * must not touch tensor storage) and `run` (execute the validated frame).
 * For the B200 artifact the scratch is DEVICE memory and `run` launches on
 * the stream found in the call's execution context.
 */
#ifndef VECOPS_B200_KERNEL_ABI_H
#define VECOPS_B200_KERNEL_ABI_H

#include "vecops_b200/call_abi.h"

#ifndef VECOPS_RUNTIME_KERNEL_ABI_H /* vecops' own header not seen */
#define VECOPS_B200_KERNEL_ABI_OWNS_RECORDS 1

#ifdef __cplusplus
extern "C" {
#endif

#define VECOPS_KERNEL_ABI_VERSION_MAJOR 1u
#define VECOPS_KERNEL_ABI_VERSION_MINOR 1u
#define VECOPS_KERNEL_QUERY_SYMBOL_V1 "vecops_kernel_query_v1"

typedef enum VecopsDimensionKind {
  VECOPS_DIM_ANY = 0,     /* unconstrained */
  VECOPS_DIM_CONST = 1,   /* must equal `value` */
  VECOPS_DIM_DYNAMIC = 2  /* lower_bound <= x <= upper_bound and x % alignment == 0 */
} VecopsDimensionKind;

typedef struct VecopsDimensionConstraint {
  uint32_t struct_size;
  uint32_t kind;
  int64_t value;
  int64_t lower_bound;
  int64_t upper_bound;
  int64_t alignment; /* positive power of two */
} VecopsDimensionConstraint;

typedef struct VecopsTensorParameter {
  uint32_t struct_size;
  uint64_t dtype_mask;   /* bit (dtype - 1) per accepted VecopsDType */
  uint32_t device_type;  /* 0 accepts any */
  int32_t device_index;  /* -1 accepts any */
  int32_t rank;
  uint32_t optional;     /* non-zero: VECOPS_VALUE_NONE accepted */
  uint32_t dimension_constraint_stride;
  const VecopsDimensionConstraint* sizes;
  const VecopsDimensionConstraint* strides;
  uint64_t required_flags;
} VecopsTensorParameter;

typedef struct VecopsScalarParameter {
  uint32_t struct_size;
  uint64_t dtype_mask;
} VecopsScalarParameter;

typedef struct VecopsParameterDescriptor {
  uint32_t struct_size;
  uint32_t kind; /* VECOPS_VALUE_TENSOR or VECOPS_VALUE_SCALAR */
  const char* name;
  union {
    VecopsTensorParameter tensor;
    VecopsScalarParameter scalar;
  } constraint;
} VecopsParameterDescriptor;

typedef int32_t (*VecopsWorkspaceFn)(const VecopsCall*, uint64_t*, VecopsError*);
typedef int32_t (*VecopsRunFn)(const VecopsCall*, VecopsError*);

typedef struct VecopsKernelDescriptorV1 {
  uint32_t struct_size;
  uint16_t abi_version_major;
  uint16_t abi_version_minor;
  const char* operator_name;
  const char* specialization_key;
  uint32_t num_parameters;
  uint32_t parameter_stride;
  const VecopsParameterDescriptor* parameters;
  VecopsWorkspaceFn workspace; /* may be NULL when no scratch is ever needed */
  VecopsRunFn run;             /* required */
  uint64_t flags;              /* must be zero in v1 */
} VecopsKernelDescriptorV1;

typedef const VecopsKernelDescriptorV1* (*VecopsKernelQueryFnV1)(void);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* VECOPS_RUNTIME_KERNEL_ABI_H */
#endif /* VECOPS_B200_KERNEL_ABI_H */
