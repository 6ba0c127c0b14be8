/*
 * C door to the matmul Operator, for embeddings that cannot include C++.
 *
 * vecops_operator_bridge_invoke_v1 has the signature and meaning of vecops'
 * process-local bridge (include/vecops/runtime/OperatorBridgeAbi.h:23-158): a
 * generated framework adapter hands over a positional VecopsCall plus named
 * specialization values, and the runtime validates, resolves and runs.  The
 * handle comes from vecops_b200_matmul_operator() instead of a Python-owned
 * registry.
 */
#ifndef VECOPS_B200_OPERATOR_BRIDGE_H
#define VECOPS_B200_OPERATOR_BRIDGE_H

#include "vecops_b200/kernel_abi.h"

#ifdef __cplusplus
extern "C" {
#endif

#ifndef VECOPS_RUNTIME_OPERATOR_BRIDGE_ABI_H
typedef enum VecopsSpecializationValueKind {
  VECOPS_SPECIALIZATION_CONST_INT = 1,
  VECOPS_SPECIALIZATION_DTYPE = 2
} VecopsSpecializationValueKind;

typedef struct VecopsSpecializationArgument {
  uint32_t struct_size;
  uint32_t kind;
  const char* name;
  union {
    int64_t integer;
    uint32_t dtype;
  } value;
} VecopsSpecializationArgument;
#endif

/* Handle of the process-wide CUDA matmul operator (created on first use). */
VECOPS_B200_EXPORT uint64_t vecops_b200_matmul_operator(void);

/* Handle of a process-wide operand-preparation operator: vecops::matmul_pack, values = {src, dst} (compensated == 0),
 * or vecops::matmul_pack_b_compensated, values = {src, dst, compensation, a_zero_point}; dst a tensor over
 * vecops_b200_matmul_packed_layout's layout (ops/MatmulPack.h:93-131, :28-35). */
VECOPS_B200_EXPORT uint64_t vecops_b200_matmul_pack_operator(int32_t compensated);

/* Handles of the operators either side of the matmul path (0 for an unknown `which`):
 *   0  vecops::matmul_batched                values = {a[B,M,K], b[B,N,K], c[B,M,N][, column_scale[N]]}; an operand every entry
 *                                            shares comes as a view with batch stride 0 (tests/ops/MatmulBatchTest.cpp:96-131)
 *   1  vecops::scaled_dot_product_attention  values = {q[H,Lq,D], k[H,Lkv,D], v[H,Lkv,Dv], out[H,Lq,Dv], scale, causal[, key_mask[Lkv]
 *                                            [, bias[H,Lq,Lkv]]]}; scratch of vecops_b200_operator_workspace bytes in the frame
 *                                            (ops/details/attention/SDPA.h:72-84)
 *   2  vecops::quantize_rows_per_row         values = {src[M,K], multipliers[M], dst[M,K][, zero_point]} (matmul/Quantization.h:76-140) */
VECOPS_B200_EXPORT uint64_t vecops_b200_caller_operator(uint32_t which);

/* Validate, resolve and run one call: values = {a, b, c[, column_scale]}.
 * Replaces vecops_operator_bridge_invoke_v1 (OperatorBridgeAbi.h:156-158). */
VECOPS_B200_EXPORT int32_t vecops_operator_bridge_invoke_v1(uint64_t handle, const VecopsCall* call,
                                                            uint32_t num_specialization_values,
                                                            const VecopsSpecializationArgument* specialization_values,
                                                            VecopsError* error);

/* Resolve only: which specialization key would serve this call.  The key is
 * written NUL-terminated (truncated to `capacity`) into `key`. */
VECOPS_B200_EXPORT int32_t vecops_b200_operator_resolve(uint64_t handle, const VecopsCall* call, char* key,
                                                        size_t capacity, VecopsError* error);

/* Device scratch in bytes the resolved executable wants for this call. */
VECOPS_B200_EXPORT int32_t vecops_b200_operator_workspace(uint64_t handle, const VecopsCall* call, uint64_t* bytes,
                                                          VecopsError* error);

/* How often vecops_operator_bridge_invoke_v1 took its two paths since the library was loaded (all threads): the full one -
 * bind, validate, dispatch, resolve, then run - and the prepared one, which re-enters an executable a previous call with
 * the same signature resolved (same operator, value kinds, tensor dtypes, devices, flags, ranks, sizes, strides and
 * address alignment; data addresses and scalar payloads are free).  Each thread keeps its last eight signatures, as
 * vecops' own framework bridge does (docs/Runtime.md:195-206).  VECOPS_B200_PREPARED_CALL=0 in the environment before the
 * first call turns the prepared path off.  Either pointer may be NULL. */
VECOPS_B200_EXPORT void vecops_b200_bridge_counters(uint64_t* slow_calls, uint64_t* prepared_calls);

/* Descriptor template of one kernel variant (VecopsB200MatmulKernel id): what
 * a one-specialization artifact's vecops_kernel_query_v1 would return, with an
 * empty specialization key.  NULL for AUTO or an id out of range. */
VECOPS_B200_EXPORT const VecopsKernelDescriptorV1* vecops_b200_matmul_descriptor(uint32_t kernel);

#ifdef __cplusplus
}
#endif

#endif /* VECOPS_B200_OPERATOR_BRIDGE_H */
