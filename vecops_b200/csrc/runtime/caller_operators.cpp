// The callers and data formats on either side of the matmul path, as operators of the runtime layer: rank-3 (batched)
// matmul, scaled dot-product attention, and the per-row quantiser of the activations.  The reference reaches all three
// through its operator layer (leading batch dimensions on ops::Matmul's operands, tests/ops/MatmulBatchTest.cpp:96-131;
// ops::scaled_dot_product_attention, include/vecops/ops/details/attention/SDPA.h:72-84; the per-row quantising transform,
// include/vecops/matmul/Quantization.h:76-140); here each is one KernelDef, one recipe over the prebuilt CUDA entry point
// and one in-process descriptor, assembled into an Operator the bridge can be handed like the matmul operator.
//
//   vecops::matmul_batched                  a[B,M,K] TA, b[B,N,K] TB, c[B,M,N] TC, column_scale[N] f32 (optional)
//                                           (an operand every entry shares comes as a view with batch stride 0)
//   vecops::scaled_dot_product_attention    q[H,Lq,D] bf16, k[H,Lkv,D] bf16, v[H,Lkv,Dv] bf16, out[H,Lq,Dv] TO, scale f32,
//                                           causal i32 (0 none, 1 top left, 2 bottom right), key_mask[Lkv] u8 (optional),
//                                           bias[H,Lq,Lkv] f32 (optional); scratch through the call's workspace
//   vecops::quantize_rows_per_row           src[M,K] f32|bf16, multipliers[M] f32, dst[M,K] u8|i8, zero_point f32
#include <array>
#include <cstddef>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "vecops_b200/matmul_cuda.h"
#include "vecops_b200/operator_bridge.h"
#include "vecops_b200/runtime/matmul_operator.h"

namespace vecops::runtime {
namespace {

struct ErrorText {
  std::array<char, 1024> text{};
  VecopsError record{};
  ErrorText() {
    record.struct_size = sizeof(VecopsError);
    record.message = text.data();
    record.message_capacity = text.size();
  }
};

std::int32_t fail(VecopsError* error, std::int32_t code, const char* message) {
  if (error != nullptr && error->struct_size >= sizeof(VecopsError)) {
    error->code = code;
    error->message_required = std::strlen(message) + 1;
    if (error->message != nullptr && error->message_capacity > 0) {
      std::strncpy(error->message, message, error->message_capacity - 1);
      error->message[error->message_capacity - 1] = '\0';
    }
  }
  return code;
}

constexpr std::uint64_t bit(std::uint32_t dtype) { return std::uint64_t{1} << (dtype - 1); }
constexpr VecopsDimensionConstraint any_dim() { return {sizeof(VecopsDimensionConstraint), VECOPS_DIM_ANY, 0, 0, 0, 1}; }

VecopsParameterDescriptor scalar_parameter(const char* name, std::uint64_t dtype_mask) {
  VecopsParameterDescriptor p{};
  p.struct_size = sizeof(VecopsParameterDescriptor);
  p.kind = VECOPS_VALUE_SCALAR;
  p.name = name;
  p.constraint.scalar.struct_size = sizeof(VecopsScalarParameter);
  p.constraint.scalar.dtype_mask = dtype_mask;
  return p;
}

VecopsParameterDescriptor tensor_parameter(const char* name, std::uint64_t dtype_mask, std::int32_t rank, const VecopsDimensionConstraint* any,
                                           bool optional, bool output) {
  VecopsParameterDescriptor p{};
  p.struct_size = sizeof(VecopsParameterDescriptor);
  p.kind = VECOPS_VALUE_TENSOR;
  p.name = name;
  auto& t = p.constraint.tensor;
  t.struct_size = sizeof(VecopsTensorParameter);
  t.dtype_mask = dtype_mask;
  t.device_type = VECOPS_DEVICE_CUDA;
  t.device_index = -1;
  t.rank = rank;
  t.optional = optional ? 1u : 0u;
  t.dimension_constraint_stride = sizeof(VecopsDimensionConstraint);
  t.sizes = any;    // every extent and stride is free at this level: the entry points check what they can serve
  t.strides = any;
  t.required_flags = output ? VECOPS_TENSOR_WRITE : VECOPS_TENSOR_READ;
  return p;
}

TensorDef tensor_def(std::string name, std::vector<DimensionDef> shape, TensorDTypeDef dtype, TensorAccess access, bool optional = false) {
  TensorDef t;
  t.name = std::move(name);
  t.strides.assign(shape.size(), DimensionDef::any());
  t.shape = std::move(shape);
  t.dtype = std::move(dtype);
  t.access = access;
  t.optional = optional;
  t.device_type = VECOPS_DEVICE_CUDA;
  t.device_index = -1;
  return t;
}
DimensionDef dim(const char* name) { return DimensionDef::named_dynamic(name, 1, 0); }

// frame access
const VecopsTensorView* tensor_at(const VecopsCall* call, std::uint32_t index) {
  if (index >= call->num_values || call->values[index].kind != VECOPS_VALUE_TENSOR) return nullptr;
  return &call->values[index].value.tensor;
}
bool absent_at(const VecopsCall* call, std::uint32_t index) { return index >= call->num_values || call->values[index].kind == VECOPS_VALUE_NONE; }
void* data_of(const VecopsTensorView& t) { return static_cast<char*>(t.data) + t.byte_offset; }
void* stream_of(const VecopsCall* call) {
  const VecopsExecutionContext* context = call->context;
  if (context != nullptr && context->struct_size >= offsetof(VecopsExecutionContext, stream) + sizeof(context->stream)) return context->stream;
  return nullptr;
}
bool asynchronous(const VecopsCall* call) {
  const VecopsExecutionContext* context = call->context;
  return context != nullptr && context->struct_size >= offsetof(VecopsExecutionContext, flags) + sizeof(context->flags) &&
         (context->flags & VECOPS_B200_CONTEXT_FLAG_ASYNC) != 0;
}
bool scalar_f32(const VecopsCall* call, std::uint32_t index, float fallback, float* out) {
  *out = fallback;
  if (absent_at(call, index)) return true;
  const VecopsValue& v = call->values[index];
  if (v.kind != VECOPS_VALUE_SCALAR) return false;
  if (v.value.scalar.dtype == VECOPS_DTYPE_F32 || v.value.scalar.dtype == VECOPS_DTYPE_F64) *out = static_cast<float>(v.value.scalar.value.f64);
  else *out = static_cast<float>(v.value.scalar.value.i64);
  return true;
}
bool scalar_i32(const VecopsCall* call, std::uint32_t index, std::int32_t fallback, std::int32_t* out) {
  *out = fallback;
  if (absent_at(call, index)) return true;
  const VecopsValue& v = call->values[index];
  if (v.kind != VECOPS_VALUE_SCALAR || v.value.scalar.dtype == VECOPS_DTYPE_F32 || v.value.scalar.dtype == VECOPS_DTYPE_F64) return false;
  *out = static_cast<std::int32_t>(v.value.scalar.value.i64);
  return true;
}


// ---------------------------------------------------------------- vecops::matmul_batched

std::int32_t batched_from_frame(const VecopsCall* call, VecopsB200Matmul* problem, VecopsB200Batch* batch, VecopsError* error) {
  if (call == nullptr || call->struct_size < sizeof(VecopsCall)) return fail(error, VECOPS_STATUS_ABI_MISMATCH, "call frame is null or too small");
  if (call->num_values < 3 || call->num_values > 4 || call->values == nullptr)
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "matmul_batched expects a, b, c and optionally column_scale");
  const VecopsTensorView *a = tensor_at(call, 0), *b = tensor_at(call, 1), *c = tensor_at(call, 2), *scale = tensor_at(call, 3);
  if (a == nullptr || b == nullptr || c == nullptr || (scale == nullptr && !absent_at(call, 3)))
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "matmul_batched operands must be tensors");
  if (a->rank != 3 || b->rank != 3 || c->rank != 3 || (scale != nullptr && scale->rank != 1))
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "matmul_batched wants rank-3 a, b, c and a rank-1 column_scale");
  const std::int64_t count = c->sizes[0];
  VecopsB200Matmul p{};
  p.struct_size = sizeof(VecopsB200Matmul);
  p.kernel = VECOPS_B200_KERNEL_AUTO;
  p.m = a->sizes[1], p.k = a->sizes[2], p.n = b->sizes[1];
  if (a->sizes[0] != count || b->sizes[0] != count || b->sizes[2] != p.k || c->sizes[1] != p.m || c->sizes[2] != p.n ||
      (scale != nullptr && scale->sizes[0] != p.n))
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "matmul_batched extents disagree: a[B,M,K] b[B,N,K] c[B,M,N] column_scale[N]");
  p.a = data_of(*a), p.a_stride_m = a->strides[1], p.a_stride_k = a->strides[2];
  p.b = data_of(*b), p.b_stride_n = b->strides[1], p.b_stride_k = b->strides[2];
  p.c = data_of(*c), p.c_stride_m = c->strides[1], p.c_stride_n = c->strides[2];
  if (scale != nullptr) {
    if (scale->strides[0] != 1 && p.n > 1) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "column_scale must be contiguous");
    p.column_scale = static_cast<const float*>(data_of(*scale));
  }
  p.a_dtype = a->dtype, p.b_dtype = b->dtype, p.c_dtype = c->dtype;
  p.device_index = c->device_index;
  p.workspace = call->workspace, p.workspace_size = call->workspace_size;
  p.stream = stream_of(call);
  if (asynchronous(call)) p.flags |= VECOPS_B200_MATMUL_FLAG_ASYNC;
  VecopsB200Batch q{};
  q.struct_size = sizeof(VecopsB200Batch);
  q.count = count;
  q.a_stride_b = a->strides[0], q.b_stride_b = b->strides[0], q.c_stride_b = c->strides[0];
  *problem = p;
  *batch = q;
  return VECOPS_STATUS_OK;
}

std::int32_t run_batched(const VecopsCall* call, VecopsError* error) {
  VecopsB200Matmul problem;
  VecopsB200Batch batch;
  if (const auto rc = batched_from_frame(call, &problem, &batch, error); rc != VECOPS_STATUS_OK) return rc;
  return vecops_b200_matmul_run_batched(&problem, &batch, nullptr, error);
}

std::int32_t workspace_batched(const VecopsCall* call, std::uint64_t* bytes, VecopsError* error) {
  VecopsB200Matmul problem;
  VecopsB200Batch batch;
  if (const auto rc = batched_from_frame(call, &problem, &batch, error); rc != VECOPS_STATUS_OK) return rc;
  // what covers both ways the batch may run: the problem with its rows stacked (matmul_cuda.h, VecopsB200Batch).  The
  // kernels that would use it run without it too, so it is what the call can use, reported as what it needs
  problem.m *= batch.count > 0 ? batch.count : 1;
  return vecops_b200_matmul_workspace(&problem, bytes, error);
}

// ---------------------------------------------------------------- vecops::scaled_dot_product_attention

std::int32_t attention_from_frame(const VecopsCall* call, VecopsB200Attention* out, VecopsError* error) {
  if (call == nullptr || call->struct_size < sizeof(VecopsCall)) return fail(error, VECOPS_STATUS_ABI_MISMATCH, "call frame is null or too small");
  if (call->num_values < 5 || call->num_values > 8 || call->values == nullptr)
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "attention expects q, k, v, out, scale and optionally causal, key_mask, bias");
  const VecopsTensorView *q = tensor_at(call, 0), *k = tensor_at(call, 1), *v = tensor_at(call, 2), *o = tensor_at(call, 3);
  const VecopsTensorView *key_mask = tensor_at(call, 6), *bias = tensor_at(call, 7);
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || (key_mask == nullptr && !absent_at(call, 6)) || (bias == nullptr && !absent_at(call, 7)))
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "attention operands must be tensors");
  if (q->rank != 3 || k->rank != 3 || v->rank != 3 || o->rank != 3 || (key_mask != nullptr && key_mask->rank != 1) || (bias != nullptr && bias->rank != 3))
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "attention wants rank-3 q, k, v, out and bias, and a rank-1 key_mask");
  float scale = 1.f;
  std::int32_t causal = 0;
  if (absent_at(call, 4) || !scalar_f32(call, 4, 1.f, &scale)) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "scale is an f32 scalar");
  if (!scalar_i32(call, 5, 0, &causal) || causal < 0 || causal > 2) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "causal is the i32 0, 1 or 2");
  VecopsB200Attention a{};
  a.struct_size = sizeof(VecopsB200Attention);
  a.causal = static_cast<std::uint32_t>(causal);
  a.heads = o->sizes[0];
  a.lq = q->sizes[1], a.dqk = q->sizes[2], a.lkv = k->sizes[1], a.dv = v->sizes[2];
  if (q->sizes[0] != a.heads || k->sizes[0] != a.heads || v->sizes[0] != a.heads || k->sizes[2] != a.dqk || v->sizes[1] != a.lkv ||
      o->sizes[1] != a.lq || o->sizes[2] != a.dv || (key_mask != nullptr && key_mask->sizes[0] != a.lkv) ||
      (bias != nullptr && (bias->sizes[0] != a.heads || bias->sizes[1] != a.lq || bias->sizes[2] != a.lkv)))
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "attention extents disagree: q[H,Lq,D] k[H,Lkv,D] v[H,Lkv,Dv] out[H,Lq,Dv] key_mask[Lkv] bias[H,Lq,Lkv]");
  a.q = data_of(*q), a.q_stride_head = q->strides[0], a.q_stride_row = q->strides[1], a.q_stride_col = q->strides[2];
  a.k = data_of(*k), a.k_stride_head = k->strides[0], a.k_stride_row = k->strides[1], a.k_stride_col = k->strides[2];
  a.v = data_of(*v), a.v_stride_head = v->strides[0], a.v_stride_row = v->strides[1], a.v_stride_col = v->strides[2];
  a.out = data_of(*o), a.out_stride_head = o->strides[0], a.out_stride_row = o->strides[1], a.out_stride_col = o->strides[2];
  a.qkv_dtype = q->dtype, a.out_dtype = o->dtype;
  if (k->dtype != q->dtype || v->dtype != q->dtype) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "q, k and v share one element type");
  if (key_mask != nullptr) {
    if (key_mask->strides[0] != 1 && a.lkv > 1) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "key_mask must be contiguous");
    a.key_mask = static_cast<const std::uint8_t*>(data_of(*key_mask));
  }
  if (bias != nullptr) {
    a.bias = static_cast<const float*>(data_of(*bias));
    a.bias_stride_head = bias->strides[0], a.bias_stride_row = bias->strides[1], a.bias_stride_col = bias->strides[2];
  }
  a.scale = scale;
  a.flags = asynchronous(call) ? VECOPS_B200_MATMUL_FLAG_ASYNC : 0;
  // scratch: the run wants it 256-byte aligned; what the frame brings is used from its first aligned byte on
  const auto address = reinterpret_cast<std::uintptr_t>(call->workspace);
  const std::uintptr_t skip = call->workspace == nullptr ? 0 : (256 - address % 256) % 256;
  a.workspace = call->workspace == nullptr || call->workspace_size <= skip ? nullptr : static_cast<char*>(call->workspace) + skip;
  a.workspace_size = a.workspace == nullptr ? 0 : call->workspace_size - skip;
  a.stream = stream_of(call);
  a.device_index = o->device_index;
  *out = a;
  return VECOPS_STATUS_OK;
}

std::int32_t run_attention(const VecopsCall* call, VecopsError* error) {
  VecopsB200Attention attention;
  if (const auto rc = attention_from_frame(call, &attention, error); rc != VECOPS_STATUS_OK) return rc;
  return vecops_b200_sdpa_run(&attention, error);
}

std::int32_t workspace_attention(const VecopsCall* call, std::uint64_t* bytes, VecopsError* error) {
  VecopsB200Attention attention;
  if (const auto rc = attention_from_frame(call, &attention, error); rc != VECOPS_STATUS_OK) return rc;
  attention.workspace = nullptr, attention.workspace_size = 0;
  const auto rc = vecops_b200_sdpa_workspace(&attention, bytes, error);
  if (rc == VECOPS_STATUS_OK && *bytes != 0) *bytes += 256;  // room to align inside whatever the caller allocates
  return rc;
}

// ---------------------------------------------------------------- vecops::quantize_rows_per_row

std::int32_t run_quantize(const VecopsCall* call, VecopsError* error) {
  if (call == nullptr || call->struct_size < sizeof(VecopsCall)) return fail(error, VECOPS_STATUS_ABI_MISMATCH, "call frame is null or too small");
  if (call->num_values < 3 || call->num_values > 4 || call->values == nullptr)
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "quantize_rows_per_row expects src, multipliers, dst and optionally zero_point");
  const VecopsTensorView *src = tensor_at(call, 0), *multipliers = tensor_at(call, 1), *dst = tensor_at(call, 2);
  float zero_point = 0.f;
  if (src == nullptr || multipliers == nullptr || dst == nullptr || !scalar_f32(call, 3, 0.f, &zero_point))
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "quantize_rows_per_row takes three tensors and an f32 scalar");
  if (src->rank != 2 || dst->rank != 2 || multipliers->rank != 1 || dst->sizes[0] != src->sizes[0] || dst->sizes[1] != src->sizes[1] ||
      multipliers->sizes[0] != src->sizes[0] || (multipliers->strides[0] != 1 && src->sizes[0] > 1) || (dst->strides[1] != 1 && dst->sizes[1] > 1))
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "quantize_rows_per_row wants src[M,K], contiguous multipliers[M] and a K-contiguous dst[M,K]");
  const auto rc = vecops_b200_quantize_rows_per_row(data_of(*src), src->dtype, src->strides[0], src->strides[1], data_of(*dst), dst->dtype,
                                                    dst->strides[0], src->sizes[0], src->sizes[1], static_cast<const float*>(data_of(*multipliers)),
                                                    zero_point, stream_of(call), error);
  if (rc != VECOPS_STATUS_OK || asynchronous(call)) return rc;
  return vecops_b200_stream_synchronize(stream_of(call), error);
}

std::int32_t workspace_none(const VecopsCall*, std::uint64_t* bytes, VecopsError*) {
  if (bytes != nullptr) *bytes = 0;
  return VECOPS_STATUS_OK;
}


// ---------------------------------------------------------------- one recipe, one descriptor, one provider per operator

struct CallerDescriptor {
  VecopsDimensionConstraint any[4];
  VecopsParameterDescriptor parameters[8];
  VecopsKernelDescriptorV1 descriptor;
};

struct CallerSpec {
  const char* operator_name;
  const char* recipe_id;
  KernelDef (*definition)();
  const CallerDescriptor* (*descriptor)();
  // the frame as the entry point will read it: NOT_APPLICABLE / INVALID_ARGUMENT with its reason, before anything is launched
  std::int32_t (*check)(const VecopsCall* call, VecopsError* error);
};

CallerDescriptor* new_descriptor(const char* operator_name, std::uint32_t parameters, VecopsWorkspaceFn workspace, VecopsRunFn run) {
  auto* v = new CallerDescriptor{};  // lives for the life of the process, like a DSO's static descriptor
  for (auto& d : v->any) d = any_dim();
  auto& d = v->descriptor;
  d.struct_size = sizeof(VecopsKernelDescriptorV1);
  d.abi_version_major = VECOPS_KERNEL_ABI_VERSION_MAJOR;
  d.abi_version_minor = VECOPS_KERNEL_ABI_VERSION_MINOR;
  d.operator_name = operator_name;
  d.specialization_key = "";
  d.num_parameters = parameters;
  d.parameter_stride = sizeof(VecopsParameterDescriptor);
  d.parameters = v->parameters;
  d.workspace = workspace;
  d.run = run;
  d.flags = 0;
  return v;
}

constexpr std::uint64_t kFloats = bit(VECOPS_DTYPE_F32) | bit(VECOPS_DTYPE_BF16) | bit(VECOPS_DTYPE_F16);
constexpr std::uint64_t kBytes = bit(VECOPS_DTYPE_I8) | bit(VECOPS_DTYPE_U8);

const CallerDescriptor* batched_descriptor() {
  static const CallerDescriptor* const built = [] {
    auto* v = new_descriptor("vecops::matmul_batched", 4, &workspace_batched, &run_batched);
    v->parameters[0] = tensor_parameter("a", kFloats | kBytes, 3, v->any, false, false);
    v->parameters[1] = tensor_parameter("b", kFloats | kBytes, 3, v->any, false, false);
    v->parameters[2] = tensor_parameter("c", kFloats | bit(VECOPS_DTYPE_I32), 3, v->any, false, true);
    v->parameters[3] = tensor_parameter("column_scale", bit(VECOPS_DTYPE_F32), 1, v->any, true, false);
    return v;
  }();
  return built;
}

const CallerDescriptor* attention_descriptor() {
  static const CallerDescriptor* const built = [] {
    auto* v = new_descriptor("vecops::scaled_dot_product_attention", 8, &workspace_attention, &run_attention);
    v->parameters[0] = tensor_parameter("q", bit(VECOPS_DTYPE_BF16), 3, v->any, false, false);
    v->parameters[1] = tensor_parameter("k", bit(VECOPS_DTYPE_BF16), 3, v->any, false, false);
    v->parameters[2] = tensor_parameter("v", bit(VECOPS_DTYPE_BF16), 3, v->any, false, false);
    v->parameters[3] = tensor_parameter("out", bit(VECOPS_DTYPE_F32) | bit(VECOPS_DTYPE_BF16), 3, v->any, false, true);
    v->parameters[4] = scalar_parameter("scale", bit(VECOPS_DTYPE_F32));
    v->parameters[5] = scalar_parameter("causal", bit(VECOPS_DTYPE_I32));
    v->parameters[6] = tensor_parameter("key_mask", bit(VECOPS_DTYPE_U8), 1, v->any, true, false);
    v->parameters[7] = tensor_parameter("bias", bit(VECOPS_DTYPE_F32), 3, v->any, true, false);
    return v;
  }();
  return built;
}

const CallerDescriptor* quantize_descriptor() {
  static const CallerDescriptor* const built = [] {
    auto* v = new_descriptor("vecops::quantize_rows_per_row", 4, &workspace_none, &run_quantize);
    v->parameters[0] = tensor_parameter("src", bit(VECOPS_DTYPE_F32) | bit(VECOPS_DTYPE_BF16), 2, v->any, false, false);
    v->parameters[1] = tensor_parameter("multipliers", bit(VECOPS_DTYPE_F32), 1, v->any, false, false);
    v->parameters[2] = tensor_parameter("dst", kBytes, 2, v->any, false, true);
    v->parameters[3] = scalar_parameter("zero_point", bit(VECOPS_DTYPE_F32));
    return v;
  }();
  return built;
}

std::int32_t check_batched(const VecopsCall* call, VecopsError* error) {
  VecopsB200Matmul problem;
  VecopsB200Batch batch;
  if (const auto rc = batched_from_frame(call, &problem, &batch, error); rc != VECOPS_STATUS_OK) return rc;
  std::uint32_t kernel = 0;
  return vecops_b200_matmul_select(&problem, &kernel, error);  // the dtype row must be one the matmul serves
}
std::int32_t check_attention(const VecopsCall* call, VecopsError* error) {
  VecopsB200Attention attention;
  if (const auto rc = attention_from_frame(call, &attention, error); rc != VECOPS_STATUS_OK) return rc;
  std::uint32_t strategy = 0, tiles = 0;
  return vecops_b200_sdpa_plan(&attention, &strategy, &tiles, error);
}
std::int32_t check_quantize(const VecopsCall* call, VecopsError* error) {
  if (call == nullptr || call->num_values < 3 || tensor_at(call, 0) == nullptr || tensor_at(call, 1) == nullptr || tensor_at(call, 2) == nullptr)
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "quantize_rows_per_row takes three tensors and an f32 scalar");
  return VECOPS_STATUS_OK;
}

KernelDef batched_kernel_def() {
  return KernelDef("vecops::matmul_batched",
                   {tensor_def("a", {dim("B"), dim("M"), dim("K")}, "TA", TensorAccess::Input),
                    tensor_def("b", {dim("B"), dim("N"), dim("K")}, "TB", TensorAccess::Input),
                    tensor_def("c", {dim("B"), dim("M"), dim("N")}, "TC", TensorAccess::Output),
                    tensor_def("column_scale", {dim("N")}, DType::Float32, TensorAccess::Input, true)},
                   {{"TA", SpecializationType::DType}, {"TB", SpecializationType::DType}, {"TC", SpecializationType::DType}});
}
KernelDef attention_kernel_def() {
  return KernelDef("vecops::scaled_dot_product_attention",
                   {tensor_def("q", {dim("H"), dim("Lq"), dim("D")}, DType::BFloat16, TensorAccess::Input),
                    tensor_def("k", {dim("H"), dim("Lkv"), dim("D")}, DType::BFloat16, TensorAccess::Input),
                    tensor_def("v", {dim("H"), dim("Lkv"), dim("Dv")}, DType::BFloat16, TensorAccess::Input),
                    tensor_def("out", {dim("H"), dim("Lq"), dim("Dv")}, "TO", TensorAccess::Output),
                    ValueDef{"scale", DType::Float32, Scalar::floating(1.0, DType::Float32)},
                    ValueDef{"causal", DType::Int32, Scalar::signed_integer(0, DType::Int32)},
                    tensor_def("key_mask", {dim("Lkv")}, DType::UInt8, TensorAccess::Input, true),
                    tensor_def("bias", {dim("H"), dim("Lq"), dim("Lkv")}, DType::Float32, TensorAccess::Input, true)},
                   {{"TO", SpecializationType::DType}});
}
KernelDef quantize_kernel_def() {
  return KernelDef("vecops::quantize_rows_per_row",
                   {tensor_def("src", {dim("M"), dim("K")}, "TS", TensorAccess::Input),
                    tensor_def("multipliers", {dim("M")}, DType::Float32, TensorAccess::Input),
                    tensor_def("dst", {dim("M"), dim("K")}, "TD", TensorAccess::Output),
                    ValueDef{"zero_point", DType::Float32, Scalar::floating(0.0, DType::Float32)}},
                   {{"TS", SpecializationType::DType}, {"TD", SpecializationType::DType}});
}

constexpr CallerSpec kSpecs[3] = {
    {"vecops::matmul_batched", "cuda/sm_100a/matmul_batched", &batched_kernel_def, &batched_descriptor, &check_batched},
    {"vecops::scaled_dot_product_attention", "cuda/sm_100a/sdpa", &attention_kernel_def, &attention_descriptor, &check_attention},
    {"vecops::quantize_rows_per_row", "cuda/sm_100a/quantize_rows_per_row", &quantize_kernel_def, &quantize_descriptor, &check_quantize},
};

class CallerRecipe final : public KernelRecipe {
public:
  explicit CallerRecipe(const CallerSpec& spec) : spec_(spec), definition_(std::make_shared<const KernelDef>(spec.definition())) {}
  [[nodiscard]] std::string_view id() const override { return spec_.recipe_id; }
  [[nodiscard]] Status match(const KernelCall& call) const override {
    ArgumentMetadata arguments(std::vector<Value>(call.arguments().values().begin(), call.arguments().values().end()));
    CallFrame frame(arguments);
    ErrorText error;
    if (const auto rc = spec_.check(&frame.abi(), &error.record); rc != VECOPS_STATUS_OK) return Status(StatusCode::NotApplicable, error.text.data());
    return Status::success();
  }
  [[nodiscard]] Result<BoundKernelRecipe> bind(const KernelCall& call) const override {
    auto binding = bind_kernel_call(*definition_, call);
    if (!binding) return binding.status();
    BoundKernelRecipe bound;
    bound.recipe_id = std::string(id());
    bound.specialization_key = binding.value().specialization_key;
    bound.artifact_key = std::string(id());
    return bound;
  }

private:
  const CallerSpec& spec_;
  std::shared_ptr<const KernelDef> definition_;
};

struct OwnedCallerDescriptor {
  std::string key;
  VecopsKernelDescriptorV1 descriptor;
};

class CallerProvider final : public ExecutableProvider {
public:
  explicit CallerProvider(const CallerSpec& spec) : spec_(spec) {}
  [[nodiscard]] Result<std::shared_ptr<Executable>> resolve(const BoundKernelRecipe& recipe) override {
    std::lock_guard<std::mutex> lock(mutex_);
    if (auto found = cache_.find(recipe.specialization_key); found != cache_.end()) return found->second;
    if (recipe.artifact_key != spec_.recipe_id) return Status(StatusCode::NotFound, "artifact '" + recipe.artifact_key + "' is not a prebuilt kernel of this operator");
    auto owned = std::make_shared<OwnedCallerDescriptor>();
    owned->key = recipe.specialization_key;
    owned->descriptor = spec_.descriptor()->descriptor;
    owned->descriptor.specialization_key = owned->key.c_str();
    auto module = LoadedModule::adopt(&owned->descriptor, owned);
    if (!module) return module.status();
    return cache_.emplace(recipe.specialization_key, std::make_shared<Executable>(std::move(module).value())).first->second;
  }

private:
  const CallerSpec& spec_;
  std::mutex mutex_;
  std::map<std::string, std::shared_ptr<Executable>, std::less<>> cache_;
};

std::shared_ptr<Operator> make_caller(const CallerSpec& spec) {
  std::vector<std::shared_ptr<const KernelRecipe>> recipes{std::make_shared<CallerRecipe>(spec)};
  return std::make_shared<Operator>(spec.definition(), std::move(recipes), std::make_shared<OrderedDispatchPolicy>(), std::make_shared<CallerProvider>(spec));
}

}  // namespace

std::shared_ptr<Operator> make_matmul_batched_operator() { return make_caller(kSpecs[0]); }
std::shared_ptr<Operator> make_attention_operator() { return make_caller(kSpecs[1]); }
std::shared_ptr<Operator> make_quantize_rows_per_row_operator() { return make_caller(kSpecs[2]); }

const Operator* caller_operator_of(std::uint64_t handle) {
  static const std::shared_ptr<Operator> operators[3] = {make_matmul_batched_operator(), make_attention_operator(), make_quantize_rows_per_row_operator()};
  const std::uint64_t index = handle - kCallerHandleBase;
  return index < 3 ? operators[index].get() : nullptr;
}

const KernelDef* caller_kernel_def_of(std::uint64_t handle) {
  static const KernelDef definitions[3] = {batched_kernel_def(), attention_kernel_def(), quantize_kernel_def()};
  const std::uint64_t index = handle - kCallerHandleBase;
  return index < 3 ? &definitions[index] : nullptr;
}

}  // namespace vecops::runtime

extern "C" uint64_t vecops_b200_caller_operator(uint32_t which) {
  if (which >= 3) return 0;
  (void)vecops::runtime::caller_operator_of(vecops::runtime::kCallerHandleBase + which);
  return vecops::runtime::kCallerHandleBase + which;
}
