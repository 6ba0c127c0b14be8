// CUDA matmul operator: KernelDef, recipes, dispatch policy, provider,
// descriptors and the C bridge.
#include "vecops_b200/runtime/matmul_operator.h"

#include <array>
#include <atomic>
#include <cstdlib>
#include <string>
#include <cstddef>
#include <cstring>

#include "vecops_b200/operator_bridge.h"

namespace vecops::runtime {
namespace {

constexpr const char* kOperatorName = "vecops::matmul";
constexpr std::uint32_t kVariants[] = {VECOPS_B200_KERNEL_BF16_TCGEN05, VECOPS_B200_KERNEL_I8_TCGEN05,
                                       VECOPS_B200_KERNEL_W8_SMALL_M,   VECOPS_B200_KERNEL_W8_TCGEN05,
                                       VECOPS_B200_KERNEL_F32_TF32X3,   VECOPS_B200_KERNEL_F32_SIMT,
                                       VECOPS_B200_KERNEL_GENERIC};

struct ErrorText {
  std::array<char, 1024> text{};
  VecopsError record{};
  ErrorText() {
    record.struct_size = sizeof(VecopsError);
    record.message = text.data();
    record.message_capacity = text.size();
  }
  [[nodiscard]] Status status(std::int32_t rc) const {
    if (rc == VECOPS_STATUS_OK) return Status::success();
    return Status(static_cast<StatusCode>(rc), text.data());
  }
};

std::shared_ptr<const KernelDef> shared_definition() {
  static const auto definition = std::make_shared<const KernelDef>(matmul_kernel_def());
  return definition;
}

// ---------------------------------------------------------------- descriptors

constexpr std::uint64_t bit(std::uint32_t dtype) { return std::uint64_t{1} << (dtype - 1); }
constexpr VecopsDimensionConstraint any_dim() { return {sizeof(VecopsDimensionConstraint), VECOPS_DIM_ANY, 0, 0, 0, 1}; }
constexpr VecopsDimensionConstraint const_dim(std::int64_t v) { return {sizeof(VecopsDimensionConstraint), VECOPS_DIM_CONST, v, 0, 0, 1}; }
constexpr VecopsDimensionConstraint aligned_dim(std::int64_t alignment) {
  return {sizeof(VecopsDimensionConstraint), VECOPS_DIM_DYNAMIC, 0, 0, INT64_MAX, alignment};
}

// Parameters of every matmul specialization: a, b, c, column_scale?, cin?, alpha, activation, clamp_lo, clamp_hi, row_scale?.
constexpr std::uint32_t kMatmulParameters = 10;

struct VariantDescriptor {
  VecopsDimensionConstraint a_sizes[2], a_strides[2], b_sizes[2], b_strides[2], c_sizes[2], c_strides[2], s_sizes[1], s_strides[1],
      cin_sizes[2], cin_strides[2], r_sizes[1], r_strides[1];
  VecopsParameterDescriptor parameters[kMatmulParameters];
  VecopsKernelDescriptorV1 descriptor;
};

VecopsParameterDescriptor scalar_parameter(const char* name, std::uint64_t dtype_mask) {
  VecopsParameterDescriptor p{};
  p.struct_size = sizeof(VecopsParameterDescriptor);
  p.kind = VECOPS_VALUE_SCALAR;
  p.name = name;
  p.constraint.scalar.struct_size = sizeof(VecopsScalarParameter);
  p.constraint.scalar.dtype_mask = dtype_mask;
  return p;
}

VecopsParameterDescriptor tensor_parameter(const char* name, std::uint64_t dtype_mask, std::int32_t rank,
                                           const VecopsDimensionConstraint* sizes, const VecopsDimensionConstraint* strides,
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
  t.sizes = sizes;
  t.strides = strides;
  t.required_flags = output ? VECOPS_TENSOR_WRITE : VECOPS_TENSOR_READ;
  return p;
}

std::int32_t run_with(std::uint32_t kernel, const VecopsCall* call, VecopsError* error, bool only_workspace, std::uint64_t* bytes);

template <std::uint32_t kKernel>
std::int32_t run_variant(const VecopsCall* call, VecopsError* error) {
  return run_with(kKernel, call, error, false, nullptr);
}
template <std::uint32_t kKernel>
std::int32_t workspace_variant(const VecopsCall* call, std::uint64_t* bytes, VecopsError* error) {
  return run_with(kKernel, call, error, true, bytes);
}

template <std::uint32_t kKernel>
VariantDescriptor* build_variant(std::uint64_t a_mask, std::uint64_t b_mask, std::uint64_t c_mask, std::int64_t a_pitch_align,
                                 std::int64_t b_pitch_align, std::int64_t k_align, bool contiguous_k, bool row_major_c) {
  auto* v = new VariantDescriptor{};  // lives for the life of the process, like a DSO's static descriptor
  v->a_sizes[0] = any_dim();
  v->a_sizes[1] = k_align > 1 ? aligned_dim(k_align) : any_dim();
  v->b_sizes[0] = any_dim();
  v->b_sizes[1] = v->a_sizes[1];
  v->c_sizes[0] = v->c_sizes[1] = any_dim();
  v->a_strides[0] = a_pitch_align > 1 ? aligned_dim(a_pitch_align) : any_dim();
  v->b_strides[0] = b_pitch_align > 1 ? aligned_dim(b_pitch_align) : any_dim();
  v->a_strides[1] = v->b_strides[1] = contiguous_k ? const_dim(1) : any_dim();
  v->c_strides[0] = any_dim();
  v->c_strides[1] = row_major_c ? const_dim(1) : any_dim();
  v->s_sizes[0] = any_dim();
  v->s_strides[0] = const_dim(1);
  v->parameters[0] = tensor_parameter("a", a_mask, 2, v->a_sizes, v->a_strides, false, false);
  v->parameters[1] = tensor_parameter("b", b_mask, 2, v->b_sizes, v->b_strides, false, false);
  v->parameters[2] = tensor_parameter("c", c_mask, 2, v->c_sizes, v->c_strides, false, true);
  v->parameters[3] = tensor_parameter("column_scale", bit(VECOPS_DTYPE_F32), 1, v->s_sizes, v->s_strides, true, false);
  // the fused form's accumulator input (any strides, 0 included: a bias row or a column) and output transform
  v->cin_sizes[0] = v->cin_sizes[1] = any_dim();
  v->cin_strides[0] = v->cin_strides[1] = any_dim();
  v->parameters[4] = tensor_parameter("cin", bit(VECOPS_DTYPE_F32) | bit(VECOPS_DTYPE_BF16) | bit(VECOPS_DTYPE_I32), 2, v->cin_sizes,
                                      v->cin_strides, true, false);
  v->parameters[5] = scalar_parameter("alpha", bit(VECOPS_DTYPE_F32));
  v->parameters[6] = scalar_parameter("activation", bit(VECOPS_DTYPE_I32));
  v->parameters[7] = scalar_parameter("clamp_lo", bit(VECOPS_DTYPE_F32));
  v->parameters[8] = scalar_parameter("clamp_hi", bit(VECOPS_DTYPE_F32));
  // one factor per output row: the row half of vecops' row-by-column dequantisation (matmul/Quantization.h:195-246)
  v->r_sizes[0] = any_dim();
  v->r_strides[0] = const_dim(1);
  v->parameters[9] = tensor_parameter("row_scale", bit(VECOPS_DTYPE_F32), 1, v->r_sizes, v->r_strides, true, false);
  auto& d = v->descriptor;
  d.struct_size = sizeof(VecopsKernelDescriptorV1);
  d.abi_version_major = VECOPS_KERNEL_ABI_VERSION_MAJOR;
  d.abi_version_minor = VECOPS_KERNEL_ABI_VERSION_MINOR;
  d.operator_name = kOperatorName;
  d.specialization_key = "";
  d.num_parameters = kMatmulParameters;
  d.parameter_stride = sizeof(VecopsParameterDescriptor);
  d.parameters = v->parameters;
  d.workspace = &workspace_variant<kKernel>;
  d.run = &run_variant<kKernel>;
  d.flags = 0;
  return v;
}

const VariantDescriptor* variant_descriptor(std::uint32_t kernel) {
  constexpr auto f32 = bit(VECOPS_DTYPE_F32), bf16 = bit(VECOPS_DTYPE_BF16), i8 = bit(VECOPS_DTYPE_I8),
                 u8 = bit(VECOPS_DTYPE_U8), i32 = bit(VECOPS_DTYPE_I32), f16 = bit(VECOPS_DTYPE_F16);
  static const VariantDescriptor* const table[VECOPS_B200_KERNEL_COUNT_] = {
      nullptr,
      build_variant<VECOPS_B200_KERNEL_GENERIC>(f32 | bf16 | f16 | i8 | u8, f32 | bf16 | f16 | i8 | u8, f32 | bf16 | f16 | i32, 1, 1, 1, false,
                                                false),
      build_variant<VECOPS_B200_KERNEL_F32_SIMT>(f32, f32, f32, 1, 1, 1, false, true),
      // TMA wants 16-byte row pitches: 8 bf16 elements, 16 int8 elements.  The 16-bit kernel serves bf16 and fp16 pairs
      // (never mixed: the problem record's own check refuses those).
      build_variant<VECOPS_B200_KERNEL_BF16_TCGEN05>(bf16 | f16, bf16 | f16, bf16 | f16 | f32, 8, 8, 1, true, true),
      build_variant<VECOPS_B200_KERNEL_I8_TCGEN05>(i8 | u8, i8 | u8, i32 | f32 | bf16, 16, 16, 1, true, true),
      build_variant<VECOPS_B200_KERNEL_W8_SMALL_M>(bf16, i8, bf16 | f32, 8, 16, 32, true, true),
      build_variant<VECOPS_B200_KERNEL_W8_TCGEN05>(bf16, i8, bf16 | f32, 8, 16, 32, true, true),
      build_variant<VECOPS_B200_KERNEL_F32_TF32X3>(f32, f32, f32, 1, 1, 1, false, true),
  };
  return kernel < VECOPS_B200_KERNEL_COUNT_ ? table[kernel] : nullptr;
}

// ---------------------------------------------------------------- ABI frame -> problem record

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

std::int32_t problem_from_frame(const VecopsCall* call, std::uint32_t kernel, VecopsB200Matmul* out, VecopsB200Epilogue* fused,
                                VecopsError* error) {
  if (call == nullptr || call->struct_size < sizeof(VecopsCall)) return fail(error, VECOPS_STATUS_ABI_MISMATCH, "call frame is null or too small");
  // a, b, c, then - each optional from the right - column_scale, cin (absent or VECOPS_VALUE_NONE = none), the
  // scalars alpha, activation, clamp_lo, clamp_hi (absent = 1, none, 0, 0) and row_scale (absent or NONE = none)
  if (call->num_values < 3 || call->num_values > kMatmulParameters || call->values == nullptr)
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT,
                "matmul expects a, b, c and optionally column_scale, cin, alpha, activation, clamp_lo, clamp_hi, row_scale");
  const VecopsTensorView* t[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
  const VecopsTensorView* row_scale = nullptr;
  VecopsB200Epilogue e{};
  e.struct_size = sizeof(VecopsB200Epilogue);
  e.alpha = 1.f;
  for (int i = 0; i < static_cast<int>(call->num_values); ++i) {
    const VecopsValue& value = call->values[i];
    if (i < 5) {
      if (value.kind == VECOPS_VALUE_TENSOR) t[i] = &value.value.tensor;
      else if (!(i >= 3 && value.kind == VECOPS_VALUE_NONE)) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "matmul operands must be tensors");
      continue;
    }
    if (i == 9) {
      if (value.kind == VECOPS_VALUE_NONE) continue;
      if (value.kind != VECOPS_VALUE_TENSOR || value.value.tensor.rank != 1 || value.value.tensor.dtype != VECOPS_DTYPE_F32)
        return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "row_scale is a rank-1 f32 tensor");
      row_scale = &value.value.tensor;
      continue;
    }
    if (value.kind != VECOPS_VALUE_SCALAR) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "alpha, activation, clamp_lo and clamp_hi are scalars");
    const VecopsScalar& scalar = value.value.scalar;
    const bool is_f32 = scalar.dtype == VECOPS_DTYPE_F32;
    if (i == 6) {
      // (scalars travel widened: integers in i64, floating point in f64, with the dtype tag saying what they were)
      if (scalar.dtype != VECOPS_DTYPE_I32 || scalar.value.i64 < 0) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "activation is a non-negative i32");
      e.activation = static_cast<std::uint32_t>(scalar.value.i64);
    } else {
      if (!is_f32) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "alpha, clamp_lo and clamp_hi are f32");
      (i == 5 ? e.alpha : i == 7 ? e.clamp_lo : e.clamp_hi) = static_cast<float>(scalar.value.f64);
    }
  }
  if (t[0]->rank != 2 || t[1]->rank != 2 || t[2]->rank != 2 || (t[3] != nullptr && t[3]->rank != 1) || (t[4] != nullptr && t[4]->rank != 2))
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "matmul wants rank-2 a, b, c, cin and a rank-1 column_scale");
  VecopsB200Matmul p{};
  p.struct_size = sizeof(VecopsB200Matmul);
  p.kernel = kernel;
  p.m = t[0]->sizes[0];
  p.k = t[0]->sizes[1];
  p.n = t[1]->sizes[0];
  if (t[1]->sizes[1] != p.k || t[2]->sizes[0] != p.m || t[2]->sizes[1] != p.n || (t[3] != nullptr && t[3]->sizes[0] != p.n) ||
      (t[4] != nullptr && (t[4]->sizes[0] != p.m || t[4]->sizes[1] != p.n)))
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "matmul extents disagree: a[M,K] b[N,K] c[M,N] column_scale[N] cin[M,N]");
  auto base = [](const VecopsTensorView* v) { return static_cast<char*>(v->data) + v->byte_offset; };
  p.a = base(t[0]);
  p.a_stride_m = t[0]->strides[0];
  p.a_stride_k = t[0]->strides[1];
  p.b = base(t[1]);
  p.b_stride_n = t[1]->strides[0];
  p.b_stride_k = t[1]->strides[1];
  p.c = base(t[2]);
  p.c_stride_m = t[2]->strides[0];
  p.c_stride_n = t[2]->strides[1];
  if (t[3] != nullptr) {
    if (t[3]->strides[0] != 1 && p.n > 1) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "column_scale must be contiguous");
    p.column_scale = reinterpret_cast<const float*>(base(t[3]));
  }
  if (t[4] != nullptr) {
    e.cin = base(t[4]);
    e.cin_stride_m = t[4]->strides[0];
    e.cin_stride_n = t[4]->strides[1];
    e.cin_dtype = t[4]->dtype;
  }
  if (row_scale != nullptr) {
    if (row_scale->sizes[0] != p.m || (row_scale->strides[0] != 1 && p.m > 1))
      return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "row_scale must be a contiguous tensor of M factors");
    e.row_scale = reinterpret_cast<const float*>(base(row_scale));
  }
  p.a_dtype = t[0]->dtype;
  p.b_dtype = t[1]->dtype;
  p.c_dtype = t[2]->dtype;
  p.device_index = t[2]->device_index;
  p.workspace = call->workspace;
  p.workspace_size = call->workspace_size;
  if (const VecopsExecutionContext* context = call->context) {
    // append-only record: only read what the caller's struct_size covers
    if (context->struct_size >= offsetof(VecopsExecutionContext, stream) + sizeof(context->stream)) p.stream = context->stream;
    if (context->struct_size >= offsetof(VecopsExecutionContext, flags) + sizeof(context->flags) &&
        (context->flags & VECOPS_B200_CONTEXT_FLAG_ASYNC) != 0)
      p.flags |= VECOPS_B200_MATMUL_FLAG_ASYNC;
  }
  *out = p;
  if (fused != nullptr) *fused = e;
  return VECOPS_STATUS_OK;
}

bool transform_present(const VecopsB200Epilogue& e) {
  return e.cin != nullptr || e.alpha != 1.f || e.activation != VECOPS_B200_ACTIVATION_NONE || e.row_scale != nullptr;
}

std::int32_t run_with(std::uint32_t kernel, const VecopsCall* call, VecopsError* error, bool only_workspace, std::uint64_t* bytes) {
  VecopsB200Matmul problem;
  VecopsB200Epilogue fused;
  if (const auto rc = problem_from_frame(call, kernel, &problem, &fused, error); rc != VECOPS_STATUS_OK) return rc;
  if (only_workspace) return vecops_b200_matmul_workspace(&problem, bytes, error);
  return transform_present(fused) ? vecops_b200_matmul_run_fused(&problem, &fused, error) : vecops_b200_matmul_run(&problem, error);
}

}  // namespace

// ---------------------------------------------------------------- definition

KernelDef matmul_kernel_def() {
  auto tensor = [](std::string name, std::vector<DimensionDef> shape, TensorDTypeDef dtype, TensorAccess access, bool optional) {
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
  };
  auto M = [] { return DimensionDef::named_dynamic("M", 1, 0); };
  auto N = [] { return DimensionDef::named_dynamic("N", 1, 0); };
  auto K = [] { return DimensionDef::named_dynamic("K", 1, 0); };
  return KernelDef(kOperatorName,
                   {tensor("a", {M(), K()}, "TA", TensorAccess::Input, false),
                    tensor("b", {N(), K()}, "TB", TensorAccess::Input, false),
                    tensor("c", {M(), N()}, "TC", TensorAccess::Output, false),
                    tensor("column_scale", {N()}, DType::Float32, TensorAccess::Input, true),
                    // the fused form COut = activation((CIn + A.B^T) * alpha * column_scale): vecops' explicit accumulate form
                    // (ops/Matmul.h:519-570) with the output transforms its fusion tests compose, as parameters
                    tensor("cin", {M(), N()}, TensorDTypeDef(), TensorAccess::Input, true),
                    ValueDef{"alpha", DType::Float32, Scalar::floating(1.0, DType::Float32)},
                    ValueDef{"activation", DType::Int32, Scalar::signed_integer(0, DType::Int32)},
                    ValueDef{"clamp_lo", DType::Float32, Scalar::floating(0.0, DType::Float32)},
                    ValueDef{"clamp_hi", DType::Float32, Scalar::floating(0.0, DType::Float32)},
                    tensor("row_scale", {M()}, DType::Float32, TensorAccess::Input, true)},
                   {{"TA", SpecializationType::DType}, {"TB", SpecializationType::DType}, {"TC", SpecializationType::DType}});
}

Result<VecopsB200Matmul> matmul_problem_from(std::span<const Value> values, std::uint32_t kernel) {
  ArgumentMetadata arguments(std::vector<Value>(values.begin(), values.end()));
  CallFrame frame(arguments);
  VecopsB200Matmul problem;
  ErrorText error;
  if (const auto rc = problem_from_frame(&frame.abi(), kernel, &problem, nullptr, &error.record); rc != VECOPS_STATUS_OK) return error.status(rc);
  return problem;
}

// ---------------------------------------------------------------- recipe

CudaMatmulRecipe::CudaMatmulRecipe(std::uint32_t kernel)
    : kernel_(kernel), id_(std::string("cuda/sm_100a/") + (vecops_b200_kernel_name(kernel) ? vecops_b200_kernel_name(kernel) : "?")),
      definition_(shared_definition()) {}

Status CudaMatmulRecipe::match(const KernelCall& call) const {
  auto problem = matmul_problem_from(call.arguments().values(), kernel_);
  if (!problem) return Status(StatusCode::NotApplicable, problem.status().message());
  ErrorText error;
  std::uint32_t chosen = 0;
  const auto rc = vecops_b200_matmul_select(&problem.value(), &chosen, &error.record);
  if (rc == VECOPS_STATUS_OK) return Status::success();
  // An unsupported dtype row is a property of the call, not of this recipe, but
  // another operator recipe might still serve it: report "does not apply".
  return Status(StatusCode::NotApplicable, error.text.data());
}

Result<BoundKernelRecipe> CudaMatmulRecipe::bind(const KernelCall& call) const {
  auto binding = bind_kernel_call(*definition_, call);
  if (!binding) return binding.status();
  BoundKernelRecipe bound;
  bound.recipe_id = id_;
  bound.specialization_key = binding.value().specialization_key + ";kernel=" + vecops_b200_kernel_name(kernel_);
  bound.artifact_key = id_;
  return bound;
}

// ---------------------------------------------------------------- dispatch policy

Result<std::vector<std::size_t>> MatmulRuntimeDispatch::candidates(
    const KernelCall& call, std::span<const std::shared_ptr<const KernelRecipe>> recipes) const {
  std::vector<std::size_t> order;
  std::uint32_t chosen = VECOPS_B200_KERNEL_AUTO;
  if (auto problem = matmul_problem_from(call.arguments().values(), VECOPS_B200_KERNEL_AUTO)) {
    ErrorText error;
    if (vecops_b200_matmul_select(&problem.value(), &chosen, &error.record) != VECOPS_STATUS_OK) chosen = VECOPS_B200_KERNEL_AUTO;
  }
  auto kernel_of = [&](std::size_t i) -> std::uint32_t {
    const auto* recipe = dynamic_cast<const CudaMatmulRecipe*>(recipes[i].get());
    return recipe != nullptr ? recipe->kernel() : static_cast<std::uint32_t>(VECOPS_B200_KERNEL_AUTO);
  };
  for (std::size_t i = 0; i < recipes.size(); ++i)
    if (chosen != VECOPS_B200_KERNEL_AUTO && kernel_of(i) == chosen) order.push_back(i);
  // then foreign recipes in declaration order, and the strided kernel as the safety net
  for (std::size_t i = 0; i < recipes.size(); ++i)
    if (kernel_of(i) == VECOPS_B200_KERNEL_AUTO) order.push_back(i);
  for (std::size_t i = 0; i < recipes.size(); ++i)
    if (kernel_of(i) == VECOPS_B200_KERNEL_GENERIC && chosen != VECOPS_B200_KERNEL_GENERIC) order.push_back(i);
  return order;
}

// ---------------------------------------------------------------- provider

namespace {
struct OwnedDescriptor {
  std::string key;
  VecopsKernelDescriptorV1 descriptor;
};
}  // namespace

Result<std::shared_ptr<Executable>> CudaExecutableProvider::resolve(const BoundKernelRecipe& recipe) {
  {
    std::lock_guard<std::mutex> lock(mutex_);
    if (auto found = cache_.find(recipe.specialization_key); found != cache_.end()) return found->second;
  }
  constexpr std::string_view prefix = "cuda/sm_100a/";
  if (!std::string_view(recipe.artifact_key).starts_with(prefix))
    return Status(StatusCode::NotFound, "artifact '" + recipe.artifact_key + "' is not a prebuilt sm_100a kernel");
  const std::string_view name = std::string_view(recipe.artifact_key).substr(prefix.size());
  std::uint32_t kernel = VECOPS_B200_KERNEL_AUTO;
  for (std::uint32_t k = 1; k < VECOPS_B200_KERNEL_COUNT_; ++k)
    if (name == vecops_b200_kernel_name(k)) kernel = k;
  const VariantDescriptor* variant = variant_descriptor(kernel);
  if (kernel == VECOPS_B200_KERNEL_AUTO || variant == nullptr)
    return Status(StatusCode::NotFound, "no prebuilt kernel image named '" + std::string(name) + "'");
  auto owned = std::make_shared<OwnedDescriptor>();
  owned->key = recipe.specialization_key;
  owned->descriptor = variant->descriptor;
  owned->descriptor.specialization_key = owned->key.c_str();
  auto module = LoadedModule::adopt(&owned->descriptor, owned);
  if (!module) return module.status();
  auto executable = std::make_shared<Executable>(std::move(module).value());
  std::lock_guard<std::mutex> lock(mutex_);
  // two threads may have raced to build the same key: the first one published wins
  return cache_.emplace(recipe.specialization_key, std::move(executable)).first->second;
}

std::size_t CudaExecutableProvider::cached() const {
  std::lock_guard<std::mutex> lock(mutex_);
  return cache_.size();
}

std::shared_ptr<Operator> make_matmul_operator() {
  std::vector<std::shared_ptr<const KernelRecipe>> recipes;
  for (const auto kernel : kVariants) recipes.push_back(std::make_shared<CudaMatmulRecipe>(kernel));
  return std::make_shared<Operator>(matmul_kernel_def(), std::move(recipes), std::make_shared<MatmulRuntimeDispatch>(),
                                    std::make_shared<CudaExecutableProvider>());
}

const VecopsKernelDescriptorV1* matmul_descriptor_template(std::uint32_t kernel) {
  const VariantDescriptor* variant = variant_descriptor(kernel);
  return variant != nullptr ? &variant->descriptor : nullptr;
}

// ================================================================== vecops::matmul_pack
//
// Two more operators behind the same Operator machinery: ops::matmul_pack, values = {src[R,K], dst[R,P]}, and
// ops::matmul_pack_b_compensated, values = {src, dst, compensation[R], a_zero_point} (include/vecops/ops/MatmulPack.h;
// separate operators there too, :28-35 - and a writable tensor cannot be optional in a schema).  dst must be a tensor
// over the packed layout of src - P = vecops_b200_matmul_packed_layout's pitch, strides (P, 1) - as the reference
// demands of its output (tests/ops/MatmulPackTest.cpp:461-487).  One recipe each: the layout decides the kernel inside.

namespace {

constexpr const char* kPackOperatorName = "vecops::matmul_pack";
constexpr const char* kPackCompensatedOperatorName = "vecops::matmul_pack_b_compensated";
constexpr std::uint32_t kPackParameters = 4;  // of the compensated operator; the plain one has the first two

std::int32_t pack_from_frame(const VecopsCall* call, VecopsB200Pack* out, std::int32_t* zero_point, std::int32_t** compensation,
                             VecopsError* error) {
  if (call == nullptr || call->struct_size < sizeof(VecopsCall)) return fail(error, VECOPS_STATUS_ABI_MISMATCH, "call frame is null or too small");
  if (call->num_values < 2 || call->num_values > kPackParameters || call->values == nullptr)
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "matmul_pack expects src, dst and optionally compensation, a_zero_point");
  if (call->values[0].kind != VECOPS_VALUE_TENSOR || call->values[1].kind != VECOPS_VALUE_TENSOR)
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "matmul_pack operands must be tensors");
  const VecopsTensorView& src = call->values[0].value.tensor;
  const VecopsTensorView& dst = call->values[1].value.tensor;
  if (src.rank != 2 || dst.rank != 2) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "matmul_pack wants rank-2 src and dst");
  *compensation = nullptr;
  *zero_point = 0;
  if (call->num_values > 2 && call->values[2].kind == VECOPS_VALUE_TENSOR) {
    const VecopsTensorView& row = call->values[2].value.tensor;
    if (row.rank != 1 || row.sizes[0] != src.sizes[0] || row.dtype != VECOPS_DTYPE_I32 || (row.strides[0] != 1 && row.sizes[0] > 1))
      return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "compensation must be a contiguous int32 tensor of one element per packed row");
    *compensation = reinterpret_cast<std::int32_t*>(static_cast<char*>(row.data) + row.byte_offset);
  } else if (call->num_values > 2 && call->values[2].kind != VECOPS_VALUE_NONE) {
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "compensation is a tensor or absent");
  }
  if (call->num_values > 3) {
    const VecopsValue& value = call->values[3];
    if (value.kind != VECOPS_VALUE_SCALAR || value.value.scalar.dtype != VECOPS_DTYPE_I32)
      return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "a_zero_point is an i32 scalar");
    *zero_point = static_cast<std::int32_t>(value.value.scalar.value.i64);
  }
  std::int64_t pitch = 0;
  std::uint64_t bytes = 0;
  if (const auto rc = vecops_b200_matmul_packed_layout(dst.dtype, src.sizes[0], src.sizes[1], &pitch, &bytes, error); rc != VECOPS_STATUS_OK) return rc;
  if (dst.sizes[0] != src.sizes[0] || dst.sizes[1] != pitch || (dst.strides[0] != pitch && dst.sizes[0] > 1) || (dst.strides[1] != 1 && pitch > 1))
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "dst is not a tensor over the packed layout of src ([rows, pitch], strides (pitch, 1))");
  VecopsB200Pack p{};
  p.struct_size = sizeof(VecopsB200Pack);
  p.operand = 1;
  p.rows = src.sizes[0];
  p.k = src.sizes[1];
  p.src = static_cast<const char*>(src.data) + src.byte_offset;
  p.src_stride_row = src.strides[0];
  p.src_stride_k = src.strides[1];
  p.src_dtype = src.dtype;
  p.dst_dtype = dst.dtype;
  p.dst = static_cast<char*>(dst.data) + dst.byte_offset;
  p.dst_size = bytes;
  p.device_index = dst.device_index;
  if (const VecopsExecutionContext* context = call->context)
    if (context->struct_size >= offsetof(VecopsExecutionContext, stream) + sizeof(context->stream)) p.stream = context->stream;
  *out = p;
  return VECOPS_STATUS_OK;
}

template <bool kCompensated>
std::int32_t run_pack(const VecopsCall* call, VecopsError* error) {
  VecopsB200Pack pack;
  std::int32_t zero_point = 0;
  std::int32_t* compensation = nullptr;
  if (const auto rc = pack_from_frame(call, &pack, &zero_point, &compensation, error); rc != VECOPS_STATUS_OK) return rc;
  if (kCompensated != (compensation != nullptr))
    return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, kCompensated ? "matmul_pack_b_compensated needs its compensation row" : "matmul_pack takes src and dst only");
  if (kCompensated) return vecops_b200_matmul_pack_b_compensated(&pack, zero_point, compensation, error);
  return vecops_b200_matmul_pack(&pack, error);
}

std::int32_t pack_workspace(const VecopsCall*, std::uint64_t* bytes, VecopsError*) {
  if (bytes != nullptr) *bytes = 0;  // as matmul_pack_workspace_bytes of the reference's direct plans (MatmulPackTest.cpp:178-182)
  return VECOPS_STATUS_OK;
}

struct PackDescriptor {
  VecopsDimensionConstraint sizes2[2], src_strides[2], dst_strides[2], sizes1[1], strides1[1];
  VecopsParameterDescriptor parameters[kPackParameters];
  VecopsKernelDescriptorV1 descriptor;
};

PackDescriptor* build_pack_descriptor(bool compensated) {
  auto* v = new PackDescriptor{};
  constexpr auto all = bit(VECOPS_DTYPE_F32) | bit(VECOPS_DTYPE_BF16) | bit(VECOPS_DTYPE_F16) | bit(VECOPS_DTYPE_I8) | bit(VECOPS_DTYPE_U8);
  v->sizes2[0] = v->sizes2[1] = any_dim();
  v->src_strides[0] = v->src_strides[1] = any_dim();
  v->dst_strides[0] = any_dim();
  v->dst_strides[1] = const_dim(1);
  v->sizes1[0] = any_dim();
  v->strides1[0] = const_dim(1);
  v->parameters[0] = tensor_parameter("src", compensated ? bit(VECOPS_DTYPE_I8) : all, 2, v->sizes2, v->src_strides, false, false);
  v->parameters[1] = tensor_parameter("dst", compensated ? bit(VECOPS_DTYPE_I8) : all, 2, v->sizes2, v->dst_strides, false, true);
  v->parameters[2] = tensor_parameter("compensation", bit(VECOPS_DTYPE_I32), 1, v->sizes1, v->strides1, false, true);
  v->parameters[3] = scalar_parameter("a_zero_point", bit(VECOPS_DTYPE_I32));
  auto& d = v->descriptor;
  d.struct_size = sizeof(VecopsKernelDescriptorV1);
  d.abi_version_major = VECOPS_KERNEL_ABI_VERSION_MAJOR;
  d.abi_version_minor = VECOPS_KERNEL_ABI_VERSION_MINOR;
  d.operator_name = compensated ? kPackCompensatedOperatorName : kPackOperatorName;
  d.specialization_key = "";
  d.num_parameters = compensated ? kPackParameters : 2;
  d.parameter_stride = sizeof(VecopsParameterDescriptor);
  d.parameters = v->parameters;
  d.workspace = &pack_workspace;
  d.run = compensated ? &run_pack<true> : &run_pack<false>;
  d.flags = 0;
  return v;
}

const PackDescriptor* pack_descriptor(bool compensated) {
  static const PackDescriptor* const built[2] = {build_pack_descriptor(false), build_pack_descriptor(true)};
  return built[compensated ? 1 : 0];
}

class CudaPackRecipe final : public KernelRecipe {
public:
  explicit CudaPackRecipe(bool compensated)
      : compensated_(compensated),
        definition_(std::make_shared<const KernelDef>(compensated ? matmul_pack_b_compensated_kernel_def() : matmul_pack_kernel_def())) {}
  [[nodiscard]] std::string_view id() const override { return compensated_ ? "cuda/sm_100a/matmul_pack_b_compensated" : "cuda/sm_100a/matmul_pack"; }
  [[nodiscard]] Status match(const KernelCall& call) const override {
    ArgumentMetadata arguments(std::vector<Value>(call.arguments().values().begin(), call.arguments().values().end()));
    CallFrame frame(arguments);
    VecopsB200Pack pack;
    std::int32_t zero_point = 0;
    std::int32_t* compensation = nullptr;
    ErrorText error;
    if (const auto rc = pack_from_frame(&frame.abi(), &pack, &zero_point, &compensation, &error.record); rc != VECOPS_STATUS_OK)
      return Status(StatusCode::NotApplicable, error.text.data());
    const bool same = pack.src_dtype == pack.dst_dtype;
    const bool narrowing = pack.src_dtype == VECOPS_DTYPE_F32 && (pack.dst_dtype == VECOPS_DTYPE_BF16 || pack.dst_dtype == VECOPS_DTYPE_F16);
    if (!same && !narrowing) return Status(StatusCode::NotApplicable, "matmul_pack keeps the element type or narrows f32 to bf16 / f16");
    if (compensated_ != (compensation != nullptr)) return Status(StatusCode::NotApplicable, "compensation row missing or unexpected");
    if (compensated_ && (pack.src_dtype != VECOPS_DTYPE_I8 || pack.dst_dtype != VECOPS_DTYPE_I8))
      return Status(StatusCode::NotApplicable, "the compensated form packs a signed 8-bit B");
    return Status::success();
  }
  [[nodiscard]] Result<BoundKernelRecipe> bind(const KernelCall& call) const override {
    auto binding = bind_kernel_call(*definition_, call);
    if (!binding) return binding.status();
    BoundKernelRecipe bound;
    bound.recipe_id = std::string(id());
    bound.specialization_key = binding.value().specialization_key + ";kernel=pack";
    bound.artifact_key = std::string(id());
    return bound;
  }

private:
  bool compensated_;
  std::shared_ptr<const KernelDef> definition_;
};

class CudaPackProvider final : public ExecutableProvider {
public:
  [[nodiscard]] Result<std::shared_ptr<Executable>> resolve(const BoundKernelRecipe& recipe) override {
    std::lock_guard<std::mutex> lock(mutex_);
    if (auto found = cache_.find(recipe.specialization_key); found != cache_.end()) return found->second;
    const bool compensated = recipe.artifact_key == "cuda/sm_100a/matmul_pack_b_compensated";
    if (!compensated && recipe.artifact_key != "cuda/sm_100a/matmul_pack")
      return Status(StatusCode::NotFound, "artifact '" + recipe.artifact_key + "' is not a prebuilt pack kernel");
    auto owned = std::make_shared<OwnedDescriptor>();
    owned->key = recipe.specialization_key;
    owned->descriptor = pack_descriptor(compensated)->descriptor;
    owned->descriptor.specialization_key = owned->key.c_str();
    auto module = LoadedModule::adopt(&owned->descriptor, owned);
    if (!module) return module.status();
    return cache_.emplace(recipe.specialization_key, std::make_shared<Executable>(std::move(module).value())).first->second;
  }

private:
  std::mutex mutex_;
  std::map<std::string, std::shared_ptr<Executable>, std::less<>> cache_;
};

}  // namespace

namespace {
TensorDef pack_tensor(std::string name, std::vector<DimensionDef> shape, TensorDTypeDef dtype, TensorAccess access) {
  TensorDef t;
  t.name = std::move(name);
  t.strides.assign(shape.size(), DimensionDef::any());
  t.shape = std::move(shape);
  t.dtype = std::move(dtype);
  t.access = access;
  t.optional = false;
  t.device_type = VECOPS_DEVICE_CUDA;
  t.device_index = -1;
  return t;
}
DimensionDef pack_dim(const char* name) { return DimensionDef::named_dynamic(name, 1, 0); }
}  // namespace

KernelDef matmul_pack_kernel_def() {
  return KernelDef(kPackOperatorName,
                   {pack_tensor("src", {pack_dim("R"), pack_dim("K")}, "TS", TensorAccess::Input),
                    pack_tensor("dst", {pack_dim("R"), pack_dim("P")}, "TD", TensorAccess::Output)},
                   {{"TS", SpecializationType::DType}, {"TD", SpecializationType::DType}});
}

KernelDef matmul_pack_b_compensated_kernel_def() {
  return KernelDef(kPackCompensatedOperatorName,
                   {pack_tensor("src", {pack_dim("R"), pack_dim("K")}, DType::Int8, TensorAccess::Input),
                    pack_tensor("dst", {pack_dim("R"), pack_dim("P")}, DType::Int8, TensorAccess::Output),
                    pack_tensor("compensation", {pack_dim("R")}, DType::Int32, TensorAccess::Output),
                    ValueDef{"a_zero_point", DType::Int32, Scalar::signed_integer(0, DType::Int32)}},
                   {});
}

std::shared_ptr<Operator> make_matmul_pack_operator(bool compensated) {
  std::vector<std::shared_ptr<const KernelRecipe>> recipes{std::make_shared<CudaPackRecipe>(compensated)};
  return std::make_shared<Operator>(compensated ? matmul_pack_b_compensated_kernel_def() : matmul_pack_kernel_def(), std::move(recipes),
                                    std::make_shared<OrderedDispatchPolicy>(), std::make_shared<CudaPackProvider>());
}

}  // namespace vecops::runtime

// ------------------------------------------------------------------ C bridge

using namespace vecops::runtime;

namespace {

constexpr std::uint64_t kMatmulHandle = 0x6d61746d756c0001ULL;
constexpr std::uint64_t kPackHandle = 0x6d61746d756c0002ULL;
constexpr std::uint64_t kPackCompensatedHandle = 0x6d61746d756c0003ULL;

const std::shared_ptr<Operator>& matmul_operator() {
  static const std::shared_ptr<Operator> op = make_matmul_operator();
  return op;
}

const std::shared_ptr<Operator>& pack_operator(bool compensated) {
  static const std::shared_ptr<Operator> ops[2] = {make_matmul_pack_operator(false), make_matmul_pack_operator(true)};
  return ops[compensated ? 1 : 0];
}

const Operator* operator_of(std::uint64_t handle) {
  if (handle == kMatmulHandle) return matmul_operator().get();
  if (handle == kPackHandle) return pack_operator(false).get();
  if (handle == kPackCompensatedHandle) return pack_operator(true).get();
  return caller_operator_of(handle);  // batched matmul, attention, per-row quantiser
}

std::int32_t report(VecopsError* error, const Status& status) {
  return fail(error, static_cast<std::int32_t>(status.code()), status.message().c_str());
}

// Copy the ABI frame into owned metadata (shape/stride arrays included).
std::int32_t call_from_frame(const VecopsCall* call, std::uint32_t nspec, const VecopsSpecializationArgument* specs, KernelCall* out,
                             VecopsError* error) {
  if (call == nullptr || call->struct_size < sizeof(VecopsCall)) return fail(error, VECOPS_STATUS_ABI_MISMATCH, "call frame is null or too small");
  if (call->num_values != 0 && call->values == nullptr) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "call frame has no values");
  std::vector<Value> values;
  for (std::uint32_t i = 0; i < call->num_values; ++i) {
    const VecopsValue& v = call->values[i];
    if (v.kind == VECOPS_VALUE_NONE) {
      values.emplace_back(std::monostate{});
    } else if (v.kind == VECOPS_VALUE_TENSOR) {
      const VecopsTensorView& t = v.value.tensor;
      if (t.rank != 0 && (t.sizes == nullptr || t.strides == nullptr)) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "tensor without sizes or strides");
      TensorView view;
      view.data = t.data;
      view.byte_offset = t.byte_offset;
      view.device_type = t.device_type;
      view.device_index = t.device_index;
      view.dtype = static_cast<DType>(t.dtype);
      view.sizes.assign(t.sizes, t.sizes + t.rank);
      view.strides.assign(t.strides, t.strides + t.rank);
      view.flags = t.flags;
      values.emplace_back(std::move(view));
    } else if (v.kind == VECOPS_VALUE_SCALAR) {
      Scalar s;
      s.dtype = static_cast<DType>(v.value.scalar.dtype);
      s.value = v.value.scalar.value;
      values.emplace_back(s);
    } else {
      return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "unknown value kind");
    }
  }
  SpecializationValues named;
  for (std::uint32_t i = 0; i < nspec; ++i) {
    if (specs == nullptr || specs[i].name == nullptr) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "specialization value without a name");
    if (specs[i].kind == VECOPS_SPECIALIZATION_CONST_INT) named[specs[i].name] = specs[i].value.integer;
    else if (specs[i].kind == VECOPS_SPECIALIZATION_DTYPE) named[specs[i].name] = static_cast<DType>(specs[i].value.dtype);
    else return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "unknown specialization value kind");
  }
  *out = KernelCall(ArgumentMetadata(std::move(values)), std::move(named));
  return VECOPS_STATUS_OK;
}

}  // namespace

// ---------------------------------------------------------------- prepared calls
//
// vecops' framework bridge keeps up to eight exact call signatures per thread: once a slow invocation has resolved and
// validated an Executable, a call with the same signature re-enters it directly through Executable::invoke_prevalidated
// (docs/Runtime.md:195-206).  The same here, one level down, for every caller of the C bridge.  A signature holds what
// binding, validation, dispatch and the workspace query depend on - the operator handle, each value's kind, and for
// tensors dtype, device, access flags, rank, every size and every stride - and leaves out what they do not: data
// addresses and scalar payloads.  A hit skips bind_kernel_call, schema and descriptor validation, the dispatch policy,
// the recipes and the provider; what is left is the workspace-size comparison vecops' Executable::invoke makes and the
// artifact's run callback on the caller's own frame (the callbacks of this library read frames of 3 to 10 values
// as they come: problem_from_frame fills in the defaults itself).
namespace {

constexpr std::size_t kSignatureWords = 96;  // ten values of rank <= 3 fit with room to spare; anything longer takes the slow path
constexpr int kPreparedPerThread = 8;

struct CallSignature {
  std::array<std::uint64_t, kSignatureWords> words{};
  std::size_t count = 0;
  std::uint64_t hash = 0;
  bool usable = false;
};

CallSignature signature_of(std::uint64_t handle, const VecopsCall* call, std::uint32_t num_specialization_values) {
  CallSignature s;
  if (call == nullptr || call->struct_size < sizeof(VecopsCall) || num_specialization_values != 0 ||
      (call->num_values != 0 && call->values == nullptr))
    return s;  // explicit specialization values, or a frame the slow path has to refuse in words
  auto push = [&s](std::uint64_t word) {
    if (s.count < kSignatureWords) s.words[s.count] = word;
    ++s.count;
  };
  push(handle);
  push(call->num_values);
  for (std::uint32_t i = 0; i < call->num_values; ++i) {
    const VecopsValue& v = call->values[i];
    push(v.kind);
    if (v.kind == VECOPS_VALUE_TENSOR) {
      const VecopsTensorView& t = v.value.tensor;
      if (t.rank > 8 || (t.rank != 0 && (t.sizes == nullptr || t.strides == nullptr))) return s;
      push((static_cast<std::uint64_t>(t.dtype) << 32) | t.rank);
      push((static_cast<std::uint64_t>(t.device_type) << 32) | static_cast<std::uint32_t>(t.device_index));
      push(t.flags);
      // the address and its byte offset are left out, but not how the address is aligned: the dispatch rules send
      // 16-byte aligned operands to the TMA-fed kernels and others to the strided one
      push((reinterpret_cast<std::uintptr_t>(t.data) + t.byte_offset) & 15u);
      for (std::uint32_t d = 0; d < t.rank; ++d) {
        push(static_cast<std::uint64_t>(t.sizes[d]));
        push(static_cast<std::uint64_t>(t.strides[d]));
      }
    } else if (v.kind == VECOPS_VALUE_SCALAR) {
      push(v.value.scalar.dtype);
    }
  }
  if (s.count > kSignatureWords) return s;
  std::uint64_t h = 0xcbf29ce484222325ULL;
  for (std::size_t i = 0; i < s.count; ++i) h = (h ^ s.words[i]) * 0x100000001b3ULL;
  s.hash = h;
  s.usable = true;
  return s;
}

struct PreparedCall {
  CallSignature signature;
  std::shared_ptr<Executable> executable;
  std::uint64_t workspace_bytes = 0;
};

struct PreparedCalls {
  std::array<PreparedCall, kPreparedPerThread> entries;
  int next = 0;
  const PreparedCall* find(const CallSignature& s) const {
    for (const auto& e : entries)
      if (e.executable != nullptr && e.signature.hash == s.hash && e.signature.count == s.count &&
          std::memcmp(e.signature.words.data(), s.words.data(), s.count * sizeof(std::uint64_t)) == 0)
        return &e;
    return nullptr;
  }
  void remember(const CallSignature& s, std::shared_ptr<Executable> executable, std::uint64_t bytes) {
    entries[next] = PreparedCall{s, std::move(executable), bytes};
    next = (next + 1) % kPreparedPerThread;
  }
};

thread_local PreparedCalls tl_prepared;
std::atomic<std::uint64_t> g_bridge_slow{0}, g_bridge_prepared{0};

bool prepared_calls_enabled() {
  static const bool enabled = [] {
    const char* v = std::getenv("VECOPS_B200_PREPARED_CALL");  // "0" before the first call turns the hot path off, for diagnostics
    return !(v != nullptr && v[0] == '0');
  }();
  return enabled;
}

}  // namespace

extern "C" {

uint64_t vecops_b200_matmul_operator(void) {
  (void)matmul_operator();
  return kMatmulHandle;
}

uint64_t vecops_b200_matmul_pack_operator(int32_t compensated) {
  (void)pack_operator(compensated != 0);
  return compensated != 0 ? kPackCompensatedHandle : kPackHandle;
}

int32_t vecops_operator_bridge_invoke_v1(uint64_t handle, const VecopsCall* call, uint32_t num_specialization_values,
                                         const VecopsSpecializationArgument* specialization_values, VecopsError* error) {
  const Operator* op = operator_of(handle);
  if (op == nullptr) return fail(error, VECOPS_STATUS_NOT_FOUND, "unknown operator handle");
  const CallSignature signature = prepared_calls_enabled() ? signature_of(handle, call, num_specialization_values) : CallSignature{};
  if (signature.usable) {
    if (const PreparedCall* prepared = tl_prepared.find(signature)) {
      // the one check of Executable::invoke that depends on what the signature leaves out (Executable.cpp:288-295)
      if (prepared->workspace_bytes > call->workspace_size || (prepared->workspace_bytes != 0 && call->workspace == nullptr)) {
        const std::string text = "kernel requires " + std::to_string(prepared->workspace_bytes) + " workspace bytes, but " +
                                 std::to_string(call->workspace_size) + " were supplied";
        return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, text.c_str());
      }
      g_bridge_prepared.fetch_add(1, std::memory_order_relaxed);
      const Status status = prepared->executable->invoke_prevalidated(*call);
      return status.ok() ? VECOPS_STATUS_OK : report(error, status);
    }
  }
  g_bridge_slow.fetch_add(1, std::memory_order_relaxed);
  KernelCall kernel_call;
  if (const auto rc = call_from_frame(call, num_specialization_values, specialization_values, &kernel_call, error); rc != VECOPS_STATUS_OK) return rc;
  const Status status = op->invoke(kernel_call, call->context, call->workspace, call->workspace_size);
  // Binding, validation and resolution have passed when the call succeeded or failed only inside the artifact's run
  // (a device error, no device at all): the signature is worth remembering either way.
  if (signature.usable && (status.ok() || status.code() == StatusCode::ExecutionError)) {
    if (auto executable = op->resolve(kernel_call, call->context)) {
      std::uint64_t bytes = 0;
      bool sized = true;
      if (const auto query = executable.value()->module()->descriptor().workspace) {
        std::array<char, 256> text{};
        VecopsError scratch{sizeof(VecopsError), 0, text.data(), text.size(), 0};
        sized = query(call, &bytes, &scratch) == VECOPS_STATUS_OK;
      }
      if (sized) tl_prepared.remember(signature, std::move(executable).value(), bytes);
    }
  }
  return status.ok() ? VECOPS_STATUS_OK : report(error, status);
}

void vecops_b200_bridge_counters(uint64_t* slow_calls, uint64_t* prepared_calls) {
  if (slow_calls != nullptr) *slow_calls = g_bridge_slow.load(std::memory_order_relaxed);
  if (prepared_calls != nullptr) *prepared_calls = g_bridge_prepared.load(std::memory_order_relaxed);
}

int32_t vecops_b200_operator_resolve(uint64_t handle, const VecopsCall* call, char* key, size_t capacity, VecopsError* error) {
  const Operator* op = operator_of(handle);
  if (op == nullptr) return fail(error, VECOPS_STATUS_NOT_FOUND, "unknown operator handle");
  KernelCall kernel_call;
  if (const auto rc = call_from_frame(call, 0, nullptr, &kernel_call, error); rc != VECOPS_STATUS_OK) return rc;
  auto executable = op->resolve(kernel_call, call->context);
  if (!executable) return report(error, executable.status());
  if (key != nullptr && capacity > 0) {
    const auto text = executable.value()->specialization_key();
    const size_t count = text.size() < capacity - 1 ? text.size() : capacity - 1;
    std::memcpy(key, text.data(), count);
    key[count] = '\0';
  }
  return VECOPS_STATUS_OK;
}

int32_t vecops_b200_operator_workspace(uint64_t handle, const VecopsCall* call, uint64_t* bytes, VecopsError* error) {
  const Operator* op = handle == kMatmulHandle ? matmul_operator().get() : caller_operator_of(handle);
  const KernelDef* caller_definition = handle == kMatmulHandle ? nullptr : caller_kernel_def_of(handle);
  if (op == nullptr || (handle != kMatmulHandle && caller_definition == nullptr)) return fail(error, VECOPS_STATUS_NOT_FOUND, "unknown operator handle");
  if (bytes == nullptr) return fail(error, VECOPS_STATUS_INVALID_ARGUMENT, "bytes output pointer is null");
  KernelCall kernel_call;
  if (const auto rc = call_from_frame(call, 0, nullptr, &kernel_call, error); rc != VECOPS_STATUS_OK) return rc;
  auto executable = op->resolve(kernel_call, call->context);
  if (!executable) return report(error, executable.status());
  auto bound = caller_definition != nullptr ? bind_kernel_call(*caller_definition, kernel_call) : bind_kernel_call(matmul_kernel_def(), kernel_call);
  if (!bound) return report(error, bound.status());
  auto size = executable.value()->workspace_size(bound.value().arguments, call->context);
  if (!size) return report(error, size.status());
  *bytes = size.value();
  return VECOPS_STATUS_OK;
}

const VecopsKernelDescriptorV1* vecops_b200_matmul_descriptor(uint32_t kernel) { return matmul_descriptor_template(kernel); }

}  // extern "C"
