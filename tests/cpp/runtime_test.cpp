// Host-only tests of the operator runtime (no GPU needed): binding and keys,
// schema checks, recipe/dispatch/provider protocol, descriptor validation,
// a dlopen'ed fixture artifact, and the CUDA matmul operator's resolution.
// Plain main(), like the reference's tests/runtime/RuntimeTest.cpp.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <future>
#include <string>
#include <thread>

#include "fixture_artifact.h"
#include "vecops_b200/operator_bridge.h"
#include "vecops_b200/runtime/matmul_operator.h"

using namespace vecops::runtime;

namespace {

int g_checks = 0;
void require(bool condition, const char* what) {
  ++g_checks;
  if (!condition) {
    std::fprintf(stderr, "FAIL: %s\n", what);
    std::exit(1);
  }
}

TensorView cuda2d(void* p, DType dtype, std::int64_t rows, std::int64_t cols, bool writable = false, std::int64_t pitch = -1) {
  return device_tensor(p, dtype, {rows, cols}, {pitch < 0 ? cols : pitch, 1}, 0, writable);
}

alignas(256) unsigned char g_fake_device_memory[1 << 16];  // addresses only; never dereferenced on the host path

KernelCall matmul_call(DType ta, DType tb, DType tc, std::int64_t m, std::int64_t n, std::int64_t k, bool scale = false) {
  void* base = g_fake_device_memory;
  std::vector<Value> values{cuda2d(base, ta, m, k), cuda2d(base, tb, n, k), cuda2d(base, tc, m, n, true)};
  if (scale) values.emplace_back(device_tensor(base, DType::Float32, {n}, {1}, 0));
  return KernelCall(ArgumentMetadata(std::move(values)));
}

// ------------------------------------------------------------------ binding

void test_binding_and_keys() {
  KernelDef def("test::axpy",
                {TensorDef{"x", {"N"}, {1}, "T"}, TensorDef{"y", {"N"}, {1}, "T", false, TensorAccess::InOut},
                 TensorDef{"mask", {DimensionDef::constant()}, {1}, TensorDTypeDef{}, true}},
                {{"N", SpecializationType::ConstInt}, {"T", SpecializationType::DType}});
  require(def.validate().ok(), "definition validates");
  float storage[8];
  TensorView x{storage, 0, VECOPS_DEVICE_CPU, 0, DType::Float32, {8}, {1}, VECOPS_TENSOR_READ};
  TensorView y = x;
  y.flags = VECOPS_TENSOR_READ | VECOPS_TENSOR_WRITE;
  auto bound = bind_kernel_call(def, KernelCall(make_arguments(x, y)));
  require(bound.ok(), "bind infers N and T");
  require(bound.value().specialization_key == "test::axpy;N=8;T=f32;$0=0", "key spells symbols then anonymous entries");
  require(bound.value().arguments.size() == 3, "omitted trailing optional tensor is filled in");

  TensorView mask{storage, 0, VECOPS_DEVICE_CPU, 0, DType::UInt8, {4}, {1}, VECOPS_TENSOR_READ};
  auto with_mask = bind_kernel_call(def, KernelCall(make_arguments(x, y, mask)));
  require(with_mask.ok() && with_mask.value().specialization_key == "test::axpy;N=8;T=f32;$0=1;$1=u8;$2=4",
          "optional presence, anonymous dtype and Const extent are positional");

  TensorView y_short = y;
  y_short.sizes = {4};
  auto conflict = bind_kernel_call(def, KernelCall(make_arguments(x, y_short)));
  require(!conflict.ok() && conflict.status().code() == StatusCode::InvalidArgument, "conflicting symbol is refused");

  TensorView y_readonly = x;
  auto access = bind_kernel_call(def, KernelCall(make_arguments(x, y_readonly)));
  require(!access.ok(), "InOut tensor needs write access");

  auto supplied = bind_kernel_call(def, KernelCall(make_arguments(x, y), {{"N", std::int64_t{9}}}));
  require(!supplied.ok(), "supplied symbol must agree with the observed one");
  auto unknown = bind_kernel_call(def, KernelCall(make_arguments(x, y), {{"Q", std::int64_t{1}}}));
  require(!unknown.ok(), "unknown specialization value is refused");

  // named Dynamic: checked for agreement and alignment, never part of the key
  KernelDef dyn("test::dyn", {TensorDef{"a", {DimensionDef::named_dynamic("M", 4, 0, 64)}, {1}, DType::Float32},
                              TensorDef{"b", {DimensionDef::named_dynamic("M", 4, 0, 64)}, {1}, DType::Float32}});
  auto ok = bind_kernel_call(dyn, KernelCall(make_arguments(x, x)));
  require(ok.ok() && ok.value().specialization_key == "test::dyn", "named Dynamic stays out of the key");
  TensorView odd = x;
  odd.sizes = {6};
  require(!bind_kernel_call(dyn, KernelCall(make_arguments(odd, odd))).ok(), "Dynamic alignment is enforced");
  TensorView four = x;
  four.sizes = {4};
  require(!bind_kernel_call(dyn, KernelCall(make_arguments(x, four))).ok(), "named Dynamic must agree across tensors");

  KernelDef bad("test::bad", {TensorDef{"a", {"N"}, {1}, DType::Float32}});
  require(!bad.validate().ok(), "undeclared symbol fails validation");
  KernelDef dup("test::dup", {TensorDef{"a", {1}, {1}, DType::Float32}, TensorDef{"a", {1}, {1}, DType::Float32}});
  require(!dup.validate().ok(), "duplicate parameter names fail validation");
  require(def.canonical() != dyn.canonical() && def.canonical().find("name:test::axpy") == 0, "canonical text identifies a definition");
}

// ------------------------------------------------------------------ schema

void test_schema() {
  TensorConstraint rule;
  rule.dtype_mask = dtype_bit(DType::Float32);
  rule.rank = 1;
  rule.sizes = {DimensionConstraint::dynamic(0, 16, 4)};
  rule.device_type = VECOPS_DEVICE_CUDA;
  OperatorSchema schema("test::op", {ParameterSchema{"x", rule}, ParameterSchema{"alpha", ScalarConstraint{dtype_bit(DType::Float64)}}},
                        [](std::span<const Value> values) {
                          return std::get<Scalar>(values[1]).value.f64 >= 0 ? Status::success()
                                                                            : Status(StatusCode::InvalidArgument, "alpha < 0");
                        });
  auto x = device_tensor(g_fake_device_memory, DType::Float32, {8}, {1});
  require(schema.validate(make_arguments(x, 1.0)).ok(), "schema accepts a valid call");
  require(!schema.validate(make_arguments(x)).ok(), "argument count is checked");
  require(!schema.validate(make_arguments(x, -1.0)).ok(), "relation validator runs");
  auto host = x;
  host.device_type = VECOPS_DEVICE_CPU;
  require(!schema.validate(make_arguments(host, 1.0)).ok(), "a host tensor is refused where CUDA is required");
  auto big = x;
  big.sizes = {20};
  require(!schema.validate(make_arguments(big, 1.0)).ok(), "size bound is enforced");
  auto wrong = x;
  wrong.dtype = DType::Int8;
  require(!schema.validate(make_arguments(wrong, 1.0)).ok(), "dtype mask is enforced");
  require(!schema.validate(make_arguments(x, std::int32_t{1})).ok(), "scalar dtype mask is enforced");
}

// ------------------------------------------------------------------ fixture artifact through Operator

class FixtureRecipe final : public KernelRecipe {
public:
  explicit FixtureRecipe(std::string key) : key_(std::move(key)) {}
  std::string_view id() const override { return "fixture"; }
  Status match(const KernelCall& call) const override {
    return call.arguments().size() == 0 ? Status::success() : Status(StatusCode::NotApplicable, "fixture takes no arguments");
  }
  Result<BoundKernelRecipe> bind(const KernelCall& call) const override {
    if (auto status = match(call); !status.ok()) return status;
    BoundKernelRecipe bound;
    bound.recipe_id = "fixture";
    bound.specialization_key = key_;
    bound.artifact_key = "fixture-artifact";
    return bound;
  }

private:
  std::string key_;
};

class FixedProvider final : public ExecutableProvider {
public:
  explicit FixedProvider(std::shared_ptr<Executable> executable) : executable_(std::move(executable)) {}
  Result<std::shared_ptr<Executable>> resolve(const BoundKernelRecipe&) override {
    ++resolves;
    return executable_;
  }
  int resolves = 0;

private:
  std::shared_ptr<Executable> executable_;
};

class MissingProvider final : public ExecutableProvider {
public:
  Result<std::shared_ptr<Executable>> resolve(const BoundKernelRecipe&) override {
    return Status(StatusCode::NotFound, "nothing prebuilt");
  }
};

void test_fixture_artifact(const char* fixture_path) {
  auto missing = Executable::load("/nonexistent/libnothing.so");
  require(!missing.ok() && missing.status().code() == StatusCode::LoadError, "missing DSO is a LoadError");
  auto executable = Executable::load(fixture_path);
  require(executable.ok(), "fixture DSO loads and its descriptor validates");
  require(executable.value()->operator_name() == "test::fixture" && executable.value()->specialization_key() == "fixture-v1",
          "descriptor identity is readable");

  OperatorSchema schema("test::fixture", {});
  auto provider = std::make_shared<FixedProvider>(executable.value());
  Operator op(schema, {std::make_shared<FixtureRecipe>("fixture-v1")}, std::make_shared<OrderedDispatchPolicy>(), provider);

  FixtureObservation seen;
  VecopsExecutionContext context{};
  context.struct_size = sizeof(context);
  context.stream = reinterpret_cast<void*>(0x1234);
  context.user_data = &seen;
  context.flags = VECOPS_B200_CONTEXT_FLAG_ASYNC | 7;
  unsigned char scratch[128] = {};

  auto too_small = op.invoke(ArgumentMetadata{}, scratch, 8, &context);
  require(!too_small.ok() && too_small.code() == StatusCode::InvalidArgument && seen.runs == 0,
          "too-small workspace is refused before run");
  auto status = op.invoke(ArgumentMetadata{}, scratch, sizeof(scratch), &context);
  require(status.ok(), "fixture runs through Operator::invoke");
  require(seen.runs == 1 && seen.stream == context.stream && seen.flags == context.flags, "stream and flags are forwarded untouched");
  require(seen.workspace == scratch && seen.workspace_size == sizeof(scratch) && scratch[0] == 0x5a, "workspace is forwarded");
  require(seen.workspace_queries == 2, "workspace is queried once per invoke");

  seen.fail_next_run = true;
  auto failed = op.invoke(ArgumentMetadata{}, scratch, sizeof(scratch), &context);
  require(!failed.ok() && failed.code() == StatusCode::ExecutionError && failed.message() == "boom", "callback errors carry their text");
  seen.fail_next_run = false;

  // wrong key: the provider hands back an executable for another specialization
  Operator wrong_key(schema, {std::make_shared<FixtureRecipe>("some-other-key")}, std::make_shared<OrderedDispatchPolicy>(), provider);
  auto mismatch = wrong_key.resolve(ArgumentMetadata{});
  require(!mismatch.ok() && mismatch.status().code() == StatusCode::AbiMismatch, "key mismatch is AbiMismatch");
  OperatorSchema other_schema("test::other", {});
  Operator wrong_op(other_schema, {std::make_shared<FixtureRecipe>("fixture-v1")}, std::make_shared<OrderedDispatchPolicy>(), provider);
  require(wrong_op.resolve(ArgumentMetadata{}).status().code() == StatusCode::AbiMismatch, "operator-name mismatch is AbiMismatch");

  // NotFound from the provider falls through; with no other candidate it is the final answer
  Operator nothing(schema, {std::make_shared<FixtureRecipe>("fixture-v1")}, std::make_shared<OrderedDispatchPolicy>(),
                   std::make_shared<MissingProvider>());
  require(nothing.resolve(ArgumentMetadata{}).status().code() == StatusCode::NotFound, "provider miss is NotFound");
  // NotApplicable from every recipe
  require(op.resolve(make_arguments(1.0)).status().code() != StatusCode::Ok, "a call no recipe matches does not resolve");

  // descriptor validation of in-process descriptors
  VecopsKernelDescriptorV1 broken = executable.value()->module()->descriptor();
  broken.run = nullptr;
  require(LoadedModule::adopt(&broken, nullptr).status().code() == StatusCode::AbiMismatch, "descriptor without run is refused");
  broken = executable.value()->module()->descriptor();
  broken.abi_version_major = 2;
  require(LoadedModule::adopt(&broken, nullptr).status().code() == StatusCode::AbiMismatch, "foreign ABI major is refused");
  broken = executable.value()->module()->descriptor();
  broken.flags = 4;
  require(LoadedModule::adopt(&broken, nullptr).status().code() == StatusCode::AbiMismatch, "unknown descriptor flags are refused");
}

// ------------------------------------------------------------------ the CUDA matmul operator (resolution only)

void test_matmul_operator() {
  auto op = make_matmul_operator();
  require(op->schema().name() == "vecops::matmul" && op->schema().parameters().size() == 10,
          "matmul schema has a, b, c, column_scale, cin, the four scalars of the output transform and row_scale");

  auto resolve_key = [&](const KernelCall& call) {
    auto executable = op->resolve(call);
    return executable.ok() ? std::string(executable.value()->specialization_key()) : "ERROR: " + executable.status().message();
  };
  require(resolve_key(matmul_call(DType::BFloat16, DType::BFloat16, DType::BFloat16, 4096, 4096, 4096)) ==
              "vecops::matmul;TA=bf16;TB=bf16;TC=bf16;$0=0;$1=0;$2=0;kernel=bf16_tcgen05", "C2 resolves to the tcgen05 bf16 kernel");
  require(resolve_key(matmul_call(DType::Int8, DType::Int8, DType::Int32, 4096, 14336, 4096)) ==
              "vecops::matmul;TA=i8;TB=i8;TC=i32;$0=0;$1=0;$2=0;kernel=i8_tcgen05", "C3 resolves to the tcgen05 int8 kernel");
  require(resolve_key(matmul_call(DType::BFloat16, DType::Int8, DType::BFloat16, 16, 14336, 4096, true)) ==
              "vecops::matmul;TA=bf16;TB=i8;TC=bf16;$0=1;$1=0;$2=0;kernel=w8_small_m", "C4 resolves to the weight-only kernel");
  require(resolve_key(matmul_call(DType::BFloat16, DType::Int8, DType::BFloat16, 128, 14336, 4096, true)) ==
              "vecops::matmul;TA=bf16;TB=i8;TC=bf16;$0=1;$1=0;$2=0;kernel=w8_tcgen05", "C4 at M=128 resolves to the tensor-memory weight-only kernel");
  {
    // that kernel is the one that needs device scratch: the executable reports it, and refuses to run without it
    auto call = matmul_call(DType::BFloat16, DType::Int8, DType::BFloat16, 128, 14336, 4096, true);
    auto exe = op->resolve(call);
    auto bound = bind_kernel_call(matmul_kernel_def(), call);
    require(exe.ok() && bound.ok(), "w8_tcgen05 call binds");
    auto bytes = exe.value()->workspace_size(bound.value().arguments);
    require(bytes.ok() && bytes.value() > (10u << 20), "WorkspacePlanning sizes the device scratch");
    auto refused = exe.value()->invoke(bound.value().arguments, nullptr, 0);
    require(!refused.ok() && refused.code() == StatusCode::InvalidArgument, "invoke without the scratch is refused before run");
  }
  require(resolve_key(matmul_call(DType::Float32, DType::Float32, DType::Float32, 1024, 1024, 1024)) ==
              "vecops::matmul;TA=f32;TB=f32;TC=f32;$0=0;$1=0;$2=0;kernel=f32_tf32x3", "C1 resolves to the split-operand tensor-core kernel");
  require(resolve_key(matmul_call(DType::Float32, DType::Float32, DType::Float32, 128, 1024, 1024)) ==
              "vecops::matmul;TA=f32;TB=f32;TC=f32;$0=0;$1=0;$2=0;kernel=f32_simt", "a small fp32 product resolves to the FMA kernel");
  require(resolve_key(matmul_call(DType::BFloat16, DType::BFloat16, DType::Float32, 16, 16, 35)) ==
              "vecops::matmul;TA=bf16;TB=bf16;TC=f32;$0=0;$1=0;$2=0;kernel=generic", "an unaligned K falls to the strided kernel");

  {
    // the fused form COut = activation((CIn + A.B^T) * alpha): a bias row as a stride-0 accumulator input and SiLU
    auto call = matmul_call(DType::BFloat16, DType::BFloat16, DType::BFloat16, 4096, 4096, 4096);
    std::vector<Value> fused(call.arguments().values().begin(), call.arguments().values().end());
    fused.emplace_back(std::monostate{});                                                                      // no column_scale
    fused.emplace_back(device_tensor(reinterpret_cast<void*>(0x9000), DType::Float32, {4096, 4096}, {0, 1}, 0, false));  // cin = bias row
    fused.emplace_back(Scalar::floating(1.0, DType::Float32));
    fused.emplace_back(Scalar::signed_integer(VECOPS_B200_ACTIVATION_SILU, DType::Int32));
    auto key = resolve_key(KernelCall(ArgumentMetadata(fused)));
    require(key == "vecops::matmul;TA=bf16;TB=bf16;TC=bf16;$0=0;$1=1;$2=f32;$3=0;kernel=bf16_tcgen05",
            "a fused call resolves to the same kernel; the accumulator input's presence and dtype enter the key, the scalars do not");
    std::vector<Value> bad_scalar = fused;
    bad_scalar[6] = Scalar::floating(3.0, DType::Float32);
    require(!op->resolve(KernelCall(ArgumentMetadata(bad_scalar))).ok(), "activation must be an i32");
  }

  // decode-time M varies without a new specialization
  auto first = op->resolve(matmul_call(DType::BFloat16, DType::Int8, DType::BFloat16, 1, 14336, 4096, true));
  auto second = op->resolve(matmul_call(DType::BFloat16, DType::Int8, DType::BFloat16, 16, 14336, 4096, true));
  require(first.ok() && second.ok() && first.value() == second.value(), "M is a runtime dimension: one executable serves M=1 and M=16");

  // host tensors and disagreeing extents never reach a kernel
  auto host_call = matmul_call(DType::Float32, DType::Float32, DType::Float32, 8, 8, 8);
  std::vector<Value> host_values(host_call.arguments().values().begin(), host_call.arguments().values().end());
  std::get<TensorView>(host_values[0]).device_type = VECOPS_DEVICE_CPU;
  require(op->resolve(KernelCall(ArgumentMetadata(host_values))).status().code() == StatusCode::InvalidArgument, "a host tensor is refused");
  std::vector<Value> bad(host_call.arguments().values().begin(), host_call.arguments().values().end());
  std::get<TensorView>(bad[1]).sizes = {8, 9};
  require(op->resolve(KernelCall(ArgumentMetadata(bad))).status().code() == StatusCode::InvalidArgument, "K must agree between a and b");
  require(op->resolve(matmul_call(DType::Float32, DType::BFloat16, DType::Float32, 8, 8, 8)).status().code() != StatusCode::Ok,
          "an unsupported dtype row does not resolve");

  // dispatch order: chosen variant first, strided kernel as the last candidate
  MatmulRuntimeDispatch policy;
  std::vector<std::shared_ptr<const KernelRecipe>> recipes{std::make_shared<CudaMatmulRecipe>(VECOPS_B200_KERNEL_GENERIC),
                                                           std::make_shared<CudaMatmulRecipe>(VECOPS_B200_KERNEL_BF16_TCGEN05),
                                                           std::make_shared<CudaMatmulRecipe>(VECOPS_B200_KERNEL_I8_TCGEN05)};
  auto order = policy.candidates(matmul_call(DType::BFloat16, DType::BFloat16, DType::BFloat16, 512, 512, 512), recipes);
  require(order.ok() && order.value() == std::vector<std::size_t>({1, 0}), "dispatch puts the tensor-core recipe before the strided one");
  require(!recipes[2]->match(matmul_call(DType::BFloat16, DType::BFloat16, DType::BFloat16, 512, 512, 512)).ok(),
          "the int8 recipe reports NotApplicable for a bf16 call");

  // provider: memoised per key, unknown images are NotFound, concurrent resolves share one executable
  CudaExecutableProvider provider;
  BoundKernelRecipe bound;
  bound.specialization_key = "k1";
  bound.artifact_key = "cuda/sm_100a/bf16_tcgen05";
  auto a = std::async(std::launch::async, [&] { return provider.resolve(bound); });
  auto b = std::async(std::launch::async, [&] { return provider.resolve(bound); });
  auto ra = a.get(), rb = b.get();
  require(ra.ok() && rb.ok() && ra.value() == rb.value() && provider.cached() == 1, "identical keys share one executable");
  bound.artifact_key = "cuda/sm_100a/no_such_kernel";
  bound.specialization_key = "k2";
  require(provider.resolve(bound).status().code() == StatusCode::NotFound, "an image that was not prebuilt is NotFound");
  bound.artifact_key = "cpu/avx512/whatever";
  require(provider.resolve(bound).status().code() == StatusCode::NotFound, "foreign artifact keys are NotFound");
  require(provider.cached() == 1, "misses create nothing");

  // descriptor templates state each variant's constraints
  const auto* d = vecops_b200_matmul_descriptor(VECOPS_B200_KERNEL_I8_TCGEN05);
  require(d != nullptr && d->num_parameters == 10 && d->parameters[9].constraint.tensor.optional != 0 && d->parameters[4].constraint.tensor.optional != 0 && d->parameters[6].kind == VECOPS_VALUE_SCALAR && d->parameters[0].constraint.tensor.device_type == VECOPS_DEVICE_CUDA &&
              d->parameters[0].constraint.tensor.strides[0].alignment == 16 && d->run != nullptr && d->workspace != nullptr,
          "int8 descriptor wants CUDA tensors with 16-element row pitches");
  require(vecops_b200_matmul_descriptor(VECOPS_B200_KERNEL_AUTO) == nullptr, "AUTO has no descriptor");

  // an executable validates calls against its descriptor before running
  auto exe = op->resolve(matmul_call(DType::Int8, DType::Int8, DType::Int32, 256, 256, 256));
  require(exe.ok(), "int8 call resolves");
  auto bf16_args = matmul_call(DType::BFloat16, DType::BFloat16, DType::BFloat16, 256, 256, 256, true);
  require(!exe.value()->can_invoke(bf16_args.arguments()).ok(), "descriptor dtype mask refuses a bf16 call on the int8 executable");
}

void test_invoke_without_gpu_reports_execution_error() {
  if (vecops_b200_device_count() != 0) return;  // only meaningful on a host without a GPU
  auto op = make_matmul_operator();
  auto status = op->invoke(matmul_call(DType::Float32, DType::Float32, DType::Float32, 64, 64, 64));
  require(!status.ok() && status.code() == StatusCode::ExecutionError && status.message().find("no CPU fallback") != std::string::npos,
          "without a GPU the operator fails loudly, it does not fall back");
}

}  // namespace

// ------------------------------------------------------------------ the operand-preparation operator (resolution only)

void test_matmul_pack_operator() {
  auto op = make_matmul_pack_operator();
  require(op->schema().name() == "vecops::matmul_pack" && op->schema().parameters().size() == 2, "matmul_pack schema has src and dst");
  auto compensated_op = make_matmul_pack_operator(true);
  require(compensated_op->schema().name() == "vecops::matmul_pack_b_compensated" && compensated_op->schema().parameters().size() == 4,
          "matmul_pack_b_compensated is its own operator: src, dst, compensation, a_zero_point");
  void* src = reinterpret_cast<void*>(0x10000);
  void* dst = reinterpret_cast<void*>(0x900000);
  auto resolve_key = [&](std::vector<Value> values) {
    auto executable = op->resolve(KernelCall(ArgumentMetadata(std::move(values))));
    return executable.ok() ? std::string(executable.value()->specialization_key()) : "ERROR: " + executable.status().message();
  };
  // a [K, N]-stored int8 weight (row stride 1, k stride N) into its packed form: K = 129 -> pitch 256
  std::vector<Value> plain{device_tensor(src, DType::Int8, {33, 129}, {1, 33}, 0, false), device_tensor(dst, DType::Int8, {33, 256}, {256, 1}, 0, true)};
  require(resolve_key(plain) == "vecops::matmul_pack;TD=i8;TS=i8;kernel=pack", "a pack call resolves to the one pack recipe");
  std::vector<Value> compensated = plain;
  compensated.emplace_back(device_tensor(reinterpret_cast<void*>(0xa00000), DType::Int32, {33}, {1}, 0, true));
  compensated.emplace_back(Scalar::signed_integer(3, DType::Int32));
  {
    auto executable = compensated_op->resolve(KernelCall(ArgumentMetadata(compensated)));
    require(executable.ok() && executable.value()->specialization_key() == "vecops::matmul_pack_b_compensated;kernel=pack",
            "the compensated call resolves on its own operator");
    require(!op->resolve(KernelCall(ArgumentMetadata(compensated))).ok(), "the plain operator takes src and dst only");
  }
  std::vector<Value> narrowing{device_tensor(src, DType::Float32, {5, 9}, {21, 2}, 0, false), device_tensor(dst, DType::BFloat16, {5, 64}, {64, 1}, 0, true)};
  require(resolve_key(narrowing) == "vecops::matmul_pack;TD=bf16;TS=f32;kernel=pack", "fp32 storage narrows to the bf16 compute type");
  std::vector<Value> wrong_layout{device_tensor(src, DType::Int8, {33, 129}, {129, 1}, 0, false), device_tensor(dst, DType::Int8, {33, 129}, {129, 1}, 0, true)};
  require(!op->resolve(KernelCall(ArgumentMetadata(wrong_layout))).ok(), "a destination that is not over the packed layout does not resolve");
  std::vector<Value> wrong_types{device_tensor(src, DType::Int8, {33, 129}, {129, 1}, 0, false), device_tensor(dst, DType::BFloat16, {33, 192}, {192, 1}, 0, true)};
  require(!op->resolve(KernelCall(ArgumentMetadata(wrong_types))).ok(), "int8 -> bf16 is not a packing conversion");
}

int main(int argc, char** argv) {
  if (argc < 2) {
    std::fprintf(stderr, "usage: runtime_test <fixture_artifact.so>\n");
    return 2;
  }
  test_binding_and_keys();
  test_schema();
  test_fixture_artifact(argv[1]);
  test_matmul_operator();
  test_matmul_pack_operator();
  test_invoke_without_gpu_reports_execution_error();
  std::printf("runtime_test PASS (%d checks)\n", g_checks);
  return 0;
}
