// Torch bridge: torch.ops.vecops_b200.matmul / matmul_out / sdpa hand CUDA tensors straight to the operator bridge
// (vecops_operator_bridge_invoke_v1) on the current stream - dispatcher to C++ to kernel, no Python on the hot path.
// It stands where vecops' generated Torch adapters stand (python/vecops/ops/torch.py `register` -> generated bridge
// DSO -> vecops_operator_bridge_invoke_v1, include/vecops/runtime/OperatorBridgeAbi.h:156-158).
//
// torch is plumbing here (tensors, the caching allocator for scratch, the current stream); all arithmetic is in the
// library's own kernels.  Calls are enqueued asynchronously, like any torch CUDA op.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <array>
#include <string>
#include <vector>

#include "vecops_b200/matmul_cuda.h"
#include "vecops_b200/operator_bridge.h"

namespace {

uint32_t dtype_code(at::ScalarType type) {
  switch (type) {
    case at::kFloat: return VECOPS_DTYPE_F32;
    case at::kBFloat16: return VECOPS_DTYPE_BF16;
    case at::kHalf: return VECOPS_DTYPE_F16;
    case at::kChar: return VECOPS_DTYPE_I8;
    case at::kByte: return VECOPS_DTYPE_U8;
    case at::kInt: return VECOPS_DTYPE_I32;
    default: TORCH_CHECK(false, "vecops_b200: dtype ", type, " has no vecops code on this path");
  }
}

struct ErrorText {
  std::array<char, 512> text{};
  VecopsError record{};
  ErrorText() {
    record.struct_size = sizeof(VecopsError);
    record.message = text.data();
    record.message_capacity = text.size();
  }
  void check(int32_t code, const char* what) const { TORCH_CHECK(code == VECOPS_STATUS_OK, "vecops_b200 ", what, " failed (", code, "): ", text.data()); }
};

VecopsValue tensor_value(const at::Tensor& t, bool writable) {
  VecopsValue v{};
  v.struct_size = sizeof(VecopsValue);
  v.kind = VECOPS_VALUE_TENSOR;
  VecopsTensorView& view = v.value.tensor;
  view.struct_size = sizeof(VecopsTensorView);
  view.data = t.data_ptr();
  view.byte_offset = 0;
  view.device_type = t.is_cuda() ? VECOPS_DEVICE_CUDA : VECOPS_DEVICE_CPU;
  view.device_index = t.is_cuda() ? static_cast<int32_t>(t.get_device()) : 0;
  view.dtype = dtype_code(t.scalar_type());
  view.rank = static_cast<uint32_t>(t.dim());
  view.sizes = t.sizes().data();      // owned by the tensor, which outlives the call
  view.strides = t.strides().data();
  view.flags = VECOPS_TENSOR_READ | (writable ? VECOPS_TENSOR_WRITE : 0);
  return v;
}

VecopsValue none_value() {
  VecopsValue v{};
  v.struct_size = sizeof(VecopsValue);
  v.kind = VECOPS_VALUE_NONE;
  return v;
}

VecopsValue scalar_value(uint32_t dtype, double real, int64_t integer) {
  VecopsValue v{};
  v.struct_size = sizeof(VecopsValue);
  v.kind = VECOPS_VALUE_SCALAR;
  v.value.scalar.struct_size = sizeof(VecopsScalar);
  v.value.scalar.dtype = dtype;
  if (dtype == VECOPS_DTYPE_F32) v.value.scalar.value.f64 = real;  // scalars travel widened, the tag says what they were
  else v.value.scalar.value.i64 = integer;
  return v;
}

// c = activation((cin + a . b_nk^T) * alpha * column_scale), written into `c`
void matmul_out(const at::Tensor& a, const at::Tensor& b_nk, at::Tensor& c, const c10::optional<at::Tensor>& column_scale,
                const c10::optional<at::Tensor>& cin, double alpha, int64_t activation, double clamp_lo, double clamp_hi,
                const c10::optional<at::Tensor>& row_scale) {
  TORCH_CHECK(a.is_cuda() && b_nk.is_cuda() && c.is_cuda(), "vecops_b200.matmul: CUDA tensors only (there is no CPU path)");
  TORCH_CHECK(a.dim() == 2 && b_nk.dim() == 2 && c.dim() == 2, "vecops_b200.matmul: a [M,K], b_nk [N,K], c [M,N]");
  const c10::cuda::CUDAGuard guard(c.device());
  const bool has_scale = column_scale.has_value() && column_scale->defined();
  const bool has_cin = cin.has_value() && cin->defined();
  at::Tensor cin_view;
  if (has_cin) cin_view = cin->expand({c.size(0), c.size(1)});  // a bias row or a column becomes a stride-0 view
  std::vector<VecopsValue> values{tensor_value(a, false), tensor_value(b_nk, false), tensor_value(c, true)};
  const bool has_row = row_scale.has_value() && row_scale->defined();
  const bool fused = has_cin || alpha != 1.0 || activation != 0 || has_row;
  if (has_scale || fused) values.push_back(has_scale ? tensor_value(*column_scale, false) : none_value());
  if (fused) {
    values.push_back(has_cin ? tensor_value(cin_view, false) : none_value());
    values.push_back(scalar_value(VECOPS_DTYPE_F32, alpha, 0));
    values.push_back(scalar_value(VECOPS_DTYPE_I32, 0.0, activation));
    values.push_back(scalar_value(VECOPS_DTYPE_F32, clamp_lo, 0));
    values.push_back(scalar_value(VECOPS_DTYPE_F32, clamp_hi, 0));
    if (has_row) values.push_back(tensor_value(*row_scale, false));
  }
  VecopsExecutionContext context{};
  context.struct_size = sizeof(VecopsExecutionContext);
  context.stream = at::cuda::getCurrentCUDAStream(c.get_device()).stream();
  context.flags = VECOPS_B200_CONTEXT_FLAG_ASYNC;
  VecopsCall call{};
  call.struct_size = sizeof(VecopsCall);
  call.num_values = static_cast<uint32_t>(values.size());
  call.values = values.data();
  call.context = &context;
  const uint64_t handle = vecops_b200_matmul_operator();
  ErrorText error;
  uint64_t need = 0;
  error.check(vecops_b200_operator_workspace(handle, &call, &need, &error.record), "workspace query");
  at::Tensor scratch;  // from torch's caching allocator: freed blocks are re-issued only to later work on this stream
  if (need != 0) {
    scratch = at::empty({static_cast<int64_t>(need)}, a.options().dtype(at::kByte));
    call.workspace = scratch.data_ptr();
    call.workspace_size = need;
  }
  error.check(vecops_operator_bridge_invoke_v1(handle, &call, 0, nullptr, &error.record), "matmul");
}

at::Tensor matmul(const at::Tensor& a, const at::Tensor& b_nk, const c10::optional<at::Tensor>& column_scale,
                  const c10::optional<at::Tensor>& cin, double alpha, int64_t activation, double clamp_lo, double clamp_hi,
                  c10::optional<at::ScalarType> out_dtype, const c10::optional<at::Tensor>& row_scale) {
  TORCH_CHECK(a.dim() == 2 && b_nk.dim() == 2, "vecops_b200.matmul: a [M,K], b_nk [N,K]");
  at::ScalarType type = a.scalar_type();
  if (out_dtype.has_value()) type = *out_dtype;
  else if (a.scalar_type() == at::kChar || a.scalar_type() == at::kByte) type = at::kInt;  // 8-bit operands accumulate in int32
  at::Tensor c = at::empty({a.size(0), b_nk.size(0)}, a.options().dtype(type));
  matmul_out(a, b_nk, c, column_scale, cin, alpha, activation, clamp_lo, clamp_hi, row_scale);
  return c;
}

// Scaled dot-product attention, q [H,Lq,D] | [Lq,D] (k, v likewise), bf16; masks uint8 / bool (non-zero keeps).
at::Tensor sdpa(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double scale, int64_t causal,
                const c10::optional<at::Tensor>& key_mask, const c10::optional<at::Tensor>& bias, c10::optional<at::ScalarType> out_dtype) {
  TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda(), "vecops_b200.sdpa: CUDA tensors only");
  TORCH_CHECK(q.dim() == k.dim() && q.dim() == v.dim() && (q.dim() == 2 || q.dim() == 3), "vecops_b200.sdpa: q, k, v are [L,D] or [H,L,D]");
  const c10::cuda::CUDAGuard guard(q.device());
  const bool heads = q.dim() == 3;
  const int64_t h = heads ? q.size(0) : 1;
  auto dim = [&](const at::Tensor& t, int i) { return t.size(heads ? i + 1 : i); };
  auto stride = [&](const at::Tensor& t, int i) { return t.stride(heads ? i + 1 : i); };
  TORCH_CHECK(!heads || (k.size(0) == h && v.size(0) == h), "vecops_b200.sdpa: head counts disagree (expand shared K / V to the head count)");
  std::vector<int64_t> shape = heads ? std::vector<int64_t>{h, dim(q, 0), dim(v, 1)} : std::vector<int64_t>{dim(q, 0), dim(v, 1)};
  at::Tensor out = at::empty(shape, q.options().dtype(out_dtype.has_value() ? *out_dtype : q.scalar_type()));
  VecopsB200Attention a{};
  a.struct_size = sizeof(VecopsB200Attention);
  a.causal = static_cast<uint32_t>(causal);
  a.lq = dim(q, 0), a.dqk = dim(q, 1), a.lkv = dim(v, 0), a.dv = dim(v, 1);
  TORCH_CHECK(dim(k, 0) == a.lkv && dim(k, 1) == a.dqk, "vecops_b200.sdpa: k must be [Lkv, Dqk]");
  a.q = q.data_ptr(), a.q_stride_row = stride(q, 0), a.q_stride_col = stride(q, 1);
  a.k = k.data_ptr(), a.k_stride_row = stride(k, 0), a.k_stride_col = stride(k, 1);
  a.v = v.data_ptr(), a.v_stride_row = stride(v, 0), a.v_stride_col = stride(v, 1);
  a.out = out.data_ptr(), a.out_stride_row = stride(out, 0), a.out_stride_col = stride(out, 1);
  a.qkv_dtype = dtype_code(q.scalar_type());
  a.out_dtype = dtype_code(out.scalar_type());
  at::Tensor mask_bytes, bias_view;
  if (key_mask.has_value() && key_mask->defined()) {
    mask_bytes = key_mask->to(at::kByte).contiguous();
    TORCH_CHECK(mask_bytes.dim() == 1 && mask_bytes.size(0) == a.lkv, "vecops_b200.sdpa: key_mask is [Lkv]");
    a.key_mask = static_cast<const uint8_t*>(mask_bytes.data_ptr());
  }
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->scalar_type() == at::kFloat, "vecops_b200.sdpa: bias is float32");
    bias_view = heads ? bias->expand({h, a.lq, a.lkv}) : bias->expand({a.lq, a.lkv});
    a.bias = static_cast<const float*>(bias_view.data_ptr());
    a.bias_stride_row = stride(bias_view, 0), a.bias_stride_col = stride(bias_view, 1);
    if (heads) a.bias_stride_head = bias_view.stride(0);
  }
  if (heads) {
    a.heads = h;
    a.q_stride_head = q.stride(0), a.k_stride_head = k.stride(0), a.v_stride_head = v.stride(0), a.out_stride_head = out.stride(0);
  }
  a.scale = static_cast<float>(scale);
  a.flags = VECOPS_B200_MATMUL_FLAG_ASYNC;
  a.stream = at::cuda::getCurrentCUDAStream(q.get_device()).stream();
  a.device_index = static_cast<int32_t>(q.get_device());
  ErrorText error;
  uint64_t need = 0;
  error.check(vecops_b200_sdpa_workspace(&a, &need, &error.record), "sdpa workspace query");
  at::Tensor scratch = at::empty({static_cast<int64_t>(need) + 256}, q.options().dtype(at::kByte));
  const uintptr_t base = reinterpret_cast<uintptr_t>(scratch.data_ptr());
  a.workspace = reinterpret_cast<void*>((base + 255) & ~static_cast<uintptr_t>(255));
  a.workspace_size = need;
  error.check(vecops_b200_sdpa_run(&a, &error.record), "sdpa");
  return out;
}

}  // namespace

TORCH_LIBRARY(vecops_b200, m) {
  m.def("matmul(Tensor a, Tensor b_nk, Tensor? column_scale=None, Tensor? cin=None, float alpha=1.0, int activation=0, float clamp_lo=0.0, "
        "float clamp_hi=0.0, ScalarType? out_dtype=None, Tensor? row_scale=None) -> Tensor");
  m.def("matmul_out(Tensor a, Tensor b_nk, Tensor(a!) c, Tensor? column_scale=None, Tensor? cin=None, float alpha=1.0, int activation=0, "
        "float clamp_lo=0.0, float clamp_hi=0.0, Tensor? row_scale=None) -> ()");
  m.def("sdpa(Tensor q, Tensor k, Tensor v, float scale, int causal=0, Tensor? key_mask=None, Tensor? bias=None, ScalarType? out_dtype=None) -> Tensor");
}

TORCH_LIBRARY_IMPL(vecops_b200, CUDA, m) {
  m.impl("matmul", &matmul);
  m.impl("matmul_out", &matmul_out);
  m.impl("sdpa", &sdpa);
}
