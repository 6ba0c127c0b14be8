// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// A C-callable door to the reference's own CPU matmul, compiled from the
// reference's headers where they lie (never copied into this repository) by
// oracle/build_oracle.py into oracle/_ref/libvecops_ref.so.  It validates the
// C restatement in matmul_oracle.c, generates the fixtures under tests/golden/
// and serves as the timed "reference" CPU baseline of bench.py.
//
// API usage follows the reference's own tests: tests/ops/MatmulTest.cpp:60-81
// (make_tensor / ops::matmul / required_workspace / kernel::Workspace) and
// tests/ops/MatmulConversionTestCommon.h:105-124, 664-677 (input<Compute>(t),
// output<Acc>(t, epilogue), per-column scale as a lane-local vec transform).
// AMX needs a per-thread permission request first, as in
// tests/ops/MatmulTestArch.h:22-27.
#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <thread>
#include <vector>

#include "vecops/ops/Attention.h"
#include "vecops/matmul/Quantization.h"
#include "vecops/ops/Matmul.h"
#include "vecops/ops/MatmulPack.h"

using namespace vecops;
using namespace vecops::meta;
using namespace vecops::tensor;

namespace {

bool request_amx() {
  return syscall(SYS_arch_prctl, 0x1023 /* ARCH_REQ_XCOMP_PERM */, 18 /* XFEATURE_XTILEDATA */) == 0;
}

template <class Atom, class MA, class MB, class MC, class... Epilogue>
void ref_matmul(nint_t m, nint_t n, nint_t k, const MA* a, nint_t lda, const MB* b, nint_t ldb, MC* c, nint_t ldc,
                Epilogue... epilogue) {
  auto at = make_tensor(a, make_layout(make_shape(Any{m}, Any{k}), make_strides(Any{lda}, cint<1>)));
  auto bt = make_tensor(b, make_layout(make_shape(Any{n}, Any{k}), make_strides(Any{ldb}, cint<1>)));
  auto ct = make_tensor(c, make_layout(make_shape(Any{m}, Any{n}), make_strides(Any{ldc}, cint<1>)));
  auto ai = input<typename Atom::TA>(at);
  auto bi = input<typename Atom::TB>(bt);
  auto co = output<typename Atom::TAcc>(ct, epilogue...);
  auto op = ops::matmul(ops::MatmulConfig<Atom>{});
  kernel::Workspace storage(op.required_workspace(Any{m}, Any{n}, Any{k}, ai, bi, co));
  auto view = storage.view();
  op(view, Any{m}, Any{n}, Any{k}, ai, bi, co);
}

// Run `body(n0, n1)` over [0, n) split across `threads` workers in multiples
// of 16 columns (the AMX tile width), each worker with its own AMX permission:
// the way the reference means callers to use all cores (one matmul per lane on
// a sub-view, docs/WorkspacePlanning.md:96-110).
template <class Body>
void over_columns(nint_t n, int threads, Body body) {
  threads = std::max(1, threads);
  if (threads == 1) {
    body(nint_t{0}, n);
    return;
  }
  const nint_t blocks = (n + 15) / 16;
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t) {
    const nint_t n0 = std::min(n, (blocks * t / threads) * 16);
    const nint_t n1 = std::min(n, (blocks * (t + 1) / threads) * 16);
    if (n1 <= n0) continue;
    pool.emplace_back([=] {
      request_amx();
      body(n0, n1);
    });
  }
  for (auto& worker : pool) worker.join();
}

}  // namespace

extern "C" {

int ref_available(void) { return request_amx() ? 1 : 0; }

// bf16 x bf16 -> f32 accumulate -> bf16 (c_is_bf16) or f32.  AMX_BF16F32.
int ref_matmul_bf16(int64_t m, int64_t n, int64_t k, const uint16_t* a, int64_t lda, const uint16_t* b, int64_t ldb,
                    void* c, int64_t ldc, int c_is_bf16, int threads) {
  if (!request_amx()) return 1;
  over_columns(n, threads, [=](nint_t n0, nint_t n1) {
    const auto* ap = reinterpret_cast<const bfloat16_t*>(a);
    const auto* bp = reinterpret_cast<const bfloat16_t*>(b) + n0 * ldb;
    if (c_is_bf16)
      ref_matmul<matmul::AMX_BF16F32>(m, n1 - n0, k, ap, lda, bp, ldb, reinterpret_cast<bfloat16_t*>(c) + n0, ldc);
    else
      ref_matmul<matmul::AMX_BF16F32>(m, n1 - n0, k, ap, lda, bp, ldb, reinterpret_cast<float*>(c) + n0, ldc);
  });
  return 0;
}

// 8-bit x 8-bit -> int32.  AMX_I8I32<A,B> for the four signedness pairs.
int ref_matmul_i8(int64_t m, int64_t n, int64_t k, const void* a, int64_t lda, int a_signed, const void* b, int64_t ldb,
                  int b_signed, int32_t* c, int64_t ldc, int threads) {
  if (!request_amx()) return 1;
  over_columns(n, threads, [=](nint_t n0, nint_t n1) {
    int32_t* cp = c + n0;
    if (a_signed && b_signed)
      ref_matmul<matmul::AMX_I8I32<int8_t, int8_t>>(m, n1 - n0, k, static_cast<const int8_t*>(a), lda,
                                                    static_cast<const int8_t*>(b) + n0 * ldb, ldb, cp, ldc);
    else if (a_signed)
      ref_matmul<matmul::AMX_I8I32<int8_t, uint8_t>>(m, n1 - n0, k, static_cast<const int8_t*>(a), lda,
                                                     static_cast<const uint8_t*>(b) + n0 * ldb, ldb, cp, ldc);
    else if (b_signed)
      ref_matmul<matmul::AMX_I8I32<uint8_t, int8_t>>(m, n1 - n0, k, static_cast<const uint8_t*>(a), lda,
                                                     static_cast<const int8_t*>(b) + n0 * ldb, ldb, cp, ldc);
    else
      ref_matmul<matmul::AMX_I8I32<uint8_t, uint8_t>>(m, n1 - n0, k, static_cast<const uint8_t*>(a), lda,
                                                      static_cast<const uint8_t*>(b) + n0 * ldb, ldb, cp, ldc);
  });
  return 0;
}

// Weight-only int8: bf16 activations, int8 weights read as the bf16 compute
// type, per-column f32 scale in the epilogue, bf16 store.  `scale` must have
// 64 readable floats past n (the epilogue loads whole vectors, as the
// reference tests allocate n + 64: MatmulConversionTestCommon.h:636-646).
int ref_matmul_w8(int64_t m, int64_t n, int64_t k, const uint16_t* a, int64_t lda, const int8_t* w, int64_t ldw,
                  const float* scale, uint16_t* c, int64_t ldc, int threads) {
  if (!request_amx()) return 1;
  over_columns(n, threads, [=](nint_t n0, nint_t n1) {
    const float* scales = scale + n0;
    auto epilogue = make_lane_local_vec_transform<float32_t, float32_t>(
        [scales](auto tag, auto value, const auto& context) VECOPS_KERNEL_LAMBDA {
          const auto coordinate = context.lane_coord(0);
          const nint_t column = coordinate[coordinate.size() - 1];
          return vec::mul(tag, value, vec::load(tag, scales + column));
        });
    ref_matmul<matmul::AMX_BF16F32>(m, n1 - n0, k, reinterpret_cast<const bfloat16_t*>(a), lda, w + n0 * ldw, ldw,
                                    reinterpret_cast<bfloat16_t*>(c) + n0, ldc, epilogue);
  });
  return 0;
}

// Fused forms (the reference's explicit accumulate form COut = transform(CIn + A.B^T), ops/Matmul.h:519-570, with the
// transforms its fusion tests compose: MatmulConversionTestCommon.h:623-704 scale, :705-770 bias + clamp, :1028-1160
// relu / sigmoid / silu).  One transform covers them: value * alpha * column_scale[col], then the activation.
// act: 0 none, 1 relu, 2 sigmoid, 3 silu, 4 clamp(lo, hi).  cin may be null (zero accumulator input).
int ref_matmul_bf16_fused(int64_t m, int64_t n, int64_t k, const uint16_t* a, int64_t lda, const uint16_t* b, int64_t ldb,
                          const float* cin, int64_t cin_sm, int64_t cin_sn, float alpha, const float* scale, int act, float lo,
                          float hi, void* c, int64_t ldc, int c_is_bf16) {
  if (!request_amx()) return 1;
  auto transform = make_lane_local_vec_transform<float32_t, float32_t>(
      [=](auto tag, auto value, const auto& context) VECOPS_KERNEL_LAMBDA {
        const auto coordinate = context.lane_coord(0);
        const nint_t column = coordinate[coordinate.size() - 1];
        auto x = vec::mul(tag, value, vec::fill(tag, alpha));
        if (scale != nullptr) x = vec::mul(tag, x, vec::load(tag, scale + column));
        const auto one = vec::fill(tag, 1.0f);
        if (act == 1) x = vec::max(tag, x, vec::fill(tag, 0.0f));
        if (act == 2) x = vec::div(tag, one, vec::add(tag, one, vec::exp(tag, vec::neg(tag, x))));
        if (act == 3) x = vec::mul(tag, x, vec::div(tag, one, vec::add(tag, one, vec::exp(tag, vec::neg(tag, x)))));
        if (act == 4) x = vec::min(tag, vec::max(tag, x, vec::fill(tag, lo)), vec::fill(tag, hi));
        return x;
      });
  const auto* ap = reinterpret_cast<const bfloat16_t*>(a);
  const auto* bp = reinterpret_cast<const bfloat16_t*>(b);
  auto at = make_tensor(ap, make_layout(make_shape(Any{m}, Any{k}), make_strides(Any{lda}, cint<1>)));
  auto bt = make_tensor(bp, make_layout(make_shape(Any{n}, Any{k}), make_strides(Any{ldb}, cint<1>)));
  auto ai = input<bfloat16_t>(at);
  auto bi = input<bfloat16_t>(bt);
  auto op = ops::matmul(ops::MatmulConfig<matmul::AMX_BF16F32>{});
  auto run = [&](auto co) {
    if (cin != nullptr) {
      auto cint_tensor = make_tensor(cin, make_layout(make_shape(Any{m}, Any{n}), make_strides(Any{cin_sm}, Any{cin_sn})));
      auto ci = input<float32_t>(cint_tensor);
      kernel::Workspace storage(op.required_workspace(Any{m}, Any{n}, Any{k}, ai, bi, ci, co));
      auto view = storage.view();
      op(view, Any{m}, Any{n}, Any{k}, ai, bi, ci, co);
    } else {
      kernel::Workspace storage(op.required_workspace(Any{m}, Any{n}, Any{k}, ai, bi, co));
      auto view = storage.view();
      op(view, Any{m}, Any{n}, Any{k}, ai, bi, co);
    }
  };
  if (c_is_bf16) {
    auto ct = make_tensor(reinterpret_cast<bfloat16_t*>(c), make_layout(make_shape(Any{m}, Any{n}), make_strides(Any{ldc}, cint<1>)));
    run(output<float32_t>(ct, transform));
  } else {
    auto ct = make_tensor(reinterpret_cast<float*>(c), make_layout(make_shape(Any{m}, Any{n}), make_strides(Any{ldc}, cint<1>)));
    run(output<float32_t>(ct, transform));
  }
  return 0;
}

// Native integer accumulate (MatmulConversionTestCommon.h check_native_integer_accumulate): C = Cin + A.B^T in int32.
int ref_matmul_i8_accumulate(int64_t m, int64_t n, int64_t k, const int8_t* a, int64_t lda, const int8_t* b, int64_t ldb,
                             const int32_t* cin, int64_t cin_sm, int64_t cin_sn, int32_t* c, int64_t ldc) {
  if (!request_amx()) return 1;
  auto at = make_tensor(a, make_layout(make_shape(Any{m}, Any{k}), make_strides(Any{lda}, cint<1>)));
  auto bt = make_tensor(b, make_layout(make_shape(Any{n}, Any{k}), make_strides(Any{ldb}, cint<1>)));
  auto ct = make_tensor(c, make_layout(make_shape(Any{m}, Any{n}), make_strides(Any{ldc}, cint<1>)));
  auto cin_tensor = make_tensor(cin, make_layout(make_shape(Any{m}, Any{n}), make_strides(Any{cin_sm}, Any{cin_sn})));
  auto ai = input<int8_t>(at);
  auto bi = input<int8_t>(bt);
  auto ci = input<int32_t>(cin_tensor);
  auto co = output<int32_t>(ct);
  auto op = ops::matmul(ops::MatmulConfig<matmul::AMX_I8I32<int8_t, int8_t>>{});
  kernel::Workspace storage(op.required_workspace(Any{m}, Any{n}, Any{k}, ai, bi, ci, co));
  auto view = storage.view();
  op(view, Any{m}, Any{n}, Any{k}, ai, bi, ci, co);
  return 0;
}

// The asymmetric quantised form as the reference ships it (tests/ops/MatmulConversionTestCommon.h:501-618
// check_asymmetric_quantized): fp32 A quantised on load to u8 (value * a_scale + a_zero_point, converted like the
// reference converts), s8 B read directly, an int32 correction row (-zero_point * column sums of B) as the accumulator
// input, and a dequantising output transform (accumulator * dequant) to an fp32 C.  AMX_I8I32<uint8_t, int8_t>.
int ref_matmul_quantized_u8s8(int64_t m, int64_t n, int64_t k, const float* a, int64_t lda, float a_scale, float a_zero_point,
                              const int8_t* b, int64_t ldb, const int32_t* correction, float dequant, float* c, int64_t ldc) {
  if (!request_amx()) return 1;
  auto at = make_tensor(a, make_layout(make_shape(Any{m}, Any{k}), make_strides(Any{lda}, cint<1>)));
  auto bt = make_tensor(b, make_layout(make_shape(Any{n}, Any{k}), make_strides(Any{ldb}, cint<1>)));
  auto ct = make_tensor(c, make_layout(make_shape(Any{m}, Any{n}), make_strides(Any{ldc}, cint<1>)));
  auto correction_tensor = make_tensor(correction, make_layout(make_shape(Any{m}, Any{n}), make_strides(cint<0>, cint<1>)));
  auto quantize_a = make_elementwise_vec_transform<float32_t, float32_t>([=](auto tag, auto value) VECOPS_KERNEL_LAMBDA {
    return vec::add(tag, vec::mul(tag, value, vec::fill(tag, a_scale)), vec::fill(tag, a_zero_point));
  });
  auto dequantize = make_elementwise_vec_transform<float32_t, float32_t>([=](auto tag, auto value) VECOPS_KERNEL_LAMBDA {
    return vec::mul(tag, value, vec::fill(tag, dequant));
  });
  auto ai = input<uint8_t>(at, quantize_a);
  auto bi = input<int8_t>(bt);
  auto ci = input<int32_t>(correction_tensor);
  auto co = output<int32_t>(ct, dequantize);
  auto op = ops::matmul(ops::MatmulConfig<matmul::AMX_I8I32<uint8_t, int8_t>>{});
  kernel::Workspace storage(op.required_workspace(Any{m}, Any{n}, Any{k}, ai, bi, ci, co));
  auto view = storage.view();
  op(view, Any{m}, Any{n}, Any{k}, ai, bi, ci, co);
  return 0;
}

// Per-token quantisation with the reference's own named transforms (include/vecops/matmul/Quantization.h:76-246; call
// form of tests/ops/MatmulConversionTestCommon.h:1384-1401): fp32 A quantised on load to u8 with one multiplier per
// row and a shared int32 zero point, s8 B, the int32 correction row as the accumulator input, and the row-by-column
// dequantising output transform.  `column_scales` needs 64 readable floats past n (the transform loads whole vectors).
int ref_matmul_quantized_per_row(int64_t m, int64_t n, int64_t k, const float* a, int64_t lda, const float* multipliers, int32_t zero_point,
                                 const int8_t* b, int64_t ldb, const int32_t* correction, const float* row_scales,
                                 const float* column_scales, float* c, int64_t ldc) {
  if (!request_amx()) return 1;
  auto at = make_tensor(a, make_layout(make_shape(Any{m}, Any{k}), make_strides(Any{lda}, cint<1>)));
  auto bt = make_tensor(b, make_layout(make_shape(Any{n}, Any{k}), make_strides(Any{ldb}, cint<1>)));
  auto ct = make_tensor(c, make_layout(make_shape(Any{m}, Any{n}), make_strides(Any{ldc}, cint<1>)));
  auto correction_tensor = make_tensor(correction, make_layout(make_shape(Any{m}, Any{n}), make_strides(cint<0>, cint<1>)));
  auto quantize_a = ::vecops::matmul::make_runtime_per_row_asymmetric_quantize_transform({multipliers, &zero_point, nint_t{0}});
  auto dequantize = ::vecops::matmul::make_runtime_per_row_column_dequantize_transform({row_scales, column_scales, nint_t{0}});
  auto ai = input<uint8_t>(at, quantize_a);
  auto bi = input<int8_t>(bt);
  auto ci = input<int32_t>(correction_tensor);
  auto co = output<int32_t>(ct, dequantize);
  auto op = ops::matmul(ops::MatmulConfig<matmul::AMX_I8I32<uint8_t, int8_t>>{});
  kernel::Workspace storage(op.required_workspace(Any{m}, Any{n}, Any{k}, ai, bi, ci, co));
  auto view = storage.view();
  op(view, Any{m}, Any{n}, Any{k}, ai, bi, ci, co);
  return 0;
}

// Rank-3 operands: a leading batch axis on A, B and C, any of whose strides may be 0 (a shared A, or shared weights), as
// in tests/ops/MatmulBatchTest.cpp:96-131; `bias` (optional, [N]) enters as the accumulator input with strides (0, 0, 1).
int ref_matmul_bf16_batched(int64_t batch, int64_t m, int64_t n, int64_t k, const uint16_t* a, int64_t a_sb, int64_t lda,
                            const uint16_t* b, int64_t b_sb, int64_t ldb, const float* bias, float* c, int64_t c_sb, int64_t ldc) {
  if (!request_amx()) return 1;
  auto at = make_tensor(reinterpret_cast<const bfloat16_t*>(a),
                        make_layout(make_shape(Any{batch}, Any{m}, Any{k}), make_strides(Any{a_sb}, Any{lda}, cint<1>)));
  auto bt = make_tensor(reinterpret_cast<const bfloat16_t*>(b),
                        make_layout(make_shape(Any{batch}, Any{n}, Any{k}), make_strides(Any{b_sb}, Any{ldb}, cint<1>)));
  auto ct = make_tensor(c, make_layout(make_shape(Any{batch}, Any{m}, Any{n}), make_strides(Any{c_sb}, Any{ldc}, cint<1>)));
  auto ai = input<bfloat16_t>(at);
  auto bi = input<bfloat16_t>(bt);
  auto co = output<float32_t>(ct);
  auto op = ops::matmul(ops::MatmulConfig<matmul::AMX_BF16F32>{});
  if (bias != nullptr) {
    auto bias_tensor = make_tensor(bias, make_layout(make_shape(Any{batch}, Any{m}, Any{n}), make_strides(cint<0>, cint<0>, cint<1>)));
    auto ci = input<float32_t>(bias_tensor);
    kernel::Workspace storage(op.required_workspace(Any{m}, Any{n}, Any{k}, ai, bi, ci, co));
    auto view = storage.view();
    op(view, Any{m}, Any{n}, Any{k}, ai, bi, ci, co);
  } else {
    kernel::Workspace storage(op.required_workspace(Any{m}, Any{n}, Any{k}, ai, bi, co));
    auto view = storage.view();
    op(view, Any{m}, Any{n}, Any{k}, ai, bi, co);
  }
  return 0;
}

// fp32: the reference has no fp32 matmul atom on x86; its only fp32 x fp32
// product code is the AVX-512 vector leaf (amx/Backend.h:767-901) instantiated
// with equal types.  B is [N,K] here.
int ref_matmul_f32_leaf(int64_t m, int64_t n, int64_t k, const float* a, int64_t lda, const float* b, int64_t ldb,
                        float* c, int64_t ldc, int threads) {
  over_columns(n, threads, [=](nint_t n0, nint_t n1) {
    kernel::matmul_details::amx::small_vector_dense_matmul<false, float, float, float>(a, lda, b + n0 * ldb, ldb, c + n0,
                                                                                       ldc, m, n1 - n0, k);
  });
  return 0;
}

// ops::matmul_pack_b_compensated (ops/MatmulPack.h:28-35): packs a signed 8-bit B[N,K] into the AMX blocked layout and
// emits compensation[n] = -a_zero_point * sum_k B[n,k].  The packed bytes are in the reference's own tile layout and are
// discarded here; the compensation row does not depend on that layout and is what the caller gets.  Call form as in the
// header's usage note and tests/ops/MatmulPackTest.cpp:157-186.
int ref_pack_b_compensated(int64_t n, int64_t k, const int8_t* b, int64_t ldb, int32_t a_zero_point, int32_t* compensation) {
  using Atom = matmul::AMX_I8I32<uint8_t, int8_t>;
  if (!request_amx()) return 1;
  auto layout = make_layout(make_shape(Any{n}, Any{k}), make_strides(Any{ldb}, cint<1>));
  auto input_tensor = make_tensor(b, layout);
  auto packed_layout = matmul::packed_layout<Atom, matmul::Operand::B>(layout);
  std::vector<int8_t> packed(static_cast<size_t>(numel(packed_layout)) + 64);
  auto* aligned = reinterpret_cast<int8_t*>((reinterpret_cast<uintptr_t>(packed.data()) + 63) & ~uintptr_t{63});
  auto output_tensor = make_tensor(aligned, packed_layout);
  auto compensation_tensor = make_tensor(compensation, make_layout(make_shape(Any{n})));
  auto op = ops::matmul_pack_b_compensated(ops::MatmulPackBCompensatedConfig<Atom>{.a_zero_point = a_zero_point});
  ExecutionSession execution{};
  op(execution, input_tensor, output_tensor, compensation_tensor);
  return 0;
}

// float16_t's own conversions (util/Float16.h:272-277), element by element: the part of the fp16 row that runs on
// a host without AMX-FP16.
void ref_f16_widen(const uint16_t* src, float* dst, int64_t count) {
  for (int64_t i = 0; i < count; ++i) dst[i] = static_cast<float>(float16_t::from_bits(src[i]));
}
void ref_f16_narrow(const float* src, uint16_t* dst, int64_t count) {
  for (int64_t i = 0; i < count; ++i) dst[i] = float16_t(src[i]).to_bits();
}

}  // extern "C"

// The reference's scaled dot-product attention for one head (ops/details/attention/SDPA.h:72-84), materialized strategy:
// Q[Lq,Dqk], K[Lkv,Dqk], V[Lkv,Dv] bf16, out[Lq,Dv] f32.  Call forms as in tests/ops/AttentionTest.cpp:238-241 (plain) and
// :603-607 (query mask, key mask, keep mask, bias - all four or none).  causal: 0 none, 1 top_left, 2 bottom_right.
template <ops::AttentionCausalMode Causal, ops::SDPAStrategy Strategy = ops::SDPAStrategy::materialized, int KeyValueBlock = 32>
static int ref_sdpa_typed(int64_t lq, int64_t lkv, int64_t dqk, int64_t dv, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                          const uint8_t* query_mask, const uint8_t* key_mask, const uint8_t* keep_mask, const float* bias, float scale,
                          float* out) {
  using Config = ops::AttentionConfig<ops::MatmulConfig<matmul::AMX_BF16F32>, 32, KeyValueBlock, Causal, Strategy>;
  auto qt = make_tensor(reinterpret_cast<const bfloat16_t*>(q), make_shape(Any{lq}, Any{dqk}));
  auto kt = make_tensor(reinterpret_cast<const bfloat16_t*>(k), make_shape(Any{lkv}, Any{dqk}));
  auto vt = make_tensor(reinterpret_cast<const bfloat16_t*>(v), make_shape(Any{lkv}, Any{dv}));
  auto ot = make_tensor(out, make_shape(Any{lq}, Any{dv}));
  auto op = ops::scaled_dot_product_attention(Config{});
  if (query_mask == nullptr) {
    kernel::Workspace storage(op.required_workspace(qt, kt, vt, ot));
    auto workspace = storage.view();
    op(workspace, qt, kt, vt, ot, scale);
    return 0;
  }
  auto qmt = make_tensor(reinterpret_cast<const bool*>(query_mask), make_shape(Any{lq}));
  auto kmt = make_tensor(reinterpret_cast<const bool*>(key_mask), make_shape(Any{lkv}));
  auto amt = make_tensor(reinterpret_cast<const bool*>(keep_mask), make_shape(Any{lq}, Any{lkv}));
  auto bt = make_tensor(bias, make_shape(Any{lq}, Any{lkv}));
  kernel::Workspace storage(op.required_workspace(qt, kt, vt, qmt, kmt, amt, bt, ot));
  auto workspace = storage.view();
  op(workspace, qt, kt, vt, qmt, kmt, amt, bt, ot, scale);
  return 0;
}

extern "C" {

int ref_sdpa_bf16(int64_t lq, int64_t lkv, int64_t dqk, int64_t dv, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                  const uint8_t* query_mask, const uint8_t* key_mask, const uint8_t* keep_mask, const float* bias, int causal, float scale,
                  float* out) {
  if (!request_amx()) return 1;
  if ((query_mask == nullptr) != (key_mask == nullptr) || (query_mask == nullptr) != (keep_mask == nullptr) ||
      (query_mask == nullptr) != (bias == nullptr))
    return 2;  // this door passes all four optional operands or none
  if (causal == 1) return ref_sdpa_typed<ops::AttentionCausalMode::top_left>(lq, lkv, dqk, dv, q, k, v, query_mask, key_mask, keep_mask, bias, scale, out);
  if (causal == 2) return ref_sdpa_typed<ops::AttentionCausalMode::bottom_right>(lq, lkv, dqk, dv, q, k, v, query_mask, key_mask, keep_mask, bias, scale, out);
  return ref_sdpa_typed<ops::AttentionCausalMode::none>(lq, lkv, dqk, dv, q, k, v, query_mask, key_mask, keep_mask, bias, scale, out);
}

// The same call with the streaming strategy (SDPA.h:21-25; SparseFlashAttention.h:360-545 over every key/value block):
// keys walked in blocks of 128 with a running maximum and sum, probabilities rounded to bf16 before normalisation.
int ref_sdpa_bf16_streaming(int64_t lq, int64_t lkv, int64_t dqk, int64_t dv, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                            const uint8_t* query_mask, const uint8_t* key_mask, const uint8_t* keep_mask, const float* bias, int causal,
                            float scale, float* out) {
  if (!request_amx()) return 1;
  if ((query_mask == nullptr) != (key_mask == nullptr) || (query_mask == nullptr) != (keep_mask == nullptr) ||
      (query_mask == nullptr) != (bias == nullptr))
    return 2;
  constexpr auto streaming = ops::SDPAStrategy::streaming;
  if (causal == 1)
    return ref_sdpa_typed<ops::AttentionCausalMode::top_left, streaming, 128>(lq, lkv, dqk, dv, q, k, v, query_mask, key_mask, keep_mask, bias, scale, out);
  if (causal == 2)
    return ref_sdpa_typed<ops::AttentionCausalMode::bottom_right, streaming, 128>(lq, lkv, dqk, dv, q, k, v, query_mask, key_mask, keep_mask, bias, scale, out);
  return ref_sdpa_typed<ops::AttentionCausalMode::none, streaming, 128>(lq, lkv, dqk, dv, q, k, v, query_mask, key_mask, keep_mask, bias, scale, out);
}

}  // extern "C"
