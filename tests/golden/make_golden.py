"""Generate tests/golden/*.npz by running the reference's own CPU matmul.

Needs the reference checkout (to build oracle/_ref) and a CPU with AMX; the
fixtures it writes are committed, so neither is needed to run the tests.

Inputs follow the reference tests' own deterministic patterns:
  value<T>(i, modulus)        tests/ops/MatmulTest.cpp:36-41   (a: modulus 13, b: modulus 11, :63-64)
  conversion_value<T>(i, s)   tests/ops/MatmulConversionTestCommon.h:62-70
on shapes the reference tests use (K tails, ragged M/N, all int8 signedness
pairs, GEMV orientations: MatmulTest.cpp:434-452, :1005-1023).

    python tests/golden/make_golden.py
"""
from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle.checker import (ACT_CLAMP, ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_SILU, Ref, f16_conversion_inputs,  # noqa: E402
                            f32_to_bf16_bits)

HERE = Path(__file__).resolve().parent


def value_pattern(count: int, modulus: int, dtype) -> np.ndarray:
    """value<T>(index, modulus): (index % modulus) - modulus / 2, scaled by 1/modulus for floats."""
    x = (np.arange(count, dtype=np.int64) % modulus) - modulus // 2
    if np.issubdtype(dtype, np.integer):
        return x.astype(dtype)
    return (x.astype(np.float32) / np.float32(modulus)).astype(np.float32)


def conversion_pattern(count: int, seed: int, dtype) -> np.ndarray:
    """conversion_value<T>(index, seed)."""
    index = np.arange(count, dtype=np.int64)
    if np.issubdtype(dtype, np.integer):
        low = 0 if np.issubdtype(dtype, np.unsignedinteger) else -3
        return (low + (index * 5 + seed) % 7).astype(dtype)
    return (((index * 7 + seed) % 17 - 8).astype(np.float32) / np.float32(16.0)).astype(np.float32)


def main() -> None:
    ref, why = Ref.load()
    if ref is None:
        raise SystemExit(f"reference matmul unavailable here: {why}")
    cases = {}

    # AMX_BF16F32, bf16 in / f32 out and bf16 out, microkernel shapes with K tails
    for m, n, k in [(16, 16, 35), (37, 51, 79), (1, 128, 65), (48, 16, 65), (64, 96, 256)]:
        a = f32_to_bf16_bits(value_pattern(m * k, 13, np.float32)).reshape(m, k)
        b = f32_to_bf16_bits(value_pattern(n * k, 11, np.float32)).reshape(n, k)
        cases[f"bf16_{m}x{n}x{k}"] = dict(kind="bf16", a=a, b=b, c_f32=ref.matmul_bf16(a, b, out_bf16=False),
                                          c_bf16=ref.matmul_bf16(a, b, out_bf16=True))

    # AMX_I8I32<A,B>, all four signedness pairs
    for (m, n, k), (ta, tb) in [((19, 21, 69), (np.int8, np.int8)), ((19, 21, 69), (np.int8, np.uint8)),
                                ((19, 21, 69), (np.uint8, np.int8)), ((19, 21, 69), (np.uint8, np.uint8)),
                                ((1, 128, 65), (np.int8, np.int8)), ((16, 1, 129), (np.uint8, np.int8)),
                                ((40, 48, 192), (np.int8, np.int8))]:
        a = value_pattern(m * k, 13, np.int16).astype(ta).reshape(m, k)
        b = value_pattern(n * k, 11, np.int16).astype(tb).reshape(n, k)
        name = f"i8_{np.dtype(ta).name}_{np.dtype(tb).name}_{m}x{n}x{k}"
        cases[name] = dict(kind="i8", a=a, b=b, c=ref.matmul_i8(a, b))

    # full-range int8 at one bigger shape (random, seeded)
    rng = np.random.default_rng(2)
    a = rng.integers(-128, 128, (33, 256), dtype=np.int8)
    b = rng.integers(-128, 128, (47, 256), dtype=np.int8)
    cases["i8_full_range_33x47x256"] = dict(kind="i8", a=a, b=b, c=ref.matmul_i8(a, b))

    # weight-only int8: bf16 activations, int8 weights, per-column scale, bf16 out
    rng = np.random.default_rng(3)
    for m, n, k in [(1, 48, 128), (16, 64, 256), (5, 33, 96)]:
        a = f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
        w = rng.integers(-127, 128, (n, k), dtype=np.int8)
        s = rng.uniform(0.001, 0.02, n).astype(np.float32)
        cases[f"w8_{m}x{n}x{k}"] = dict(kind="w8", a=a, b=w, scale=s, c_bf16=ref.matmul_w8(a, w, s))

    # fp32: the AVX-512 fmadd leaf (B as [N,K])
    for m, n, k in [(33, 40, 64), (7, 19, 50)]:
        a = conversion_pattern(m * k, 3, np.float32).reshape(m, k)
        b = conversion_pattern(n * k, 5, np.float32).reshape(n, k)
        cases[f"f32_{m}x{n}x{k}"] = dict(kind="f32", a=a, b=b, c=ref.matmul_f32_leaf(a, b))

    # fused forms: COut = activation((CIn + A.B^T) * alpha * column_scale), on the reference fusion tests' shapes and
    # input patterns (MatmulFusionTest.cpp:29-70; MatmulConversionTestCommon.h:705-770 bias + clamp, :1028-1160
    # relu / sigmoid / silu, :623-704 runtime and per-column scale)
    def fused_inputs(m, n, k):
        a = f32_to_bf16_bits(conversion_pattern(m * k, 3, np.float32)).reshape(m, k)
        b = f32_to_bf16_bits(conversion_pattern(n * k, 11, np.float32)).reshape(n, k)
        bias = (((np.arange(n) * 3) % 11 - 5) / 8.0).astype(np.float32)
        return a, b, bias

    def fused_case(name, m, n, k, cin=None, alpha=1.0, scale=None, act=ACT_NONE, lo=0.0, hi=0.0):
        a, b, bias = fused_inputs(m, n, k)
        if isinstance(cin, str):
            cin = {"bias": bias, "full": (((np.arange(m * n) * 5) % 13 - 6) / 4.0).astype(np.float32).reshape(m, n),
                   "column": (((np.arange(m) * 7) % 9 - 4) / 2.0).astype(np.float32).reshape(m, 1)}[cin]
        arrays = dict(kind="fused_bf16", a=a, b=b, alpha=np.float32(alpha), act=np.int32(act), lo=np.float32(lo), hi=np.float32(hi),
                      c_f32=ref.matmul_bf16_fused(a, b, cin, alpha, scale, act, lo, hi, out_bf16=False),
                      c_bf16=ref.matmul_bf16_fused(a, b, cin, alpha, scale, act, lo, hi, out_bf16=True))
        if cin is not None:
            arrays["cin"] = cin
        if scale is not None:
            arrays["scale"] = scale
        cases[f"fused_{name}_{m}x{n}x{k}"] = arrays

    fused_case("bias_clamp", 19, 23, 65, cin="bias", act=ACT_CLAMP, lo=-0.25, hi=0.25)
    for m, n, k in [(19, 23, 65), (1, 8, 129), (8, 1, 129)]:
        fused_case("relu", m, n, k, act=ACT_RELU)
        fused_case("sigmoid", m, n, k, act=ACT_SIGMOID)
    fused_case("silu", 1, 8, 129, act=ACT_SILU)
    fused_case("bias_silu", 1, 8, 129, cin="bias", act=ACT_SILU)
    fused_case("alpha", 19, 23, 65, alpha=0.75)
    fused_case("alpha_scale_relu_cin", 19, 23, 65, cin="full", alpha=0.75,
               scale=(0.5 + (np.arange(23) % 5) / 4.0).astype(np.float32), act=ACT_RELU)
    fused_case("column_cin", 19, 23, 65, cin="column")

    # native integer accumulate (check_native_integer_accumulate): C = CIn + A.B^T in int32
    for m, n, k in [(19, 23, 65), (1, 8, 129)]:
        a = conversion_pattern(m * k, 3, np.int8).reshape(m, k)
        b = conversion_pattern(n * k, 11, np.int8).reshape(n, k)
        cin = ((np.arange(m * n, dtype=np.int64) * 37) % 1001 - 500).astype(np.int32).reshape(m, n)
        cases[f"i8acc_{m}x{n}x{k}"] = dict(kind="i8acc", a=a, b=b, cin=cin, c=ref.matmul_i8_accumulate(a, b, cin))

    # the quantised form as shipped (check_asymmetric_quantized, MatmulConversionTestCommon.h:501-618): fp32 A quantised on
    # load to u8 (value * 4 + 3), s8 B, correction row -3 * column sums of B, dequantising transform * 0.0625, fp32 C
    for m, n, k in [(19, 23, 65), (32, 64, 128), (1, 8, 129)]:
        a = conversion_pattern(m * k, 3, np.float32).reshape(m, k)
        b = conversion_pattern(n * k, 11, np.int8).reshape(n, k)
        correction = (-3 * b.astype(np.int64).sum(axis=1)).astype(np.int32)
        cases[f"quant_u8s8_{m}x{n}x{k}"] = dict(kind="quant_u8s8", a=a, a_scale=np.float32(4.0), a_zero_point=np.float32(3.0), b=b,
                                                correction=correction, dequant=np.float32(0.0625),
                                                c=ref.matmul_quantized_u8s8(a, 4.0, 3.0, b, correction, 0.0625))
    rng = np.random.default_rng(4)  # out-of-range activations: the conversion saturates
    a = rng.uniform(-40, 80, (33, 96)).astype(np.float32)
    b = rng.integers(-128, 128, (47, 96), dtype=np.int8)
    correction = (-7 * b.astype(np.int64).sum(axis=1)).astype(np.int32)
    cases["quant_u8s8_saturating_33x47x96"] = dict(kind="quant_u8s8", a=a, a_scale=np.float32(2.5), a_zero_point=np.float32(7.0), b=b,
                                                   correction=correction, dequant=np.float32(0.01),
                                                   c=ref.matmul_quantized_u8s8(a, 2.5, 7.0, b, correction, 0.01))

    # rank-3 operands with a leading batch axis (tests/ops/MatmulBatchTest.cpp:96-131): a shared A (batch stride 0) against
    # batched B with a bias row; batched A against shared weights; everything batched
    def bf16_pattern(count, seed, shape):
        return f32_to_bf16_bits(conversion_pattern(count, seed, np.float32)).reshape(shape)

    batch, m, n, k = 3, 5, 23, 65
    a = bf16_pattern(m * k, 3, (m, k))
    b = bf16_pattern(batch * n * k, 11, (batch, n, k))
    bias = conversion_pattern(n, 5, np.float32)
    cases["batched_shared_a_bias_3x5x23x65"] = dict(kind="batched_bf16", a=a, b=b, bias=bias, shared=np.array("a"),
                                                    c=ref.matmul_bf16_batched(np.broadcast_to(a, (batch, m, k)), b, bias))
    a = bf16_pattern(batch * m * k, 3, (batch, m, k))
    b = bf16_pattern(n * k, 11, (n, k))
    cases["batched_shared_b_3x5x23x65"] = dict(kind="batched_bf16", a=a, b=b, shared=np.array("b"),
                                               c=ref.matmul_bf16_batched(a, np.broadcast_to(b, (batch, n, k))))
    batch, m, n, k = 4, 19, 21, 72
    a = bf16_pattern(batch * m * k, 3, (batch, m, k))
    b = bf16_pattern(batch * n * k, 11, (batch, n, k))
    cases["batched_4x19x21x72"] = dict(kind="batched_bf16", a=a, b=b, shared=np.array(""), c=ref.matmul_bf16_batched(a, b))

    # scaled dot-product attention, one head (ops/details/attention/SDPA.h): the reference tests' own operand patterns
    # (tests/ops/AttentionTest.cpp:256-286 tail shapes; :568-612 masks, bias and a fully masked query row) and seeded cases
    # with causal modes
    def attention_case(name, q, k, v, scale, causal=0, **optional):
        out = ref.sdpa_bf16(q, k, v, scale, causal=causal, **optional)
        # the same call by the reference's streaming strategy (key blocks of 128): probabilities are rounded to bf16 before
        # the normalisation there, after it in the materialized strategy, so the two outputs differ by 2e-3 .. 4e-3
        out_streaming = ref.sdpa_bf16(q, k, v, scale, causal=causal, streaming=True, **optional)
        cases[name] = dict(kind="sdpa_bf16", q=q, k=k, v=v, scale=np.float32(scale), causal=np.int32(causal), out=out,
                           out_streaming=out_streaming, **optional)

    lq, lkv, dqk, dv = 5, 7, 8, 6
    q = f32_to_bf16_bits((((np.arange(lq * dqk) * 3) % 11 - 5) / 8).astype(np.float32)).reshape(lq, dqk)
    k = f32_to_bf16_bits((((np.arange(lkv * dqk) * 5) % 13 - 6) / 8).astype(np.float32)).reshape(lkv, dqk)
    v = f32_to_bf16_bits((((np.arange(lkv * dv) * 7) % 17 - 8) / 16).astype(np.float32)).reshape(lkv, dv)
    attention_case("sdpa_tail_5x7x8x6", q, k, v, 0.375)
    lq, lkv, d = 3, 5, 8
    q = f32_to_bf16_bits(np.full((lq, d), 0.25, np.float32))
    k = f32_to_bf16_bits(np.full((lkv, d), 0.5, np.float32))
    v = f32_to_bf16_bits(((np.arange(lkv * d) % 9 - 4) / 8).astype(np.float32)).reshape(lkv, d)
    keep = np.ones((lq, lkv), np.uint8)
    keep[2, 3] = 0
    attention_case("sdpa_masks_bias_3x5x8x8", q, k, v, 0.5, query_mask=np.array([1, 0, 1], np.uint8), key_mask=np.array([1, 1, 0, 1, 1], np.uint8),
                   keep_mask=keep, bias=((np.arange(lq * lkv) % lkv) * 0.125).astype(np.float32).reshape(lq, lkv))
    rng = np.random.default_rng(41)
    for name, (lq, lkv, dqk, dv), causal, optional in [("sdpa_bottom_right_33x70x16x24", (33, 70, 16, 24), 2, False),
                                                         ("sdpa_top_left_40x40x64x64", (40, 40, 64, 64), 1, False),
                                                         ("sdpa_masks_bottom_right_37x53x32x40", (37, 53, 32, 40), 2, True),
                                                         ("sdpa_masks_130x257x64x64", (130, 257, 64, 64), 0, True)]:
        q = f32_to_bf16_bits(rng.standard_normal((lq, dqk)).astype(np.float32))
        k = f32_to_bf16_bits(rng.standard_normal((lkv, dqk)).astype(np.float32))
        v = f32_to_bf16_bits(rng.standard_normal((lkv, dv)).astype(np.float32))
        extra = {}
        if optional:
            extra = dict(query_mask=(rng.random(lq) > 0.2).astype(np.uint8), key_mask=(rng.random(lkv) > 0.2).astype(np.uint8),
                         keep_mask=(rng.random((lq, lkv)) > 0.1).astype(np.uint8), bias=rng.uniform(-1, 1, (lq, lkv)).astype(np.float32))
        attention_case(name, q, k, v, 1.0 / np.sqrt(dqk), causal, **extra)

    # per-token quantisation with the reference's named transforms (matmul/Quantization.h:76-246): the reference test's own
    # operand pattern (tests/ops/MatmulConversionTestCommon.h:1455-1480: multipliers 4 << (row % 2), logical values
    # ((row*k + kk) % 7 - 3) / multiplier, zero point 7, column scales 0.03125 + (col % 5) / 128) and a seeded case
    def per_row_case(name, a, multipliers, zero_point, b, row_scales, column_scales):
        correction = (-zero_point * b.astype(np.int64).sum(axis=1)).astype(np.int32)
        cases[name] = dict(kind="quant_per_row", a=a, multipliers=multipliers, zero_point=np.int32(zero_point), b=b, correction=correction,
                           row_scales=row_scales, column_scales=column_scales,
                           c=ref.matmul_quantized_per_row(a, multipliers, zero_point, b, correction, row_scales, column_scales))

    for m, n, k in [(19, 23, 65), (1, 8, 129), (33, 47, 96)]:
        multipliers = np.array([4 << (r % 2) for r in range(m)], np.float32)
        a = (((np.arange(m * k) % 7) - 3).reshape(m, k) / multipliers[:, None]).astype(np.float32)
        b = conversion_pattern(n * k, 11, np.int8).reshape(n, k)
        per_row_case(f"quant_per_row_{m}x{n}x{k}", a, multipliers, 7, b, (1.0 / multipliers).astype(np.float32),
                     (0.03125 + (np.arange(n) % 5) * 0.0078125).astype(np.float32))
    rng = np.random.default_rng(43)
    m, n, k = 37, 51, 128
    multipliers = rng.uniform(10, 40, m).astype(np.float32)
    per_row_case("quant_per_row_seeded_37x51x128", rng.uniform(-3, 3, (m, k)).astype(np.float32), multipliers, 100,
                 rng.integers(-128, 128, (n, k), dtype=np.int8), (1.0 / multipliers).astype(np.float32), rng.uniform(0.01, 0.05, n).astype(np.float32))

    # ops::matmul_pack_b_compensated (ops/MatmulPack.h:28-35): the compensation row -a_zero_point * sum_k B[n,k], which does
    # not depend on the packed layout.  The reference test's own case (tests/ops/MatmulPackTest.cpp:354-376: N=33, K=129,
    # values (n*17 + k*3) % 61 - 30, zero point 3, rows on a pitch of K+3) and seeded ones with extreme values and a long K
    def compensation_case(name, b, zero_point):  # `b` may be a view with a row pitch larger than K
        cases[name] = dict(kind="pack_comp", b=np.ascontiguousarray(b), zero_point=np.int32(zero_point),
                           compensation=ref.pack_compensation(b, zero_point))

    n, k = 33, 129
    storage = np.full((n, k + 3), -99, dtype=np.int8)
    storage[:, :k] = ((np.arange(n)[:, None] * 17 + np.arange(k)[None, :] * 3) % 61 - 30).astype(np.int8)
    compensation_case("pack_comp_33x129_zp3", storage[:, :k], 3)
    rng = np.random.default_rng(47)
    compensation_case("pack_comp_seeded_24x4099_zp128", rng.integers(-128, 128, (24, 4099), dtype=np.int8), 128)
    extreme = np.full((19, 512), -128, dtype=np.int8)
    extreme[1::2] = 127
    compensation_case("pack_comp_extremes_19x512_zp255", extreme, 255)
    compensation_case("pack_comp_zero_point_0_16x64", rng.integers(-128, 128, (16, 64), dtype=np.int8), 0)

    # float16_t's widening and narrowing (util/Float16.h:272-277) over the whole sweep, as digests: the part of the
    # AMX_F16F32 row a host without AMX-FP16 can run
    patterns, floats = f16_conversion_inputs()
    cases["f16_conversions"] = dict(kind="f16_convert",
                                    widen_sha256=np.array(hashlib.sha256(ref.f16_widen(patterns).tobytes()).hexdigest()),
                                    narrow_sha256=np.array(hashlib.sha256(ref.f16_narrow(floats).tobytes()).hexdigest()))

    for name, arrays in cases.items():
        kind = arrays.pop("kind")
        np.savez_compressed(HERE / f"{name}.npz", kind=np.array(kind), **arrays)
    total = sum(p.stat().st_size for p in HERE.glob("*.npz"))
    print(f"wrote {len(cases)} fixtures, {total / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
