"""The CPU checker against the reference: committed fixtures (outputs of the
reference's own ops::matmul) and, where this host can run it, the reference
library itself."""
import hashlib

import numpy as np
import pytest

from oracle.checker import Ref, bf16_bits_to_f32, f16_conversion_inputs, f32_to_bf16_bits, rel_frobenius
from tests.helpers import TOL_BF16, TOL_F32


def test_bf16_rounding_rule(port):
    # round-to-nearest-even on the bit pattern, NaN -> 0x7fc0 (util/BFloat16.h:25-37)
    samples = np.array([0.0, -0.0, 1.0, 1.00390625, 1.005859375, 3.14159265, -2.5e-40, 6.5e4, 3.38e38, np.inf, -np.inf],
                       dtype=np.float32)
    bits = f32_to_bf16_bits(samples)
    for value, got in zip(samples, bits):
        assert port.lib.oracle_f32_to_bf16(float(value)) == int(got)
    assert f32_to_bf16_bits(np.array([np.nan], dtype=np.float32))[0] == 0x7FC0
    assert port.lib.oracle_f32_to_bf16(float("nan")) == 0x7FC0
    # ties go to even: 1 + 2^-8 is exactly between 1.0 and 1 + 2^-7
    assert f32_to_bf16_bits(np.array([1.00390625], dtype=np.float32))[0] == 0x3F80
    assert f32_to_bf16_bits(np.array([1.01171875], dtype=np.float32))[0] == 0x3F82


def test_port_matches_golden_fixtures(port, golden):
    checked = 0
    for name, case in golden.items():
        kind = str(case["kind"])
        if kind == "f16_convert":
            # float16_t's own conversions, recorded as digests over the whole sweep (every pattern, every tie)
            patterns, floats = f16_conversion_inputs()
            assert hashlib.sha256(port.f16_widen(patterns).tobytes()).hexdigest() == str(case["widen_sha256"]), name
            assert hashlib.sha256(port.f16_narrow(floats).tobytes()).hexdigest() == str(case["narrow_sha256"]), name
            checked += 1
            continue
        if kind == "sdpa_bf16":
            # the caller one step up: outputs of the reference's own attention (materialized strategy)
            got = port.sdpa_bf16(case["q"], case["k"], case["v"], float(case["scale"]), case.get("query_mask"), case.get("key_mask"),
                                 case.get("keep_mask"), case.get("bias"), int(case["causal"]))
            assert rel_frobenius(got, case["out"]) <= 1e-5, name  # the reference's fast exp is the only difference
            assert np.array_equal((got == 0).all(axis=1), (case["out"] == 0).all(axis=1)), name  # fully masked rows are exactly zero
            # ... and of its streaming strategy (key blocks of 128, probabilities rounded before the normalisation)
            streamed = port.sdpa_bf16_streaming(case["q"], case["k"], case["v"], float(case["scale"]), case.get("query_mask"),
                                                case.get("key_mask"), case.get("keep_mask"), case.get("bias"), int(case["causal"]))
            assert rel_frobenius(streamed, case["out_streaming"]) <= 1e-5, name
            assert np.array_equal((streamed == 0).all(axis=1), (case["out_streaming"] == 0).all(axis=1)), name
            # the two strategies round probabilities at different scalings: they agree to a few 1e-3, not to 1e-5
            assert 1e-4 < rel_frobenius(case["out_streaming"], case["out"]) < 5e-3, name
            checked += 1
            continue
        if kind == "pack_comp":
            # the compensation row the reference's own ops::matmul_pack_b_compensated emitted (it does not depend on the
            # packed layout, which is the reference's tile layout there and TMA's row layout here)
            from oracle.checker import pack_compensation
            assert np.array_equal(pack_compensation(case["b"], int(case["zero_point"])), case["compensation"]), name
            checked += 1
            continue
        if kind == "quant_per_row":
            quantized = port.quantize_rows_per_row(case["a"], case["multipliers"], float(case["zero_point"]))
            got = port.matmul_i8_dequant_rows(quantized, case["b"], case["correction"], case["row_scales"], case["column_scales"])
            assert np.array_equal(got, case["c"]), name
            checked += 1
            continue
        a, b = case["a"], case["b"]
        if kind == "i8":
            assert np.array_equal(port.matmul_i8(a, b), case["c"]), name
        elif kind == "f32":
            assert rel_frobenius(port.matmul_f32(a, b), case["c"]) <= TOL_F32, name
        elif kind == "bf16":
            assert rel_frobenius(port.matmul_bf16(a, b, None, False), case["c_f32"]) <= 1e-6, name
            got = bf16_bits_to_f32(port.matmul_bf16(a, b, None, True))
            assert rel_frobenius(got, bf16_bits_to_f32(case["c_bf16"])) <= TOL_BF16, name
        elif kind == "w8":
            got = bf16_bits_to_f32(port.matmul_w8(a, b, case["scale"], True))
            assert rel_frobenius(got, bf16_bits_to_f32(case["c_bf16"])) <= TOL_BF16, name
        elif kind == "fused_bf16":
            args = dict(cin=case.get("cin"), alpha=float(case["alpha"]), scale=case.get("scale"), act=int(case["act"]),
                        lo=float(case["lo"]), hi=float(case["hi"]))
            assert rel_frobenius(port.matmul_bf16_fused(a, b, out_bf16=False, **args), case["c_f32"]) <= 1e-6, name
            got = bf16_bits_to_f32(port.matmul_bf16_fused(a, b, out_bf16=True, **args))
            assert rel_frobenius(got, bf16_bits_to_f32(case["c_bf16"])) <= TOL_BF16, name
        elif kind == "i8acc":
            assert np.array_equal(port.matmul_i8_accumulate(a, b, case["cin"]), case["c"]), name
        elif kind == "batched_bf16":
            # the reference's rank-3 form is one product per batch index, a leading stride of 0 sharing an operand
            batch = case["c"].shape[0]
            for i in range(batch):
                ai = a if a.ndim == 2 else a[i]
                bi = b if b.ndim == 2 else b[i]
                got = port.matmul_bf16_fused(ai, bi, case.get("bias"), out_bf16=False)
                assert rel_frobenius(got, case["c"][i]) <= 1e-6, name
        elif kind == "quant_u8s8":
            quantized = port.quantize_rows(a, float(case["a_scale"]), float(case["a_zero_point"]))
            got = port.matmul_i8_dequant(quantized, b, case["correction"], float(case["dequant"]))
            assert np.array_equal(got, case["c"]), name
        else:
            raise AssertionError(f"unknown fixture kind {kind}")
        checked += 1
    assert checked >= 48


def test_int32_accumulator_wraps(port):
    # K = 262145 of 127*127 overflows int32 and must wrap (tests/ops/MatmulTest.cpp:1025-1055)
    k = 262145
    for dtype, value in ((np.int8, 127), (np.uint8, 255)):
        a = np.full((1, k), value, dtype=dtype)
        expected = np.uint32((value * value * k) % (1 << 32)).astype(np.int32)
        assert port.matmul_i8(a, a)[0, 0] == expected


def test_empty_and_degenerate_shapes(port):
    a = np.zeros((3, 0), dtype=np.float32)
    b = np.zeros((5, 0), dtype=np.float32)
    assert np.array_equal(port.matmul_f32(a, b), np.zeros((3, 5), dtype=np.float32))  # K = 0 -> zeros
    assert port.matmul_i8(np.zeros((0, 4), np.int8), np.zeros((2, 4), np.int8)).shape == (0, 2)


def test_strided_b_is_the_nk_view_of_a_kn_matrix(port):
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (9, 20)).astype(np.float32)
    b_kn = rng.uniform(-1, 1, (20, 13)).astype(np.float32)
    want = (a.astype(np.float64) @ b_kn.astype(np.float64)).astype(np.float32)
    assert rel_frobenius(port.matmul_f32(a, b_kn.T), want) <= 1e-7


def test_port_against_reference_library_live(port):
    ref, why = Ref.load()
    if ref is None:
        pytest.skip(f"reference matmul cannot run on this host: {why}")
    rng = np.random.default_rng(11)
    a = f32_to_bf16_bits(rng.standard_normal((96, 320), dtype=np.float32))
    b = f32_to_bf16_bits(rng.standard_normal((80, 320), dtype=np.float32))
    assert rel_frobenius(bf16_bits_to_f32(port.matmul_bf16(a, b)), bf16_bits_to_f32(ref.matmul_bf16(a, b, threads=2))) <= TOL_BF16
    ai = rng.integers(-128, 128, (70, 448), dtype=np.int8)
    bi = rng.integers(-128, 128, (50, 448), dtype=np.int8)
    assert np.array_equal(port.matmul_i8(ai, bi), ref.matmul_i8(ai, bi, threads=2))
    w = rng.integers(-127, 128, (64, 320), dtype=np.int8)
    s = rng.uniform(0.001, 0.02, 64).astype(np.float32)
    got = bf16_bits_to_f32(port.matmul_w8(a[:16], w, s))
    assert rel_frobenius(got, bf16_bits_to_f32(ref.matmul_w8(a[:16], w, s))) <= TOL_BF16


def test_pack_compensation_against_reference_library_live():
    ref, why = Ref.load()
    if ref is None:
        pytest.skip(f"reference matmul cannot run on this host: {why}")
    from oracle.checker import pack_compensation
    rng = np.random.default_rng(21)
    for n, k, zp in [(1, 1, 9), (17, 63, -4), (64, 1024, 77), (5, 70000, 255)]:
        b = rng.integers(-128, 128, (n, k), dtype=np.int8)
        assert np.array_equal(pack_compensation(b, zp), ref.pack_compensation(b, zp)), (n, k, zp)
    padded = rng.integers(-128, 128, (12, 100), dtype=np.int8)   # rows on a pitch larger than K
    assert np.array_equal(pack_compensation(padded[:, :90], 3), ref.pack_compensation(padded[:, :90], 3))


def test_fp16_product_against_numpy(port):
    # the fp16 row's restatement (conversions pinned by the fixture above) against a float64 numpy product
    rng = np.random.default_rng(11)
    a = rng.standard_normal((19, 65)).astype(np.float16)
    b = rng.standard_normal((23, 65)).astype(np.float16)
    want = a.astype(np.float64) @ b.astype(np.float64).T
    got = port.matmul_f16(a.view(np.uint16), b.view(np.uint16), out_f16=False)
    assert np.array_equal(got, want.astype(np.float32))
    got16 = port.matmul_f16(a.view(np.uint16), b.view(np.uint16), out_f16=True)
    assert np.array_equal(got16, want.astype(np.float32).astype(np.float16).view(np.uint16))


def test_pack_restatement_follows_the_reference_tests_expectations():
    # the strided conversion case of tests/ops/MatmulPackTest.cpp:221-262: 5 x 9 fp32 values s*17 + k + 0.25 with StrideK 2,
    # packed as bf16: every position holds the converted logical element, zero past the extents
    from oracle.checker import pack_compensation, pack_rows, packed_pitch
    spatial, k = 5, 9
    storage = np.full(spatial * (2 * k + 3), -999.0, dtype=np.float32)
    view = np.lib.stride_tricks.as_strided(storage, (spatial, k), ((2 * k + 3) * 4, 8))
    view[...] = np.arange(spatial)[:, None] * 17 + np.arange(k)[None, :] + 0.25
    packed = pack_rows(view, "bf16")
    assert packed.shape == (spatial, 64) and packed_pitch(2, k) == 64
    assert np.array_equal(packed[:, :k], f32_to_bf16_bits(np.ascontiguousarray(view)))
    assert not packed[:, k:].any()
    logical = ((np.arange(33)[:, None] * 17 + np.arange(129)[None, :] * 3) % 61 - 30).astype(np.int8)
    assert np.array_equal(pack_compensation(logical, 3), -3 * logical.astype(np.int32).sum(axis=1))
