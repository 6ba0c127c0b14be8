"""Parity of the CUDA kernels with the CPU checker, through the C ABI.

Every case calls `vecops_b200_matmul_run` (directly or through the operator
bridge) on device tensors and compares with the checker on the same seeded
inputs: bit-exact for int32 results, relative Frobenius error within the stated
tolerance for floating-point results.
"""
import ctypes
from ctypes import byref

import numpy as np
import pytest
import torch

import vecops_b200
from oracle.checker import bf16_bits_to_f32, f32_to_bf16_bits, rel_frobenius
from tests.helpers import TOL_BF16, TOL_F32, bf16_result_to_numpy, to_device
from vecops_b200 import capi, harness

pytestmark = pytest.mark.gpu

K = capi  # kernel ids live there


def run_case(kind, a, b, scale=None, out_bf16=True, kernel=capi.KERNEL_AUTO, b_kn=False, ldc_pad=0):
    """Run on the GPU; returns a numpy result in the checker's representation."""
    m, n = a.shape[0], b.shape[0]
    da = to_device(a, bf16=kind in ("bf16", "w8"))
    if b_kn:  # store B as a row-major [K,N] matrix and hand over its [N,K] view
        db = to_device(np.ascontiguousarray(b.T), bf16=kind == "bf16").t()
    else:
        db = to_device(b, bf16=kind == "bf16")
    ds = to_device(scale) if scale is not None else None
    out_dtype = {"f32": torch.float32, "i8": torch.int32}.get(kind, torch.bfloat16 if out_bf16 else torch.float32)
    storage = torch.full((m, n + ldc_pad), -3, dtype=out_dtype, device="cuda")
    c = storage[:, :n]
    vecops_b200.matmul(da, db, c, ds, kernel=kernel)
    torch.cuda.synchronize()
    if ldc_pad:
        assert bool((storage[:, n:] == -3).all()), "kernel wrote outside its C columns"
    return bf16_result_to_numpy(c) if out_dtype == torch.bfloat16 else c.contiguous().cpu().numpy()


def check(kind, got, want, name=""):
    if kind == "i8":
        assert np.array_equal(got, want), f"{name}: int32 results differ"
    elif kind == "f32":
        assert rel_frobenius(got, want) <= TOL_F32, name
    else:
        g = bf16_bits_to_f32(got) if got.dtype == np.uint16 else got
        w = bf16_bits_to_f32(want) if want.dtype == np.uint16 else want
        assert rel_frobenius(g, w) <= TOL_BF16, name


def inputs(kind, m, n, k, rng, a_dtype=np.int8, b_dtype=np.int8):
    if kind == "f32":
        return rng.uniform(-1, 1, (m, k)).astype(np.float32), rng.uniform(-1, 1, (n, k)).astype(np.float32), None
    if kind == "bf16":
        return (f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32)),
                f32_to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32)), None)
    if kind == "i8":
        lo_a, hi_a = (-128, 128) if a_dtype == np.int8 else (0, 256)
        lo_b, hi_b = (-128, 128) if b_dtype == np.int8 else (0, 256)
        return rng.integers(lo_a, hi_a, (m, k)).astype(a_dtype), rng.integers(lo_b, hi_b, (n, k)).astype(b_dtype), None
    if kind == "w8":
        return (f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32)), rng.integers(-127, 128, (n, k), dtype=np.int8),
                rng.uniform(0.001, 0.02, n).astype(np.float32))
    raise ValueError(kind)


def oracle(kind, port, a, b, scale, out_bf16=True):
    from tests.helpers import oracle_for
    return oracle_for(kind, port, a, b, scale, out_bf16)


# ------------------------------------------------------------------ golden fixtures (outputs of the reference itself)

def test_golden_fixtures_through_automatic_dispatch(golden):
    for name, case in golden.items():
        kind = str(case["kind"])
        if kind in ("fused_bf16", "i8acc", "quant_u8s8", "batched_bf16", "f16_convert", "sdpa_bf16", "quant_per_row", "pack_comp"):
            continue  # the fused forms have their own tests below; the conversion digests are the checker's own
        a, b = case["a"], case["b"]
        if kind == "i8":
            check(kind, run_case(kind, a, b), case["c"], name)
        elif kind == "f32":
            check(kind, run_case(kind, a, b), case["c"], name)
        elif kind == "bf16":
            check(kind, run_case(kind, a, b, out_bf16=False), case["c_f32"], name)
            check(kind, run_case(kind, a, b, out_bf16=True), case["c_bf16"], name)
        else:
            check(kind, run_case(kind, a, b, case["scale"]), case["c_bf16"], name)


# ------------------------------------------------------------------ each kernel, forced, over shapes with tails

TC_SHAPES = [(128, 256, 64), (128, 256, 512), (512, 1024, 512), (200, 328, 200), (1, 256, 128), (129, 257, 72), (640, 768, 1032)]


@pytest.fixture(params=["single", "pair"])
def cta_form(request, monkeypatch):
    """Run the tcgen05 GEMM as single CTAs on 128x256 tiles, or as CTA pairs on 256x256 tiles (cta_group::2)."""
    monkeypatch.setenv("VECOPS_B200_GEMM_PAIR", "1" if request.param == "pair" else "0")
    return request.param


@pytest.fixture(params=["mixed", "tmem", "tmem_pair"])
def w8_form(request, monkeypatch):
    """The weight-only tensor-core kernel id in its forms: the default (weights widened into shared memory as the N operand of
    the dense GEMM's MMAs, tiles cut along K), and the older one (weights widened into tensor memory as the M operand,
    stream-K) on 128-row tiles per CTA or on 256-row tiles per CTA pair."""
    if request.param != "mixed":
        monkeypatch.setenv("VECOPS_B200_W8TC_FORM", "tmem")
        monkeypatch.setenv("VECOPS_B200_W8TC_PAIR", "1" if request.param == "tmem_pair" else "0")
    return request.param


@pytest.mark.parametrize("m,n,k", TC_SHAPES)
@pytest.mark.parametrize("out_bf16", [True, False])
def test_bf16_tcgen05(port, cta_form, m, n, k, out_bf16):
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    a, b, _ = inputs("bf16", m, n, k, rng)
    check("bf16", run_case("bf16", a, b, out_bf16=out_bf16, kernel=K.KERNEL_BF16_TCGEN05), oracle("bf16", port, a, b, None, out_bf16))


def test_bf16_tcgen05_scale_and_padded_c(port, cta_form):
    rng = np.random.default_rng(21)
    a, b, _ = inputs("bf16", 300, 520, 264, rng)
    scale = rng.uniform(0.5, 2.0, 520).astype(np.float32)
    for out_bf16 in (True, False):
        got = run_case("bf16", a, b, scale, out_bf16, K.KERNEL_BF16_TCGEN05, ldc_pad=24)
        check("bf16", got, oracle("bf16", port, a, b, scale, out_bf16))


def test_bf16_tcgen05_direct_epilogue_for_unaligned_c(port, cta_form):
    # a C row pitch that is not a multiple of 16 bytes cannot use TMA stores: the direct path must serve it
    rng = np.random.default_rng(22)
    a, b, _ = inputs("bf16", 150, 300, 128, rng)
    got = run_case("bf16", a, b, None, True, K.KERNEL_BF16_TCGEN05, ldc_pad=3)
    check("bf16", got, oracle("bf16", port, a, b, None, True))


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (384, 512, 1024), (150, 300, 272), (1, 512, 4096), (257, 129, 48)])
@pytest.mark.parametrize("a_dtype,b_dtype", [(np.int8, np.int8), (np.uint8, np.int8), (np.int8, np.uint8), (np.uint8, np.uint8)])
def test_i8_tcgen05_all_signedness_pairs(port, cta_form, m, n, k, a_dtype, b_dtype):
    rng = np.random.default_rng(m + n + k)
    a, b, _ = inputs("i8", m, n, k, rng, a_dtype, b_dtype)
    check("i8", run_case("i8", a, b, kernel=K.KERNEL_I8_TCGEN05), port.matmul_i8(a, b))


@pytest.mark.parametrize("m", [1, 3, 8, 16, 17, 32, 40, 128])
def test_w8_small_m(port, m):
    rng = np.random.default_rng(100 + m)
    a, w, s = inputs("w8", m, 208, 512, rng)
    check("w8", run_case("w8", a, w, s, kernel=K.KERNEL_W8_SMALL_M), port.matmul_w8(a, w, s))


def test_w8_small_m_ragged_n_no_scale_f32_out(port):
    rng = np.random.default_rng(9)
    a, w, s = inputs("w8", 5, 77, 96, rng)
    check("w8", run_case("w8", a, w, None, False, K.KERNEL_W8_SMALL_M), port.matmul_w8(a, w, None, False))
    check("w8", run_case("w8", a, w, s, True, K.KERNEL_W8_SMALL_M, ldc_pad=5), port.matmul_w8(a, w, s, True))


@pytest.mark.parametrize("m", [1, 16, 17, 32, 48, 100, 128])
@pytest.mark.parametrize("n,k", [(128, 128), (256, 512), (300, 208), (1024, 1024), (2048, 384), (4096, 2048)])  # the last: 9 CTAs per tile
def test_w8_tcgen05(port, w8_form, m, n, k):
    # weights widened into tensor memory; stream-K partial sums through device scratch
    rng = np.random.default_rng(1000 * m + n + k)
    a, w, s = inputs("w8", m, n, k, rng)
    check("w8", run_case("w8", a, w, s, kernel=K.KERNEL_W8_TCGEN05), port.matmul_w8(a, w, s), f"m={m} n={n} k={k}")


def test_w8_tcgen05_f32_out_no_scale_padded_c(port, w8_form):
    rng = np.random.default_rng(77)
    a, w, s = inputs("w8", 40, 640, 768, rng)
    check("w8", run_case("w8", a, w, None, False, K.KERNEL_W8_TCGEN05, ldc_pad=7), port.matmul_w8(a, w, None, False))


@pytest.mark.parametrize("m,n,k", [(129, 512, 1024), (300, 1000, 528), (1024, 768, 256)])
def test_w8_tcgen05_more_than_one_row_tile(port, m, n, k):
    # the default form walks row tiles like the dense GEMM: M > 128 is served too (each row tile widens the weights again)
    rng = np.random.default_rng(m + n + k)
    a, w, s = inputs("w8", m, n, k, rng)
    check("w8", run_case("w8", a, w, s, kernel=K.KERNEL_W8_TCGEN05), port.matmul_w8(a, w, s), f"m={m} n={n} k={k}")


def test_w8_tcgen05_runs_whole_tiles_without_scratch(port):
    # no workspace: the tiles are not cut along K; same result within tolerance, and with scratch the query is non-zero
    rng = np.random.default_rng(31)
    a, w, s = inputs("w8", 64, 1024, 2048, rng)
    da, dw, ds = to_device(a, True), to_device(w), to_device(s)
    c = torch.zeros((64, 1024), dtype=torch.bfloat16, device="cuda")
    problem = vecops_b200.matmul_problem(da, dw, c, ds, kernel=K.KERNEL_W8_TCGEN05)
    assert harness.workspace_bytes(problem) > 0 and problem.workspace is None
    harness.run(problem)
    check("w8", bf16_result_to_numpy(c), port.matmul_w8(a, w, s))


def test_w8_tcgen05_older_form_refuses_a_missing_workspace(monkeypatch):
    monkeypatch.setenv("VECOPS_B200_W8TC_FORM", "tmem")
    a = torch.zeros((32, 256), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((256, 256), dtype=torch.int8, device="cuda")
    c = torch.zeros((32, 256), dtype=torch.bfloat16, device="cuda")
    problem = vecops_b200.matmul_problem(a, w, c, kernel=K.KERNEL_W8_TCGEN05)
    assert harness.workspace_bytes(problem) > 0
    with pytest.raises(capi.VecopsB200Error) as info:
        harness.run(problem)
    assert info.value.code == capi.INVALID_ARGUMENT and "workspace" in info.value.message


@pytest.mark.parametrize("m,n,k", [(64, 64, 64), (200, 300, 100), (130, 70, 45), (1, 1000, 333), (1024, 1024, 1024), (128, 192, 48), (64, 64, 16)])
@pytest.mark.parametrize("b_kn", [True, False])
def test_f32_simt(port, m, n, k, b_kn):
    rng = np.random.default_rng(m + 2 * n + 3 * k)
    a, b, _ = inputs("f32", m, n, k, rng)
    check("f32", run_case("f32", a, b, kernel=K.KERNEL_F32_SIMT, b_kn=b_kn), port.matmul_f32(a, b))


@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (1024, 1024, 1024), (300, 520, 77), (129, 257, 1000), (64, 2048, 4096)])
@pytest.mark.parametrize("b_kn", [True, False])
def test_f32_tf32x3(port, m, n, k, b_kn):
    # fp32 as three tf32 products of split operands on the tensor cores: inside the fp32 bar of 1e-5 (2e-6 to 4e-6 in fact),
    # any K (zero-padded to k-blocks by the split), either storage of B
    rng = np.random.default_rng(m + 2 * n + 3 * k)
    a, b, _ = inputs("f32", m, n, k, rng)
    got = run_case("f32", a, b, kernel=K.KERNEL_F32_TF32X3, b_kn=b_kn)
    want = port.matmul_f32(a, b)
    assert rel_frobenius(got, want) <= TOL_F32, f"m={m} n={n} k={k}"


def test_f32_tf32x3_keeps_small_values_and_large_ranges(port):
    # rows spanning many orders of magnitude: the split is per element, so no element loses bits to its neighbours
    rng = np.random.default_rng(3)
    m, n, k = 256, 384, 512
    a = (rng.uniform(-1, 1, (m, k)) * 10.0 ** rng.integers(-6, 7, (m, k))).astype(np.float32)
    b = (rng.uniform(-1, 1, (n, k)) * 10.0 ** rng.integers(-6, 7, (n, k))).astype(np.float32)
    got = run_case("f32", a, b, kernel=K.KERNEL_F32_TF32X3)
    assert rel_frobenius(got, port.matmul_f32(a, b)) <= TOL_F32
    # and without the scratch the automatic choice is the FMA kernel, with it the split route: both inside the bar
    da, db = to_device(a), to_device(b)
    c = torch.empty((m, n), dtype=torch.float32, device="cuda")
    problem = harness.matmul_problem(da, db, c)
    harness.run(problem)
    assert rel_frobenius(c.cpu().numpy(), port.matmul_f32(a, b)) <= TOL_F32
    scratch = harness.attach_workspace(problem, da.device)
    assert scratch is not None
    before = capi.library().vecops_b200_launch_count()
    harness.run(problem)
    assert capi.library().vecops_b200_launch_count() - before == 2  # the operand split and the product
    assert rel_frobenius(c.cpu().numpy(), port.matmul_f32(a, b)) <= TOL_F32


@pytest.mark.parametrize("kind", ["f32", "bf16", "i8", "w8"])
def test_strided_kernel_on_reference_test_shapes(port, kind):
    # ragged shapes and K tails the reference exercises (tests/ops/MatmulTest.cpp:434-452)
    for m, n, k in [(16, 16, 35), (37, 51, 79), (1, 48, 79), (512, 1, 256), (96, 16, 67)]:
        rng = np.random.default_rng(m * n + k)
        a, b, s = inputs(kind, m, n, k, rng, np.uint8, np.int8)
        got = run_case(kind, a, b, s, kernel=K.KERNEL_GENERIC, b_kn=(kind == "f32"), ldc_pad=1)
        check(kind, got, oracle(kind, port, a, b, s))


def test_fused_allgather_epilogue_stores_the_slab_into_every_destination(port, cta_form):
    # Two destinations on ONE GPU stand in for two ranks' result matrices: the epilogue must place this
    # rank's [M, n] slab at columns [col0, col0 + n) of both, and touch nothing else.
    from vecops_b200 import sharding
    rng = np.random.default_rng(88)
    m, n, k, n_total, col0 = 384, 512, 256, 1536, 768
    a, b, _ = inputs("bf16", m, n, k, rng)
    da, db = to_device(a, True), to_device(b, True)
    for out_dtype in (torch.bfloat16, torch.float32):
        full = [torch.full((m, n_total), -3.0, dtype=out_dtype, device="cuda") for _ in range(2)]
        gemm = sharding.FusedGatherGemm(da, db, [t.data_ptr() for t in full], n_total, n_total, col0, out_dtype)
        gemm.launch()
        torch.cuda.synchronize()
        want = port.matmul_bf16(a, b, None, out_dtype == torch.bfloat16)
        for t in full:
            slab = t[:, col0:col0 + n]
            got = bf16_result_to_numpy(slab) if out_dtype == torch.bfloat16 else slab.contiguous().cpu().numpy()
            check("bf16", got, want)
            assert bool((t[:, :col0] == -3).all()) and bool((t[:, col0 + n:] == -3).all())


@pytest.mark.parametrize("route,lanes", [(K.PUSH_KERNEL, 1), (K.PUSH_COPY_ENGINE, 1), (K.PUSH_COPY_ENGINE, 2), (K.PUSH_KERNEL, 2)])
def test_pipelined_gather_pushes_the_slab_behind_the_next_product(port, route, lanes):
    # One GPU stands in for three ranks: rank 1's double-buffered result and two "peers'" results are three local
    # tensors, the barrier is a no-op.  After every step the copy it filled must hold the slab at [col0, col0 + n) in
    # the rank's own result AND in both peers', nothing else may have been touched, and five steps in a row (each
    # result copy reused twice) must give the product of THAT step's operands.
    from vecops_b200 import sharding
    rng = np.random.default_rng(89)
    m, n, k, n_total, col0 = 384, 512, 256, 1536, 512
    a, b, _ = inputs("bf16", m, n, k, rng)
    da, db = to_device(a, True), to_device(b, True)
    results = [torch.full((2, m, n_total), -3.0, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    bases = [t.data_ptr() for t in results]  # indexed by rank: this rank is 1
    gemm = sharding.PipelinedGatherGemm(da, db, results[1], bases, rank=1, col0=col0, barrier=lambda: None, route=route, lanes=lanes)
    before = capi.library().vecops_b200_launch_count()
    for step in range(5):
        if step == 3:  # new operand values in place: later steps must follow them
            a2, b2, _ = inputs("bf16", m, n, k, np.random.default_rng(90))
            gemm.join()
            torch.cuda.synchronize()
            da.copy_(to_device(a2, True))
            db.copy_(to_device(b2, True))
            a, b = a2, b2
        half = gemm.launch()
        assert half == step % 2
        gemm.join()
        torch.cuda.synchronize()
        want = port.matmul_bf16(a, b, None, True)
        for t in results:
            check("bf16", bf16_result_to_numpy(t[half][:, col0:col0 + n]), want)
            assert bool((t[half][:, :col0] == -3).all()) and bool((t[half][:, col0 + n:] == -3).all())
    expected = 5 * (1 + (lanes if route == K.PUSH_KERNEL else 0))  # the GEMM, and one push kernel per lane
    assert capi.library().vecops_b200_launch_count() - before == expected
    status, error = ctypes.c_uint32(1), capi.ErrorBuffer()
    error.raise_for(capi.library().vecops_b200_take_device_status(0, ctypes.byref(status), ctypes.byref(error.record)))
    assert status.value == 0


def test_push_columns_refuses_what_it_cannot_send():
    src = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    dst = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    error = capi.ErrorBuffer()
    lib = capi.library()
    one = (ctypes.c_void_p * 1)(dst.data_ptr())
    same = (ctypes.c_void_p * 1)(src.data_ptr())
    nine = (ctypes.c_void_p * 9)(*[dst.data_ptr()] * 9)
    assert lib.vecops_b200_push_columns(src.data_ptr(), nine, 9, 64, 0, 8, 64, 2, K.PUSH_KERNEL, None, ctypes.byref(error.record)) == capi.INVALID_ARGUMENT
    assert lib.vecops_b200_push_columns(src.data_ptr(), same, 1, 64, 0, 8, 64, 2, K.PUSH_KERNEL, None, ctypes.byref(error.record)) == capi.INVALID_ARGUMENT
    assert lib.vecops_b200_push_columns(src.data_ptr(), one, 1, 64, 32, 8, 64, 2, K.PUSH_KERNEL, None, ctypes.byref(error.record)) == capi.INVALID_ARGUMENT
    assert lib.vecops_b200_push_columns(src.data_ptr(), one, 1, 64, 4, 8, 8, 2, K.PUSH_KERNEL, None, ctypes.byref(error.record)) == capi.INVALID_ARGUMENT  # 8-byte offset
    assert lib.vecops_b200_push_columns(src.data_ptr(), one, 1, 64, 0, 8, 64, 2, 7, None, ctypes.byref(error.record)) == capi.INVALID_ARGUMENT
    assert lib.vecops_b200_push_columns(src.data_ptr(), one, 1, 64, 0, 0, 64, 2, K.PUSH_KERNEL, None, ctypes.byref(error.record)) == capi.OK


def test_int32_accumulators_wrap_like_the_reference(port):
    # K = 262145 of 127*127 (and 255*255) overflows int32 and must wrap (tests/ops/MatmulTest.cpp:1025-1055)
    k = 262145
    for dtype, value in ((np.int8, 127), (np.uint8, 255)):
        a = np.full((1, k), value, dtype=dtype)
        got = run_case("i8", a, a)
        assert got[0, 0] == np.uint32((value * value * k) % (1 << 32)).astype(np.int32)


def test_empty_reduction_stores_zeros_and_empty_outputs_are_no_ops():
    a = torch.empty((5, 0), dtype=torch.bfloat16, device="cuda")
    b = torch.empty((7, 0), dtype=torch.bfloat16, device="cuda")
    c = torch.full((5, 7), 9.0, dtype=torch.bfloat16, device="cuda")
    vecops_b200.matmul(a, b, c)
    assert bool((c == 0).all())  # K == 0 -> C = 0 (ops/Matmul.h:41-43)
    vecops_b200.matmul(torch.empty((0, 8), dtype=torch.float32, device="cuda"), torch.empty((4, 8), dtype=torch.float32, device="cuda"),
                       torch.empty((0, 4), dtype=torch.float32, device="cuda"))


def test_full_range_int8_extremes(port):
    # -128 * -128 * K: the largest magnitudes the int8 path can see
    a = np.full((128, 4096), -128, dtype=np.int8)
    b = np.full((256, 4096), -128, dtype=np.int8)
    b[::2] = 127
    check("i8", run_case("i8", a, b, kernel=K.KERNEL_I8_TCGEN05), port.matmul_i8(a, b))


# ------------------------------------------------------------------ the operator path (bridge -> Operator -> provider -> descriptor.run)

def _tensor_value(t, writable=False, keep=None):
    sizes = (ctypes.c_int64 * t.dim())(*t.shape)
    strides = (ctypes.c_int64 * t.dim())(*t.stride())
    keep.extend([sizes, strides])
    v = capi.VecopsValue()
    v.struct_size = ctypes.sizeof(capi.VecopsValue)
    v.kind = capi.VALUE_TENSOR
    tv = v.value.tensor
    tv.struct_size = ctypes.sizeof(capi.VecopsTensorView)
    tv.data = t.data_ptr()
    tv.byte_offset = 0
    tv.device_type = capi.DEVICE_CUDA if t.is_cuda else capi.DEVICE_CPU
    tv.device_index = t.device.index if t.is_cuda else 0
    tv.dtype = vecops_b200.torch_dtype_code(t.dtype)
    tv.rank = t.dim()
    tv.sizes = sizes
    tv.strides = strides
    tv.flags = capi.TENSOR_READ | (capi.TENSOR_WRITE if writable else 0)
    return v


def bridge_call(a, b, c, scale=None, stream=None, asynchronous=False):
    keep = []
    values = [_tensor_value(a, keep=keep), _tensor_value(b, keep=keep), _tensor_value(c, True, keep=keep)]
    if scale is not None:
        values.append(_tensor_value(scale, keep=keep))
    array = (capi.VecopsValue * len(values))(*values)
    context = capi.VecopsExecutionContext()
    context.struct_size = ctypes.sizeof(context)
    context.stream = stream.cuda_stream if stream is not None else None
    context.flags = capi.CONTEXT_FLAG_ASYNC if asynchronous else 0
    call = capi.VecopsCall(ctypes.sizeof(capi.VecopsCall), len(values), array, None, 0, ctypes.pointer(context))
    keep.extend([array, context])
    return call, keep


def bridge_lib():
    lib = capi.library()
    lib.vecops_b200_matmul_operator.restype = ctypes.c_uint64
    lib.vecops_operator_bridge_invoke_v1.argtypes = [ctypes.c_uint64, ctypes.POINTER(capi.VecopsCall), ctypes.c_uint32, ctypes.c_void_p,
                                                     ctypes.POINTER(capi.VecopsError)]
    lib.vecops_b200_operator_resolve.argtypes = [ctypes.c_uint64, ctypes.POINTER(capi.VecopsCall), ctypes.c_char_p, ctypes.c_size_t,
                                                 ctypes.POINTER(capi.VecopsError)]
    return lib, lib.vecops_b200_matmul_operator()


@pytest.mark.parametrize("kind,m,n,k", [("bf16", 256, 512, 256), ("i8", 256, 512, 256), ("w8", 16, 256, 512), ("f32", 96, 80, 64),
                                        ("bf16", 16, 16, 35)])
def test_operator_bridge_invokes_the_selected_kernel(port, kind, m, n, k):
    lib, handle = bridge_lib()
    rng = np.random.default_rng(k)
    a, b, s = inputs(kind, m, n, k, rng)
    da = to_device(a, bf16=kind in ("bf16", "w8"))
    db = to_device(b, bf16=kind == "bf16")
    ds = to_device(s) if s is not None else None
    out_dtype = {"f32": torch.float32, "i8": torch.int32}.get(kind, torch.bfloat16)
    c = torch.zeros((m, n), dtype=out_dtype, device="cuda")
    call, keep = bridge_call(da, db, c, ds)
    error = capi.ErrorBuffer()
    key = ctypes.create_string_buffer(256)
    error.raise_for(lib.vecops_b200_operator_resolve(handle, byref(call), key, 256, byref(error.record)))
    assert key.value.decode().startswith("vecops::matmul;TA=")
    before = lib.vecops_b200_launch_count()
    error.raise_for(lib.vecops_operator_bridge_invoke_v1(handle, byref(call), 0, None, byref(error.record)))
    assert lib.vecops_b200_launch_count() == before + 1
    got = bf16_result_to_numpy(c) if out_dtype == torch.bfloat16 else c.cpu().numpy()
    check(kind, got, oracle(kind, port, a, b, s))


def test_operator_bridge_sizes_and_uses_device_scratch(port):
    # M = 40 weight-only: resolves to the stream-K kernel, whose descriptor reports the scratch it needs
    lib, handle = bridge_lib()
    lib.vecops_b200_operator_workspace.argtypes = [ctypes.c_uint64, ctypes.POINTER(capi.VecopsCall), ctypes.POINTER(ctypes.c_uint64),
                                                   ctypes.POINTER(capi.VecopsError)]
    rng = np.random.default_rng(40)
    a, w, s = inputs("w8", 40, 512, 1024, rng)
    da, dw, ds = to_device(a, True), to_device(w), to_device(s)
    c = torch.zeros((40, 512), dtype=torch.bfloat16, device="cuda")
    call, keep = bridge_call(da, dw, c, ds)
    error = capi.ErrorBuffer()
    key = ctypes.create_string_buffer(256)
    error.raise_for(lib.vecops_b200_operator_resolve(handle, byref(call), key, 256, byref(error.record)))
    assert key.value.decode().endswith("kernel=w8_tcgen05")
    need = ctypes.c_uint64(0)
    error.raise_for(lib.vecops_b200_operator_workspace(handle, byref(call), byref(need), byref(error.record)))
    assert need.value > 0
    assert lib.vecops_operator_bridge_invoke_v1(handle, byref(call), 0, None, byref(error.record)) == capi.INVALID_ARGUMENT
    scratch = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    call.workspace, call.workspace_size = scratch.data_ptr(), need.value
    for _ in range(2):  # the scratch is reusable as is: flags carry a per-launch nonce
        c.zero_()
        error.raise_for(lib.vecops_operator_bridge_invoke_v1(handle, byref(call), 0, None, byref(error.record)))
        check("w8", bf16_result_to_numpy(c), port.matmul_w8(a, w, s))


def test_operator_bridge_async_on_a_side_stream(port):
    lib, handle = bridge_lib()
    rng = np.random.default_rng(3)
    a, b, _ = inputs("bf16", 512, 512, 512, rng)
    da, db = to_device(a, True), to_device(b, True)
    c = torch.zeros((512, 512), dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    call, keep = bridge_call(da, db, c, stream=stream, asynchronous=True)
    error = capi.ErrorBuffer()
    # eight tiles on 148 SMs are cut along K: the executable asks for the scratch the slices meet in, as the contract has it
    lib.vecops_b200_operator_workspace.argtypes = [ctypes.c_uint64, ctypes.POINTER(capi.VecopsCall), ctypes.POINTER(ctypes.c_uint64),
                                                   ctypes.POINTER(capi.VecopsError)]
    need = ctypes.c_uint64(0)
    error.raise_for(lib.vecops_b200_operator_workspace(handle, byref(call), byref(need), byref(error.record)))
    assert need.value > 0
    assert lib.vecops_operator_bridge_invoke_v1(handle, byref(call), 0, None, byref(capi.ErrorBuffer().record)) == capi.INVALID_ARGUMENT  # none given
    scratch = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    call.workspace, call.workspace_size = scratch.data_ptr(), need.value
    error.raise_for(lib.vecops_operator_bridge_invoke_v1(handle, byref(call), 0, None, byref(error.record)))
    stream.synchronize()
    status = ctypes.c_uint32(1)
    error.raise_for(lib.vecops_b200_take_device_status(0, byref(status), byref(error.record)))
    assert status.value == 0
    check("bf16", bf16_result_to_numpy(c), port.matmul_bf16(a, b))


def test_operator_bridge_refuses_host_tensors_and_bad_handles():
    lib, handle = bridge_lib()
    a = torch.zeros((8, 8), dtype=torch.float32)
    c = torch.zeros((8, 8), dtype=torch.float32)
    call, keep = bridge_call(a, a, c)
    error = capi.ErrorBuffer()
    assert lib.vecops_operator_bridge_invoke_v1(handle, byref(call), 0, None, byref(error.record)) == capi.INVALID_ARGUMENT
    assert b"wrong device" in error.text.value
    assert lib.vecops_operator_bridge_invoke_v1(12345, byref(call), 0, None, byref(error.record)) == capi.NOT_FOUND


# ------------------------------------------------------------------ tail tiles cut along K (partials meet in device scratch)

def _tail_split_case(kind, m, n, k, out_bf16, monkeypatch, port):
    rng = np.random.default_rng(m + 3 * n + 7 * k)
    a, b, _ = inputs(kind, m, n, k, rng)
    kernel = K.KERNEL_I8_TCGEN05 if kind == "i8" else K.KERNEL_BF16_TCGEN05
    # the harness attaches the scratch the workspace query asks for: a non-zero answer means the tail is split
    da, db = to_device(a, bf16=kind == "bf16"), to_device(b, bf16=kind == "bf16")
    out_dtype = torch.int32 if kind == "i8" else (torch.bfloat16 if out_bf16 else torch.float32)
    probe = harness.matmul_problem(da, db, torch.empty((m, n), dtype=out_dtype, device="cuda"), kernel=kernel)
    assert harness.workspace_bytes(probe) > 0, "shape does not leave a splittable tail on this GPU"
    split = run_case(kind, a, b, out_bf16=out_bf16, kernel=kernel)
    again = run_case(kind, a, b, out_bf16=out_bf16, kernel=kernel)
    assert np.array_equal(split, again), "the split tail must be reproducible run to run"
    monkeypatch.setenv("VECOPS_B200_TAIL_SPLIT", "0")
    whole = run_case(kind, a, b, out_bf16=out_bf16, kernel=kernel)
    monkeypatch.delenv("VECOPS_B200_TAIL_SPLIT")
    rows = np.unique(np.concatenate([np.linspace(0, m - 1, 24).astype(np.int64), np.arange(m - 8, m)]))
    want = oracle(kind, port, a[rows], b, None, out_bf16)
    if kind == "i8":
        assert np.array_equal(split, whole)
        assert np.array_equal(split[rows], want)
    else:
        check(kind, split, whole)
        check(kind, split[rows], want)


@pytest.mark.parametrize("m,n,k,out_bf16", [
    (1536, 3584, 1024, True),    # 168 tiles: 20 tail tiles, 4 slices each on 148 SMs (pairs: 84 tiles, 10 in the tail)
    (1536, 3584, 1024, False),
    (1024, 6912, 512, True),     # 216 tiles: 68 tail tiles, 2 slices each
    (1000, 6900, 520, False),    # the same grid with ragged M, N and K
])
def test_bf16_tcgen05_tail_split(port, monkeypatch, cta_form, m, n, k, out_bf16):
    _tail_split_case("bf16", m, n, k, out_bf16, monkeypatch, port)


@pytest.mark.parametrize("m,n,k", [
    (512, 10496, 4096),          # 164 tiles: 16 tail tiles, 8 slices each
    (1536, 3584, 2048),          # 20 tail tiles, 4 slices each
    (1000, 6900, 1040),          # 68 tail tiles, 2 slices, ragged
])
def test_i8_tcgen05_tail_split(port, monkeypatch, cta_form, m, n, k):
    _tail_split_case("i8", m, n, k, True, monkeypatch, port)


def test_tcgen05_tail_runs_whole_without_scratch(port):
    # no workspace supplied: same result, tail tiles computed whole
    rng = np.random.default_rng(5)
    a, b, _ = inputs("i8", 1536, 3584, 1024, rng)
    da, db = to_device(a), to_device(b)
    c = torch.empty((1536, 3584), dtype=torch.int32, device="cuda")
    problem = harness.matmul_problem(da, db, c, kernel=K.KERNEL_I8_TCGEN05)
    error = capi.ErrorBuffer()
    error.raise_for(capi.library().vecops_b200_matmul_run(byref(problem), byref(error.record)))
    rows = np.arange(1400, 1536)
    assert np.array_equal(c.cpu().numpy()[rows], port.matmul_i8(a[rows], b))


# ------------------------------------------------------------------ fused forms: COut = activation((CIn + A.B^T) * alpha * scale)

def _fused_gpu(kind, a, b, out_dtype, kernel, cin=None, alpha=1.0, scale=None, act=capi.ACTIVATION_NONE, lo=0.0, hi=0.0):
    m, n = a.shape[0], b.shape[0]
    da, db = to_device(a, bf16=kind == "bf16"), to_device(b, bf16=kind == "bf16")
    dcin = None
    if cin is not None:
        dcin = to_device(cin, bf16=cin.dtype == np.uint16)
    ds = to_device(scale) if scale is not None else None
    c = torch.full((m, n), -3, dtype=out_dtype, device="cuda")
    vecops_b200.matmul(da, db, c, ds, kernel=kernel, cin=dcin, alpha=alpha, activation=act, clamp_lo=lo, clamp_hi=hi)
    torch.cuda.synchronize()
    return bf16_result_to_numpy(c) if out_dtype == torch.bfloat16 else c.cpu().numpy()


def test_fused_golden_fixtures(golden):
    # outputs of the reference's own explicit-accumulate form with composed output transforms
    seen = 0
    for name, case in golden.items():
        kind = str(case["kind"])
        if kind == "fused_bf16":
            args = dict(cin=case.get("cin"), alpha=float(case["alpha"]), scale=case.get("scale"), act=int(case["act"]),
                        lo=float(case["lo"]), hi=float(case["hi"]))
            # (the reference tests' shapes have odd K: rows TMA cannot address, so these run on the strided kernel; the
            # tensor-core epilogue is checked against the restatement in the next test)
            for kernel in (K.KERNEL_AUTO, K.KERNEL_GENERIC):
                check("bf16", _fused_gpu("bf16", case["a"], case["b"], torch.float32, kernel, **args), case["c_f32"], name)
                check("bf16", _fused_gpu("bf16", case["a"], case["b"], torch.bfloat16, kernel, **args), case["c_bf16"], name)
            seen += 1
        elif kind == "i8acc":
            for kernel in (K.KERNEL_AUTO, K.KERNEL_GENERIC):
                got = _fused_gpu("i8", case["a"], case["b"], torch.int32, kernel, cin=case["cin"])
                assert np.array_equal(got, case["c"]), name
            seen += 1
    assert seen >= 14


@pytest.mark.parametrize("m,n,k", [(300, 520, 264), (1536, 3584, 1024)])  # the second: split tail tiles on 148 SMs
def test_fused_bf16_tcgen05_against_the_checker(port, cta_form, m, n, k):
    from oracle.checker import ACT_CLAMP, ACT_RELU, ACT_SIGMOID, ACT_SILU
    rng = np.random.default_rng(m + n)
    a, b, _ = inputs("bf16", m, n, k, rng)
    a = f32_to_bf16_bits(bf16_bits_to_f32(a) * 0.1)
    bias = rng.uniform(-1, 1, n).astype(np.float32)
    full_bf16 = f32_to_bf16_bits(rng.uniform(-2, 2, (m, n)).astype(np.float32))
    scale = rng.uniform(0.5, 2.0, n).astype(np.float32)
    rows = np.unique(np.concatenate([np.linspace(0, m - 1, 16).astype(np.int64), np.arange(m - 4, m)]))
    cases = [dict(cin=bias, act=ACT_RELU), dict(cin=bias, act=ACT_SILU, alpha=0.5), dict(act=ACT_SIGMOID, scale=scale),
             dict(cin=full_bf16, act=ACT_CLAMP, lo=-0.5, hi=0.75, scale=scale, alpha=1.5)]
    for kw in cases:
        cin = kw.get("cin")
        cin_rows = None if cin is None else (cin if cin.ndim == 1 else cin[rows])
        for out_bf16 in (True, False):
            got = _fused_gpu("bf16", a, b, torch.bfloat16 if out_bf16 else torch.float32, K.KERNEL_BF16_TCGEN05, cin=cin,
                             alpha=kw.get("alpha", 1.0), scale=kw.get("scale"), act=kw.get("act", 0), lo=kw.get("lo", 0.0), hi=kw.get("hi", 0.0))
            want = port.matmul_bf16_fused(a[rows], b, cin_rows, kw.get("alpha", 1.0), kw.get("scale"), kw.get("act", 0), kw.get("lo", 0.0),
                                          kw.get("hi", 0.0), out_bf16=out_bf16)
            check("bf16", got[rows], want, str(kw.keys()))


def test_fused_f32_and_weight_only_and_empty_reduction(port):
    from oracle.checker import ACT_RELU, ACT_SILU
    rng = np.random.default_rng(9)
    a = rng.uniform(-1, 1, (130, 70)).astype(np.float32)
    b = rng.uniform(-1, 1, (200, 70)).astype(np.float32)
    bias = rng.uniform(-1, 1, 200).astype(np.float32)
    got = _fused_gpu("f32", a, b, torch.float32, K.KERNEL_F32_SIMT, cin=bias, act=ACT_SILU, alpha=0.25)
    assert rel_frobenius(got, port.matmul_f32_fused(a, b, bias, 0.25, None, ACT_SILU)) <= 1e-5
    # weight-only problems take the fused form in their own kernels: streaming (M <= 16), general, and tensor-core
    bias_w = rng.uniform(-1, 1, 2048).astype(np.float32)
    for m, kernel in ((16, K.KERNEL_W8_SMALL_M), (40, K.KERNEL_W8_SMALL_M), (40, K.KERNEL_W8_TCGEN05), (128, K.KERNEL_AUTO)):
        aw, w, s = inputs("w8", m, 2048, 1024, rng)
        da, dw, ds = to_device(aw, True), to_device(w), to_device(s)
        c = torch.zeros((m, 2048), dtype=torch.bfloat16, device="cuda")
        vecops_b200.matmul(da, dw, c, ds, kernel=kernel, cin=to_device(bias_w), alpha=0.5, activation=ACT_SILU)
        want = port.matmul_bf16_fused(aw, f32_to_bf16_bits(w.astype(np.float32)), bias_w, 0.5, s, ACT_SILU)
        check("w8", bf16_result_to_numpy(c), want, f"m={m} kernel={kernel}")
    # K == 0: the result is transform(CIn)
    e = torch.zeros((4, 8), dtype=torch.float32, device="cuda")
    vecops_b200.matmul(torch.zeros((4, 0), device="cuda"), torch.zeros((8, 0), device="cuda"), e, cin=to_device(bias[:8].copy()), alpha=2.0)
    assert np.allclose(e.cpu().numpy(), np.broadcast_to(bias[:8] * 2.0, (4, 8)))


def test_fused_i8_tcgen05_accumulates_into_an_int32_input(port, cta_form):
    rng = np.random.default_rng(12)
    m, n, k = 1536, 3584, 1024   # split tail tiles too
    a, b, _ = inputs("i8", m, n, k, rng)
    cin = rng.integers(-2**31, 2**31, (m, n), dtype=np.int64).astype(np.int32)
    got = _fused_gpu("i8", a, b, torch.int32, K.KERNEL_I8_TCGEN05, cin=cin)
    rows = np.unique(np.concatenate([np.linspace(0, m - 1, 12).astype(np.int64), np.arange(m - 4, m)]))
    assert np.array_equal(got[rows], port.matmul_i8_accumulate(a[rows], b, cin[rows]))
    row_cin = cin[:1].copy()
    got = _fused_gpu("i8", a, b, torch.int32, K.KERNEL_I8_TCGEN05, cin=row_cin)
    assert np.array_equal(got[rows], port.matmul_i8_accumulate(a[rows], b, row_cin))


def test_fused_form_refuses_what_int32_accumulators_cannot_do():
    a = torch.zeros((16, 64), dtype=torch.int8, device="cuda")
    c = torch.zeros((16, 16), dtype=torch.int32, device="cuda")
    with pytest.raises(capi.VecopsB200Error) as info:
        vecops_b200.matmul(a, a, c, activation=capi.ACTIVATION_RELU)
    assert info.value.code == capi.INVALID_ARGUMENT
    with pytest.raises(capi.VecopsB200Error) as info:
        vecops_b200.matmul(a, a, c, cin=torch.zeros((16, 16), dtype=torch.float32, device="cuda"))
    assert info.value.code == capi.INVALID_ARGUMENT


def _scalar_value(dtype_code, value):
    v = capi.VecopsValue()
    v.struct_size = ctypes.sizeof(capi.VecopsValue)
    v.kind = capi.VALUE_SCALAR
    v.value.scalar.struct_size = ctypes.sizeof(capi.VecopsScalar)
    v.value.scalar.dtype = dtype_code
    if dtype_code == capi.DTYPE_F32:
        v.value.scalar.value.f64 = float(value)   # scalars travel widened, the dtype tag says what they were
    else:
        v.value.scalar.value.i64 = int(value)
    return v


def test_operator_bridge_carries_the_fused_form(port):
    # a, b, c, column_scale = none, cin = a bias row (stride 0), alpha, activation, clamp_lo, clamp_hi
    from oracle.checker import ACT_CLAMP
    lib, handle = bridge_lib()
    rng = np.random.default_rng(31)
    m, n, k = 300, 520, 264
    a, b, _ = inputs("bf16", m, n, k, rng)
    a = f32_to_bf16_bits(bf16_bits_to_f32(a) * 0.1)
    bias = rng.uniform(-1, 1, n).astype(np.float32)
    da, db, dbias = to_device(a, True), to_device(b, True), to_device(bias)
    c = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    keep = []
    none = capi.VecopsValue()
    none.struct_size = ctypes.sizeof(capi.VecopsValue)
    none.kind = capi.VALUE_NONE
    values = [_tensor_value(da, keep=keep), _tensor_value(db, keep=keep), _tensor_value(c, True, keep=keep), none,
              _tensor_value(dbias.expand(m, n), keep=keep), _scalar_value(capi.DTYPE_F32, 0.5), _scalar_value(capi.DTYPE_I32, ACT_CLAMP),
              _scalar_value(capi.DTYPE_F32, -0.75), _scalar_value(capi.DTYPE_F32, 1.25)]
    array = (capi.VecopsValue * len(values))(*values)
    context = capi.VecopsExecutionContext()
    context.struct_size = ctypes.sizeof(context)
    call = capi.VecopsCall(ctypes.sizeof(capi.VecopsCall), len(values), array, None, 0, ctypes.pointer(context))
    error = capi.ErrorBuffer()
    key = ctypes.create_string_buffer(256)
    error.raise_for(lib.vecops_b200_operator_resolve(handle, byref(call), key, 256, byref(error.record)))
    assert key.value.decode() == "vecops::matmul;TA=bf16;TB=bf16;TC=bf16;$0=0;$1=1;$2=f32;$3=0;kernel=bf16_tcgen05"
    error.raise_for(lib.vecops_operator_bridge_invoke_v1(handle, byref(call), 0, None, byref(error.record)))
    want = port.matmul_bf16_fused(a, b, bias, 0.5, None, ACT_CLAMP, -0.75, 1.25)
    check("bf16", bf16_result_to_numpy(c), want)


# ------------------------------------------------------------------ the quantised form as the reference ships it

def _quantized_gpu(a_f32, a_scale, a_zp, b, dequant, kernel, out_dtype=torch.float32, scale=None, act=0):
    """quantise-on-load pre-pass, correction row, u8 x s8 product with int32 accumulate, dequantising transform."""
    m, k = a_f32.shape
    n = b.shape[0]
    da = to_device(a_f32)
    qa = torch.empty((m, k), dtype=torch.uint8, device="cuda")
    harness.quantize_rows(da, qa, a_scale, a_zp)
    db = to_device(b)
    correction = torch.empty(n, dtype=torch.int32, device="cuda")
    harness.column_correction(db, int(a_zp), correction)
    c = torch.full((m, n), -3, dtype=out_dtype, device="cuda")
    ds = to_device(scale) if scale is not None else None
    vecops_b200.matmul(qa, db, c, ds, kernel=kernel, cin=correction, alpha=dequant, activation=act)
    torch.cuda.synchronize()
    return qa.cpu().numpy(), correction.cpu().numpy(), (bf16_result_to_numpy(c) if out_dtype == torch.bfloat16 else c.cpu().numpy())


def test_quantized_golden_fixtures(golden, port):
    seen = 0
    for name, case in golden.items():
        if str(case["kind"]) != "quant_u8s8":
            continue
        for kernel in (K.KERNEL_AUTO, K.KERNEL_GENERIC):
            qa, correction, got = _quantized_gpu(case["a"], float(case["a_scale"]), float(case["a_zero_point"]), case["b"],
                                                 float(case["dequant"]), kernel)
            assert np.array_equal(qa, port.quantize_rows(case["a"], float(case["a_scale"]), float(case["a_zero_point"]))), name
            assert np.array_equal(correction, case["correction"]), name
            assert np.array_equal(got, case["c"]), name   # integers converted and multiplied by a power of two: exact
        seen += 1
    assert seen >= 4


@pytest.mark.parametrize("m,n,k", [(384, 512, 1024), (1536, 3584, 1024)])  # the second: split tail tiles
def test_quantized_form_on_the_tensor_cores(port, cta_form, m, n, k):
    from oracle.checker import ACT_RELU
    rng = np.random.default_rng(m + k)
    a = rng.uniform(-30, 60, (m, k)).astype(np.float32)
    b = rng.integers(-128, 128, (n, k), dtype=np.int8)
    scale = rng.uniform(0.5, 2.0, n).astype(np.float32)
    rows = np.unique(np.concatenate([np.linspace(0, m - 1, 12).astype(np.int64), np.arange(m - 4, m)]))
    for out_dtype in (torch.float32, torch.bfloat16):
        qa, correction, got = _quantized_gpu(a, 2.0, 5.0, b, 0.01, K.KERNEL_I8_TCGEN05, out_dtype, scale, ACT_RELU)
        assert np.array_equal(qa, port.quantize_rows(a, 2.0, 5.0))
        assert np.array_equal(correction, (-5 * b.astype(np.int64).sum(axis=1)).astype(np.int32))
        want = port.matmul_i8_dequant(qa[rows], b, correction, 0.01, scale, ACT_RELU, out_bf16=out_dtype == torch.bfloat16)
        if out_dtype == torch.float32:
            assert rel_frobenius(got[rows], want) <= 1e-6
        else:
            check("bf16", got[rows], want)
    # the plain call of this dtype row: C = float(A . B^T)
    da, db = to_device(qa), to_device(b)
    c = torch.empty((m, n), dtype=torch.float32, device="cuda")
    vecops_b200.matmul(da, db, c, kernel=K.KERNEL_I8_TCGEN05)
    assert np.array_equal(c.cpu().numpy()[rows], port.matmul_i8(qa[rows], b).astype(np.float32))


# ------------------------------------------------------------------ rank-3 operands (a leading batch axis)

def test_batched_golden_fixtures(golden):
    seen = 0
    for name, case in golden.items():
        if str(case["kind"]) != "batched_bf16":
            continue
        batch, m, n = case["c"].shape
        a, b = to_device(case["a"], True), to_device(case["b"], True)
        a3 = a.expand(batch, *a.shape) if a.dim() == 2 else a
        b3 = b.expand(batch, *b.shape) if b.dim() == 2 else b
        c = torch.full((batch, m, n), -3.0, dtype=torch.float32, device="cuda")
        bias = to_device(case["bias"]) if "bias" in case else None
        harness.matmul_batched(a3, b3, c, cin=bias)
        torch.cuda.synchronize()
        check("bf16", c.cpu().numpy().reshape(batch * m, n), case["c"].reshape(batch * m, n), name)
        seen += 1
    assert seen >= 3


def test_batched_on_the_tensor_cores(port):
    rng = np.random.default_rng(17)
    batch, m, n, k = 3, 256, 512, 264
    a = f32_to_bf16_bits(rng.standard_normal((batch, m, k), dtype=np.float32))
    b = f32_to_bf16_bits(rng.standard_normal((batch, n, k), dtype=np.float32))
    bias = rng.uniform(-1, 1, n).astype(np.float32)
    da, db, dbias = to_device(a, True), to_device(b, True), to_device(bias)
    # everything batched, a bias row and ReLU: one launch per entry
    c = torch.zeros((batch, m, n), dtype=torch.bfloat16, device="cuda")
    before = capi.library().vecops_b200_launch_count()
    harness.matmul_batched(da, db, c, cin=dbias, activation=capi.ACTIVATION_RELU)
    assert capi.library().vecops_b200_launch_count() - before == batch
    for i in range(batch):
        check("bf16", bf16_result_to_numpy(c[i]), port.matmul_bf16_fused(a[i], b[i], bias, 1.0, None, 1), f"entry {i}")
    # shared weights, A and C stacked densely: ONE launch with M * batch rows
    c2 = torch.zeros((batch, m, n), dtype=torch.bfloat16, device="cuda")
    before = capi.library().vecops_b200_launch_count()
    harness.matmul_batched(da, db[0].expand(batch, n, k), c2, cin=dbias)
    assert capi.library().vecops_b200_launch_count() - before == 1
    for i in range(batch):
        check("bf16", bf16_result_to_numpy(c2[i]), port.matmul_bf16_fused(a[i], b[0], bias), f"stacked entry {i}")
    # a shared A against batched int8 weights (weight-only row), per-entry launches
    w = rng.integers(-127, 128, (batch, 256, 512), dtype=np.int8)
    aw = f32_to_bf16_bits(rng.standard_normal((16, 512), dtype=np.float32))
    s = rng.uniform(0.001, 0.02, 256).astype(np.float32)
    cw = torch.zeros((batch, 16, 256), dtype=torch.bfloat16, device="cuda")
    harness.matmul_batched(to_device(aw, True).expand(batch, 16, 512), to_device(w), cw, to_device(s))
    for i in range(batch):
        check("w8", bf16_result_to_numpy(cw[i]), port.matmul_w8(aw, w[i], s), f"w8 entry {i}")


# ------------------------------------------------------------------ fp16 operands (the reference's AMX_F16F32 row)

def _f16_gpu(a_bits, b_bits, out_f16, kernel, ldc_pad=0, **fused):
    m, n = a_bits.shape[0], b_bits.shape[0]
    da = to_device(a_bits).view(torch.float16)
    db = to_device(b_bits).view(torch.float16)
    cin = fused.pop("cin", None)
    scale = fused.pop("scale", None)
    storage = torch.full((m, n + ldc_pad), -3, dtype=torch.float16 if out_f16 else torch.float32, device="cuda")
    c = storage[:, :n]
    vecops_b200.matmul(da, db, c, to_device(scale) if scale is not None else None, kernel=kernel,
                       cin=to_device(cin) if cin is not None else None, **fused)
    torch.cuda.synchronize()
    if ldc_pad:
        assert bool((storage[:, n:] == -3).all()), "kernel wrote outside its C columns"
    return c.contiguous().float().cpu().numpy()


def _f16_inputs(m, n, k, rng):
    a = rng.standard_normal((m, k), dtype=np.float32).astype(np.float16).view(np.uint16)
    b = rng.standard_normal((n, k), dtype=np.float32).astype(np.float16).view(np.uint16)
    return a, b


def _f16_want(port, a, b, out_f16, **kw):
    want = port.matmul_f16(a, b, out_f16=out_f16, **kw)
    return want.view(np.float16).astype(np.float32) if out_f16 else want


@pytest.mark.parametrize("m,n,k", TC_SHAPES)
@pytest.mark.parametrize("out_f16", [True, False])
def test_f16_tcgen05(port, cta_form, m, n, k, out_f16):
    # the 16-bit tensor-core kernel with fp16 formats in the instruction descriptor and fp16 tensor maps
    rng = np.random.default_rng(m * 5 + n * 3 + k)
    a, b = _f16_inputs(m, n, k, rng)
    got = _f16_gpu(a, b, out_f16, K.KERNEL_BF16_TCGEN05)
    assert rel_frobenius(got, _f16_want(port, a, b, out_f16)) <= TOL_BF16


def test_f16_precision_is_fp16_not_bf16(port):
    # values with ten mantissa bits: a kernel that read them as bf16, or narrowed them to bf16, would miss by ~4e-3
    rng = np.random.default_rng(3)
    a = (1.0 + rng.integers(0, 1024, (128, 256)) / 1024.0).astype(np.float16).view(np.uint16)
    b = (1.0 + rng.integers(0, 1024, (256, 256)) / 1024.0).astype(np.float16).view(np.uint16)
    for kernel in (K.KERNEL_BF16_TCGEN05, K.KERNEL_GENERIC):
        got = _f16_gpu(a, b, False, kernel)
        assert rel_frobenius(got, _f16_want(port, a, b, False)) <= 1e-5  # fp32 summation order only
        got = _f16_gpu(a, b, True, kernel)
        assert rel_frobenius(got, _f16_want(port, a, b, True)) <= 3e-4  # one fp16 rounding of the result on both sides


def test_f16_ragged_strided_and_fused(port):
    from oracle.checker import ACT_RELU, ACT_SILU
    rng = np.random.default_rng(8)
    # shapes TMA cannot address run on the strided kernel through automatic dispatch
    for m, n, k in [(19, 23, 65), (1, 8, 129), (8, 1, 129), (37, 51, 79)]:
        a, b = _f16_inputs(m, n, k, rng)
        for out_f16 in (True, False):
            got = _f16_gpu(a, b, out_f16, K.KERNEL_AUTO, ldc_pad=3)
            assert rel_frobenius(got, _f16_want(port, a, b, out_f16)) <= TOL_BF16
    # fused output transform on both kernels
    m, n, k = 300, 520, 264
    a, b = _f16_inputs(m, n, k, rng)
    a = (a.view(np.float16).astype(np.float32) * 0.1).astype(np.float16).view(np.uint16)
    bias = rng.uniform(-1, 1, n).astype(np.float32)
    scale = rng.uniform(0.5, 2.0, n).astype(np.float32)
    for kernel in (K.KERNEL_BF16_TCGEN05, K.KERNEL_GENERIC):
        for out_f16 in (True, False):
            got = _f16_gpu(a, b, out_f16, kernel, cin=bias, scale=scale, alpha=0.5, activation=capi.ACTIVATION_SILU)
            want = _f16_want(port, a, b, out_f16, cin=bias, scale=scale, alpha=0.5, act=ACT_SILU)
            assert rel_frobenius(got, want) <= TOL_BF16
            got = _f16_gpu(a, b, out_f16, kernel, activation=capi.ACTIVATION_RELU)
            assert rel_frobenius(got, _f16_want(port, a, b, out_f16, act=ACT_RELU)) <= TOL_BF16


def test_f16_mixed_with_bf16_is_refused():
    a = torch.zeros((128, 64), dtype=torch.float16, device="cuda")
    b = torch.zeros((256, 64), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((128, 256), dtype=torch.float32, device="cuda")
    with pytest.raises(capi.VecopsB200Error):
        vecops_b200.matmul(a, b, c)
    with pytest.raises(capi.VecopsB200Error):  # fp16 operands narrow to fp16 or stay fp32, never bf16
        vecops_b200.matmul(a, a[:64].contiguous(), torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda"))


# ------------------------------------------------------------------ prepared operands (the reference's ops::matmul_pack)

def _torch_of(array, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(array)).cuda()
    return t.view(dtype) if dtype is not None else t


def _strided_source(logical, layout, canary):
    """A device tensor view equal to `logical` [rows, K] under one of the source layouts the pack must serve."""
    rows, k = logical.shape
    if layout == "k_contiguous":
        return _torch_of(logical)
    if layout == "k_contiguous_odd_pitch":        # row pitch K + 3, view starts one element in: nothing is 16-byte aligned
        storage = np.full(rows * (k + 3) + 1, canary, dtype=logical.dtype)
        host = np.lib.stride_tricks.as_strided(storage[1:], (rows, k), ((k + 3) * logical.itemsize, logical.itemsize))
        host[...] = logical
        return torch.as_strided(_torch_of(storage), (rows, k), (k + 3, 1), 1)
    if layout == "row_contiguous":                # stored [K, rows] row-major, handed over as its transposed view
        return _torch_of(np.ascontiguousarray(logical.T)).t()
    if layout == "row_contiguous_odd_pitch":
        storage = np.full(k * (rows + 5) + 3, canary, dtype=logical.dtype)
        host = np.lib.stride_tricks.as_strided(storage[3:], (rows, k), (logical.itemsize, (rows + 5) * logical.itemsize))
        host[...] = logical
        return torch.as_strided(_torch_of(storage), (rows, k), (1, rows + 5), 3)
    if layout == "both_strided":                  # StrideK = 2, row pitch 2K + 3 (tests/ops/MatmulPackTest.cpp:221-237)
        storage = np.full(rows * (2 * k + 3), canary, dtype=logical.dtype)
        host = np.lib.stride_tricks.as_strided(storage, (rows, k), ((2 * k + 3) * logical.itemsize, 2 * logical.itemsize))
        host[...] = logical
        return torch.as_strided(_torch_of(storage), (rows, k), (2 * k + 3, 2), 0)
    raise ValueError(layout)


PACK_LAYOUTS = ["k_contiguous", "k_contiguous_odd_pitch", "row_contiguous", "row_contiguous_odd_pitch", "both_strided"]
PACK_SHAPES = [(16, 32), (17, 33), (19, 35), (1, 1), (16, 64), (31, 79), (129, 65), (300, 1000), (1024, 512), (5, 9)]


@pytest.mark.parametrize("layout", PACK_LAYOUTS)
@pytest.mark.parametrize("dtype,narrow", [(np.int8, None), (np.uint8, None), (np.uint16, None), (np.float32, None), (np.float32, "bf16"),
                                          (np.float32, "f16")])
def test_pack_brings_every_layout_into_the_packed_form(layout, dtype, narrow):
    from oracle.checker import pack_rows
    rng = np.random.default_rng(17)
    torch_out = {None: None, "bf16": torch.bfloat16, "f16": torch.float16}[narrow]
    for rows, k in PACK_SHAPES:
        if dtype == np.float32:
            logical = (rng.standard_normal((rows, k)) * 3).astype(np.float32)
        else:
            info = np.iinfo(dtype)
            logical = rng.integers(info.min, int(info.max) + 1, (rows, k)).astype(dtype)
        source = _strided_source(logical, layout, canary=dtype(77))
        if dtype == np.uint16:
            source = source.view(torch.bfloat16)  # any 2-byte type: a bit copy
        packed = harness.pack_operand(source, torch_out)
        torch.cuda.synchronize()
        want = pack_rows(logical, narrow)
        assert packed.stride(0) == want.shape[1] and packed.stride(1) == 1, (rows, k)
        whole = torch.as_strided(packed, (rows, want.shape[1]), (want.shape[1], 1))
        got = whole.contiguous().view(torch.int16 if want.itemsize == 2 else whole.dtype).cpu().numpy().view(want.dtype)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), f"{layout} {dtype} {narrow} rows={rows} k={k}"


def test_packed_layout_sizes_and_refusals():
    assert harness.packed_layout(torch.int8, 33, 129) == (256, 33 * 256)
    assert harness.packed_layout(torch.bfloat16, 19, 35) == (64, 19 * 128)
    assert harness.packed_layout(torch.float32, 5, 32) == (32, 5 * 128)
    assert harness.packed_layout(torch.bfloat16, 7, 0) == (0, 0)          # a zero-K packed layout is empty
    assert harness.packed_layout(torch.int8, 0, 64) == (128, 0)
    harness.pack_operand(torch.empty((0, 64), dtype=torch.int8, device="cuda"))  # zero extents touch no memory
    harness.pack_operand(torch.empty((9, 0), dtype=torch.bfloat16, device="cuda"))
    lib = capi.library()
    src = torch.zeros((64, 64), dtype=torch.int8, device="cuda")
    dst = torch.zeros((64, 128), dtype=torch.int8, device="cuda")

    def record(source, destination, size, dst_dtype=capi.DTYPE_I8):
        return capi.VecopsB200Pack(ctypes.sizeof(capi.VecopsB200Pack), 1, 64, 64, source.data_ptr(), 64, 1, capi.DTYPE_I8, dst_dtype,
                                   destination.data_ptr(), size, -1, 0, None)

    for bad in (record(src, dst, 64 * 128 - 1),                      # undersized destination
                record(src, src, 64 * 128),                          # aliasing
                record(src, dst, 64 * 128, capi.DTYPE_BF16)):        # int8 -> bf16 is not a packing conversion
        error = capi.ErrorBuffer()
        assert lib.vecops_b200_matmul_pack(byref(bad), byref(error.record)) == capi.INVALID_ARGUMENT
    error = capi.ErrorBuffer()
    misaligned = capi.VecopsB200Pack(ctypes.sizeof(capi.VecopsB200Pack), 1, 32, 64, src.data_ptr(), 64, 1, capi.DTYPE_I8, capi.DTYPE_I8,
                                     dst.data_ptr() + 4, 32 * 128, -1, 0, None)
    assert lib.vecops_b200_matmul_pack(byref(misaligned), byref(error.record)) == capi.INVALID_ARGUMENT


def test_packed_operands_reach_the_tensor_core_kernels(port):
    # a [K, N]-stored weight and an odd K both send the raw views to the strided kernel; their packed forms run on tcgen05
    rng = np.random.default_rng(23)
    m, n, k = 256, 512, 325
    a, b, _ = inputs("bf16", m, n, k, rng)
    da = to_device(a, bf16=True)
    db_kn = to_device(np.ascontiguousarray(b.T), bf16=True).t()           # [N, K] view of a [K, N] matrix
    c = torch.empty((m, n), dtype=torch.float32, device="cuda")
    assert vecops_b200.select_kernel(vecops_b200.matmul_problem(da, db_kn, c)) == K.KERNEL_GENERIC
    pa, pb = harness.pack_operand(da, operand=0), harness.pack_operand(db_kn)
    assert vecops_b200.select_kernel(vecops_b200.matmul_problem(pa, pb, c)) == K.KERNEL_BF16_TCGEN05
    vecops_b200.matmul(pa, pb, c)
    torch.cuda.synchronize()
    check("bf16", c.cpu().numpy(), port.matmul_bf16(a, b, None, False))
    # fp32 storage narrowed to the bf16 compute type while packing (memory type != compute type)
    a32, b32 = bf16_bits_to_f32(a) * 1.001, bf16_bits_to_f32(b) * 0.999
    pa = harness.pack_operand(torch.from_numpy(a32).cuda(), torch.bfloat16, operand=0)
    pb = harness.pack_operand(torch.from_numpy(np.ascontiguousarray(b32.T)).cuda().t(), torch.bfloat16)
    vecops_b200.matmul(pa, pb, c)
    torch.cuda.synchronize()
    check("bf16", c.cpu().numpy(), port.matmul_bf16(f32_to_bf16_bits(a32), f32_to_bf16_bits(b32), None, False))
    # int8: bit-exact, and equal to what the raw strided views give
    ai = rng.integers(-128, 128, (m, k)).astype(np.int8)
    bi = rng.integers(-128, 128, (n, k)).astype(np.int8)
    dai, dbi = to_device(ai), to_device(np.ascontiguousarray(bi.T)).t()
    ci_raw = torch.empty((m, n), dtype=torch.int32, device="cuda")
    ci_packed = torch.empty((m, n), dtype=torch.int32, device="cuda")
    vecops_b200.matmul(dai, dbi, ci_raw)
    pai, pbi = harness.pack_operand(dai, operand=0), harness.pack_operand(dbi)
    assert vecops_b200.select_kernel(vecops_b200.matmul_problem(pai, pbi, ci_packed)) == K.KERNEL_I8_TCGEN05
    vecops_b200.matmul(pai, pbi, ci_packed)
    torch.cuda.synchronize()
    want = port.matmul_i8(ai, bi)
    assert np.array_equal(ci_packed.cpu().numpy(), want) and np.array_equal(ci_raw.cpu().numpy(), want)


def test_pack_b_compensated_emits_the_zero_point_row(port):
    from oracle.checker import pack_compensation, pack_rows
    # the reference test's own case: N=33, K=129, row pitch K+3, a_zero_point 3, values (n*17 + k*3) % 61 - 30
    # (tests/ops/MatmulPackTest.cpp:354-376); the row after the compensation keeps its canary (:217)
    n, k, zp = 33, 129, 3
    logical = ((np.arange(n)[:, None] * 17 + np.arange(k)[None, :] * 3) % 61 - 30).astype(np.int8)
    source = _strided_source(logical, "k_contiguous_odd_pitch", np.int8(-99))
    pitch, size = harness.packed_layout(torch.int8, n, k)
    storage = torch.zeros(n * pitch, dtype=torch.int8, device="cuda")
    compensation = torch.full((n + 1,), 0x13579bdf, dtype=torch.int32, device="cuda")
    record = capi.VecopsB200Pack(ctypes.sizeof(capi.VecopsB200Pack), 1, n, k, source.data_ptr(), source.stride(0), source.stride(1), capi.DTYPE_I8,
                                 capi.DTYPE_I8, storage.data_ptr(), size, -1, 0, None)
    error = capi.ErrorBuffer()
    error.raise_for(capi.library().vecops_b200_matmul_pack_b_compensated(byref(record), zp, compensation.data_ptr(), byref(error.record)))
    torch.cuda.synchronize()
    assert np.array_equal(storage.view(n, pitch).cpu().numpy(), pack_rows(logical))
    assert np.array_equal(compensation[:n].cpu().numpy(), pack_compensation(logical, zp))
    assert int(compensation[n]) == 0x13579bdf
    # and used: u8 A (zero point 3) x packed s8 B with the row as the accumulator input equals the product of the centred values
    rng = np.random.default_rng(4)
    a_u8 = rng.integers(0, 256, (21, k)).astype(np.uint8)
    packed, row = harness.pack_operand(source, zero_point=zp)
    c = torch.empty((21, n), dtype=torch.int32, device="cuda")
    vecops_b200.matmul(harness.pack_operand(to_device(a_u8), operand=0), packed, c, cin=row)
    torch.cuda.synchronize()
    centred = (a_u8.astype(np.int64) - zp) @ logical.astype(np.int64).T
    assert np.array_equal(c.cpu().numpy(), centred.astype(np.int32))
    # zero extents (tests/ops/MatmulPackTest.cpp:401-434): K == 0 gives an all-zero row
    empty = torch.empty((7, 0), dtype=torch.int8, device="cuda")
    _, row0 = harness.pack_operand(empty, zero_point=5)
    torch.cuda.synchronize()
    assert bool((row0 == 0).all()) and row0.numel() == 7


def test_pack_b_compensated_golden_fixtures(golden):
    """The compensation rows the reference's own ops::matmul_pack_b_compensated emitted, bit for bit, and the packed
    operand beside them (every position the logical element, zero past K)."""
    from oracle.checker import pack_rows
    seen = 0
    for name, case in golden.items():
        if str(case["kind"]) != "pack_comp":
            continue
        b, zp = case["b"], int(case["zero_point"])
        packed, row = harness.pack_operand(to_device(b), zero_point=zp)
        torch.cuda.synchronize()
        assert np.array_equal(row.cpu().numpy(), case["compensation"]), name
        assert np.array_equal(packed.cpu().numpy(), pack_rows(b)[:, :b.shape[1]]), name
        seen += 1
    assert seen >= 4


def test_pack_operator_through_the_bridge():
    # vecops::matmul_pack behind the same Operator machinery: {src, dst} and {src, dst, compensation, a_zero_point}
    from oracle.checker import pack_compensation, pack_rows
    lib, _ = bridge_lib()
    lib.vecops_b200_matmul_pack_operator.restype = ctypes.c_uint64
    lib.vecops_b200_matmul_pack_operator.argtypes = [ctypes.c_int32]
    handle = lib.vecops_b200_matmul_pack_operator(0)
    compensated_handle = lib.vecops_b200_matmul_pack_operator(1)
    rng = np.random.default_rng(31)
    n, k = 200, 333
    logical = rng.integers(-128, 128, (n, k)).astype(np.int8)
    source = to_device(np.ascontiguousarray(logical.T)).t()            # a [K, N]-stored weight
    pitch, _ = harness.packed_layout(torch.int8, n, k)
    dst = torch.full((n, pitch), 55, dtype=torch.int8, device="cuda")
    row = torch.zeros(n, dtype=torch.int32, device="cuda")

    def frame(values, keep):
        array = (capi.VecopsValue * len(values))(*values)
        context = capi.VecopsExecutionContext()
        context.struct_size = ctypes.sizeof(context)
        context.stream = None
        keep.extend([array, context])
        return capi.VecopsCall(ctypes.sizeof(capi.VecopsCall), len(values), array, None, 0, ctypes.pointer(context))

    keep = []
    call = frame([_tensor_value(source, keep=keep), _tensor_value(dst, True, keep=keep)], keep)
    error = capi.ErrorBuffer()
    key = ctypes.create_string_buffer(256)
    error.raise_for(lib.vecops_b200_operator_resolve(handle, byref(call), key, 256, byref(error.record)))
    assert key.value.decode() == "vecops::matmul_pack;TD=i8;TS=i8;kernel=pack", key.value
    error.raise_for(lib.vecops_operator_bridge_invoke_v1(handle, byref(call), 0, None, byref(error.record)))
    torch.cuda.synchronize()
    assert np.array_equal(dst.cpu().numpy(), pack_rows(logical))
    dst.fill_(55)
    call = frame([_tensor_value(source, keep=keep), _tensor_value(dst, True, keep=keep), _tensor_value(row, True, keep=keep),
                  _scalar_value(capi.DTYPE_I32, 7)], keep)
    assert lib.vecops_operator_bridge_invoke_v1(handle, byref(call), 0, None, byref(capi.ErrorBuffer().record)) != capi.OK  # its own operator
    error.raise_for(lib.vecops_operator_bridge_invoke_v1(compensated_handle, byref(call), 0, None, byref(error.record)))
    torch.cuda.synchronize()
    assert np.array_equal(dst.cpu().numpy(), pack_rows(logical))
    assert np.array_equal(row.cpu().numpy(), pack_compensation(logical, 7))
    # a destination that is not a tensor over the packed layout is refused
    wrong = torch.zeros((n, k), dtype=torch.int8, device="cuda")
    call = frame([_tensor_value(source, keep=keep), _tensor_value(wrong, True, keep=keep)], keep)
    error = capi.ErrorBuffer()
    assert lib.vecops_operator_bridge_invoke_v1(handle, byref(call), 0, None, byref(error.record)) != capi.OK


# ------------------------------------------------------------------ the caller one step up: scaled dot-product attention

SDPA_STRATEGIES = [capi.SDPA_MATERIALIZED, capi.SDPA_STREAMING]


def _launches() -> int:
    capi.library().vecops_b200_launch_count.restype = ctypes.c_uint64
    return capi.library().vecops_b200_launch_count()


def _sdpa_gpu(case_or_kwargs, out_dtype=torch.float32, strategy=capi.SDPA_AUTOMATIC):
    c = case_or_kwargs
    q, k, v = (to_device(c[name], bf16=True) for name in ("q", "k", "v"))
    out = torch.full((q.shape[0], v.shape[1]), -99, dtype=out_dtype, device="cuda")
    optional = {name: to_device(np.ascontiguousarray(c[name])) for name in ("query_mask", "key_mask", "keep_mask", "bias") if c.get(name) is not None}
    harness.sdpa(q, k, v, out, float(c["scale"]), causal=int(c.get("causal", 0)), strategy=strategy, **optional)
    torch.cuda.synchronize()
    return bf16_bits_to_f32(bf16_result_to_numpy(out)) if out_dtype == torch.bfloat16 else out.cpu().numpy()


def _stream_cut(lq, lkv, causal, asked):
    """128-key tiles per work item the streaming launch uses when VECOPS_B200_SDPA_CHUNK_TILES asks for `asked`: a query
    block's keys are never cut into more than 32 chunks, and a chunk is never longer than the block with the most keys."""
    last = lkv - 1 if causal == 0 else min(lkv - 1, lq - 1 + (lkv - lq if causal == 2 else 0))
    most = max(1, last // 128 + 1) if last >= 0 else 1
    return min(max(asked, -(-most // 32)), most)


def _sdpa_want(port, strategy, q, k, v, scale, cut=0, **kwargs):
    """The checker's result for the strategy: the two differ in where probabilities are rounded to bf16 (2e-3 .. 4e-3 apart,
    as the reference's own two strategies are), so each kernel is held to the restatement of ITS strategy - for the
    streaming one with the same cut of the keys into chunks."""
    if strategy == capi.SDPA_STREAMING:
        return port.sdpa_bf16_streaming(q, k, v, scale, chunk_blocks=cut, **kwargs)
    return port.sdpa_bf16(q, k, v, scale, **kwargs)


@pytest.mark.parametrize("strategy,cut", [(capi.SDPA_MATERIALIZED, 0), (capi.SDPA_STREAMING, 1000), (capi.SDPA_STREAMING, 1)])
def test_sdpa_golden_fixtures(golden, port, monkeypatch, strategy, cut):
    # outputs of the reference's own scaled_dot_product_attention, by its materialized and by its streaming strategy, on
    # its tests' operand patterns and on seeded cases
    monkeypatch.setenv("VECOPS_B200_SDPA_CHUNK_TILES", str(cut))
    seen = 0
    for name, case in golden.items():
        if str(case["kind"]) != "sdpa_bf16":
            continue
        got = _sdpa_gpu(case, strategy=strategy)
        want = case["out"] if strategy == capi.SDPA_MATERIALIZED else case["out_streaming"]
        if cut == 1:  # every 128-key tile on its own SM, merged at the end: the reference has no such cut, the restatement does
            optional = {n: case[n] for n in ("query_mask", "key_mask", "keep_mask", "bias") if case.get(n) is not None}
            want = port.sdpa_bf16_streaming(case["q"], case["k"], case["v"], float(case["scale"]), causal=int(case["causal"]), chunk_blocks=1, **optional)
        assert rel_frobenius(got, want) <= TOL_BF16, name
        assert np.array_equal((got == 0).all(axis=1), (want == 0).all(axis=1)), name  # fully masked rows are exactly zero
        seen += 1
    assert seen >= 6


@pytest.mark.parametrize("lq,lkv,dqk,dv,causal", [(512, 768, 64, 64, 0), (1024, 1024, 128, 128, 2), (300, 520, 72, 40, 1), (1, 2048, 128, 128, 0),
                                                    (257, 129, 64, 96, 2), (40, 9000, 64, 64, 0)])  # the last: rows too long for registers
@pytest.mark.parametrize("strategy", SDPA_STRATEGIES)
def test_sdpa_against_the_checker(port, monkeypatch, lq, lkv, dqk, dv, causal, strategy):
    # sizes at which both products run on the tensor-core kernels (and ragged ones that do not)
    monkeypatch.setenv("VECOPS_B200_SDPA_CHUNK_TILES", "2")
    cut = _stream_cut(lq, lkv, causal, 2)
    rng = np.random.default_rng(lq + lkv)
    case = dict(q=f32_to_bf16_bits(rng.standard_normal((lq, dqk)).astype(np.float32)),
                k=f32_to_bf16_bits(rng.standard_normal((lkv, dqk)).astype(np.float32)),
                v=f32_to_bf16_bits(rng.standard_normal((lkv, dv)).astype(np.float32)), scale=1.0 / np.sqrt(dqk), causal=causal)
    rows = np.unique(np.concatenate([np.linspace(0, lq - 1, 24).astype(np.int64), np.arange(max(0, lq - 3), lq)]))
    got = _sdpa_gpu(case, strategy=strategy)
    # rows of attention are independent: the checker runs on a sample of query rows (causal cuts are per row, so the
    # sample keeps its row indices through a keep mask instead)
    last = np.arange(lq)[:, None] + (0 if causal == 1 else lkv - lq)
    keep = np.ones((lq, lkv), np.uint8) if causal == 0 else (np.arange(lkv)[None, :] <= last).astype(np.uint8)
    want = _sdpa_want(port, strategy, case["q"][rows], case["k"], case["v"], case["scale"], cut, keep_mask=keep[rows])
    assert rel_frobenius(got[rows], want) <= TOL_BF16
    # with every optional operand, bf16 out
    case.update(query_mask=(rng.random(lq) > 0.1).astype(np.uint8), key_mask=(rng.random(lkv) > 0.1).astype(np.uint8),
                keep_mask=(rng.random((lq, lkv)) > 0.05).astype(np.uint8), bias=rng.uniform(-1, 1, (lq, lkv)).astype(np.float32))
    got = _sdpa_gpu(case, torch.bfloat16, strategy=strategy)
    combined = (keep & case["keep_mask"])[rows]
    want = _sdpa_want(port, strategy, case["q"][rows], case["k"], case["v"], case["scale"], cut, query_mask=case["query_mask"][rows],
                      key_mask=case["key_mask"], keep_mask=combined, bias=case["bias"][rows], out_bf16=True)
    assert rel_frobenius(got[rows], bf16_bits_to_f32(want)) <= 3e-3  # one more bf16 rounding of the output on both sides


def test_sdpa_degenerate_extents_and_refusals():
    q = torch.zeros((4, 8), dtype=torch.bfloat16, device="cuda")
    out = torch.full((4, 8), 7.0, dtype=torch.float32, device="cuda")
    harness.sdpa(q, torch.zeros((0, 8), dtype=torch.bfloat16, device="cuda"), torch.zeros((0, 8), dtype=torch.bfloat16, device="cuda"), out, 1.0)
    torch.cuda.synchronize()
    assert bool((out == 0).all())  # no key: every row is an all-dropped row
    harness.sdpa(q[:0], q, q, out[:0], 1.0)  # no query: nothing to write
    with pytest.raises(capi.VecopsB200Error):
        harness.sdpa(q.float(), q.float(), q.float(), out, 1.0)  # fp32 q, k, v are not served
    record = harness.sdpa_record(q, q, q, out, 1.0, strategy=capi.SDPA_MATERIALIZED)
    error = capi.ErrorBuffer()
    assert capi.library().vecops_b200_sdpa_run(byref(record), byref(error.record)) == capi.INVALID_ARGUMENT  # no scratch given
    # the streaming kernel needs scratch only where it cuts a query block's keys into chunks, and does not cut without it
    k = torch.randn((1024, 8), device="cuda").to(torch.bfloat16)
    record = harness.sdpa_record(q, k, k, out, 1.0, strategy=capi.SDPA_STREAMING)
    assert harness.sdpa_plan(record) == (capi.SDPA_STREAMING, 1)
    assert capi.library().vecops_b200_sdpa_run(byref(record), byref(error.record)) == capi.OK
    reference = torch.softmax((q.float() @ k.float().t()), dim=1) @ k.float()
    assert torch.allclose(out, reference, atol=2e-2)


def test_sdpa_strategy_choice():
    """Automatic takes the streaming kernel (a pack of V and one launch for all heads) whenever it can serve the call and the
    composition through the matmul path (four launches per head) otherwise; a forced streaming call that cannot be
    served says so instead of running something else."""
    q = torch.randn((3, 256, 64), device="cuda").to(torch.bfloat16)
    out = torch.empty((3, 256, 64), dtype=torch.float32, device="cuda")
    before = _launches()
    harness.sdpa(q, q, q, out, 0.125)
    assert _launches() - before == 1 + 1  # the attention launch for all heads, the merge of the key chunks
    before = _launches()
    harness.sdpa(q, q, q, out, 0.125, strategy=capi.SDPA_MATERIALIZED)
    assert _launches() - before == 3 * 4
    strided = torch.randn((64, 256), device="cuda").to(torch.bfloat16).t()  # [256, 64] with the head dim strided
    out2 = torch.empty((256, 64), dtype=torch.float32, device="cuda")
    before = _launches()
    harness.sdpa(strided, strided, strided, out2, 0.125)
    assert _launches() - before == 4
    with pytest.raises(capi.VecopsB200Error) as info:
        harness.sdpa(strided, strided, strided, out2, 0.125, strategy=capi.SDPA_STREAMING)
    assert info.value.code == capi.NOT_APPLICABLE
    torch.cuda.synchronize()


@pytest.mark.parametrize("lq,lkv,d,causal,heads", [(4096, 4096, 128, 2, 1),   # every query block's keys cut into chunks that meet in scratch
                                                   (128, 8192, 64, 0, 2),     # one query block per head, 32 chunks each (decode-like)
                                                   (1000, 3000, 128, 1, 3)])  # ragged edges, top-left cut: late blocks see few keys
def test_sdpa_streaming_chunks_merge(port, monkeypatch, lq, lkv, d, causal, heads):
    monkeypatch.setenv("VECOPS_B200_SDPA_CHUNK_TILES", "4")
    cut = _stream_cut(lq, lkv, causal, 4)
    rng = np.random.default_rng(lq + lkv + heads)
    qh = f32_to_bf16_bits(rng.standard_normal((heads, lq, d)).astype(np.float32))
    kh = f32_to_bf16_bits(rng.standard_normal((heads, lkv, d)).astype(np.float32))
    vh = f32_to_bf16_bits(rng.standard_normal((heads, lkv, d)).astype(np.float32))
    out = torch.full((heads, lq, d), -99, dtype=torch.float32, device="cuda")
    scale = 1.0 / np.sqrt(d)
    for repeat in range(2):  # the second call finds the first one's counters and partial records in its scratch
        harness.sdpa(to_device(qh, bf16=True), to_device(kh, bf16=True), to_device(vh, bf16=True), out, scale, causal=causal,
                     strategy=capi.SDPA_STREAMING)
        torch.cuda.synchronize()
        rows = np.unique(np.concatenate([np.linspace(0, lq - 1, 20).astype(np.int64), np.arange(max(0, lq - 2), lq)]))
        last = np.arange(lq)[:, None] + (0 if causal == 1 else lkv - lq)
        keep = np.ones((lq, lkv), np.uint8) if causal == 0 else (np.arange(lkv)[None, :] <= last).astype(np.uint8)
        for h in range(heads):
            want = port.sdpa_bf16_streaming(qh[h][rows], kh[h], vh[h], scale, keep_mask=keep[rows], chunk_blocks=cut)
            assert rel_frobenius(out[h].cpu().numpy()[rows], want) <= TOL_BF16, (repeat, h)


def _frame_of(values, keep, workspace=None):
    array = (capi.VecopsValue * len(values))(*values)
    context = capi.VecopsExecutionContext()
    context.struct_size = ctypes.sizeof(context)
    context.stream = None
    keep.extend([array, context, workspace])
    return capi.VecopsCall(ctypes.sizeof(capi.VecopsCall), len(values), array, workspace.data_ptr() if workspace is not None else None,
                           workspace.numel() if workspace is not None else 0, ctypes.pointer(context))


def _none_value():
    v = capi.VecopsValue()
    v.struct_size = ctypes.sizeof(capi.VecopsValue)
    v.kind = capi.VALUE_NONE
    return v


def test_callers_through_the_operator_layer(port, golden, monkeypatch):
    """Rank-3 matmul, attention and the per-row quantiser as operators behind vecops_operator_bridge_invoke_v1: the same
    frames, keys and errors as the matmul operator's, held to the reference-made fixtures."""
    lib, _ = bridge_lib()
    lib.vecops_b200_caller_operator.restype = ctypes.c_uint64
    lib.vecops_b200_caller_operator.argtypes = [ctypes.c_uint32]
    lib.vecops_b200_operator_workspace.argtypes = [ctypes.c_uint64, ctypes.POINTER(capi.VecopsCall), ctypes.POINTER(ctypes.c_uint64),
                                                   ctypes.POINTER(capi.VecopsError)]
    batched, attention, quantize = (lib.vecops_b200_caller_operator(i) for i in range(3))
    assert batched and attention and quantize and lib.vecops_b200_caller_operator(3) == 0
    error = capi.ErrorBuffer()
    key = ctypes.create_string_buffer(256)
    # rank-3 matmul: the reference's own batch fixtures, shared weights as a stride-0 view
    for name, case in golden.items():
        if str(case["kind"]) != "batched_bf16":
            continue
        if "bias" in case:
            continue  # (an accumulator input is the fused form's: the C entry point takes it, this operator does not)
        batch = case["c"].shape[0]
        a = to_device(case["a"], bf16=True)
        b = to_device(case["b"], bf16=True)
        a = a.expand(batch, *a.shape) if a.dim() == 2 else a
        b = b.expand(batch, *b.shape) if b.dim() == 2 else b
        c = torch.full((batch, a.shape[1], b.shape[1]), -5.0, dtype=torch.float32, device="cuda")
        keep = []
        call = _frame_of([_tensor_value(a, keep=keep), _tensor_value(b, keep=keep), _tensor_value(c, True, keep=keep)], keep)
        error.raise_for(lib.vecops_b200_operator_resolve(batched, byref(call), key, 256, byref(error.record)))
        assert key.value.decode().startswith("vecops::matmul_batched;TA=bf16;TB=bf16;TC=f32"), key.value
        error.raise_for(lib.vecops_operator_bridge_invoke_v1(batched, byref(call), 0, None, byref(error.record)))
        torch.cuda.synchronize()
        assert rel_frobenius(c.cpu().numpy(), case["c"]) <= TOL_BF16, name
    # a rank-2 operand is not this operator's
    keep = []
    flat = torch.zeros((4, 8), dtype=torch.bfloat16, device="cuda")
    call = _frame_of([_tensor_value(flat, keep=keep), _tensor_value(flat, keep=keep), _tensor_value(flat, True, keep=keep)], keep)
    assert lib.vecops_operator_bridge_invoke_v1(batched, byref(call), 0, None, byref(capi.ErrorBuffer().record)) != capi.OK
    # attention: one fixture with masks and bias as a single head, scratch as the workspace query sizes it
    monkeypatch.setenv("VECOPS_B200_SDPA_CHUNK_TILES", "1000")
    case = golden["sdpa_masks_130x257x64x64"]
    q, k, v = (to_device(case[n], bf16=True).unsqueeze(0) for n in ("q", "k", "v"))
    out = torch.full((1, q.shape[1], v.shape[2]), -5.0, dtype=torch.float32, device="cuda")
    key_mask, bias = to_device(case["key_mask"]), to_device(case["bias"]).unsqueeze(0)
    keep = []
    values = [_tensor_value(q, keep=keep), _tensor_value(k, keep=keep), _tensor_value(v, keep=keep), _tensor_value(out, True, keep=keep),
              _scalar_value(capi.DTYPE_F32, float(case["scale"])), _scalar_value(capi.DTYPE_I32, int(case["causal"])),
              _tensor_value(key_mask, keep=keep), _tensor_value(bias, keep=keep)]
    call = _frame_of(values, keep)
    need = ctypes.c_uint64(0)
    error.raise_for(lib.vecops_b200_operator_workspace(attention, byref(call), byref(need), byref(error.record)))
    scratch = torch.empty(max(need.value, 1), dtype=torch.uint8, device="cuda")
    call = _frame_of(values, keep, scratch if need.value else None)
    error.raise_for(lib.vecops_operator_bridge_invoke_v1(attention, byref(call), 0, None, byref(error.record)))
    torch.cuda.synchronize()
    want = port.sdpa_bf16_streaming(case["q"], case["k"], case["v"], float(case["scale"]), key_mask=case["key_mask"], bias=case["bias"],
                                    causal=int(case["causal"]))
    assert rel_frobenius(out[0].cpu().numpy(), want) <= TOL_BF16
    # the per-row quantiser: the reference's own per-token fixture, bit for bit
    case = next(c for c in golden.values() if str(c["kind"]) == "quant_per_row")
    src, multipliers = to_device(case["a"]), to_device(case["multipliers"])
    dst = torch.zeros(case["a"].shape, dtype=torch.uint8, device="cuda")
    keep = []
    call = _frame_of([_tensor_value(src, keep=keep), _tensor_value(multipliers, keep=keep), _tensor_value(dst, True, keep=keep),
                      _scalar_value(capi.DTYPE_F32, float(case["zero_point"]))], keep)
    error.raise_for(lib.vecops_operator_bridge_invoke_v1(quantize, byref(call), 0, None, byref(error.record)))
    assert np.array_equal(dst.cpu().numpy(), port.quantize_rows_per_row(case["a"], case["multipliers"], float(case["zero_point"])))


@pytest.mark.parametrize("strategy", SDPA_STRATEGIES)
def test_sdpa_heads_in_one_call(port, monkeypatch, strategy):
    monkeypatch.setenv("VECOPS_B200_SDPA_CHUNK_TILES", "1000")  # 160 keys: two tiles, kept together
    # [heads, L, D] operands; K and V shared by pairs of heads (grouped-query: head stride via expanded views), one mask for all
    rng = np.random.default_rng(77)
    heads, lq, lkv, d = 4, 96, 160, 64
    qh = f32_to_bf16_bits(rng.standard_normal((heads, lq, d)).astype(np.float32))
    kh = f32_to_bf16_bits(rng.standard_normal((heads // 2, lkv, d)).astype(np.float32))
    vh = f32_to_bf16_bits(rng.standard_normal((heads // 2, lkv, d)).astype(np.float32))
    key_mask = (rng.random(lkv) > 0.2).astype(np.uint8)
    bias = rng.uniform(-1, 1, (heads, lq, lkv)).astype(np.float32)
    q = to_device(qh, bf16=True)
    k = to_device(kh, bf16=True).repeat_interleave(2, dim=0)       # heads 0,1 -> group 0; heads 2,3 -> group 1
    v = to_device(vh, bf16=True).repeat_interleave(2, dim=0)
    out = torch.full((heads, lq, d), -99, dtype=torch.float32, device="cuda")
    harness.sdpa(q, k, v, out, 0.125, key_mask=to_device(key_mask), bias=to_device(bias), causal=capi.CAUSAL_BOTTOM_RIGHT, strategy=strategy)
    torch.cuda.synchronize()
    for h in range(heads):
        want = _sdpa_want(port, strategy, qh[h], kh[h // 2], vh[h // 2], 0.125, key_mask=key_mask, bias=bias[h], causal=2)
        assert rel_frobenius(out[h].cpu().numpy(), want) <= TOL_BF16, h
    # a head stride of 0 shares K and V between all heads
    shared_k, shared_v = to_device(kh[:1], bf16=True).expand(heads, lkv, d), to_device(vh[:1], bf16=True).expand(heads, lkv, d)
    harness.sdpa(q, shared_k, shared_v, out, 0.125, strategy=strategy)
    torch.cuda.synchronize()
    for h in (0, heads - 1):
        assert rel_frobenius(out[h].cpu().numpy(), _sdpa_want(port, strategy, qh[h], kh[0], vh[0], 0.125)) <= TOL_BF16, h



@pytest.mark.parametrize("b_kn", [True, False])
def test_f32_whole_tile_form_agrees_with_the_general_kernel(port, b_kn, monkeypatch):
    # shapes made of whole 64 x 64 x 16 tiles run on the 8 x 8-per-thread kernel; the switch keeps the general one
    from oracle.checker import ACT_SILU
    rng = np.random.default_rng(12)
    a, b, _ = inputs("f32", 192, 256, 80, rng)
    want = port.matmul_f32(a, b)
    fast = run_case("f32", a, b, kernel=K.KERNEL_F32_SIMT, b_kn=b_kn)
    monkeypatch.setenv("VECOPS_B200_F32_TILE8", "0")
    general = run_case("f32", a, b, kernel=K.KERNEL_F32_SIMT, b_kn=b_kn)
    monkeypatch.delenv("VECOPS_B200_F32_TILE8")
    assert rel_frobenius(fast, want) <= TOL_F32 and rel_frobenius(general, want) <= TOL_F32
    assert rel_frobenius(fast, general) <= 1e-6  # the same fp32 FMAs in the same k order
    bias = rng.uniform(-1, 1, 256).astype(np.float32)
    got = _fused_gpu("f32", a, b, torch.float32, K.KERNEL_F32_SIMT, cin=bias, act=ACT_SILU, alpha=0.25)
    assert rel_frobenius(got, port.matmul_f32_fused(a, b, bias, 0.25, None, ACT_SILU)) <= 1e-5


# ------------------------------------------------------------------ per-token quantisation: row multipliers in, row-by-column scales out

def _per_row_gpu(a, multipliers, zero_point, b, correction, row_scales, column_scales, kernel, out_dtype=torch.float32):
    m, k = a.shape
    n = b.shape[0]
    qa = torch.empty((m, k), dtype=torch.uint8, device="cuda")
    harness.quantize_rows(to_device(a), qa, to_device(np.ascontiguousarray(multipliers, dtype=np.float32)), float(zero_point))
    c = torch.full((m, n), -3, dtype=out_dtype, device="cuda")
    vecops_b200.matmul(qa, to_device(b), c, to_device(column_scales), kernel=kernel, cin=to_device(correction),
                       row_scale=to_device(np.ascontiguousarray(row_scales, dtype=np.float32)))
    torch.cuda.synchronize()
    return qa.cpu().numpy(), (bf16_result_to_numpy(c) if out_dtype == torch.bfloat16 else c.cpu().numpy())


def test_per_row_quantised_golden_fixtures(port, golden):
    # outputs of the reference's own per-row quantise / row-by-column dequantise transforms: bit-exact
    seen = 0
    for name, case in golden.items():
        if str(case["kind"]) != "quant_per_row":
            continue
        for kernel in (K.KERNEL_AUTO, K.KERNEL_GENERIC):
            quantized, got = _per_row_gpu(case["a"], case["multipliers"], int(case["zero_point"]), case["b"], case["correction"], case["row_scales"],
                                          case["column_scales"], kernel)
            assert np.array_equal(quantized, port.quantize_rows_per_row(case["a"], case["multipliers"], float(case["zero_point"]))), name
            assert np.array_equal(got, case["c"]), name
        seen += 1
    assert seen >= 4


def test_per_row_scales_on_the_tensor_core_kernels(port, cta_form):
    from oracle.checker import pack_compensation
    rng = np.random.default_rng(61)
    m, n, k = 300, 520, 256
    a = rng.uniform(-3, 3, (m, k)).astype(np.float32)
    multipliers = rng.uniform(10, 40, m).astype(np.float32)
    b = rng.integers(-128, 128, (n, k), dtype=np.int8)
    correction = pack_compensation(b, 100)
    rows, cols = (1.0 / multipliers).astype(np.float32), rng.uniform(0.01, 0.05, n).astype(np.float32)
    quantized = port.quantize_rows_per_row(a, multipliers, 100.0)
    for out_dtype in (torch.float32, torch.bfloat16):
        got_q, got = _per_row_gpu(a, multipliers, 100, b, correction, rows, cols, K.KERNEL_I8_TCGEN05, out_dtype)
        assert np.array_equal(got_q, quantized)
        want = port.matmul_i8_dequant_rows(quantized, b, correction, rows, cols, out_bf16=out_dtype == torch.bfloat16)
        assert np.array_equal(got, want), out_dtype
    # float rows take the row factor too: bf16 product, and the weight-only kernels (which compute the product transposed)
    ab, bb, _ = inputs("bf16", m, n, k, rng)
    row = rng.uniform(0.5, 2.0, m).astype(np.float32)
    c = torch.empty((m, n), dtype=torch.float32, device="cuda")
    vecops_b200.matmul(to_device(ab, bf16=True), to_device(bb, bf16=True), c, to_device(cols), kernel=K.KERNEL_BF16_TCGEN05, row_scale=to_device(row))
    torch.cuda.synchronize()
    want = port.matmul_bf16(ab, bb, None, False) * row[:, None] * cols[None, :]
    assert rel_frobenius(c.cpu().numpy(), want) <= TOL_BF16
    for mw, kernel in ((16, K.KERNEL_AUTO), (8, K.KERNEL_W8_SMALL_M), (96, K.KERNEL_W8_TCGEN05)):
        aw, w, s = inputs("w8", mw, 512, 1024, rng)
        roww = rng.uniform(0.5, 2.0, mw).astype(np.float32)
        cw = torch.empty((mw, 512), dtype=torch.float32, device="cuda")
        vecops_b200.matmul(to_device(aw, bf16=True), to_device(w), cw, to_device(s), kernel=kernel, row_scale=to_device(roww))
        torch.cuda.synchronize()
        wantw = port.matmul_w8(aw, w, s, False) * roww[:, None]
        assert rel_frobenius(cw.cpu().numpy(), wantw) <= TOL_BF16, mw
    # the plain int32 row refuses a row factor
    with pytest.raises(capi.VecopsB200Error):
        vecops_b200.matmul(to_device(quantized), to_device(b), torch.empty((m, n), dtype=torch.int32, device="cuda"), row_scale=to_device(rows))


# ------------------------------------------------------------------ the Torch operators (dispatcher -> C++ -> operator bridge)

def test_torch_ops_reach_the_kernels(port):
    from oracle.checker import ACT_SILU
    from vecops_b200 import torch_ops
    torch_ops.load()
    ops = torch.ops.vecops_b200
    lib = capi.library()
    rng = np.random.default_rng(88)
    m, n, k = 256, 512, 256
    a, b, _ = inputs("bf16", m, n, k, rng)
    da, db = to_device(a, bf16=True), to_device(b, bf16=True)
    before = lib.vecops_b200_launch_count()
    c = ops.matmul(da, db)
    torch.cuda.synchronize()
    assert lib.vecops_b200_launch_count() == before + 1 and c.dtype == torch.bfloat16
    check("bf16", bf16_result_to_numpy(c), port.matmul_bf16(a, b))
    # fused form with a bias row, f32 out, under a side stream
    bias = rng.uniform(-1, 1, n).astype(np.float32)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        c32 = ops.matmul(da, db, None, to_device(bias), 0.5, capi.ACTIVATION_SILU, 0.0, 0.0, torch.float32)
    side.synchronize()
    check("bf16", c32.cpu().numpy(), port.matmul_bf16_fused(a, b, bias, 0.5, None, ACT_SILU, out_bf16=False))
    # int8 -> int32, into a caller's tensor; weight-only int8 with its scratch from torch's allocator
    ai, bi, _ = inputs("i8", m, n, k, rng)
    ci = torch.empty((m, n), dtype=torch.int32, device="cuda")
    ops.matmul_out(to_device(ai), to_device(bi), ci)
    aw, w, s = inputs("w8", 64, 512, 1024, rng)
    cw = ops.matmul(to_device(aw, bf16=True), to_device(w), to_device(s))
    torch.cuda.synchronize()
    assert np.array_equal(ci.cpu().numpy(), port.matmul_i8(ai, bi))
    check("w8", bf16_result_to_numpy(cw), port.matmul_w8(aw, w, s))
    # per-token quantised product through the operator layer: u8 x s8, correction row, row and column factors -> f32, bit-exact
    from oracle.checker import pack_compensation
    aq = rng.integers(0, 256, (m, k)).astype(np.uint8)
    bq = rng.integers(-128, 128, (n, k), dtype=np.int8)
    correction = pack_compensation(bq, 9)
    row_factors, column_factors = rng.uniform(0.01, 0.1, m).astype(np.float32), rng.uniform(0.01, 0.05, n).astype(np.float32)
    cq = ops.matmul(to_device(aq), to_device(bq), to_device(column_factors), to_device(correction), 1.0, 0, 0.0, 0.0, torch.float32,
                    to_device(row_factors))
    torch.cuda.synchronize()
    assert np.array_equal(cq.cpu().numpy(), port.matmul_i8_dequant_rows(aq, bq, correction, row_factors, column_factors))
    # attention over heads
    heads, length, d = 2, 192, 64
    q, kk, v = (f32_to_bf16_bits(rng.standard_normal((heads, length, d)).astype(np.float32)) for _ in range(3))
    out = ops.sdpa(to_device(q, bf16=True), to_device(kk, bf16=True), to_device(v, bf16=True), 0.125, capi.CAUSAL_BOTTOM_RIGHT, None, None, torch.float32)
    torch.cuda.synchronize()
    for h in range(heads):  # six tiles on 148 SMs: the automatic cut is one tile per work item, and the restatement gets the same
        assert rel_frobenius(out[h].cpu().numpy(), port.sdpa_bf16_streaming(q[h], kk[h], v[h], 0.125, causal=2, chunk_blocks=_stream_cut(length, length, 2, 1))) <= TOL_BF16
    # a captured CUDA graph replays the operator
    static_c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ops.matmul_out(da, db, static_c)  # warm-up outside the capture (first-use set-up)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.matmul_out(da, db, static_c)
    static_c.zero_()
    graph.replay()
    torch.cuda.synchronize()
    check("bf16", bf16_result_to_numpy(static_c), port.matmul_bf16(a, b))
    with pytest.raises(RuntimeError):
        ops.matmul(torch.zeros(4, 4), torch.zeros(4, 4))  # no CPU implementation


def test_numpy_face(port):
    from vecops_b200 import numpy_ops
    rng = np.random.default_rng(5)
    a, b, _ = inputs("bf16", 200, 328, 200, rng)
    check("bf16", numpy_ops.matmul(a, b, bf16=True), port.matmul_bf16(a, b))
    check("bf16", numpy_ops.matmul(a, b, bf16=True, out_dtype=np.float32), port.matmul_bf16(a, b, None, False))
    af, bf, _ = inputs("f32", 96, 80, 64, rng)
    check("f32", numpy_ops.matmul(af, bf), port.matmul_f32(af, bf))
    ai, bi, _ = inputs("i8", 64, 48, 100, rng, np.uint8, np.int8)
    assert np.array_equal(numpy_ops.matmul(ai, bi), port.matmul_i8(ai, bi))
    aw, w, s = inputs("w8", 4, 256, 512, rng)
    check("w8", numpy_ops.matmul(aw, w, s, bf16=True), port.matmul_w8(aw, w, s))
