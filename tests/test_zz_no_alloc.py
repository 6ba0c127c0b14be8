"""The entry point for callers that must not allocate: vecops_b200_matmul_w8_static_scratch.

Some users of this library run where device allocation at call time is off the table - a decode loop over a
memory pool that was sealed at start-up, an embedding whose allocator must not be re-entered from inside an
operator, a latency budget with no room for an allocation's implicit synchronisation.  For them the weight-only
int8 tensor-core kernel keeps its scratch (stream-K partial sums, flags, the fp16 activations) in a fixed 8 MiB
array inside the library.  This test drives that entry point through the C ABI and checks it against the ordinary
entry point (caller-provided workspace), twice in a row, because the array is shared by all calls and keeps what
the previous call left in it.

The file name sorts last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes
from ctypes import byref

import numpy as np
import pytest
import torch

import vecops_b200
from oracle.checker import bf16_bits_to_f32, f32_to_bf16_bits, rel_frobenius
from tests.helpers import TOL_BF16, bf16_result_to_numpy, to_device
from vecops_b200 import capi, harness

pytestmark = pytest.mark.gpu


def static_scratch_entry():
    lib = capi.library()
    lib.vecops_b200_matmul_w8_static_scratch.argtypes = [ctypes.POINTER(capi.VecopsB200Matmul), ctypes.POINTER(capi.VecopsError)]
    lib.vecops_b200_matmul_w8_static_scratch.restype = ctypes.c_int32
    return lib.vecops_b200_matmul_w8_static_scratch


def test_static_scratch_matches_the_workspace_entry_point_twice_in_a_row(port):
    entry = static_scratch_entry()
    rng = np.random.default_rng(2024)
    # two different problems back to back: the second call finds the first one's leftovers in the shared array
    for m, n, k in [(48, 1024, 2048), (33, 1408, 1024)]:
        a = f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
        w = rng.integers(-127, 128, (n, k), dtype=np.int8)
        s = rng.uniform(0.001, 0.02, n).astype(np.float32)
        da, dw, ds = to_device(a, True), to_device(w), to_device(s)

        reference = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        vecops_b200.matmul(da, dw, reference, ds, kernel=capi.KERNEL_W8_TCGEN05)  # existing entry point, caller workspace
        want = bf16_bits_to_f32(bf16_result_to_numpy(reference))

        for repeat in range(2):
            got = torch.full((m, n), -5.0, dtype=torch.bfloat16, device="cuda")
            problem = vecops_b200.matmul_problem(da, dw, got, ds, stream=torch.cuda.current_stream())
            assert problem.workspace is None and problem.workspace_size == 0  # nothing is handed in
            error = capi.ErrorBuffer()
            error.raise_for(entry(byref(problem), byref(error.record)))
            torch.cuda.synchronize()
            result = bf16_bits_to_f32(bf16_result_to_numpy(got))
            assert rel_frobenius(result, want) <= TOL_BF16, f"m={m} n={n} k={k} repeat={repeat}"
        # and both agree with the CPU checker
        assert rel_frobenius(want, bf16_bits_to_f32(port.matmul_w8(a, w, s))) <= TOL_BF16


def test_static_scratch_refuses_what_does_not_fit():
    entry = static_scratch_entry()
    a = torch.zeros((128, 4096), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((256, 4096), dtype=torch.int8, device="cuda")
    c = torch.zeros((128, 256), dtype=torch.bfloat16, device="cuda")
    problem = vecops_b200.matmul_problem(a, w, c)
    error = capi.ErrorBuffer()
    assert entry(byref(problem), byref(error.record)) == capi.INVALID_ARGUMENT
    assert b"built-in array" in error.text.value
    # and a dtype row it does not serve
    b16 = torch.zeros((256, 4096), dtype=torch.bfloat16, device="cuda")
    problem = vecops_b200.matmul_problem(a, b16, c)
    assert entry(byref(problem), byref(error.record)) == capi.INVALID_ARGUMENT


def test_static_scratch_allocates_nothing_and_serves_its_other_forms(port):
    """What the entry point promises beyond the numbers: no device memory is taken by a call once the one-time set-up is
    behind it, the fp32-output and the synchronous forms work, and inputs it cannot serve come back with a message."""
    entry = static_scratch_entry()
    rng = np.random.default_rng(7)
    m, n, k = 24, 640, 1024
    a = f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
    w = rng.integers(-127, 128, (n, k), dtype=np.int8)
    s = rng.uniform(0.001, 0.02, n).astype(np.float32)
    da, dw, ds = to_device(a, True), to_device(w), to_device(s)
    want = port.matmul_w8(a, w, s, False)
    got = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    error = capi.ErrorBuffer()

    # synchronous call (flags = 0), fp32 output; also the call that performs the set-up if nothing did before
    problem = vecops_b200.matmul_problem(da, dw, got, ds, stream=torch.cuda.current_stream())
    assert problem.flags == 0
    error.raise_for(entry(byref(problem), byref(error.record)))
    assert rel_frobenius(got.cpu().numpy(), want) <= TOL_BF16

    # a second call takes no device memory: free memory as the driver reports it is unchanged
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    got.zero_()
    torch.cuda.synchronize()
    error.raise_for(entry(byref(problem), byref(error.record)))
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "a call after the set-up must not allocate device memory"
    assert rel_frobenius(got.cpu().numpy(), want) <= TOL_BF16

    # K not a multiple of 8: not this kernel's problem, said so in words
    odd = vecops_b200.matmul_problem(da[:, :1020], dw[:, :1020], got, ds)
    assert entry(byref(odd), byref(error.record)) == capi.NOT_APPLICABLE
    assert len(error.text.value) > 0
