"""The benchmark configurations at their full sizes.

The CPU checker cannot finish a 4096^3 product in seconds, so full-size parity
uses (a) the checker on sampled output rows and (b) size-independent checksum
identities over ALL outputs, computed from the inputs in float64 / int64:

    sum_n C[m,n] = A[m,:] . (sum_n B[n,:])        (row checksum)
    sum_m C[m,n] = (sum_m A[m,:]) . B[n,:]        (column checksum)

For int8 both identities are exact integers (no wrap at these sizes), so every
int32 output is covered bit-exactly in aggregate.  For the floating-point
configurations the checksums are taken on a second run of the same kernel
with an fp32 store: rounding each output to bf16 (2^-9 relative, random sign)
does not average out against a random-sign checksum, so a checksum of bf16
outputs could not hold the 1e-3 bound even for a perfect kernel.
"""
import numpy as np
import pytest
import torch

import vecops_b200
from oracle.checker import bf16_bits_to_f32, rel_frobenius
from tests.helpers import TOL_BF16, TOL_F32, bf16_result_to_numpy, to_device
from vecops_b200 import capi, workloads

pytestmark = pytest.mark.gpu


def sample_rows(m, count=24):
    return np.unique(np.linspace(0, m - 1, count).astype(np.int64))


def test_c1_fp32_1024(port):
    w = workloads.WORKLOADS["c1_f32_1024"]
    a, b_nk = workloads.make_a(w), workloads.make_b_nk(w)
    b_kn = to_device(np.ascontiguousarray(b_nk.T))            # stored [K,N] row-major, as the configuration says
    c = torch.empty((w.m, w.n), dtype=torch.float32, device="cuda")
    vecops_b200.matmul(to_device(a), b_kn.t(), c)
    assert rel_frobenius(c.cpu().numpy(), port.matmul_f32(a, b_nk)) <= TOL_F32


def test_c2_bf16_4096(port):
    w = workloads.WORKLOADS["c2_bf16_4096"]
    a, b = workloads.make_a(w), workloads.make_b_nk(w)
    c = torch.empty((w.m, w.n), dtype=torch.bfloat16, device="cuda")
    vecops_b200.matmul(to_device(a, True), to_device(b, True), c)
    got = bf16_bits_to_f32(bf16_result_to_numpy(c))
    rows = sample_rows(w.m)
    assert rel_frobenius(got[rows], bf16_bits_to_f32(port.matmul_bf16(a[rows], b))) <= TOL_BF16
    c32 = torch.empty((w.m, w.n), dtype=torch.float32, device="cuda")
    vecops_b200.matmul(to_device(a, True), to_device(b, True), c32)
    af, bfl = bf16_bits_to_f32(a).astype(np.float64), bf16_bits_to_f32(b).astype(np.float64)
    assert rel_frobenius(c32.sum(dim=1, dtype=torch.float64).cpu().numpy(), af @ bfl.sum(axis=0)) <= TOL_BF16
    assert rel_frobenius(c32.sum(dim=0, dtype=torch.float64).cpu().numpy(), bfl @ af.sum(axis=0)) <= TOL_BF16


def test_c3_int8_4096x14336x4096(port):
    w = workloads.WORKLOADS["c3_i8_4096x14336x4096"]
    a, b = workloads.make_a(w), workloads.make_b_nk(w)
    c = torch.empty((w.m, w.n), dtype=torch.int32, device="cuda")
    vecops_b200.matmul(to_device(a), to_device(b), c)
    rows = sample_rows(w.m, 16)
    assert np.array_equal(c[torch.from_numpy(rows).cuda()].cpu().numpy(), port.matmul_i8(a[rows], b))
    a64, b64 = a.astype(np.int64), b.astype(np.int64)
    assert np.array_equal(c.sum(dim=1, dtype=torch.int64).cpu().numpy(), a64 @ b64.sum(axis=0))
    assert np.array_equal(c.sum(dim=0, dtype=torch.int64).cpu().numpy(), b64 @ a64.sum(axis=0))


@pytest.mark.parametrize("name", ["c4_w8_m1", "c4_w8_m16", "c4_w8_m128"])
def test_c4_weight_only_int8(port, name):
    w = workloads.WORKLOADS[name]
    a, wt, s = workloads.make_a(w), workloads.make_b_nk(w), workloads.make_scale(w)
    c = torch.empty((w.m, w.n), dtype=torch.bfloat16, device="cuda")
    vecops_b200.matmul(to_device(a, True), to_device(wt), c, to_device(s))
    got = bf16_bits_to_f32(bf16_result_to_numpy(c))
    rows = sample_rows(w.m, 16)
    assert rel_frobenius(got[rows], bf16_bits_to_f32(port.matmul_w8(a[rows], wt, s))) <= TOL_BF16
    # row checksum over all N columns (fp32 store), scale folded into the weights
    c32 = torch.empty((w.m, w.n), dtype=torch.float32, device="cuda")
    vecops_b200.matmul(to_device(a, True), to_device(wt), c32, to_device(s))
    af = bf16_bits_to_f32(a).astype(np.float64)
    weighted = (wt.astype(np.float64) * s.astype(np.float64)[:, None]).sum(axis=0)
    assert rel_frobenius(c32.sum(dim=1, dtype=torch.float64).cpu().numpy(), af @ weighted) <= TOL_BF16


def test_c5_one_rank_slab_of_the_sharded_gemm(port):
    # what one of 8 GPUs computes: all of A against its 6656 rows of B
    from vecops_b200 import sharding
    w = workloads.WORKLOADS["c5_bf16_16384x53248x8192"]
    n0, n1 = sharding.column_partition(w.n, 8, 5)
    assert n1 - n0 == 6656
    a, b = workloads.make_a(w), workloads.make_b_nk(w, n0, n1)
    c = torch.empty((w.m, n1 - n0), dtype=torch.bfloat16, device="cuda")
    vecops_b200.matmul(to_device(a, True), to_device(b, True), c)
    rows = sample_rows(w.m, 12)
    got = bf16_bits_to_f32(bf16_result_to_numpy(c[torch.from_numpy(rows).cuda()]))
    assert rel_frobenius(got, bf16_bits_to_f32(port.matmul_bf16(a[rows], b))) <= TOL_BF16
    del c
    c32 = torch.empty((w.m, n1 - n0), dtype=torch.float32, device="cuda")
    vecops_b200.matmul(to_device(a, True), to_device(b, True), c32)
    af, bfl = bf16_bits_to_f32(a).astype(np.float64), bf16_bits_to_f32(b).astype(np.float64)
    assert rel_frobenius(c32.sum(dim=0, dtype=torch.float64).cpu().numpy(), bfl @ af.sum(axis=0)) <= TOL_BF16
