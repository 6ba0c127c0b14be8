"""Captured launches of the kernels whose CTAs exchange partial sums through device scratch, replayed with new inputs.

A captured CUDA graph freezes every kernel argument, the 64-bit nonce of the scratch flags included, and the scratch
keeps what the previous replay left in it.  A flag that stayed "published" after a replay would let the next replay
add partial sums before they are written - stale ones whenever the inputs changed in between, which no test that
replays once, or replays unchanged inputs, can see.  Each case below captures ONE launch over static buffers, then
replays it several times, writing different operands into the buffers before every replay, and holds every replay to
the CPU checker.
"""
import ctypes
from ctypes import byref

import numpy as np
import pytest
import torch

import vecops_b200
from oracle.checker import bf16_bits_to_f32, f32_to_bf16_bits, rel_frobenius
from tests.helpers import TOL_BF16, bf16_result_to_numpy
from vecops_b200 import capi, harness

pytestmark = pytest.mark.gpu

REPLAYS = 4


def _capture(launch):
    """Warm the launch up once on a side stream (one-time set-up must not fall inside a capture), then capture it."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launch(side)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            launch(side)
    torch.cuda.current_stream().wait_stream(side)
    return graph


def _status() -> int:
    word = ctypes.c_uint32(0)
    error = capi.ErrorBuffer()
    capi.library().vecops_b200_take_device_status(0, byref(word), byref(error.record))
    return word.value


@pytest.mark.parametrize("m,n,k,out_dtype", [
    (128, 256, 4096, torch.bfloat16),    # one tile cut along K over four CTAs: every slice meets in the first round
    (256, 512, 2048, torch.float32),     # four tiles, eight slices each
    (2048, 4864, 1024, torch.bfloat16),  # pairs: 152 tiles on 74 pairs, the 4 tail tiles cut four ways
])
def test_replayed_split_k_bf16_gemm_follows_its_inputs(port, m, n, k, out_dtype):
    rng = np.random.default_rng(m + n + k)
    a = torch.zeros((m, k), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((n, k), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((m, n), dtype=out_dtype, device="cuda")
    scratch_holder = {}

    def launch(stream):
        problem = harness.matmul_problem(a, b, c, kernel=capi.KERNEL_BF16_TCGEN05, stream=stream, asynchronous=True)
        if "scratch" not in scratch_holder:
            scratch_holder["scratch"] = harness.attach_workspace(problem, a.device)
            assert scratch_holder["scratch"] is not None, "this shape is expected to be cut along K"
        ws = scratch_holder["scratch"]
        problem.workspace, problem.workspace_size = ws.data_ptr(), ws.numel()
        harness.run(problem)

    graph = _capture(launch)
    rows = np.unique(np.linspace(0, m - 1, 12).astype(np.int64))
    for replay in range(REPLAYS):
        host_a = f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
        host_b = f32_to_bf16_bits(rng.standard_normal((n, k), dtype=np.float32))
        a.copy_(torch.from_numpy(host_a).cuda().view(torch.bfloat16))
        b.copy_(torch.from_numpy(host_b).cuda().view(torch.bfloat16))
        c.fill_(-7)
        graph.replay()
        torch.cuda.synchronize()
        assert _status() == 0
        out_bf16 = out_dtype == torch.bfloat16
        want = port.matmul_bf16(host_a[rows], host_b, None, out_bf16)
        got = c[torch.from_numpy(rows).cuda()]
        got = bf16_bits_to_f32(bf16_result_to_numpy(got)) if out_bf16 else got.cpu().numpy()
        want = bf16_bits_to_f32(want) if out_bf16 else want
        assert rel_frobenius(got, want) <= TOL_BF16, f"replay {replay}"


def _w8_inputs(rng, m, n, k):
    return (f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32)), rng.integers(-127, 128, (n, k), dtype=np.int8),
            rng.uniform(0.001, 0.02, n).astype(np.float32))


@pytest.mark.parametrize("form", ["workspace", "static_scratch"])
@pytest.mark.parametrize("m,n,k", [(48, 1024, 2048),    # 128 units on 128 CTAs: one unit each, fifteen contributors per tile
                                   (80, 2048, 1024)])   # the most activation rows the built-in scratch array holds at this K
def test_replayed_w8_tcgen05_follows_its_inputs(port, form, m, n, k):
    rng = np.random.default_rng(17 * m + n + k)
    a = torch.zeros((m, k), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((n, k), dtype=torch.int8, device="cuda")
    s = torch.zeros(n, dtype=torch.float32, device="cuda")
    c = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    lib = capi.library()
    lib.vecops_b200_matmul_w8_static_scratch.argtypes = [ctypes.POINTER(capi.VecopsB200Matmul), ctypes.POINTER(capi.VecopsError)]
    lib.vecops_b200_matmul_w8_static_scratch.restype = ctypes.c_int32
    holder = {}

    def launch(stream):
        problem = harness.matmul_problem(a, w, c, s, kernel=capi.KERNEL_W8_TCGEN05, stream=stream, asynchronous=True)
        error = capi.ErrorBuffer()
        if form == "workspace":
            if "scratch" not in holder:
                holder["scratch"] = harness.attach_workspace(problem, a.device)
            ws = holder["scratch"]
            problem.workspace, problem.workspace_size = ws.data_ptr(), ws.numel()
            error.raise_for(lib.vecops_b200_matmul_run(byref(problem), byref(error.record)))
        else:
            problem.kernel = capi.KERNEL_AUTO
            error.raise_for(lib.vecops_b200_matmul_w8_static_scratch(byref(problem), byref(error.record)))

    graph = _capture(launch)
    for replay in range(REPLAYS):
        host_a, host_w, host_s = _w8_inputs(rng, m, n, k)
        a.copy_(torch.from_numpy(host_a).cuda().view(torch.bfloat16))
        w.copy_(torch.from_numpy(host_w).cuda())
        s.copy_(torch.from_numpy(host_s).cuda())
        c.fill_(-7)
        graph.replay()
        torch.cuda.synchronize()
        assert _status() == 0
        got = bf16_bits_to_f32(bf16_result_to_numpy(c))
        want = bf16_bits_to_f32(port.matmul_w8(host_a, host_w, host_s))
        assert rel_frobenius(got, want) <= TOL_BF16, f"{form} replay {replay}"


def test_automatic_weight_only_dispatch_runs_without_a_workspace(port):
    """The reference's matmul needs no workspace: a weight-only call with 16 < M <= 128 that brings none is served by a
    kernel that needs none, while the same call with the scratch the query reports takes the tensor-core kernel."""
    rng = np.random.default_rng(64)
    m, n, k = 64, 1024, 1024
    host_a, host_w, host_s = _w8_inputs(rng, m, n, k)
    a = torch.from_numpy(host_a).cuda().view(torch.bfloat16)
    w, s = torch.from_numpy(host_w).cuda(), torch.from_numpy(host_s).cuda()
    want = bf16_bits_to_f32(port.matmul_w8(host_a, host_w, host_s))
    for with_workspace in (False, True):
        c = torch.full((m, n), -3.0, dtype=torch.bfloat16, device="cuda")
        problem = harness.matmul_problem(a, w, c, s, stream=torch.cuda.current_stream())
        scratch = harness.attach_workspace(problem, a.device) if with_workspace else None
        assert with_workspace == (scratch is not None)
        harness.run(problem)
        torch.cuda.synchronize()
        assert rel_frobenius(bf16_bits_to_f32(bf16_result_to_numpy(c)), want) <= TOL_BF16, f"workspace={with_workspace}"
        del scratch


def test_replayed_streaming_attention_follows_its_inputs(port):
    """The streaming attention kernel and the merge of its key chunks (a programmatic dependent) captured once and replayed
    with new operands: the chunk records in scratch are rewritten by every launch and nothing else lives there."""
    rng = np.random.default_rng(11)
    heads, lq, lkv, d = 2, 384, 1024, 64
    q = torch.zeros((heads, lq, d), dtype=torch.bfloat16, device="cuda")
    k = torch.zeros((heads, lkv, d), dtype=torch.bfloat16, device="cuda")
    v = torch.zeros((heads, lkv, d), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((heads, lq, d), dtype=torch.float32, device="cuda")
    holder = {}

    def launch(stream):
        record = harness.sdpa_record(q, k, v, out, 0.125, causal=capi.CAUSAL_BOTTOM_RIGHT, stream=stream, asynchronous=True,
                                     strategy=capi.SDPA_STREAMING)
        if "scratch" not in holder:
            need = ctypes.c_uint64(0)
            error = capi.ErrorBuffer()
            error.raise_for(capi.library().vecops_b200_sdpa_workspace(byref(record), byref(need), byref(error.record)))
            assert need.value > 0, "this shape is expected to be cut into key chunks"
            holder["scratch"] = torch.empty(need.value + 256, dtype=torch.uint8, device="cuda")
            holder["need"] = need.value
            holder["tiles"] = harness.sdpa_plan(record)[1]
        scratch = holder["scratch"]
        record.workspace, record.workspace_size = scratch.data_ptr() + (-scratch.data_ptr()) % 256, holder["need"]
        error = capi.ErrorBuffer()
        error.raise_for(capi.library().vecops_b200_sdpa_run(byref(record), byref(error.record)))

    graph = _capture(launch)
    rows = np.unique(np.linspace(0, lq - 1, 10).astype(np.int64))
    last = np.arange(lq)[:, None] + (lkv - lq)
    keep = (np.arange(lkv)[None, :] <= last).astype(np.uint8)
    for replay in range(REPLAYS):
        host = [f32_to_bf16_bits(rng.standard_normal(t.shape).astype(np.float32)) for t in (q, k, v)]
        for tensor, values in zip((q, k, v), host):
            tensor.copy_(torch.from_numpy(values).cuda().view(torch.bfloat16))
        out.fill_(-7)
        graph.replay()
        torch.cuda.synchronize()
        assert _status() == 0
        for head in range(heads):
            want = port.sdpa_bf16_streaming(host[0][head][rows], host[1][head], host[2][head], 0.125, keep_mask=keep[rows], chunk_blocks=holder["tiles"])
            assert rel_frobenius(out[head].cpu().numpy()[rows], want) <= TOL_BF16, f"replay {replay} head {head}"
