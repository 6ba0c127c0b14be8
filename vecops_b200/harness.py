"""Test/benchmark harness over the C ABI: torch tensors in, ``vecops_b200_matmul_run`` underneath.

torch is used for device memory and streams only; all arithmetic happens in the
library's own kernels.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_int64, c_uint32, c_uint64

from . import capi


def torch_dtype_code(dtype) -> int:
    import torch
    table = {torch.float32: capi.DTYPE_F32, torch.bfloat16: capi.DTYPE_BF16, torch.int8: capi.DTYPE_I8,
             torch.uint8: capi.DTYPE_U8, torch.int32: capi.DTYPE_I32, torch.float16: capi.DTYPE_F16}
    if dtype not in table:
        raise ValueError(f"dtype {dtype} has no vecops code on this path")
    return table[dtype]


def matmul_problem(a, b_nk, c, scale=None, kernel: int = capi.KERNEL_AUTO, stream=None, asynchronous: bool = False,
                   workspace=None) -> capi.VecopsB200Matmul:
    """Describe C[M,N] = A[M,K] . B[N,K]^T over 2-D torch tensors (any strides)."""
    if a.dim() != 2 or b_nk.dim() != 2 or c.dim() != 2:
        raise ValueError("a, b and c must be 2-D")
    m, k = a.shape
    n, kb = b_nk.shape
    if kb != k or tuple(c.shape) != (m, n):
        raise ValueError(f"shape mismatch: a{tuple(a.shape)} b{tuple(b_nk.shape)} c{tuple(c.shape)}")
    p = capi.VecopsB200Matmul()
    p.struct_size = ctypes.sizeof(capi.VecopsB200Matmul)
    p.kernel = kernel
    p.m, p.n, p.k = m, n, k
    p.a, p.a_stride_m, p.a_stride_k = a.data_ptr(), a.stride(0), a.stride(1)
    p.b, p.b_stride_n, p.b_stride_k = b_nk.data_ptr(), b_nk.stride(0), b_nk.stride(1)
    p.c, p.c_stride_m, p.c_stride_n = c.data_ptr(), c.stride(0), c.stride(1)
    p.column_scale = scale.data_ptr() if scale is not None else None
    if workspace is not None:
        p.workspace, p.workspace_size = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    p.stream = stream.cuda_stream if stream is not None else None
    p.a_dtype, p.b_dtype, p.c_dtype = torch_dtype_code(a.dtype), torch_dtype_code(b_nk.dtype), torch_dtype_code(c.dtype)
    p.device_index = a.device.index if a.is_cuda and a.device.index is not None else -1
    p.flags = capi.MATMUL_FLAG_ASYNC if asynchronous else 0
    return p


def select_kernel(problem: capi.VecopsB200Matmul) -> int:
    error = capi.ErrorBuffer()
    out = c_uint32(0)
    error.raise_for(capi.library().vecops_b200_matmul_select(byref(problem), byref(out), byref(error.record)))
    return out.value


def workspace_bytes(problem: capi.VecopsB200Matmul) -> int:
    error = capi.ErrorBuffer()
    out = c_uint64(0)
    error.raise_for(capi.library().vecops_b200_matmul_workspace(byref(problem), byref(out), byref(error.record)))
    return out.value


def attach_workspace(problem: capi.VecopsB200Matmul, device):
    """Allocate the device scratch the chosen kernel asks for (torch owns the memory) and point the problem at it.

    Returns the buffer (keep it alive until the launch has finished) or None when no scratch is needed."""
    import torch
    need = workspace_bytes(problem)
    if need == 0:
        return None
    buffer = torch.empty(need, dtype=torch.uint8, device=device)
    problem.workspace, problem.workspace_size = buffer.data_ptr(), need
    return buffer


def epilogue_record(cin=None, alpha: float = 1.0, activation: int = capi.ACTIVATION_NONE, clamp_lo: float = 0.0,
                    clamp_hi: float = 0.0, rows: int | None = None, cols: int | None = None, row_scale=None) -> capi.VecopsB200Epilogue:
    """The fused output transform: COut = activation((CIn + A.B^T) * alpha * row_scale[m] * column_scale[n]).

    `cin` is a torch tensor broadcastable to [rows, cols] (a bias row [cols], a column [rows, 1], or the full matrix);
    `row_scale` a contiguous float32 tensor with one factor per output row."""
    e = capi.VecopsB200Epilogue()
    e.struct_size = ctypes.sizeof(capi.VecopsB200Epilogue)
    e.activation, e.alpha, e.clamp_lo, e.clamp_hi = activation, alpha, clamp_lo, clamp_hi
    if cin is not None:
        view = cin.expand(rows, cols) if tuple(cin.shape) != (rows, cols) else cin
        e.cin, e.cin_stride_m, e.cin_stride_n = view.data_ptr(), view.stride(0), view.stride(1)
        e.cin_dtype = torch_dtype_code(view.dtype)
    if row_scale is not None:
        e.row_scale = row_scale.data_ptr()
    return e


def run(problem: capi.VecopsB200Matmul, epilogue: capi.VecopsB200Epilogue | None = None) -> None:
    error = capi.ErrorBuffer()
    if epilogue is None:
        error.raise_for(capi.library().vecops_b200_matmul_run(byref(problem), byref(error.record)))
    else:
        error.raise_for(capi.library().vecops_b200_matmul_run_fused(byref(problem), byref(epilogue), byref(error.record)))


def matmul(a, b_nk, c, scale=None, kernel: int = capi.KERNEL_AUTO, stream=None, asynchronous: bool = False, cin=None,
           alpha: float = 1.0, activation: int = capi.ACTIVATION_NONE, clamp_lo: float = 0.0, clamp_hi: float = 0.0, row_scale=None) -> None:
    """Run C = A . B^T (or its fused form, see epilogue_record) on the GPU through the C ABI; raises VecopsB200Error."""
    import torch
    if stream is None and a.is_cuda:
        stream = torch.cuda.current_stream(a.device)
    problem = matmul_problem(a, b_nk, c, scale, kernel, stream, asynchronous)
    fused = cin is not None or alpha != 1.0 or activation != capi.ACTIVATION_NONE or row_scale is not None
    epilogue = epilogue_record(cin, alpha, activation, clamp_lo, clamp_hi, c.shape[0], c.shape[1], row_scale) if fused else None
    # freed after the call: torch's allocator re-issues the block only to later work on the same stream
    scratch = attach_workspace(problem, a.device) if a.is_cuda else None
    run(problem, epilogue)
    del scratch


def matmul_batched(a3, b3, c3, scale=None, kernel: int = capi.KERNEL_AUTO, stream=None, cin=None, alpha: float = 1.0,
                   activation: int = capi.ACTIVATION_NONE, clamp_lo: float = 0.0, clamp_hi: float = 0.0) -> None:
    """Rank-3 operands a3 [B,M,K], b3 [B,N,K], c3 [B,M,N] (expanded views share an operand across the batch: stride 0).

    `cin`: a bias row [N], or a tensor broadcastable to [B,M,N]."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream(c3.device)
    count, m, n = c3.shape
    problem = matmul_problem(a3[0], b3[0], c3[0], scale, kernel, stream, False)
    batch = capi.VecopsB200Batch(ctypes.sizeof(capi.VecopsB200Batch), 0, count, a3.stride(0), b3.stride(0), c3.stride(0), 0)
    fused = cin is not None or alpha != 1.0 or activation != capi.ACTIVATION_NONE
    epilogue = None
    if fused:
        view = None
        if cin is not None:
            view = cin.expand(count, m, n)
            batch.cin_stride_b = view.stride(0)
            view = view[0]
        epilogue = epilogue_record(view, alpha, activation, clamp_lo, clamp_hi, m, n)
    # scratch for either way the library may run it: stacked into one product, or entry by entry
    stacked = matmul_problem(a3[0], b3[0], c3[0], scale, kernel, stream, False)
    stacked.m = m * count
    need = max(workspace_bytes(problem), workspace_bytes(stacked))
    scratch = torch.empty(need, dtype=torch.uint8, device=c3.device) if need else None
    if scratch is not None:
        problem.workspace, problem.workspace_size = scratch.data_ptr(), need
    error = capi.ErrorBuffer()
    error.raise_for(capi.library().vecops_b200_matmul_run_batched(byref(problem), byref(batch), byref(epilogue) if epilogue is not None else None,
                                                                 byref(error.record)))
    del scratch


def quantize_rows(src, dst, scale, zero_point: float, stream=None) -> None:
    """dst[m,k] = convert(src[m,k] * scale + zero_point): src f32 or bf16 [M,K], dst u8 or i8 with K-contiguous rows.
    `scale`: a number, or a contiguous float32 tensor of one multiplier per row (per-token quantisation)."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream(src.device)
    error = capi.ErrorBuffer()
    if isinstance(scale, torch.Tensor):
        error.raise_for(capi.library().vecops_b200_quantize_rows_per_row(src.data_ptr(), torch_dtype_code(src.dtype), src.stride(0), src.stride(1),
                                                                        dst.data_ptr(), torch_dtype_code(dst.dtype), dst.stride(0), src.shape[0],
                                                                        src.shape[1], scale.data_ptr(), zero_point, stream.cuda_stream,
                                                                        byref(error.record)))
        return
    error.raise_for(capi.library().vecops_b200_quantize_rows(src.data_ptr(), torch_dtype_code(src.dtype), src.stride(0), src.stride(1),
                                                            dst.data_ptr(), torch_dtype_code(dst.dtype), dst.stride(0), src.shape[0],
                                                            src.shape[1], scale, zero_point, stream.cuda_stream, byref(error.record)))


def packed_layout(dtype, rows: int, k: int) -> tuple[int, int]:
    """(pitch in elements, bytes) of the packed form of a [rows, K] operand of torch dtype `dtype`."""
    pitch, size = c_int64(0), c_uint64(0)
    error = capi.ErrorBuffer()
    error.raise_for(capi.library().vecops_b200_matmul_packed_layout(torch_dtype_code(dtype), rows, k, byref(pitch), byref(size),
                                                                    byref(error.record)))
    return pitch.value, size.value


def pack_operand(view, dtype=None, operand: int = 1, zero_point: int | None = None, stream=None):
    """Prepare one matmul operand: any strided [rows, K] view (a `.t()` of a [K, N]-stored weight included) -> its packed form,
    K-contiguous rows on a 128-byte pitch, optionally narrowed from fp32 to `dtype` (bf16 / fp16).

    Returns the packed operand as a [rows, K] tensor view (row stride = pitch) to hand to `matmul` in place of `view`;
    with `zero_point` (signed 8-bit B only) returns (packed, compensation) where compensation[n] = -zero_point * sum_k B[n,k]."""
    import torch
    if view.dim() != 2:
        raise ValueError("operand must be 2-D")
    dtype = dtype or view.dtype
    rows, k = view.shape
    pitch, size = packed_layout(dtype, rows, k)
    storage = torch.empty((rows, pitch), dtype=dtype, device=view.device)
    if stream is None:
        stream = torch.cuda.current_stream(view.device)
    record = capi.VecopsB200Pack(ctypes.sizeof(capi.VecopsB200Pack), operand, rows, k, view.data_ptr(), view.stride(0), view.stride(1),
                                 torch_dtype_code(view.dtype), torch_dtype_code(dtype), storage.data_ptr(), size,
                                 view.device.index if view.device.index is not None else -1, 0, stream.cuda_stream)
    error = capi.ErrorBuffer()
    if zero_point is None:
        error.raise_for(capi.library().vecops_b200_matmul_pack(byref(record), byref(error.record)))
        return storage[:, :k]
    compensation = torch.empty(rows, dtype=torch.int32, device=view.device)
    error.raise_for(capi.library().vecops_b200_matmul_pack_b_compensated(byref(record), zero_point, compensation.data_ptr(), byref(error.record)))
    return storage[:, :k], compensation


def sdpa_record(q, k, v, out, scale: float, query_mask=None, key_mask=None, keep_mask=None, bias=None, causal: int = 0, stream=None,
                asynchronous: bool = False, strategy: int = 0) -> capi.VecopsB200Attention:
    """Describe scaled dot-product attention: q [Lq,Dqk], k [Lkv,Dqk], v [Lkv,Dv] bf16, out [Lq,Dv] f32 or bf16; masks
    uint8 / bool tensors (non-zero keeps), bias float32 [Lq,Lkv].  With a leading head axis on q, k, v and out (and
    optionally on the masks and the bias) all heads are served by the call; `.expand`ed views share an operand.
    `strategy`: capi.SDPA_AUTOMATIC (streaming kernel when it can serve the call), SDPA_MATERIALIZED or SDPA_STREAMING."""
    a = capi.VecopsB200Attention()
    a.struct_size = ctypes.sizeof(capi.VecopsB200Attention)
    a.causal = causal
    a.strategy = strategy
    if q.dim() == 3:  # [heads, L, D]; expanded views (head stride 0) share an operand between heads
        a.heads = out.shape[0]
        a.q_stride_head, a.k_stride_head, a.v_stride_head, a.out_stride_head = q.stride(0), k.stride(0), v.stride(0), out.stride(0)
        for name, tensor in (("query_mask", query_mask), ("key_mask", key_mask), ("keep", keep_mask), ("bias", bias)):
            if tensor is not None and tensor.dim() == (3 if name in ("keep", "bias") else 2):
                setattr(a, f"{name}_stride_head", tensor.stride(0))
        q, k, v, out = q[0], k[0], v[0], out[0]
        query_mask = query_mask[0] if query_mask is not None and query_mask.dim() == 2 else query_mask
        key_mask = key_mask[0] if key_mask is not None and key_mask.dim() == 2 else key_mask
        keep_mask = keep_mask[0] if keep_mask is not None and keep_mask.dim() == 3 else keep_mask
        bias = bias[0] if bias is not None and bias.dim() == 3 else bias
    a.lq, a.dqk = q.shape
    a.lkv, a.dv = v.shape
    if tuple(k.shape) != (a.lkv, a.dqk) or tuple(out.shape) != (a.lq, a.dv):
        raise ValueError(f"shape mismatch: q{tuple(q.shape)} k{tuple(k.shape)} v{tuple(v.shape)} out{tuple(out.shape)}")
    a.q, a.q_stride_row, a.q_stride_col = q.data_ptr(), q.stride(0), q.stride(1)
    a.k, a.k_stride_row, a.k_stride_col = k.data_ptr(), k.stride(0), k.stride(1)
    a.v, a.v_stride_row, a.v_stride_col = v.data_ptr(), v.stride(0), v.stride(1)
    a.out, a.out_stride_row, a.out_stride_col = out.data_ptr(), out.stride(0), out.stride(1)
    a.qkv_dtype, a.out_dtype = torch_dtype_code(q.dtype), torch_dtype_code(out.dtype)
    if query_mask is not None:
        a.query_mask = query_mask.data_ptr()
    if key_mask is not None:
        a.key_mask = key_mask.data_ptr()
    if keep_mask is not None:
        a.keep_mask, a.keep_stride_row, a.keep_stride_col = keep_mask.data_ptr(), keep_mask.stride(0), keep_mask.stride(1)
    if bias is not None:
        a.bias, a.bias_stride_row, a.bias_stride_col = bias.data_ptr(), bias.stride(0), bias.stride(1)
    a.scale = scale
    a.flags = capi.MATMUL_FLAG_ASYNC if asynchronous else 0
    a.stream = stream.cuda_stream if stream is not None else None
    a.device_index = out.device.index if out.is_cuda and out.device.index is not None else -1
    return a


def sdpa_plan(record: capi.VecopsB200Attention) -> tuple[int, int]:
    """(strategy, 128-key tiles per work item) the library takes for the record; pure host logic."""
    strategy, tiles = ctypes.c_uint32(0), ctypes.c_uint32(0)
    error = capi.ErrorBuffer()
    error.raise_for(capi.library().vecops_b200_sdpa_plan(byref(record), byref(strategy), byref(tiles), byref(error.record)))
    return strategy.value, tiles.value


def sdpa(q, k, v, out, scale: float, **kwargs) -> None:
    """Run attention on the GPU through the C ABI (the streaming kernel, or two products through the matmul path around a row softmax)."""
    import torch
    kwargs.setdefault("stream", torch.cuda.current_stream(out.device) if out.is_cuda else None)
    record = sdpa_record(q, k, v, out, scale, **kwargs)
    need = c_uint64(0)
    error = capi.ErrorBuffer()
    error.raise_for(capi.library().vecops_b200_sdpa_workspace(byref(record), byref(need), byref(error.record)))
    scratch = torch.empty(max(need.value, 256) + 256, dtype=torch.uint8, device=out.device)
    offset = (-scratch.data_ptr()) % 256
    record.workspace, record.workspace_size = scratch.data_ptr() + offset, need.value
    error.raise_for(capi.library().vecops_b200_sdpa_run(byref(record), byref(error.record)))
    del scratch


def column_correction(b_nk, zero_point: int, out, stream=None) -> None:
    """out[n] = -zero_point * sum_k B[n,k] (int32), the accumulator-input row of an asymmetric 8-bit product."""
    import torch
    if stream is None:
        stream = torch.cuda.current_stream(b_nk.device)
    error = capi.ErrorBuffer()
    error.raise_for(capi.library().vecops_b200_column_correction(b_nk.data_ptr(), torch_dtype_code(b_nk.dtype), b_nk.stride(0), b_nk.shape[0],
                                                                b_nk.shape[1], zero_point, out.data_ptr(), stream.cuda_stream,
                                                                byref(error.record)))


class PreparedMatmul:
    """One problem record built once and launched many times (keeps per-launch host cost to a single C call)."""

    def __init__(self, a, b_nk, c, scale=None, kernel: int = capi.KERNEL_AUTO, stream=None, asynchronous: bool = True,
                 epilogue: capi.VecopsB200Epilogue | None = None, keep=()) -> None:
        import torch
        if stream is None and a.is_cuda:
            stream = torch.cuda.current_stream(a.device)
        self.tensors = (a, b_nk, c, scale)  # keep the storage alive
        self.keep = keep                    # ... and whatever else the launch reads (the epilogue's accumulator input)
        self.epilogue = epilogue
        self.problem = matmul_problem(a, b_nk, c, scale, kernel, stream, asynchronous)
        self.scratch = attach_workspace(self.problem, a.device) if a.is_cuda else None  # one buffer per prepared launch
        self.error = capi.ErrorBuffer()
        self._run = capi.library().vecops_b200_matmul_run
        self._problem_ref = byref(self.problem)
        self._error_ref = byref(self.error.record)

    def launch(self) -> None:
        if self.epilogue is None:
            rc = self._run(self._problem_ref, self._error_ref)
        else:
            rc = capi.library().vecops_b200_matmul_run_fused(self._problem_ref, byref(self.epilogue), self._error_ref)
        if rc != capi.OK:
            self.error.raise_for(rc)


def capture_graph(launches, stream=None):
    """Capture a sequence of PreparedMatmul launches into one CUDA graph; returns the torch.cuda.CUDAGraph."""
    import torch
    side = stream or torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        prepared = [PreparedMatmul(*p.tensors, kernel=p.problem.kernel, stream=side, epilogue=p.epilogue, keep=p.keep) for p in launches]
        for p in prepared:  # warm up outside capture: one-time attribute and tensor-map set-up
            p.launch()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for p in prepared:
                p.launch()
    torch.cuda.current_stream().wait_stream(side)
    graph._vecops_keepalive = prepared
    return graph
