"""Column sharding of a large GEMM over the GPUs of one node.

C[:, n0:n1] = A . B[n0:n1, :]^T has no cross-shard reduction: rank r keeps rows
[n0, n1) of B resident, A is replicated, and the only exchange is an all-gather
of the finished [M, N/p] output slabs.  A column slab is not contiguous inside
the row-major [M, N] result, so the gather lands in a [p, M, N/p] staging
buffer and one kernel per slab places it into the final matrix.
"""
from __future__ import annotations

from typing import Callable

TILE_N = 256  # partition in whole output tiles of the tensor-core kernel


def column_partition(n: int, world: int, rank: int, align: int = TILE_N) -> tuple[int, int]:
    """Columns [n0, n1) owned by `rank`: whole `align`-wide blocks, spread as evenly as possible."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    blocks = (n + align - 1) // align
    base, extra = divmod(blocks, world)
    first = rank * base + min(rank, extra)
    count = base + (1 if rank < extra else 0)
    return min(n, first * align), min(n, (first + count) * align)


def uniform_partition(n: int, world: int, align: int = TILE_N) -> bool:
    """True when every rank owns the same number of columns (all_gather_into_tensor needs that)."""
    widths = {column_partition(n, world, r, align)[1] - column_partition(n, world, r, align)[0] for r in range(world)}
    return len(widths) == 1


def gather_columns(slab, full, staging, world: int, group=None, place: Callable | None = None) -> None:
    """All-gather every rank's [M, w] slab and place slab r at columns [r*w, (r+1)*w) of `full` [M, N].

    `staging` is a [world, M, w] buffer.  `place(full, col0, slab_r)` copies one slab into the result;
    on CUDA tensors the caller passes the library's placement kernel.
    """
    import torch.distributed as dist
    m, w = slab.shape
    if tuple(staging.shape) != (world, m, w):
        raise ValueError(f"staging must be [{world}, {m}, {w}]")
    if world == 1:
        staging[0].copy_(slab)
    else:
        # concatenated form: rank r lands in rows [r*M, (r+1)*M) of the flattened staging buffer
        dist.all_gather_into_tensor(staging.view(world * m, w), slab.contiguous(), group=group)
    for r in range(world):
        place(full, r * w, staging[r])


def cuda_place(stream=None) -> Callable:
    """Placement through the library's own kernel (vecops_b200_place_columns)."""
    from ctypes import byref

    from . import capi

    def place(full, col0, slab):
        import torch
        error = capi.ErrorBuffer()
        s = stream if stream is not None else torch.cuda.current_stream(full.device)
        rc = capi.library().vecops_b200_place_columns(full.data_ptr(), full.stride(0), col0, slab.data_ptr(), slab.stride(0),
                                                      slab.shape[0], slab.shape[1], full.element_size(), s.cuda_stream,
                                                      byref(error.record))
        error.raise_for(rc)

    return place


class FusedGatherGemm:
    """This rank's slab GEMM with the all-gather fused into its epilogue (vecops_b200_matmul_allgather_run).

    `destinations` are the full [M, N] result tensors of every rank as seen from this process: the local tensor
    and peer views of the others (torch symmetric memory, CUDA IPC) - or, with `multicast`, the single NVSwitch
    multicast address of the result.  Built once, launched many times.
    """

    def __init__(self, a, b_slab, destination_ptrs, n_total: int, ldc: int, col0: int, out_dtype, stream=None, multicast: bool = False) -> None:
        import ctypes

        import torch

        from . import capi, harness
        self.keep = (a, b_slab)
        m, n = a.shape[0], b_slab.shape[0]
        # problem->c is ignored by the fused entry point; a 1-element placeholder keeps the record well formed
        self.placeholder = torch.empty((m, n), dtype=out_dtype, device="meta")
        problem = capi.VecopsB200Matmul()
        problem.struct_size = ctypes.sizeof(capi.VecopsB200Matmul)
        problem.kernel = capi.KERNEL_BF16_TCGEN05
        problem.m, problem.n, problem.k = m, n, a.shape[1]
        problem.a, problem.a_stride_m, problem.a_stride_k = a.data_ptr(), a.stride(0), a.stride(1)
        problem.b, problem.b_stride_n, problem.b_stride_k = b_slab.data_ptr(), b_slab.stride(0), b_slab.stride(1)
        problem.c, problem.c_stride_m, problem.c_stride_n = None, n, 1
        stream = stream if stream is not None else torch.cuda.current_stream(a.device)
        problem.stream = stream.cuda_stream
        problem.a_dtype, problem.b_dtype = harness.torch_dtype_code(a.dtype), harness.torch_dtype_code(b_slab.dtype)
        problem.c_dtype = harness.torch_dtype_code(out_dtype)
        problem.device_index = a.device.index
        problem.flags = capi.MATMUL_FLAG_ASYNC
        self.problem = problem
        self.scratch = harness.attach_workspace(problem, a.device)  # partial sums of a split tail wave meet here
        self.pointers = (ctypes.c_void_p * len(destination_ptrs))(*destination_ptrs)
        self.gather = capi.VecopsB200Gather(ctypes.sizeof(capi.VecopsB200Gather), len(destination_ptrs), self.pointers, n_total, ldc, col0,
                                            capi.GATHER_MULTICAST if multicast else 0, 0)
        self.error = capi.ErrorBuffer()
        self._run = capi.library().vecops_b200_matmul_allgather_run
        self._args = (ctypes.byref(self.problem), ctypes.byref(self.gather), ctypes.byref(self.error.record))

    def launch(self) -> None:
        rc = self._run(*self._args)
        if rc != 0:
            self.error.raise_for(rc)


def peer_order(rank: int, world: int) -> list[int]:
    """The order in which `rank` sends to its peers: from the next rank on, wrapping round.  In phase j every rank r
    sends to (r + 1 + j) mod world, so each receiver has exactly one sender per phase when the ranks run in step."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    return [(rank + 1 + j) % world for j in range(world - 1)]


class PipelinedGatherGemm:
    """The column-sharded product with its gather run BEHIND the next product.

    Two copies of the full [M, N] result live in symmetric memory and steps alternate between them.  Step i: the slab
    GEMM stores this rank's columns into its own copy at full speed (compute stream); an event later, on a second
    stream, the slab is pushed to the same columns of every peer's copy (vecops_b200_push_columns, peers visited from
    the next rank on) and one device barrier orders the ranks - while the compute stream is already running the GEMM
    of step i+1.  A copy is written again two steps later, after its own push and barrier have finished.

    `results` is the symmetric [2, M, N] tensor, `peer_bases` every rank's base address of it as seen from here
    (handle.buffer_ptrs), `barrier` a callable that enqueues the ranks' device barrier on the CURRENT torch stream.
    """

    def __init__(self, a, b_slab, results, peer_bases, rank: int, col0: int, barrier: Callable, compute_stream=None,
                 route: int = 0, lanes: int = 1) -> None:
        import ctypes

        import torch

        from . import capi, harness
        if results.dim() != 3 or results.shape[0] != 2:
            raise ValueError("results must be [2, M, N]")
        world = len(peer_bases)
        m, n_total = results.shape[1], results.shape[2]
        n = b_slab.shape[0]
        self.device = a.device
        self.compute = compute_stream if compute_stream is not None else torch.cuda.current_stream(a.device)
        self.send = torch.cuda.Stream(a.device)
        self.results, self.barrier, self.route = results, barrier, route
        self.prepared = [harness.PreparedMatmul(a, b_slab, results[half][:, col0:col0 + n], None, stream=self.compute) for half in (0, 1)]
        half_bytes = m * n_total * results.element_size()
        order = peer_order(rank, world)
        self.peers = [(ctypes.c_void_p * max(1, len(order)))(*[int(peer_bases[r]) + half * half_bytes for r in order]) for half in (0, 1)]
        self.count = len(order)
        # `lanes` > 1: the peers are dealt over that many side streams, so that copies to different peers overlap
        self.lanes = max(1, min(lanes, self.count))
        self.single = [[(ctypes.c_void_p * 1)(int(peer_bases[r]) + half * half_bytes) for r in order] for half in (0, 1)]
        self.lane_streams = [torch.cuda.Stream(a.device) for _ in range(self.lanes)] if self.lanes > 1 else []
        self.fork = torch.cuda.Event()
        self.lane_done = [torch.cuda.Event() for _ in self.lane_streams]
        self.shape = (n_total, col0, m, n, results.element_size())
        self.computed = [torch.cuda.Event(), torch.cuda.Event()]
        self.gathered = [torch.cuda.Event(), torch.cuda.Event()]
        self.steps = 0
        self.error = capi.ErrorBuffer()
        self._push = capi.library().vecops_b200_push_columns

    def launch(self) -> int:
        """Enqueue one step; returns which copy of the result it fills (complete on every rank once `join` has been
        waited for, or once the NEXT step using that copy starts)."""
        half = self.steps & 1
        if self.steps >= 2:
            self.compute.wait_event(self.gathered[half])  # the push that read this copy two steps ago has finished
        self.prepared[half].launch()
        self.computed[half].record(self.compute)
        self.send.wait_event(self.computed[half])
        self.gather_alone(half)
        self.gathered[half].record(self.send)
        self.steps += 1
        return half

    def gather_alone(self, half: int = 0) -> None:
        """Enqueue only the push and the barrier of one copy on the send stream (for timing the transfer by itself)."""
        import ctypes

        import torch
        ld, col0, rows, cols, elem = self.shape
        source, error = self.results[half].data_ptr(), ctypes.byref(self.error.record)

        def push(pointers, count, stream):
            rc = self._push(source, pointers, count, ld, col0, rows, cols, elem, self.route, stream.cuda_stream, error)
            if rc != 0:
                self.error.raise_for(rc)

        if self.count and self.lanes <= 1:
            push(self.peers[half], self.count, self.send)
        elif self.count:
            self.fork.record(self.send)
            for lane, stream in enumerate(self.lane_streams):
                stream.wait_event(self.fork)
                for j in range(lane, self.count, self.lanes):
                    push(self.single[half][j], 1, stream)
                self.lane_done[lane].record(stream)
                self.send.wait_event(self.lane_done[lane])
        with torch.cuda.stream(self.send):
            self.barrier()

    def join(self) -> None:
        """The compute stream waits for the gather of the last step enqueued."""
        if self.steps:
            self.compute.wait_event(self.gathered[(self.steps - 1) & 1])


def symmetric_result(m: int, n: int, dtype, device, group=None, copies: int = 0):
    """Allocate the full [M, N] result (or `copies` of it, [copies, M, N]) in symmetric memory; returns (tensor, handle)
    with handle.buffer_ptrs = every rank's base address of it."""
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    tensor = symm_mem.empty((copies, m, n) if copies else (m, n), dtype=dtype, device=device)
    handle = symm_mem.rendezvous(tensor, group if group is not None else dist.group.WORLD)
    return tensor, handle
