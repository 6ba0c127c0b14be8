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
