"""Column-sharded GEMM logic on CPU ranks (gloo, world size 2 and 3): partition,
all-gather into the staging buffer, placement into the row-major result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vecops_b200 import sharding


def test_partition_covers_all_columns_in_whole_tiles():
    for n, world in [(53248, 8), (53248, 4), (53248, 2), (53248, 1), (1000, 3), (256, 4), (14336, 8)]:
        edges = [sharding.column_partition(n, world, r) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == n
        for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
            assert a1 == b0 and a0 <= a1
        for n0, n1 in edges[:-1]:
            assert n0 % sharding.TILE_N == 0 and n1 % sharding.TILE_N == 0
    # the benchmark's sharded configuration splits evenly at every GPU count
    assert all(sharding.uniform_partition(53248, p) for p in (1, 2, 4, 8))
    assert sharding.column_partition(53248, 8, 3) == (3 * 6656, 4 * 6656)
    with pytest.raises(ValueError):
        sharding.column_partition(10, 2, 2)


def test_peer_order_gives_every_receiver_one_sender_per_phase():
    # the pipelined gather sends a rank's slab to its peers one after the other: in phase j the senders must hit
    # distinct receivers, nobody sends to itself, and over all phases everybody reaches everybody else once
    for world in (1, 2, 3, 4, 8):
        orders = [sharding.peer_order(r, world) for r in range(world)]
        for r, order in enumerate(orders):
            assert sorted(order) == [p for p in range(world) if p != r]
        for phase in range(world - 1):
            assert sorted(order[phase] for order in orders) == list(range(world))
    with pytest.raises(ValueError):
        sharding.peer_order(2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, m: int, n: int, k: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.checker import Port
        checker = Port()
        rng = np.random.default_rng(5)
        a = rng.integers(-8, 8, (m, k)).astype(np.float32)       # replicated
        b = rng.integers(-8, 8, (n, k)).astype(np.float32)
        n0, n1 = sharding.column_partition(n, world, rank, align=16)
        slab = torch.from_numpy(checker.matmul_f32(a, b[n0:n1]))  # this rank's [M, w] output slab
        full = torch.zeros((m, n), dtype=torch.float32)
        staging = torch.empty((world, m, n1 - n0), dtype=torch.float32)

        def place(dst, col0, src):
            dst[:, col0:col0 + src.shape[1]].copy_(src)

        sharding.gather_columns(slab, full, staging, world, place=place)
        want = checker.matmul_f32(a, b)
        results[rank] = bool(np.array_equal(full.numpy(), want))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_gemm_gathers_to_the_full_product(world):
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 24, 16 * world * 2, 40, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(results.get(r) for r in range(world)), dict(results)
