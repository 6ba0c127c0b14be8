"""Seeded synthetic inputs for the benchmark configurations.

The reference measures on no external dataset; its matmul benchmark catalog is
synthetic shapes (benchmarks/ops/matmul-otherlibs/Cases.h:42-45).  The five
configurations below are the shapes, dtypes, layouts, value distributions and
seeds this build is measured on.  Generation is blocked (one PRNG stream per
1024-row block) so that any row range of an operand can be produced on its own,
which is how a rank of a column-sharded run gets exactly its slab of B.

bfloat16 tensors are produced as uint16 bit patterns (round-to-nearest-even).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

BLOCK_ROWS = 1024


@dataclass(frozen=True)
class Workload:
    name: str
    kind: str          # "f32" | "bf16" | "i8" | "w8"
    m: int
    n: int
    k: int
    seed: int
    b_layout: str      # "nk" (B stored [N,K], K-contiguous) or "kn" (B stored [K,N] row-major)
    description: str

    @property
    def flops(self) -> float:
        return 2.0 * self.m * self.n * self.k

    @property
    def algorithmic_bytes(self) -> int:
        """Bytes one launch must move at minimum: each operand read once, C written once."""
        if self.kind == "f32":
            return 4 * (self.m * self.k + self.n * self.k + self.m * self.n)
        if self.kind == "bf16":
            return 2 * (self.m * self.k + self.n * self.k + self.m * self.n)
        if self.kind == "i8":
            return self.m * self.k + self.n * self.k + 4 * self.m * self.n
        if self.kind == "w8":
            return self.n * self.k + 4 * self.n + 2 * self.m * self.k + 2 * self.m * self.n
        raise ValueError(self.kind)


WORKLOADS = {
    w.name: w
    for w in [
        Workload("c1_f32_1024", "f32", 1024, 1024, 1024, 0, "kn",
                 "FP32 GEMM M=N=K=1024, A[M,K], B[K,N] row-major, U(-1,1)"),
        Workload("c2_bf16_4096", "bf16", 4096, 4096, 4096, 1, "nk",
                 "BF16 GEMM M=N=K=4096, fp32 accumulate, bf16 out, B stored [N,K], N(0,1)"),
        Workload("c3_i8_4096x14336x4096", "i8", 4096, 14336, 4096, 2, "nk",
                 "INT8xINT8->INT32 GEMM M=4096 N=14336 K=4096, uniform [-128,127]"),
        Workload("c4_w8_m1", "w8", 1, 14336, 4096, 3, "nk", "weight-only int8 decode GEMM, M=1, N=14336, K=4096"),
        Workload("c4_w8_m16", "w8", 16, 14336, 4096, 3, "nk", "weight-only int8 decode GEMM, M=16, N=14336, K=4096"),
        Workload("c4_w8_m128", "w8", 128, 14336, 4096, 3, "nk", "weight-only int8 decode GEMM, M=128, N=14336, K=4096"),
        Workload("c5_bf16_16384x53248x8192", "bf16", 16384, 53248, 8192, 4, "nk",
                 "large BF16 GEMM M=16384 N=53248 K=8192, B split by N across GPUs, N(0,0.02)"),
    ]
}


def f32_to_bf16_bits(values: np.ndarray) -> np.ndarray:
    values = np.ascontiguousarray(values, dtype=np.float32)
    bits = values.view(np.uint32)
    bias = ((bits >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    out = ((bits + bias) >> np.uint32(16)).astype(np.uint16)
    out[np.isnan(values)] = 0x7FC0
    return out


def _blocked(rows: int, cols: int, row0: int, row1: int, seed: int, stream: int, draw) -> np.ndarray:
    """Rows [row0,row1) of a (rows x cols) matrix whose 1024-row blocks each own a PRNG stream."""
    pieces = []
    first = row0 // BLOCK_ROWS
    last = (row1 - 1) // BLOCK_ROWS if row1 > row0 else first - 1
    for block in range(first, last + 1):
        lo, hi = block * BLOCK_ROWS, min(rows, (block + 1) * BLOCK_ROWS)
        rng = np.random.Generator(np.random.PCG64([seed, stream, block]))
        data = draw(rng, (hi - lo, cols))
        pieces.append(data[max(row0, lo) - lo:min(row1, hi) - lo])
    if not pieces:
        return draw(np.random.Generator(np.random.PCG64([seed, stream, 0])), (0, cols))
    return np.concatenate(pieces, axis=0)


def _normal_bf16(std: float):
    return lambda rng, shape: f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32) * np.float32(std))


def _uniform_f32(rng, shape):
    return rng.uniform(-1.0, 1.0, shape).astype(np.float32)


def _int8(lo: int, hi: int):
    return lambda rng, shape: rng.integers(lo, hi + 1, shape, dtype=np.int8)


def make_a(w: Workload, row0: int = 0, row1: int | None = None) -> np.ndarray:
    """Rows [row0,row1) of A[M,K]."""
    row1 = w.m if row1 is None else row1
    draw = {"f32": _uniform_f32, "bf16": _normal_bf16(0.02 if w.seed == 4 else 1.0), "i8": _int8(-128, 127),
            "w8": _normal_bf16(1.0)}[w.kind]
    return _blocked(w.m, w.k, row0, row1, w.seed, 0, draw)


def make_b_nk(w: Workload, row0: int = 0, row1: int | None = None) -> np.ndarray:
    """Rows [row0,row1) of B addressed as [N,K] (for the "kn" layout transpose the result's view yourself)."""
    row1 = w.n if row1 is None else row1
    draw = {"f32": _uniform_f32, "bf16": _normal_bf16(0.02 if w.seed == 4 else 1.0), "i8": _int8(-128, 127),
            "w8": _int8(-127, 127)}[w.kind]
    return _blocked(w.n, w.k, row0, row1, w.seed, 1, draw)


def make_scale(w: Workload, row0: int = 0, row1: int | None = None) -> np.ndarray | None:
    """Per-output-channel fp32 scales (weight-only int8 only)."""
    if w.kind != "w8":
        return None
    row1 = w.n if row1 is None else row1
    rng = np.random.Generator(np.random.PCG64([w.seed, 2, 0]))
    return rng.uniform(0.001, 0.02, w.n).astype(np.float32)[row0:row1]


def scaled(w: Workload, m: int | None = None, n: int | None = None, k: int | None = None) -> Workload:
    """The same workload at reduced extents (parity cases the CPU checker finishes in seconds)."""
    return Workload(w.name + "_scaled", w.kind, m or w.m, n or w.n, k or w.k, w.seed, w.b_layout, w.description)
