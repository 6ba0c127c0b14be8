"""vecops_b200: the vecops matmul operator rebuilt for NVIDIA B200 (sm_100a).

The product is the shared library ``lib/libvecops_b200.so`` (hand-written CUDA
kernels behind a C ABI, plus a C++ host runtime that mirrors vecops' operator
API).  This package only builds it, loads it and offers a small harness used by
the tests and the benchmark.
"""
from . import capi  # noqa: F401
from .harness import matmul, matmul_problem, select_kernel, torch_dtype_code  # noqa: F401

__all__ = ["capi", "matmul", "matmul_problem", "select_kernel", "torch_dtype_code"]
