"""torch.ops.vecops_b200.* - the Torch face of the library.

``load()`` registers three operators implemented in C++ (csrc/torch/torch_bridge.cpp) for CUDA tensors:

    torch.ops.vecops_b200.matmul(a, b_nk, column_scale=None, cin=None, alpha=1.0, activation=0, clamp_lo=0.0, clamp_hi=0.0, out_dtype=None, row_scale=None)
    torch.ops.vecops_b200.matmul_out(a, b_nk, c, column_scale=None, cin=None, alpha=1.0, activation=0, clamp_lo=0.0, clamp_hi=0.0, row_scale=None)
    torch.ops.vecops_b200.sdpa(q, k, v, scale, causal=0, key_mask=None, bias=None, out_dtype=None)

A call goes dispatcher -> C++ -> operator bridge -> kernel on the current CUDA stream; Python is not on that path.
They stand where vecops' generated Torch adapters stand (python/vecops/ops/torch.py ``register``).  There is no CPU
implementation: a CPU tensor raises torch's "could not run ... with arguments from the 'CPU' backend".
"""
from __future__ import annotations

from pathlib import Path

LIBRARY_PATH = Path(__file__).resolve().parent / "lib" / "libvecops_b200_torch.so"
_loaded = False


def load() -> None:
    """Register the operators (idempotent); raises if the library has not been built."""
    global _loaded
    if _loaded:
        return
    import torch
    if not LIBRARY_PATH.exists():
        raise RuntimeError(f"{LIBRARY_PATH} is missing: build it with `python -m vecops_b200._build --torch`")
    torch.ops.load_library(str(LIBRARY_PATH))
    _loaded = True
