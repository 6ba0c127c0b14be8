"""Host arrays in, host array out: the NumPy face of the library (the place of vecops' NumPy bridge, python/vecops/ops).

The operands are copied to the GPU, the product runs on the library's kernels through the C ABI and the result is copied
back - there is no CPU implementation behind this, and without a B200 the call raises.  bfloat16 has no NumPy dtype:
pass uint16 bit patterns with ``bf16=True``.
"""
from __future__ import annotations

import numpy as np


def matmul(a: np.ndarray, b_nk: np.ndarray, column_scale: np.ndarray | None = None, *, bf16: bool = False, out_dtype=None,
           cin: np.ndarray | None = None, alpha: float = 1.0, activation: int = 0, device: int = 0) -> np.ndarray:
    """C[M,N] = activation((cin + A[M,K] . B[N,K]^T) * alpha * column_scale).

    dtypes: float32 x float32 -> float32; float16 x float16 -> float16 | float32; uint16 (bf16 bits, ``bf16=True``) x uint16
    -> uint16 bits | float32; uint16 bf16 bits x int8 (weight-only) -> the same; int8 / uint8 x int8 / uint8 -> int32, or
    float32 through the dequantising transform (``out_dtype=np.float32``)."""
    import torch

    from . import harness
    if not torch.cuda.is_available():
        raise RuntimeError("vecops_b200.numpy_ops.matmul needs a CUDA device: there is no CPU path")
    dev = torch.device("cuda", device)

    def up(x, as_bf16):
        t = torch.from_numpy(np.ascontiguousarray(x)).to(dev)
        return t.view(torch.bfloat16) if as_bf16 else t

    da = up(a, bf16 and a.dtype == np.uint16)
    db = up(b_nk, bf16 and b_nk.dtype == np.uint16)
    if out_dtype is None:
        torch_out = torch.int32 if a.dtype in (np.int8, np.uint8) else da.dtype
    else:
        torch_out = {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16, np.dtype(np.int32): torch.int32,
                     np.dtype(np.uint16): torch.bfloat16}[np.dtype(out_dtype)]
    c = torch.empty((a.shape[0], b_nk.shape[0]), dtype=torch_out, device=dev)
    harness.matmul(da, db, c, up(column_scale, False) if column_scale is not None else None,
                   cin=up(cin, bf16 and cin.dtype == np.uint16) if cin is not None else None, alpha=alpha, activation=activation)
    torch.cuda.synchronize(dev)
    if torch_out == torch.bfloat16:
        return c.view(torch.int16).cpu().numpy().view(np.uint16)
    return c.cpu().numpy()
