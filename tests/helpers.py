"""Shared pieces of the parity tests."""
from __future__ import annotations

import numpy as np

# Tolerances of the parity contract (relative Frobenius error against the CPU checker).
TOL_BF16 = 1e-3   # bf16 in, fp32 accumulate (also weight-only int8)
TOL_F32 = 1e-5    # fp32 GEMM
# int8 x int8 -> int32 must be bit-exact.


def oracle_for(kind: str, port, a, b, scale=None, out_bf16=True):
    if kind == "bf16":
        return port.matmul_bf16(a, b, scale, out_bf16)
    if kind == "w8":
        return port.matmul_w8(a, b, scale, out_bf16)
    if kind == "i8":
        return port.matmul_i8(a, b)
    if kind == "f32":
        return port.matmul_f32(a, b)
    raise ValueError(kind)


def to_device(array: np.ndarray, bf16: bool = False):
    import torch
    tensor = torch.from_numpy(np.ascontiguousarray(array)).cuda()
    return tensor.view(torch.bfloat16) if bf16 else tensor


def bf16_result_to_numpy(tensor) -> np.ndarray:
    import torch
    return tensor.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
