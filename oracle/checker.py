"""numpy front end of the checker libraries (test infrastructure, not product code).

``Port``  wraps the C restatement (``liboracle.so``).
``Ref``   wraps the reference's own CPU matmul (``_ref/libvecops_ref.so``) when it
          was built and this host's CPU can run it.

bfloat16 tensors travel as ``uint16`` bit patterns.  Only tests, the smoke check
and the CPU-baseline legs of the benchmark may import this module.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int64, c_void_p

import numpy as np

from . import build_oracle

_I64 = c_int64
_P = c_void_p


def _ptr(array: np.ndarray | None):
    return None if array is None else array.ctypes.data_as(c_void_p)


def f32_to_bf16_bits(values: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (NaN -> 0x7fc0).

    Same rule as include/vecops/util/BFloat16.h:25-37 of the reference.
    """
    values = np.ascontiguousarray(values, dtype=np.float32)
    bits = values.view(np.uint32)
    bias = ((bits >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    out = ((bits + bias) >> np.uint32(16)).astype(np.uint16)
    out[np.isnan(values)] = 0x7FC0
    return out


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def rel_frobenius(got: np.ndarray, want: np.ndarray) -> float:
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    denom = float(np.linalg.norm(want))
    return float(np.linalg.norm(got - want)) / (denom if denom > 0 else 1.0)


def _strides(array: np.ndarray) -> tuple[int, int]:
    item = array.itemsize
    return array.strides[0] // item, array.strides[1] // item


ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_SILU, ACT_CLAMP = range(5)
_F = ctypes.c_float


def f16_conversion_inputs() -> tuple[np.ndarray, np.ndarray]:
    """(every fp16 bit pattern, float32 inputs for the narrowing) - the sweep the fp16 conversions are pinned on:
    each fp16 value exactly, the tie above it and the floats either side of the tie, 2^20 random bit patterns, and
    the edges of the range (2^-25, 65520, infinities, NaNs)."""
    patterns = np.arange(65536, dtype=np.uint16)
    base = patterns.view(np.float16).astype(np.float32).view(np.uint32)
    rng = np.random.default_rng(5)
    bits = np.concatenate([
        base, base + np.uint32(0x1000), base + np.uint32(0x0fff), base + np.uint32(0x1001),
        rng.integers(0, 2**32, 1 << 20, dtype=np.uint64).astype(np.uint32),
        np.array([0x33000000, 0x33000001, 0x32ffffff, 0x477fe000, 0x477fefff, 0x477ff000, 0x477ff001, 0x7f800000, 0xff800000,
                  0x7fc00000, 0x7f800001], dtype=np.uint32)])
    return patterns, bits.view(np.float32)


def packed_pitch(itemsize: int, k: int) -> int:
    """Elements per row of the packed form: K rounded up to whole 128-byte lines."""
    per_line = 128 // itemsize
    return (k + per_line - 1) // per_line * per_line


def pack_rows(view: np.ndarray, narrow: str | None = None) -> np.ndarray:
    """Restatement of operand packing as the reference's tests state it (tests/ops/MatmulPackTest.cpp:186-207): every
    packed position holds the logical element (row, k) - converted to the compute type - or zero past the extents.
    Here the packed form is [rows, pitch], K-contiguous.  `narrow`: None (same type), "bf16" or "f16" for a float32
    view (returned as uint16 bit patterns)."""
    rows, k = view.shape
    if narrow == "bf16":
        values = f32_to_bf16_bits(np.ascontiguousarray(view, dtype=np.float32))
    elif narrow == "f16":
        values = np.ascontiguousarray(view, dtype=np.float32).astype(np.float16).view(np.uint16)
    else:
        values = np.ascontiguousarray(view)
    out = np.zeros((rows, packed_pitch(values.itemsize, k)), dtype=values.dtype)
    out[:, :k] = values
    return out


def pack_compensation(b_nk: np.ndarray, a_zero_point: int) -> np.ndarray:
    """-a_zero_point * sum_k B[n,k] as int32 (tests/ops/MatmulPackTest.cpp:209-216)."""
    return (-int(a_zero_point) * b_nk.astype(np.int64).sum(axis=1)).astype(np.int32)


def _cin_view(cin, m: int, n: int):
    """(array viewed as [m, n] with possibly zero strides, kind) - kind 1 for bf16 bits, else 0."""
    if cin is None:
        return None, 0
    kind = 1 if cin.dtype == np.uint16 else 0
    return np.broadcast_to(cin, (m, n)), kind


class Port:
    """The C restatement.  Every method returns a fresh C-contiguous result."""

    def __init__(self) -> None:
        path = build_oracle.build_port()
        self.lib = ctypes.CDLL(str(path))
        self.lib.oracle_threads.restype = c_int
        self.lib.oracle_f32_to_bf16.restype = ctypes.c_uint16
        self.lib.oracle_f32_to_bf16.argtypes = [ctypes.c_float]
        self.lib.oracle_matmul_f32.argtypes = [_I64] * 3 + [_P, _I64, _I64, _P, _I64, _I64, _P, _I64, _I64]
        self.lib.oracle_matmul_bf16.argtypes = [_I64] * 3 + [_P, _I64, _I64, _P, _I64, _I64, _P, _P, _I64, _I64, c_int]
        self.lib.oracle_matmul_i8.argtypes = [_I64] * 3 + [_P, _I64, _I64, c_int, _P, _I64, _I64, c_int, _P, _I64, _I64]
        self.lib.oracle_matmul_w8.argtypes = [_I64] * 3 + [_P, _I64, _I64, _P, _I64, _I64, _P, _P, _I64, _I64, c_int]
        _F = ctypes.c_float
        self.lib.oracle_matmul_bf16_fused.argtypes = [_I64] * 3 + [_P, _I64, _I64, _P, _I64, _I64, _P, c_int, _I64, _I64, _F, _P, c_int, _F, _F,
                                                                  _P, _I64, _I64, c_int]
        self.lib.oracle_matmul_f32_fused.argtypes = [_I64] * 3 + [_P, _I64, _I64, _P, _I64, _I64, _P, _I64, _I64, _F, _P, c_int, _F, _F, _P,
                                                                 _I64, _I64]
        self.lib.oracle_matmul_i8_accumulate.argtypes = [_I64] * 3 + [_P, _I64, _I64, c_int, _P, _I64, _I64, c_int, _P, _I64, _I64, _P, _I64,
                                                                     _I64]

        self.lib.oracle_f32_to_f16.restype = ctypes.c_uint16
        self.lib.oracle_f32_to_f16.argtypes = [ctypes.c_float]
        self.lib.oracle_f16_to_f32.restype = ctypes.c_float
        self.lib.oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
        self.lib.oracle_f16_widen.argtypes = [_P, _P, _I64]
        self.lib.oracle_f16_narrow.argtypes = [_P, _P, _I64]
        self.lib.oracle_matmul_f16_fused.argtypes = [_I64] * 3 + [_P, _I64, _I64, _P, _I64, _I64, _P, _I64, _I64, _F, _P, c_int, _F, _F, _P,
                                                                 _I64, _I64, c_int]
        self.lib.oracle_sdpa_bf16.argtypes = [_I64] * 4 + [_P, _I64, _P, _I64, _P, _I64, _P, _P, _P, _I64, _P, _I64, c_int, _F, _P, _I64, c_int]
        self.lib.oracle_sdpa_bf16_streaming.argtypes = ([_I64] * 4 + [_P, _I64, _P, _I64, _P, _I64, _P, _P, _P, _I64, _P, _I64, c_int, _F, _I64, _I64,
                                                         _P, _I64, c_int])
        self.lib.oracle_quantize_rows_per_row.argtypes = [_I64, _I64, _P, _I64, _I64, _P, _F, _P, _I64, _I64, c_int]
        self.lib.oracle_matmul_i8_dequant_rows.argtypes = [_I64] * 3 + [_P, _I64, _I64, c_int, _P, _I64, _I64, c_int, _P, _I64, _I64, _P, _P, _P,
                                                                       _I64, _I64, c_int]
        self.lib.oracle_quantize_rows.argtypes = [_I64, _I64, _P, _I64, _I64, _F, _F, _P, _I64, _I64, c_int]
        self.lib.oracle_matmul_i8_dequant.argtypes = [_I64] * 3 + [_P, _I64, _I64, c_int, _P, _I64, _I64, c_int, _P, _I64, _I64, _F, _P, c_int,
                                                                  _F, _F, _P, _I64, _I64, c_int]

    @property
    def threads(self) -> int:
        return int(self.lib.oracle_threads())

    def matmul_f32(self, a: np.ndarray, b_nk: np.ndarray) -> np.ndarray:
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.float32)
        self.lib.oracle_matmul_f32(m, n, k, _ptr(a), *_strides(a), _ptr(b_nk), *_strides(b_nk), _ptr(c), n, 1)
        return c

    def matmul_bf16(self, a: np.ndarray, b_nk: np.ndarray, scale: np.ndarray | None = None,
                    out_bf16: bool = True) -> np.ndarray:
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.uint16 if out_bf16 else np.float32)
        self.lib.oracle_matmul_bf16(m, n, k, _ptr(a), *_strides(a), _ptr(b_nk), *_strides(b_nk), _ptr(scale), _ptr(c),
                                    n, 1, int(out_bf16))
        return c

    def matmul_i8(self, a: np.ndarray, b_nk: np.ndarray) -> np.ndarray:
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.int32)
        self.lib.oracle_matmul_i8(m, n, k, _ptr(a), *_strides(a), int(a.dtype == np.int8), _ptr(b_nk), *_strides(b_nk),
                                  int(b_nk.dtype == np.int8), _ptr(c), n, 1)
        return c

    def matmul_w8(self, a: np.ndarray, w_nk: np.ndarray, scale: np.ndarray | None, out_bf16: bool = True) -> np.ndarray:
        m, k = a.shape
        n = w_nk.shape[0]
        c = np.empty((m, n), dtype=np.uint16 if out_bf16 else np.float32)
        self.lib.oracle_matmul_w8(m, n, k, _ptr(a), *_strides(a), _ptr(w_nk), *_strides(w_nk), _ptr(scale), _ptr(c), n,
                                  1, int(out_bf16))
        return c


    # ---- fused forms: COut = activation((CIn + A.B^T) * alpha * column_scale)

    def matmul_bf16_fused(self, a, b_nk, cin=None, alpha=1.0, scale=None, act=ACT_NONE, lo=0.0, hi=0.0, out_bf16=True):
        """`cin`: None, or an [M,N]-broadcastable float32 / uint16 (bf16 bits) array; its strides may be zero."""
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.uint16 if out_bf16 else np.float32)
        cin_view, kind = _cin_view(cin, m, n)
        self.lib.oracle_matmul_bf16_fused(m, n, k, _ptr(a), *_strides(a), _ptr(b_nk), *_strides(b_nk), _ptr(cin_view), kind,
                                          *(_strides(cin_view) if cin_view is not None else (0, 0)), float(alpha), _ptr(scale), int(act),
                                          float(lo), float(hi), _ptr(c), n, 1, int(out_bf16))
        return c

    def f16_widen(self, bits: np.ndarray) -> np.ndarray:
        bits = np.ascontiguousarray(bits, dtype=np.uint16)
        out = np.empty(bits.shape, dtype=np.float32)
        self.lib.oracle_f16_widen(_ptr(bits), _ptr(out), bits.size)
        return out

    def f16_narrow(self, values: np.ndarray) -> np.ndarray:
        values = np.ascontiguousarray(values, dtype=np.float32)
        out = np.empty(values.shape, dtype=np.uint16)
        self.lib.oracle_f16_narrow(_ptr(values), _ptr(out), values.size)
        return out

    def matmul_f16(self, a, b_nk, cin=None, alpha=1.0, scale=None, act=ACT_NONE, lo=0.0, hi=0.0, out_f16=True):
        """fp16 bit patterns (uint16) in; fp16 bits or float32 out.  `cin`: None or an [M,N]-broadcastable float32 array."""
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.uint16 if out_f16 else np.float32)
        cin_view, kind = _cin_view(cin, m, n)
        assert kind == 0, "the fp16 form takes an f32 accumulator input"
        self.lib.oracle_matmul_f16_fused(m, n, k, _ptr(a), *_strides(a), _ptr(b_nk), *_strides(b_nk), _ptr(cin_view),
                                         *(_strides(cin_view) if cin_view is not None else (0, 0)), float(alpha), _ptr(scale), int(act),
                                         float(lo), float(hi), _ptr(c), n, 1, int(out_f16))
        return c

    def sdpa_bf16(self, q, k, v, scale, query_mask=None, key_mask=None, keep_mask=None, bias=None, causal=0, out_bf16=False):
        """One head: q [Lq,Dqk], k [Lkv,Dqk], v [Lkv,Dv] as bf16 bits; masks uint8 (non-zero keeps); bias float32 [Lq,Lkv]."""
        q, k, v = (np.ascontiguousarray(x) for x in (q, k, v))
        lq, dqk = q.shape
        lkv, dv = v.shape
        out = np.empty((lq, dv), dtype=np.uint16 if out_bf16 else np.float32)
        keep_mask = None if keep_mask is None else np.ascontiguousarray(keep_mask, dtype=np.uint8)
        bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        query_mask = None if query_mask is None else np.ascontiguousarray(query_mask, dtype=np.uint8)
        key_mask = None if key_mask is None else np.ascontiguousarray(key_mask, dtype=np.uint8)
        self.lib.oracle_sdpa_bf16(lq, lkv, dqk, dv, _ptr(q), dqk, _ptr(k), dqk, _ptr(v), dv, _ptr(query_mask), _ptr(key_mask),
                                  _ptr(keep_mask), lkv, _ptr(bias), lkv, int(causal), float(scale), _ptr(out), dv, int(out_bf16))
        return out

    def sdpa_bf16_streaming(self, q, k, v, scale, query_mask=None, key_mask=None, keep_mask=None, bias=None, causal=0, out_bf16=False,
                            block=128, chunk_blocks=0):
        """The same head by the streaming strategy: keys in blocks of `block`, probabilities rounded to bf16 before the
        normalisation; `chunk_blocks` > 0 cuts the keys into chunks of that many blocks whose states are merged at the end."""
        q, k, v = (np.ascontiguousarray(x) for x in (q, k, v))
        lq, dqk = q.shape
        lkv, dv = v.shape
        out = np.empty((lq, dv), dtype=np.uint16 if out_bf16 else np.float32)
        keep_mask = None if keep_mask is None else np.ascontiguousarray(keep_mask, dtype=np.uint8)
        bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        query_mask = None if query_mask is None else np.ascontiguousarray(query_mask, dtype=np.uint8)
        key_mask = None if key_mask is None else np.ascontiguousarray(key_mask, dtype=np.uint8)
        self.lib.oracle_sdpa_bf16_streaming(lq, lkv, dqk, dv, _ptr(q), dqk, _ptr(k), dqk, _ptr(v), dv, _ptr(query_mask), _ptr(key_mask),
                                            _ptr(keep_mask), lkv, _ptr(bias), lkv, int(causal), float(scale), int(block), int(chunk_blocks),
                                            _ptr(out), dv, int(out_bf16))
        return out

    def matmul_f32_fused(self, a, b_nk, cin=None, alpha=1.0, scale=None, act=ACT_NONE, lo=0.0, hi=0.0):
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.float32)
        cin_view, _ = _cin_view(cin, m, n)
        self.lib.oracle_matmul_f32_fused(m, n, k, _ptr(a), *_strides(a), _ptr(b_nk), *_strides(b_nk), _ptr(cin_view),
                                         *(_strides(cin_view) if cin_view is not None else (0, 0)), float(alpha), _ptr(scale), int(act),
                                         float(lo), float(hi), _ptr(c), n, 1)
        return c

    def matmul_i8_accumulate(self, a, b_nk, cin):
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.int32)
        cin_view, _ = _cin_view(cin, m, n)
        self.lib.oracle_matmul_i8_accumulate(m, n, k, _ptr(a), *_strides(a), int(a.dtype == np.int8), _ptr(b_nk), *_strides(b_nk),
                                             int(b_nk.dtype == np.int8), _ptr(cin_view),
                                             *(_strides(cin_view) if cin_view is not None else (0, 0)), _ptr(c), n, 1)
        return c


    # ---- the quantised form: 8-bit operands, int32 accumulate + int32 accumulator input, float output transform

    def quantize_rows(self, a_f32, scale, zero_point, signed=False):
        m, k = a_f32.shape
        out = np.empty((m, k), dtype=np.int8 if signed else np.uint8)
        self.lib.oracle_quantize_rows(m, k, _ptr(a_f32), *_strides(a_f32), float(scale), float(zero_point), _ptr(out), k, 1, int(signed))
        return out

    def quantize_rows_per_row(self, a_f32, multipliers, zero_point, signed=False):
        m, k = a_f32.shape
        out = np.empty((m, k), dtype=np.int8 if signed else np.uint8)
        multipliers = np.ascontiguousarray(multipliers, dtype=np.float32)
        self.lib.oracle_quantize_rows_per_row(m, k, _ptr(a_f32), *_strides(a_f32), _ptr(multipliers), float(zero_point), _ptr(out), k, 1,
                                              int(signed))
        return out

    def matmul_i8_dequant_rows(self, a, b_nk, cin, row_scale, column_scale, out_bf16=False):
        """int32 product plus the int32 accumulator input, then value * row_scale[row] * column_scale[col]."""
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.uint16 if out_bf16 else np.float32)
        cin_view, _ = _cin_view(cin, m, n)
        self.lib.oracle_matmul_i8_dequant_rows(m, n, k, _ptr(a), *_strides(a), int(a.dtype == np.int8), _ptr(b_nk), *_strides(b_nk),
                                               int(b_nk.dtype == np.int8), _ptr(cin_view),
                                               *(_strides(cin_view) if cin_view is not None else (0, 0)), _ptr(row_scale), _ptr(column_scale),
                                               _ptr(c), n, 1, int(out_bf16))
        return c

    def matmul_i8_dequant(self, a, b_nk, cin=None, alpha=1.0, scale=None, act=ACT_NONE, lo=0.0, hi=0.0, out_bf16=False):
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.uint16 if out_bf16 else np.float32)
        cin_view, _ = _cin_view(cin, m, n)
        self.lib.oracle_matmul_i8_dequant(m, n, k, _ptr(a), *_strides(a), int(a.dtype == np.int8), _ptr(b_nk), *_strides(b_nk),
                                          int(b_nk.dtype == np.int8), _ptr(cin_view),
                                          *(_strides(cin_view) if cin_view is not None else (0, 0)), float(alpha), _ptr(scale), int(act),
                                          float(lo), float(hi), _ptr(c), n, 1, int(out_bf16))
        return c


class Ref:
    """The reference's own ops::matmul.  ``Ref.load()`` returns None when unavailable here."""

    def __init__(self, lib: ctypes.CDLL) -> None:
        self.lib = lib
        lib.ref_available.restype = c_int
        lib.ref_matmul_bf16.argtypes = [_I64] * 3 + [_P, _I64, _P, _I64, _P, _I64, c_int, c_int]
        lib.ref_matmul_i8.argtypes = [_I64] * 3 + [_P, _I64, c_int, _P, _I64, c_int, _P, _I64, c_int]
        lib.ref_matmul_w8.argtypes = [_I64] * 3 + [_P, _I64, _P, _I64, _P, _P, _I64, c_int]
        lib.ref_matmul_f32_leaf.argtypes = [_I64] * 3 + [_P, _I64, _P, _I64, _P, _I64, c_int]
        _F = ctypes.c_float
        if hasattr(lib, "ref_matmul_bf16_fused"):
            lib.ref_matmul_bf16_fused.argtypes = [_I64] * 3 + [_P, _I64, _P, _I64, _P, _I64, _I64, _F, _P, c_int, _F, _F, _P, _I64, c_int]
            lib.ref_matmul_i8_accumulate.argtypes = [_I64] * 3 + [_P, _I64, _P, _I64, _P, _I64, _I64, _P, _I64]
        if hasattr(lib, "ref_matmul_bf16_batched"):
            lib.ref_matmul_bf16_batched.argtypes = [_I64] * 4 + [_P, _I64, _I64, _P, _I64, _I64, _P, _P, _I64, _I64]
        if hasattr(lib, "ref_matmul_quantized_per_row"):
            lib.ref_matmul_quantized_per_row.argtypes = [_I64] * 3 + [_P, _I64, _P, ctypes.c_int32, _P, _I64, _P, _P, _P, _P, _I64]
        if hasattr(lib, "ref_sdpa_bf16"):
            lib.ref_sdpa_bf16.argtypes = [_I64] * 4 + [_P] * 7 + [c_int, ctypes.c_float, _P]
        if hasattr(lib, "ref_sdpa_bf16_streaming"):
            lib.ref_sdpa_bf16_streaming.argtypes = [_I64] * 4 + [_P] * 7 + [c_int, ctypes.c_float, _P]
        if hasattr(lib, "ref_f16_widen"):
            lib.ref_f16_widen.argtypes = [_P, _P, _I64]
            lib.ref_f16_narrow.argtypes = [_P, _P, _I64]
        if hasattr(lib, "ref_matmul_quantized_u8s8"):
            lib.ref_matmul_quantized_u8s8.argtypes = [_I64] * 3 + [_P, _I64, _F, _F, _P, _I64, _P, _F, _P, _I64]
        if hasattr(lib, "ref_pack_b_compensated"):
            lib.ref_pack_b_compensated.argtypes = [_I64, _I64, _P, _I64, ctypes.c_int32, _P]

    def sdpa_bf16(self, q, k, v, scale, query_mask=None, key_mask=None, keep_mask=None, bias=None, causal=0, streaming=False):
        """The reference's own attention (materialized strategy, or streaming over key blocks of 128); the four optional
        operands come all together or not at all."""
        q, k, v = (np.ascontiguousarray(x) for x in (q, k, v))
        lq, dqk = q.shape
        lkv, dv = v.shape
        out = np.full((lq, dv), -99.0, dtype=np.float32)
        optional = [None if x is None else np.ascontiguousarray(x, dtype=t)
                    for x, t in ((query_mask, np.uint8), (key_mask, np.uint8), (keep_mask, np.uint8), (bias, np.float32))]
        door = self.lib.ref_sdpa_bf16_streaming if streaming else self.lib.ref_sdpa_bf16
        rc = door(lq, lkv, dqk, dv, _ptr(q), _ptr(k), _ptr(v), *[_ptr(x) for x in optional], int(causal), float(scale), _ptr(out))
        assert rc == 0, rc
        return out

    def f16_widen(self, bits: np.ndarray) -> np.ndarray:
        bits = np.ascontiguousarray(bits, dtype=np.uint16)
        out = np.empty(bits.shape, dtype=np.float32)
        self.lib.ref_f16_widen(_ptr(bits), _ptr(out), bits.size)
        return out

    def f16_narrow(self, values: np.ndarray) -> np.ndarray:
        values = np.ascontiguousarray(values, dtype=np.float32)
        out = np.empty(values.shape, dtype=np.uint16)
        self.lib.ref_f16_narrow(_ptr(values), _ptr(out), values.size)
        return out

    def matmul_bf16_batched(self, a3, b3, bias=None):
        """Rank-3 bf16 operands [B,M,K] x [B,N,K] -> f32 [B,M,N]; a leading stride may be 0 (np.broadcast_to views)."""
        batch, m, k = a3.shape
        n = b3.shape[1]
        c = np.empty((batch, m, n), dtype=np.float32)
        item = a3.itemsize
        assert a3.strides[2] == item and b3.strides[2] == item
        rc = self.lib.ref_matmul_bf16_batched(batch, m, n, k, _ptr(a3), a3.strides[0] // item, a3.strides[1] // item, _ptr(b3),
                                              b3.strides[0] // item, b3.strides[1] // item, _ptr(bias), _ptr(c), m * n, n)
        assert rc == 0
        return c

    def matmul_quantized_per_row(self, a_f32, multipliers, zero_point, b_nk, correction, row_scales, column_scales):
        """Per-token quantisation with the reference's named transforms; fp32 C."""
        m, k = a_f32.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.float32)
        padded = np.concatenate([np.asarray(column_scales, np.float32), np.zeros(64, np.float32)])
        multipliers = np.ascontiguousarray(multipliers, dtype=np.float32)
        row_scales = np.ascontiguousarray(row_scales, dtype=np.float32)
        rc = self.lib.ref_matmul_quantized_per_row(m, n, k, _ptr(a_f32), self._rows(a_f32), _ptr(multipliers), int(zero_point), _ptr(b_nk),
                                                   self._rows(b_nk), _ptr(correction), _ptr(row_scales), _ptr(padded), _ptr(c), n)
        assert rc == 0
        return c

    def matmul_quantized_u8s8(self, a_f32, a_scale, a_zero_point, b_nk, correction, dequant):
        """fp32 A quantised on load to u8, s8 B, int32 correction row, dequantising output transform, fp32 C."""
        m, k = a_f32.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.float32)
        rc = self.lib.ref_matmul_quantized_u8s8(m, n, k, _ptr(a_f32), self._rows(a_f32), float(a_scale), float(a_zero_point), _ptr(b_nk),
                                                self._rows(b_nk), _ptr(correction), float(dequant), _ptr(c), n)
        assert rc == 0
        return c

    def matmul_bf16_fused(self, a, b_nk, cin=None, alpha=1.0, scale=None, act=ACT_NONE, lo=0.0, hi=0.0, out_bf16=True):
        """The reference's explicit accumulate form with one composed output transform; `cin` float32 or None.
        `scale` needs 64 readable floats past n (the transform loads whole vectors)."""
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.uint16 if out_bf16 else np.float32)
        cin_view, kind = _cin_view(cin, m, n)
        assert kind == 0, "the reference driver takes an f32 accumulator input"
        padded = None if scale is None else np.concatenate([scale.astype(np.float32), np.zeros(64, np.float32)])
        rc = self.lib.ref_matmul_bf16_fused(m, n, k, _ptr(a), self._rows(a), _ptr(b_nk), self._rows(b_nk), _ptr(cin_view),
                                            *(_strides(cin_view) if cin_view is not None else (0, 0)), float(alpha), _ptr(padded), int(act),
                                            float(lo), float(hi), _ptr(c), n, int(out_bf16))
        assert rc == 0
        return c

    def matmul_i8_accumulate(self, a, b_nk, cin):
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.int32)
        cin_view, _ = _cin_view(cin, m, n)
        rc = self.lib.ref_matmul_i8_accumulate(m, n, k, _ptr(a), self._rows(a), _ptr(b_nk), self._rows(b_nk), _ptr(cin_view),
                                               *_strides(cin_view), _ptr(c), n)
        assert rc == 0
        return c

    @staticmethod
    def load() -> tuple["Ref | None", str]:
        build_oracle.build_ref()
        ok, why = build_oracle.ref_runnable_here()
        if not ok:
            return None, why
        try:
            lib = ctypes.CDLL(str(build_oracle.REF_LIB))
        except OSError as error:
            return None, f"cannot load reference library: {error}"
        ref = Ref(lib)
        if not lib.ref_available():
            return None, "the kernel refused AMX tile permission (arch_prctl)"
        return ref, ""

    @staticmethod
    def default_threads() -> int:
        return max(1, len(os.sched_getaffinity(0)))

    @staticmethod
    def _rows(array: np.ndarray) -> int:
        assert array.strides[1] == array.itemsize, "reference driver wants K-contiguous operands"
        return array.strides[0] // array.itemsize

    def matmul_bf16(self, a, b_nk, out_bf16=True, threads=1):
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.uint16 if out_bf16 else np.float32)
        rc = self.lib.ref_matmul_bf16(m, n, k, _ptr(a), self._rows(a), _ptr(b_nk), self._rows(b_nk), _ptr(c), n,
                                      int(out_bf16), threads)
        assert rc == 0
        return c

    def matmul_i8(self, a, b_nk, threads=1):
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.int32)
        rc = self.lib.ref_matmul_i8(m, n, k, _ptr(a), self._rows(a), int(a.dtype == np.int8), _ptr(b_nk),
                                    self._rows(b_nk), int(b_nk.dtype == np.int8), _ptr(c), n, threads)
        assert rc == 0
        return c

    def matmul_w8(self, a, w_nk, scale, threads=1):
        m, k = a.shape
        n = w_nk.shape[0]
        padded = np.zeros(n + 64, dtype=np.float32)
        padded[:n] = scale
        c = np.empty((m, n), dtype=np.uint16)
        rc = self.lib.ref_matmul_w8(m, n, k, _ptr(a), self._rows(a), _ptr(w_nk), self._rows(w_nk), _ptr(padded), _ptr(c),
                                    n, threads)
        assert rc == 0
        return c

    def pack_compensation(self, b_nk: np.ndarray, a_zero_point: int) -> np.ndarray:
        """The compensation row the reference's ops::matmul_pack_b_compensated emits for a signed 8-bit B[N,K]
        (ops/MatmulPack.h:28-35); its packed bytes, in the AMX tile layout, are dropped."""
        n, k = b_nk.shape
        out = np.full(n, 0x13579bdf, dtype=np.int32)
        rc = self.lib.ref_pack_b_compensated(n, k, _ptr(b_nk), self._rows(b_nk), int(a_zero_point), _ptr(out))
        assert rc == 0
        return out

    def matmul_f32_leaf(self, a, b_nk, threads=1):
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.float32)
        rc = self.lib.ref_matmul_f32_leaf(m, n, k, _ptr(a), self._rows(a), _ptr(b_nk), self._rows(b_nk), _ptr(c), n,
                                          threads)
        assert rc == 0
        return c
