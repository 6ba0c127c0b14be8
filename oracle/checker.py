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


class Ref:
    """The reference's own ops::matmul.  ``Ref.load()`` returns None when unavailable here."""

    def __init__(self, lib: ctypes.CDLL) -> None:
        self.lib = lib
        lib.ref_available.restype = c_int
        lib.ref_matmul_bf16.argtypes = [_I64] * 3 + [_P, _I64, _P, _I64, _P, _I64, c_int, c_int]
        lib.ref_matmul_i8.argtypes = [_I64] * 3 + [_P, _I64, c_int, _P, _I64, c_int, _P, _I64, c_int]
        lib.ref_matmul_w8.argtypes = [_I64] * 3 + [_P, _I64, _P, _I64, _P, _P, _I64, c_int]
        lib.ref_matmul_f32_leaf.argtypes = [_I64] * 3 + [_P, _I64, _P, _I64, _P, _I64, c_int]

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

    def matmul_f32_leaf(self, a, b_nk, threads=1):
        m, k = a.shape
        n = b_nk.shape[0]
        c = np.empty((m, n), dtype=np.float32)
        rc = self.lib.ref_matmul_f32_leaf(m, n, k, _ptr(a), self._rows(a), _ptr(b_nk), self._rows(b_nk), _ptr(c), n,
                                          threads)
        assert rc == 0
        return c
