"""ctypes view of the C ABI in ``include/vecops_b200/*.h``.

The host side of this project is C++ (as in vecops); Python appears only as the
test and benchmark harness, and it reaches the kernels through the same
``extern "C"`` entry points a vecops build would bind.  Loading fails loudly
when the library has not been built: there is no fallback path.
"""
from __future__ import annotations

import ctypes
from ctypes import (POINTER, Structure, Union, byref, c_char, c_char_p, c_int32, c_int64, c_size_t, c_uint16, c_uint32,
                    c_uint64, c_void_p, c_float)
from pathlib import Path

LIBRARY_PATH = Path(__file__).resolve().parent / "lib" / "libvecops_b200.so"

# VecopsStatusCode
OK, INVALID_ARGUMENT, NOT_APPLICABLE, NOT_FOUND, ABI_MISMATCH, LOAD_ERROR, EXECUTION_ERROR, INTERNAL_ERROR = range(8)
STATUS_NAMES = ["OK", "INVALID_ARGUMENT", "NOT_APPLICABLE", "NOT_FOUND", "ABI_MISMATCH", "LOAD_ERROR", "EXECUTION_ERROR",
                "INTERNAL_ERROR"]
# VecopsDType
DTYPE_I8, DTYPE_U8, DTYPE_I32, DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 2, 3, 6, 10, 11, 12
DEVICE_CPU, DEVICE_CUDA = 1, 2
VALUE_NONE, VALUE_TENSOR, VALUE_SCALAR = 0, 1, 2
TENSOR_READ, TENSOR_WRITE = 1, 2
# VecopsB200MatmulKernel
KERNEL_AUTO, KERNEL_GENERIC, KERNEL_F32_SIMT, KERNEL_BF16_TCGEN05, KERNEL_I8_TCGEN05, KERNEL_W8_SMALL_M, KERNEL_W8_TCGEN05, KERNEL_F32_TF32X3 = range(8)
MATMUL_FLAG_ASYNC = 1
CONTEXT_FLAG_ASYNC = 1 << 32


class VecopsError(Structure):
    _fields_ = [("struct_size", c_uint32), ("code", c_int32), ("message", c_void_p), ("message_capacity", c_size_t),
                ("message_required", c_size_t)]


class VecopsTensorView(Structure):
    _fields_ = [("struct_size", c_uint32), ("data", c_void_p), ("byte_offset", c_uint64), ("device_type", c_uint32),
                ("device_index", c_int32), ("dtype", c_uint32), ("rank", c_uint32), ("sizes", POINTER(c_int64)),
                ("strides", POINTER(c_int64)), ("flags", c_uint64)]


class VecopsScalarStorage(Union):
    _fields_ = [("i64", c_int64), ("u64", c_uint64), ("f64", ctypes.c_double)]


class VecopsScalar(Structure):
    _fields_ = [("struct_size", c_uint32), ("dtype", c_uint32), ("value", VecopsScalarStorage)]


class _ValueUnion(Union):
    _fields_ = [("tensor", VecopsTensorView), ("scalar", VecopsScalar)]


class VecopsValue(Structure):
    _fields_ = [("struct_size", c_uint32), ("kind", c_uint32), ("value", _ValueUnion)]


class VecopsExecutionContext(Structure):
    _fields_ = [("struct_size", c_uint32), ("requested_threads", c_uint32), ("stream", c_void_p), ("user_data", c_void_p),
                ("flags", c_uint64), ("workspace_provider", c_void_p), ("thread_pool", c_void_p),
                ("allocation_observer", c_void_p)]


class VecopsCall(Structure):
    _fields_ = [("struct_size", c_uint32), ("num_values", c_uint32), ("values", POINTER(VecopsValue)),
                ("workspace", c_void_p), ("workspace_size", c_uint64), ("context", POINTER(VecopsExecutionContext))]


class VecopsB200Matmul(Structure):
    _fields_ = [("struct_size", c_uint32), ("kernel", c_uint32), ("m", c_int64), ("n", c_int64), ("k", c_int64),
                ("a", c_void_p), ("a_stride_m", c_int64), ("a_stride_k", c_int64),
                ("b", c_void_p), ("b_stride_n", c_int64), ("b_stride_k", c_int64),
                ("c", c_void_p), ("c_stride_m", c_int64), ("c_stride_n", c_int64),
                ("column_scale", c_void_p), ("workspace", c_void_p), ("workspace_size", c_uint64), ("stream", c_void_p),
                ("a_dtype", c_uint32), ("b_dtype", c_uint32), ("c_dtype", c_uint32), ("device_index", c_int32),
                ("flags", c_uint32), ("reserved", c_uint32)]


class VecopsB200Epilogue(Structure):
    _fields_ = [("struct_size", c_uint32), ("activation", c_uint32), ("cin", c_void_p), ("cin_stride_m", c_int64),
                ("cin_stride_n", c_int64), ("cin_dtype", c_uint32), ("alpha", c_float), ("clamp_lo", c_float),
                ("clamp_hi", c_float), ("reserved", c_uint32), ("row_scale", c_void_p)]


ACTIVATION_NONE, ACTIVATION_RELU, ACTIVATION_SIGMOID, ACTIVATION_SILU, ACTIVATION_CLAMP = range(5)


class VecopsB200Batch(Structure):
    _fields_ = [("struct_size", c_uint32), ("reserved", c_uint32), ("count", c_int64), ("a_stride_b", c_int64), ("b_stride_b", c_int64),
                ("c_stride_b", c_int64), ("cin_stride_b", c_int64)]


class VecopsB200Pack(Structure):
    _fields_ = [("struct_size", c_uint32), ("operand", c_uint32), ("rows", c_int64), ("k", c_int64), ("src", c_void_p),
                ("src_stride_row", c_int64), ("src_stride_k", c_int64), ("src_dtype", c_uint32), ("dst_dtype", c_uint32), ("dst", c_void_p),
                ("dst_size", c_uint64), ("device_index", c_int32), ("flags", c_uint32), ("stream", c_void_p)]


class VecopsB200Attention(Structure):
    _fields_ = [("struct_size", c_uint32), ("causal", c_uint32), ("lq", c_int64), ("lkv", c_int64), ("dqk", c_int64), ("dv", c_int64),
                ("q", c_void_p), ("q_stride_row", c_int64), ("q_stride_col", c_int64), ("k", c_void_p), ("k_stride_row", c_int64),
                ("k_stride_col", c_int64), ("v", c_void_p), ("v_stride_row", c_int64), ("v_stride_col", c_int64), ("out", c_void_p),
                ("out_stride_row", c_int64), ("out_stride_col", c_int64), ("qkv_dtype", c_uint32), ("out_dtype", c_uint32),
                ("query_mask", c_void_p), ("key_mask", c_void_p), ("keep_mask", c_void_p), ("keep_stride_row", c_int64),
                ("keep_stride_col", c_int64), ("bias", c_void_p), ("bias_stride_row", c_int64), ("bias_stride_col", c_int64),
                ("scale", c_float), ("flags", c_uint32), ("workspace", c_void_p), ("workspace_size", c_uint64), ("stream", c_void_p),
                ("device_index", c_int32), ("strategy", c_uint32), ("heads", c_int64), ("q_stride_head", c_int64), ("k_stride_head", c_int64),
                ("v_stride_head", c_int64), ("out_stride_head", c_int64), ("query_mask_stride_head", c_int64),
                ("key_mask_stride_head", c_int64), ("keep_stride_head", c_int64), ("bias_stride_head", c_int64)]


CAUSAL_NONE, CAUSAL_TOP_LEFT, CAUSAL_BOTTOM_RIGHT = 0, 1, 2
SDPA_AUTOMATIC, SDPA_MATERIALIZED, SDPA_STREAMING = 0, 1, 2  # VecopsB200SdpaStrategy


class VecopsB200Gather(Structure):
    _fields_ = [("struct_size", c_uint32), ("world", c_int32), ("c", POINTER(c_void_p)), ("n_total", c_int64), ("ldc", c_int64),
                ("col0", c_int64), ("flags", c_uint32), ("reserved", c_uint32)]


PUSH_KERNEL, PUSH_COPY_ENGINE = 0, 1
GATHER_MULTICAST = 1


class VecopsB200DeviceInfo(Structure):
    _fields_ = [("struct_size", c_uint32), ("sm_major", c_int32), ("sm_minor", c_int32), ("sm_count", c_int32),
                ("l2_bytes", c_uint64), ("hbm_bytes", c_uint64), ("smem_per_block_optin", c_uint64), ("name", c_char * 64)]


class VecopsB200Error(RuntimeError):
    def __init__(self, code: int, message: str) -> None:
        super().__init__(f"{STATUS_NAMES[code] if 0 <= code < len(STATUS_NAMES) else code}: {message}")
        self.code = code
        self.message = message


class ErrorBuffer:
    """Caller-owned VecopsError with a 1 KiB message buffer (the size vecops' runtime uses)."""

    def __init__(self) -> None:
        self.text = ctypes.create_string_buffer(1024)
        self.record = VecopsError(ctypes.sizeof(VecopsError), 0, ctypes.cast(self.text, c_void_p), 1024, 0)

    def raise_for(self, code: int) -> None:
        if code != OK:
            raise VecopsB200Error(code, self.text.value.decode(errors="replace"))


_LIB = None


def library() -> ctypes.CDLL:
    """Load libvecops_b200.so once; raise if it has not been built."""
    global _LIB
    if _LIB is None:
        if not LIBRARY_PATH.exists():
            raise RuntimeError(f"{LIBRARY_PATH} is missing: build it with `python -m vecops_b200._build` "
                               "(there is no fallback path)")
        lib = ctypes.CDLL(str(LIBRARY_PATH))
        e = POINTER(VecopsError)
        lib.vecops_b200_matmul_select.argtypes = [POINTER(VecopsB200Matmul), POINTER(c_uint32), e]
        lib.vecops_b200_matmul_workspace.argtypes = [POINTER(VecopsB200Matmul), POINTER(c_uint64), e]
        lib.vecops_b200_matmul_run.argtypes = [POINTER(VecopsB200Matmul), e]
        lib.vecops_b200_matmul_run_fused.argtypes = [POINTER(VecopsB200Matmul), POINTER(VecopsB200Epilogue), e]
        lib.vecops_b200_matmul_run_batched.argtypes = [POINTER(VecopsB200Matmul), POINTER(VecopsB200Batch), POINTER(VecopsB200Epilogue), e]
        lib.vecops_b200_quantize_rows.argtypes = [c_void_p, c_uint32, c_int64, c_int64, c_void_p, c_uint32, c_int64, c_int64, c_int64, c_float,
                                                  c_float, c_void_p, e]
        lib.vecops_b200_quantize_rows_per_row.argtypes = [c_void_p, c_uint32, c_int64, c_int64, c_void_p, c_uint32, c_int64, c_int64, c_int64,
                                                          c_void_p, c_float, c_void_p, e]
        lib.vecops_b200_column_correction.argtypes = [c_void_p, c_uint32, c_int64, c_int64, c_int64, c_int32, c_void_p, c_void_p, e]
        lib.vecops_b200_matmul_packed_layout.argtypes = [c_uint32, c_int64, c_int64, POINTER(c_int64), POINTER(c_uint64), e]
        lib.vecops_b200_matmul_pack.argtypes = [POINTER(VecopsB200Pack), e]
        lib.vecops_b200_matmul_pack_b_compensated.argtypes = [POINTER(VecopsB200Pack), c_int32, c_void_p, e]
        lib.vecops_b200_sdpa_workspace.argtypes = [POINTER(VecopsB200Attention), POINTER(c_uint64), e]
        lib.vecops_b200_sdpa_run.argtypes = [POINTER(VecopsB200Attention), e]
        lib.vecops_b200_sdpa_plan.argtypes = [POINTER(VecopsB200Attention), POINTER(c_uint32), POINTER(c_uint32), e]
        lib.vecops_b200_matmul_allgather_run.argtypes = [POINTER(VecopsB200Matmul), POINTER(VecopsB200Gather), e]
        lib.vecops_b200_kernel_name.argtypes = [c_uint32]
        lib.vecops_b200_kernel_name.restype = c_char_p
        lib.vecops_b200_device_count.restype = c_int32
        lib.vecops_b200_device_info.argtypes = [c_int32, POINTER(VecopsB200DeviceInfo), e]
        lib.vecops_b200_launch_count.restype = c_uint64
        lib.vecops_b200_stream_synchronize.argtypes = [c_void_p, e]
        lib.vecops_b200_take_device_status.argtypes = [c_int32, POINTER(c_uint32), e]
        lib.vecops_b200_place_columns.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                                                  c_uint32, c_void_p, e]
        lib.vecops_b200_push_columns.argtypes = [c_void_p, POINTER(c_void_p), c_int32, c_int64, c_int64, c_int64, c_int64,
                                                 c_uint32, c_uint32, c_void_p, e]
        _LIB = lib
    return _LIB
