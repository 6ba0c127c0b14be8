"""Host-only checks of the C ABI: the library loads without a GPU, exports every
declared symbol, and the dispatch rules / argument checks behave."""
import ctypes
import re
from ctypes import byref, c_uint32, c_uint64
from pathlib import Path

import pytest
import torch

import vecops_b200
from vecops_b200 import capi, harness

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    names = set()
    for header in (ROOT / "include" / "vecops_b200").glob("*.h"):
        text = header.read_text()
        names.update(re.findall(r"VECOPS_B200_EXPORT[^;{]*?\b(vecops_[a-z0-9_]+)\s*\(", text, flags=re.S))
    return names


def test_library_exports_every_declared_symbol(library):
    names = declared_symbols()
    assert {"vecops_b200_matmul_run", "vecops_b200_matmul_select", "vecops_b200_matmul_workspace",
            "vecops_operator_bridge_invoke_v1", "vecops_b200_matmul_operator"} <= names
    for name in sorted(names):
        assert hasattr(library, name), f"{name} is declared in include/ but not exported"


def test_record_sizes_match_the_c_layout():
    # 64-bit layouts of the vecops records the artifact exchanges with its caller
    assert ctypes.sizeof(capi.VecopsError) == 32
    assert ctypes.sizeof(capi.VecopsTensorView) == 64
    assert ctypes.sizeof(capi.VecopsScalar) == 16
    assert ctypes.sizeof(capi.VecopsValue) == 72
    assert ctypes.sizeof(capi.VecopsExecutionContext) == 56
    assert ctypes.sizeof(capi.VecopsCall) == 40


def _problem(m, n, k, a_dtype, b_dtype, c_dtype, **kw):
    a = torch.empty((m, k), dtype=a_dtype)
    b = torch.empty((n, k), dtype=b_dtype)
    c = torch.empty((m, n), dtype=c_dtype)
    keep = (a, b, c)
    p = vecops_b200.matmul_problem(a, b, c, **kw)
    p._keep = keep
    return p


def _name(kernel):
    return capi.library().vecops_b200_kernel_name(kernel).decode()


def test_dispatch_rules_pick_the_tensor_core_kernels_for_the_benchmark_shapes(library):
    assert _name(vecops_b200.select_kernel(_problem(4096, 4096, 4096, torch.bfloat16, torch.bfloat16, torch.bfloat16))) == "bf16_tcgen05"
    assert _name(vecops_b200.select_kernel(_problem(4096, 14336, 4096, torch.int8, torch.int8, torch.int32))) == "i8_tcgen05"
    assert _name(vecops_b200.select_kernel(_problem(4096, 256, 512, torch.uint8, torch.int8, torch.int32))) == "i8_tcgen05"
    for m in (1, 16):
        assert _name(vecops_b200.select_kernel(_problem(m, 14336, 4096, torch.bfloat16, torch.int8, torch.bfloat16))) == "w8_small_m"
    assert _name(vecops_b200.select_kernel(_problem(128, 14336, 4096, torch.bfloat16, torch.int8, torch.bfloat16))) == "w8_tcgen05"
    # fp32: the split-operand tensor-core route is what the rules prefer for a product this size (a launch takes it when the
    # caller brings its scratch, the FMA kernel otherwise); small products stay on the FMA kernel
    assert _name(vecops_b200.select_kernel(_problem(1024, 1024, 1024, torch.float32, torch.float32, torch.float32))) == "f32_tf32x3"
    assert _name(vecops_b200.select_kernel(_problem(128, 1024, 1024, torch.float32, torch.float32, torch.float32))) == "f32_simt"
    assert harness.workspace_bytes(_problem(1024, 1024, 1024, torch.float32, torch.float32, torch.float32)) >= 2 * 1024 * 3 * 1024 * 4


def test_dispatch_rules_route_ragged_and_tiny_problems_to_the_strided_kernel(library):
    # K = 35 bf16 rows are 70 bytes apart: not addressable by TMA
    assert _name(vecops_b200.select_kernel(_problem(16, 16, 35, torch.bfloat16, torch.bfloat16, torch.float32))) == "generic"
    # tiny outputs (area rule), as vecops sends them to its small-vector leaves
    assert _name(vecops_b200.select_kernel(_problem(4, 8, 4096, torch.bfloat16, torch.bfloat16, torch.bfloat16))) == "generic"
    # int32 wrap semantic: very long K stays on the wrapping integer kernel
    assert _name(vecops_b200.select_kernel(_problem(256, 256, 262144, torch.int8, torch.int8, torch.int32))) == "generic"
    # weight-only with K not a multiple of 32
    assert _name(vecops_b200.select_kernel(_problem(4, 64, 72, torch.bfloat16, torch.int8, torch.bfloat16))) == "generic"


def test_forced_kernel_that_cannot_serve_is_not_applicable(library):
    p = _problem(16, 16, 35, torch.bfloat16, torch.bfloat16, torch.float32, kernel=capi.KERNEL_BF16_TCGEN05)
    with pytest.raises(capi.VecopsB200Error) as info:
        vecops_b200.select_kernel(p)
    assert info.value.code == capi.NOT_APPLICABLE


def test_unsupported_dtype_row_is_invalid_argument(library):
    p = _problem(8, 8, 8, torch.float32, torch.bfloat16, torch.float32)
    with pytest.raises(capi.VecopsB200Error) as info:
        vecops_b200.select_kernel(p)
    assert info.value.code == capi.INVALID_ARGUMENT


def test_short_record_is_an_abi_mismatch(library):
    p = _problem(8, 8, 8, torch.float32, torch.float32, torch.float32)
    p.struct_size = 16
    with pytest.raises(capi.VecopsB200Error) as info:
        vecops_b200.select_kernel(p)
    assert info.value.code == capi.ABI_MISMATCH


def test_error_text_is_truncated_to_the_callers_buffer(library):
    p = _problem(8, 8, 8, torch.float32, torch.bfloat16, torch.float32)
    text = ctypes.create_string_buffer(12)
    record = capi.VecopsError(ctypes.sizeof(capi.VecopsError), 0, ctypes.cast(text, ctypes.c_void_p), 12, 0)
    out = c_uint32(0)
    rc = library.vecops_b200_matmul_select(byref(p), byref(out), byref(record))
    assert rc == capi.INVALID_ARGUMENT and record.code == capi.INVALID_ARGUMENT
    assert len(text.value) == 11 and record.message_required > 12


def test_workspace_query_is_pure_host_logic(library):
    p = _problem(16, 14336, 4096, torch.bfloat16, torch.int8, torch.bfloat16)
    assert harness.workspace_bytes(p) == 0
    # the weight-only tensor-core kernel cuts each of its 56 tiles of 256 weight rows in two along K (112 CTAs on 148 SMs)
    # and the slices meet in device scratch: one [128 x 256] 32-bit accumulator and four flags per slice
    p = _problem(128, 14336, 4096, torch.bfloat16, torch.int8, torch.bfloat16)
    assert harness.workspace_bytes(p) == 112 * (128 * 256 * 4 + 4 * 8)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_run_without_a_gpu_fails_loudly_instead_of_falling_back(library):
    assert library.vecops_b200_device_count() == 0
    p = _problem(64, 64, 64, torch.float32, torch.float32, torch.float32)
    with pytest.raises(capi.VecopsB200Error) as info:
        harness.run(p)
    assert info.value.code == capi.EXECUTION_ERROR
    assert "no CPU fallback" in info.value.message


def test_torch_operator_library_registers_its_schemas():
    # host-only: the library loads without a GPU, the three operators exist, and a CPU tensor is refused (no CPU path)
    import pytest
    import torch

    from vecops_b200 import _build, torch_ops
    _build.build_torch_bridge()
    torch_ops.load()
    schema = str(torch.ops.vecops_b200.matmul.default._schema)
    assert "Tensor? column_scale=None" in schema and "Tensor? cin=None" in schema
    assert "Tensor(a!) c" in str(torch.ops.vecops_b200.matmul_out.default._schema)
    assert "int causal=0" in str(torch.ops.vecops_b200.sdpa.default._schema)
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.vecops_b200.matmul(torch.zeros(4, 4), torch.zeros(4, 4))


def test_ctypes_records_match_the_header(tmp_path):
    # the header compiled by gcc is the authority: sizes and the offsets of late fields of every record the Python binding mirrors
    import subprocess
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    records = {"VecopsB200Matmul": "reserved", "VecopsB200Epilogue": "row_scale", "VecopsB200Batch": "cin_stride_b", "VecopsB200Pack": "stream",
               "VecopsB200Attention": "bias_stride_head", "VecopsB200Gather": "flags"}
    lines = "".join(f'  printf("{name} %zu %zu\\n", sizeof({name}), offsetof({name}, {field}));\n' for name, field in records.items())
    source = tmp_path / "sizes.c"
    source.write_text('#include <stddef.h>\n#include <stdio.h>\n#include "vecops_b200/matmul_cuda.h"\nint main(void) {\n' + lines + "  return 0;\n}\n")
    binary = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c11", f"-I{root / 'include'}", str(source), "-o", str(binary)], check=True)
    out = subprocess.run([str(binary)], check=True, capture_output=True, text=True).stdout.split("\n")
    for line in filter(None, out):
        name, size, offset = line.split()
        record = getattr(capi, name)
        assert ctypes.sizeof(record) == int(size), name
        assert getattr(record, records[name]).offset == int(offset), name


def _abi_probe_source(headers: list[str], records: dict[str, list[str]], constants: list[str]) -> str:
    lines = ["#include <stddef.h>", "#include <stdio.h>", *[f'#include "{h}"' for h in headers], "int main(void) {"]
    for name, fields in records.items():
        lines.append(f'  printf("{name} size %zu\\n", sizeof({name}));')
        lines += [f'  printf("{name}.{field} %zu\\n", offsetof({name}, {field}));' for field in fields]
    lines += [f'  printf("{c} %lld\\n", (long long)({c}));' for c in constants]
    return "\n".join(lines + ["  return 0;", "}", ""])


def test_abi_records_equal_the_reference_headers(tmp_path):
    """With the reference checkout at hand, the same probe - sizeof and offsetof of every field of every ABI record, and the
    value of every enumerator - is compiled against this repository's headers and against the reference's own
    (runtime/CallAbi.h, KernelAbi.h, OperatorBridgeAbi.h): the two printouts must be equal line for line."""
    import re
    import subprocess
    from pathlib import Path

    from oracle import build_oracle
    reference = build_oracle.REFERENCE_ROOT / "include"
    if not (reference / "vecops" / "runtime" / "CallAbi.h").exists():
        pytest.skip("no reference checkout (set VECOPS_REFERENCE_ROOT)")
    root = Path(__file__).resolve().parents[1]
    ours = ["vecops_b200/call_abi.h", "vecops_b200/kernel_abi.h", "vecops_b200/operator_bridge.h"]
    theirs = ["vecops/runtime/CallAbi.h", "vecops/runtime/KernelAbi.h", "vecops/runtime/OperatorBridgeAbi.h"]
    text = "".join((root / "include" / h).read_text() for h in ours)
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    records: dict[str, list[str]] = {}
    for match in re.finditer(r"typedef (?:struct|union) (Vecops\w+) \{(.*?)\n\} \1;", text, flags=re.S):
        body = re.sub(r"union \{(.*?)\} (\w+);", lambda m: f"int {m.group(2)};" + "".join(
            f"int {m.group(2)}.{inner};" for inner in re.findall(r"(\w+)\s*;", m.group(1))), match.group(2), flags=re.S)
        records[match.group(1)] = re.findall(r"([\w.]+)\s*(?:\[\w*\])?;", body)
    constants = [c for c in re.findall(r"\b(VECOPS_[A-Z0-9_]+)\s*=", text)]
    constants += ["VECOPS_KERNEL_ABI_VERSION_MAJOR", "VECOPS_KERNEL_ABI_VERSION_MINOR"]
    assert len(records) >= 12 and all(records.values()) and len(constants) >= 30
    assert {"VecopsCall", "VecopsValue", "VecopsTensorView", "VecopsExecutionContext", "VecopsError", "VecopsKernelDescriptorV1",
            "VecopsParameterDescriptor", "VecopsSpecializationArgument"} <= set(records)
    assert "value.tensor" in records["VecopsValue"]
    outputs = []
    for tag, headers, include in (("ours", ours, root / "include"), ("reference", theirs, reference)):
        source = tmp_path / f"probe_{tag}.c"
        source.write_text(_abi_probe_source(headers, records, constants))
        binary = tmp_path / f"probe_{tag}"
        subprocess.run(["gcc", "-std=c11", f"-I{include}", str(source), "-o", str(binary)], check=True)
        outputs.append(subprocess.run([str(binary)], check=True, capture_output=True, text=True).stdout.splitlines())
    assert len(outputs[0]) > 100
    assert outputs[0] == outputs[1]


def _frame(shapes_dtypes, base_address):
    """A VecopsCall over fake CUDA tensors (binding and validation never touch the storage): [(shape, dtype code, writable)]."""
    keep, values = [], []
    for index, (shape, dtype, writable) in enumerate(shapes_dtypes):
        sizes = (ctypes.c_int64 * len(shape))(*shape)
        contiguous = [1] * len(shape)
        for d in range(len(shape) - 2, -1, -1):
            contiguous[d] = contiguous[d + 1] * shape[d + 1]
        strides = (ctypes.c_int64 * len(shape))(*contiguous)
        keep += [sizes, strides]
        v = capi.VecopsValue()
        v.struct_size = ctypes.sizeof(capi.VecopsValue)
        v.kind = capi.VALUE_TENSOR
        t = v.value.tensor
        t.struct_size = ctypes.sizeof(capi.VecopsTensorView)
        t.data, t.byte_offset = base_address + (index << 24), 0
        t.device_type, t.device_index = capi.DEVICE_CUDA, 0
        t.dtype, t.rank, t.sizes, t.strides = dtype, len(shape), sizes, strides
        t.flags = capi.TENSOR_READ | (capi.TENSOR_WRITE if writable else 0)
        values.append(v)
    array = (capi.VecopsValue * len(values))(*values)
    frame = capi.VecopsCall(ctypes.sizeof(capi.VecopsCall), len(values), array, None, 0, None)
    keep.append(array)
    return frame, keep


@pytest.mark.skipif(torch.cuda.is_available(), reason="counts bridge paths on a host where every run ends in 'no device'")
def test_bridge_re_enters_a_prepared_call_on_an_identical_signature(library):
    """vecops' framework bridge keeps eight call signatures per thread and re-enters a resolved executable on a match
    (docs/Runtime.md:195-206); so does this bridge.  Without a GPU every call gets as far as the artifact's run callback
    and fails there - after binding, validation and resolution, which is all this test is about."""
    library.vecops_b200_matmul_operator.restype = ctypes.c_uint64
    library.vecops_operator_bridge_invoke_v1.argtypes = [ctypes.c_uint64, ctypes.POINTER(capi.VecopsCall), ctypes.c_uint32, ctypes.c_void_p,
                                                         ctypes.POINTER(capi.VecopsError)]
    library.vecops_b200_bridge_counters.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]
    library.vecops_b200_bridge_counters.restype = None
    handle = library.vecops_b200_matmul_operator()

    def counters():
        slow, prepared = ctypes.c_uint64(0), ctypes.c_uint64(0)
        library.vecops_b200_bridge_counters(byref(slow), byref(prepared))
        return slow.value, prepared.value

    def invoke(frame):
        error = capi.ErrorBuffer()
        return library.vecops_operator_bridge_invoke_v1(handle, byref(frame), 0, None, byref(error.record)), error.text.value

    decode = [((16, 4096), capi.DTYPE_BF16, False), ((14336, 4096), capi.DTYPE_I8, False), ((16, 14336), capi.DTYPE_BF16, True),
              ((14336,), capi.DTYPE_F32, False)]
    frame, keep = _frame(decode, 0x7f0000000000)
    slow0, prepared0 = counters()
    rc, text = invoke(frame)
    assert rc == capi.EXECUTION_ERROR and b"no CPU fallback" in text
    assert counters() == (slow0 + 1, prepared0)
    # the same signature at other addresses: no bind, no validation, no dispatch - straight to the executable
    other, keep2 = _frame(decode, 0x7e0000000000)
    for step in range(3):
        rc, text = invoke(other if step % 2 else frame)
        assert rc == capi.EXECUTION_ERROR and b"no CPU fallback" in text
    assert counters() == (slow0 + 1, prepared0 + 3)
    # another M is another signature (sizes are part of it), and so is an operand that is no longer 16-byte aligned
    longer, keep3 = _frame([((17, 4096), capi.DTYPE_BF16, False), decode[1], ((17, 14336), capi.DTYPE_BF16, True), decode[3]], 0x7f0000000000)
    invoke(longer)
    assert counters() == (slow0 + 2, prepared0 + 3)
    shifted, keep4 = _frame(decode, 0x7f0000000008)
    invoke(shifted)
    assert counters() == (slow0 + 3, prepared0 + 3)
    # a call the slow path refuses is not remembered: it is refused again, in words, by the slow path
    bad, keep5 = _frame([((16, 4096), capi.DTYPE_BF16, False), ((14336, 4000), capi.DTYPE_I8, False), ((16, 14336), capi.DTYPE_BF16, True)], 0x7f0000000000)
    for _ in range(2):
        rc, text = invoke(bad)
        assert rc != capi.OK and rc != capi.EXECUTION_ERROR
    assert counters() == (slow0 + 5, prepared0 + 3)
    # nine signatures push the first out of the thread's eight slots
    for m in range(1, 9):
        extra, _keep = _frame([((m, 256), capi.DTYPE_F32, False), ((64, 256), capi.DTYPE_F32, False), ((m, 64), capi.DTYPE_F32, True)], 0x7f0000000000)
        invoke(extra)
    slow1, prepared1 = counters()
    invoke(frame)
    assert counters() == (slow1 + 1, prepared1)


def test_caller_operators_bind_and_fail_loudly_without_a_gpu(library):
    """The operators either side of the matmul path (rank-3 matmul, attention, the per-row quantiser) are reachable through
    the bridge: handles exist, frames bind and resolve on the host, and a frame of the wrong shape names its fault."""
    library.vecops_b200_caller_operator.restype = ctypes.c_uint64
    library.vecops_b200_caller_operator.argtypes = [ctypes.c_uint32]
    library.vecops_operator_bridge_invoke_v1.argtypes = [ctypes.c_uint64, ctypes.POINTER(capi.VecopsCall), ctypes.c_uint32, ctypes.c_void_p,
                                                         ctypes.POINTER(capi.VecopsError)]
    library.vecops_b200_operator_resolve.argtypes = [ctypes.c_uint64, ctypes.POINTER(capi.VecopsCall), ctypes.c_char_p, ctypes.c_size_t,
                                                     ctypes.POINTER(capi.VecopsError)]
    handles = [library.vecops_b200_caller_operator(i) for i in range(3)]
    assert all(handles) and len(set(handles)) == 3 and library.vecops_b200_caller_operator(7) == 0
    batched = handles[0]
    frame, keep = _frame([((3, 16, 64), capi.DTYPE_BF16, False), ((3, 32, 64), capi.DTYPE_BF16, False), ((3, 16, 32), capi.DTYPE_F32, True)],
                         0x7f0000000000)
    key = ctypes.create_string_buffer(256)
    error = capi.ErrorBuffer()
    assert library.vecops_b200_operator_resolve(batched, byref(frame), key, 256, byref(error.record)) == capi.OK, error.text.value
    assert key.value.decode().startswith("vecops::matmul_batched;TA=bf16;TB=bf16;TC=f32")
    if not torch.cuda.is_available():
        rc = library.vecops_operator_bridge_invoke_v1(batched, byref(frame), 0, None, byref(error.record))
        assert rc == capi.EXECUTION_ERROR and b"no CPU fallback" in error.text.value
    # extents that disagree are named, and a rank-2 frame belongs to the plain matmul operator
    wrong, keep2 = _frame([((3, 16, 64), capi.DTYPE_BF16, False), ((3, 32, 48), capi.DTYPE_BF16, False), ((3, 16, 32), capi.DTYPE_F32, True)],
                          0x7f0000000000)
    error = capi.ErrorBuffer()
    assert library.vecops_operator_bridge_invoke_v1(batched, byref(wrong), 0, None, byref(error.record)) != capi.OK
    flat, keep3 = _frame([((16, 64), capi.DTYPE_BF16, False), ((32, 64), capi.DTYPE_BF16, False), ((16, 32), capi.DTYPE_F32, True)], 0x7f0000000000)
    assert library.vecops_operator_bridge_invoke_v1(batched, byref(flat), 0, None, byref(capi.ErrorBuffer().record)) != capi.OK


def test_push_columns_checks_its_arguments_and_fails_loudly_without_a_gpu(library):
    # argument checks come first and need no device; a well-formed push on a box without a GPU is an error, never a host copy
    addresses = (ctypes.c_void_p * 2)(0x7f0000100000, 0x7f0000200000)
    source = ctypes.c_void_p(0x7f0000000000)

    def push(count=2, ld=1024, col0=256, rows=64, cols=256, elem=2, route=capi.PUSH_KERNEL, dst=addresses):
        error = capi.ErrorBuffer()
        return library.vecops_b200_push_columns(source, dst, count, ld, col0, rows, cols, elem, route, None, byref(error.record)), error.text.value

    assert push(count=9)[0] == capi.INVALID_ARGUMENT
    assert push(col0=900)[0] == capi.INVALID_ARGUMENT            # the slab would leave the row
    assert push(route=5)[0] == capi.INVALID_ARGUMENT
    assert push(dst=(ctypes.c_void_p * 2)(0x7f0000100000, 0x7f0000000000))[0] == capi.INVALID_ARGUMENT  # the source among the destinations
    assert push(rows=0)[0] == capi.OK
    if library.vecops_b200_device_count() == 0:
        for route in (capi.PUSH_KERNEL, capi.PUSH_COPY_ENGINE):
            rc, text = push(route=route)
            assert rc == capi.EXECUTION_ERROR and b"no CPU fallback" in text
