"""Build recipes for the checker libraries (test infrastructure, not product code).

* ``liboracle.so``  - the C restatement in ``matmul_oracle.c`` (always built).
* ``_ref/libvecops_ref.so`` - the reference's own CPU matmul, compiled from the
  reference checkout where it lies (only when that checkout is present; the
  prebuilt file travels with the repository snapshot otherwise).  The recipe is
  the reference's compile line for header consumers (src/CMakeLists.txt:14-32:
  C++20, both include roots, -Wno-ignored-attributes) without its CMake build.

Run ``python oracle/build_oracle.py`` to (re)build both.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
# the reference checkout: $VECOPS_REFERENCE_ROOT, else a directory named "reference" beside this repository
REFERENCE_ROOT = Path(os.environ.get("VECOPS_REFERENCE_ROOT", str(HERE.parent.parent / "reference")))
PORT_LIB = HERE / "liboracle.so"
REF_DIR = HERE / "_ref"
REF_LIB = REF_DIR / "libvecops_ref.so"
REF_FLAGS = REF_DIR / "cpu_flags.txt"

# ISA features the reference build may use; the run host must have all of the
# ones the build host had, or the library is not loaded there.
ISA_FLAGS = (
    "avx512f", "avx512bw", "avx512vl", "avx512dq", "avx512cd", "avx512_vnni", "avx512_bf16", "avx512_fp16",
    "avx512vbmi", "avx512_vbmi2", "avx512ifma", "avx512_bitalg", "avx512_vpopcntdq", "amx_tile", "amx_bf16",
    "amx_int8", "avx2", "fma", "bmi2", "avx_vnni", "gfni", "vaes", "vpclmulqdq", "movdiri", "movdir64b", "serialize",
    "cldemote", "waitpkg", "avx512_vp2intersect", "amx_fp16", "avx_ifma", "rdpid", "sha_ni", "clwb", "pku",
)


def host_cpu_flags() -> set[str]:
    try:
        for line in Path("/proc/cpuinfo").read_text().splitlines():
            if line.startswith("flags"):
                return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def _newer(target: Path, sources: list[Path]) -> bool:
    return target.exists() and all(target.stat().st_mtime >= s.stat().st_mtime for s in sources if s.exists())


def build_port(force: bool = False) -> Path:
    source = HERE / "matmul_oracle.c"
    if not force and _newer(PORT_LIB, [source]):
        return PORT_LIB
    # x86-64-v3 (AVX2) keeps the checker runnable on any host of this decade.
    command = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC", "-o", str(PORT_LIB), str(source), "-lm"]
    subprocess.run(command, check=True)
    return PORT_LIB


def reference_present() -> bool:
    return (REFERENCE_ROOT / "include" / "vecops" / "ops" / "Matmul.h").exists()


def build_ref(force: bool = False) -> Path | None:
    """Compile the reference's matmul behind ref_driver.cpp; None when the checkout is absent."""
    if not reference_present():
        return REF_LIB if REF_LIB.exists() else None
    source = HERE / "ref_driver.cpp"
    if not force and _newer(REF_LIB, [source]) and REF_FLAGS.exists():
        return REF_LIB
    REF_DIR.mkdir(exist_ok=True)
    sources = [REFERENCE_ROOT / "src" / name
               for name in ("MatmulRuntimeDispatch.cpp", "CacheInfo.cpp", "Assertion.cpp", "Parallel.cpp", "NativeThreadPool.cpp")]
    command = ["g++", "-std=c++20", "-O3", "-march=native", "-Wno-ignored-attributes", "-shared", "-fPIC",
               f"-I{REFERENCE_ROOT / 'include'}", f"-I{REFERENCE_ROOT / 'include' / 'vecops'}", str(source),
               *map(str, sources), "-ldl", "-lpthread", "-o", str(REF_LIB)]
    subprocess.run(command, check=True)
    flags = host_cpu_flags()
    REF_FLAGS.write_text(" ".join(sorted(f for f in ISA_FLAGS if f in flags)) + "\n")
    return REF_LIB


def ref_runnable_here() -> tuple[bool, str]:
    """Can the prebuilt reference library run on this host's CPU?"""
    if not REF_LIB.exists() or not REF_FLAGS.exists():
        return False, "oracle/_ref is not built"
    needed = set(REF_FLAGS.read_text().split())
    missing = sorted(needed - host_cpu_flags())
    if missing:
        return False, "host CPU lacks " + ",".join(missing)
    return True, ""


if __name__ == "__main__":
    force = "--force" in sys.argv
    print("port:", build_port(force))
    print("ref :", build_ref(force))
