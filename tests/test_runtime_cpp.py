"""Builds and runs the C++ host-runtime test binary (tests/cpp/runtime_test.cpp)."""
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
CPP = ROOT / "tests" / "cpp"
OUT = ROOT / "build" / "tests"


def test_cpp_runtime_suite(library):
    from vecops_b200 import _build
    OUT.mkdir(parents=True, exist_ok=True)
    fixture = OUT / "libfixture_artifact.so"
    binary = OUT / "runtime_test"
    include = ["-I", str(ROOT / "include"), "-I", str(CPP)]
    subprocess.run(["g++", "-std=c++20", "-O1", "-fPIC", "-shared", *include, str(CPP / "fixture_artifact.cpp"), "-o", str(fixture)],
                   check=True)
    subprocess.run(["g++", "-std=c++20", "-O1", "-Wall", *include, str(CPP / "runtime_test.cpp"), "-o", str(binary),
                    f"-L{_build.LIB_DIR}", "-lvecops_b200", f"-Wl,-rpath,{_build.LIB_DIR}", "-lpthread", "-ldl"], check=True)
    result = subprocess.run([str(binary), str(fixture)], capture_output=True, text=True, timeout=120)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "runtime_test PASS" in result.stdout
