import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def port():
    from oracle.checker import Port
    return Port()


@pytest.fixture(scope="session")
def library():
    from vecops_b200 import _build, capi
    _build.build()
    return capi.library()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    cases = {}
    for path in sorted((ROOT / "tests" / "golden").glob("*.npz")):
        with np.load(path) as data:
            cases[path.stem] = {key: data[key] for key in data.files}
    assert cases, "no golden fixtures found"
    return cases
