import importlib.util
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
FIXTURES = os.path.join(GOLDEN, "fixtures")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


def load_package():
    """The package directory is named ncnn-compiler_b200; import it as ncnn_compiler_b200."""
    if "ncnn_compiler_b200" in sys.modules:
        return sys.modules["ncnn_compiler_b200"]
    d = os.path.join(ROOT, "ncnn-compiler_b200")
    spec = importlib.util.spec_from_file_location("ncnn_compiler_b200", os.path.join(d, "__init__.py"),
                                                  submodule_search_locations=[d])
    module = importlib.util.module_from_spec(spec)
    sys.modules["ncnn_compiler_b200"] = module
    spec.loader.exec_module(module)
    return module


def load_oracle():
    """oracle/ is test infrastructure: the checker, never the thing under test."""
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    if os.path.join(ROOT, "oracle") not in sys.path:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ncnn_oracle
    return ncnn_oracle


def ensure_built():
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import __graft_entry__
    __graft_entry__.build()


@pytest.fixture(scope="session")
def pkg():
    ensure_built()
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    return load_oracle()


def rel_l2(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-30))


def fixture(name):
    return os.path.join(FIXTURES, name + ".param"), os.path.join(FIXTURES, name + ".bin")
