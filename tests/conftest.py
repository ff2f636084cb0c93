import importlib.util
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load_package():
    """Imports the hyphen-named package directory as module ``aet_cnn_b200``."""
    if "aet_cnn_b200" in sys.modules:
        return sys.modules["aet_cnn_b200"]
    pkg_dir = os.path.join(ROOT, "aet-cnn_b200")
    spec = importlib.util.spec_from_file_location("aet_cnn_b200", os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["aet_cnn_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def aet():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    from oracle import binding
    binding.build()
    return binding.Oracle("parity")


@pytest.fixture(scope="session")
def oracle64():
    from oracle import binding
    binding.build()
    return binding.Oracle("acc64")


@pytest.fixture(scope="session")
def ctx(aet):
    c = aet.Context(0)
    yield c
    c.close()


def rel_l2(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    d = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / d) if d > 0 else float(np.linalg.norm(a - b))


def max_rel(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    m = np.max(np.abs(b))
    return float(np.max(np.abs(a - b)) / m) if m > 0 else float(np.max(np.abs(a - b)))
