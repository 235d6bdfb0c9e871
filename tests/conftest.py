import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load_package():
    """Imports the package directory ``flux2.c_b200`` (not a valid dotted name) as ``flux2_c_b200``."""
    name = "flux2_c_b200"
    if name in sys.modules:
        return sys.modules[name]
    pkg_dir = os.path.join(ROOT, "flux2.c_b200")
    spec = importlib.util.spec_from_file_location(name, os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def fx():
    return load_package()


@pytest.fixture(scope="session")
def ctx(fx):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    c = fx.Context(0)
    yield c
    c.close()
