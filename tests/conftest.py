import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "edge-fm-x_b200", "python")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def built():
    """The in-tree libraries; built here when absent (nvcc cross-compiles without a GPU)."""
    import importlib.util
    lib = os.path.join(ROOT, "edge-fm-x_b200", "lib", "libefm_b200.so")
    mod_dir = os.path.join(ROOT, "edge-fm-x_b200", "python")
    have_mod = os.path.isdir(mod_dir) and any(f.startswith("edge_fm.") for f in os.listdir(mod_dir))
    if not (os.path.exists(lib) and have_mod):
        spec = importlib.util.spec_from_file_location("efm_build", os.path.join(ROOT, "edge-fm-x_b200", "build.py"))
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        m.build_engine()
    return lib
