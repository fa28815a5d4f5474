import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "selective-attention-freezing_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")
    # a fresh checkout has no built library (it is kept out of history): build it once when a compiler is here
    lib = os.path.join(PKG, "lib", "libsaf_b200.so")
    if not os.path.exists(lib):
        import shutil
        if shutil.which("nvcc"):
            import importlib.util
            spec = importlib.util.spec_from_file_location("graft_entry_for_tests", os.path.join(ROOT, "__graft_entry__.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build()


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)
