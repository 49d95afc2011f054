import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def import_extension():
    """The compiled `mla_bwd_cuda` module; built in place first (`python setup.py build_ext --inplace`, about a minute)
    when the tree does not hold it yet.  There is no Python stand-in: a failed build fails the test."""
    import importlib
    import subprocess
    try:
        return importlib.import_module("mla_bwd_cuda")
    except ImportError:
        res = subprocess.run([sys.executable, "setup.py", "build_ext", "--inplace"], cwd=ROOT, capture_output=True, text=True)
        assert res.returncode == 0, "building mla_bwd_cuda failed:\n" + (res.stdout + res.stderr)[-3000:]
        importlib.invalidate_caches()
        return importlib.import_module("mla_bwd_cuda")
