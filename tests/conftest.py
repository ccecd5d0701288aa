"""Test configuration.

Markers: ``gpu`` -- needs a B200; everything else runs on CPU.  GPU tests call the CUDA kernels
through the C ABI and compare against the CPU oracle; they are skipped (not passed) when no CUDA
device exists.
"""

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)
    yield


@pytest.fixture(scope="session")
def kernel_lib():
    """The built C-ABI library (builds it in-tree if it is missing and nvcc is present)."""
    from iree_turbine_b200 import _launcher

    if not _launcher.lib_path().exists():
        import importlib.util

        spec = importlib.util.spec_from_file_location(
            "b200k_build", os.path.join(ROOT, "iree-turbine_b200", "csrc", "build.py")
        )
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    return _launcher.lib()
