"""Test set-up: the repository and the tests' own helpers on the import path, the ``gpu`` marker,
and a skip for GPU tests on a machine without a CUDA device."""
import pathlib
import sys

import pytest

_HERE = pathlib.Path(__file__).resolve().parent
for _folder in (_HERE.parent, _HERE):
    if str(_folder) not in sys.path:
        sys.path.insert(0, str(_folder))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    gpu_tests = [item for item in items if item.get_closest_marker("gpu") is not None]
    if not gpu_tests:
        return
    import torch

    if not torch.cuda.is_available():
        reason = pytest.mark.skip(reason="this test needs a CUDA device and there is none")
        for item in gpu_tests:
            item.add_marker(reason)
