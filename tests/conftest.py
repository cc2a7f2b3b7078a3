import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _experts_kernel_choice():
    """D2D_TEST_EXPERTS_KERNEL=2 runs the whole suite with the bf16 expert kernel gathering
    its token rows by TMA (tile::gather4) instead of the default 16-byte cp.async, so that
    every parity case reaches both row paths."""
    import os
    which = int(os.environ.get("D2D_TEST_EXPERTS_KERNEL", "0"))
    if which:
        from d2dmoe_b200 import _capi
        _capi.lib.d2d_debug_select_experts_kernel(which)
    yield
