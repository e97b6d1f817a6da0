import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "open-jev-fast_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _device_wait_limit():
    """OJB_TEST_WAIT_MS=<ms> shortens the limit of the kernels' bounded device-side waits for the whole run (a protocol mistake
    in a kernel under development then ends its launch after that time with a status word instead of after the default 2 s)."""
    ms = os.environ.get("OJB_TEST_WAIT_MS")
    if ms:
        import ctypes
        from ojb200 import _lib
        _lib.lib().ojb_gemm_set_wait_limit_ms(ctypes.c_int32(int(ms)))
    yield
