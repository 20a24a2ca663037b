import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    from __graft_entry__ import load_package
    return load_package()


@pytest.fixture(scope="session")
def orc():
    import parity
    return parity.oracle()


@pytest.fixture(scope="session")
def golden():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="session")
def dev(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    d = torch.device("cuda:0")
    torch.cuda.set_device(d)
    pkg.use_torch_stream()
    return d


@pytest.fixture(autouse=True)
def _clean_device_error(request, pkg):
    """After every GPU test the kernels' bounded-wait error word must be clean."""
    pkg.lib.hd_cuda_clear_error()
    yield
    if request.node.get_closest_marker("gpu"):
        import torch
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            assert pkg.lib.o1_device_error() == 0, "a kernel reported a bounded-wait timeout"
