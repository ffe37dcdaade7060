import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return ROOT / "tests" / "golden"


@pytest.fixture(autouse=True)
def no_kernel_left_work_undone(request):
    """After every GPU test: the device's kernel status word (infiniopGetKernelStatus) must read 0 - no
    worker gave up a wait, no checked index lay outside the pool.  Tests that provoke a flag read (and so
    clear) it themselves."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import torch

    if not torch.cuda.is_available():
        return
    import abi

    if abi._handle is not None:  # the test went through the C ABI on device 0
        torch.cuda.synchronize()
        assert abi.kernel_status() == 0, "a kernel of this test reported that it could not do all of its work"
