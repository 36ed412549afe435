import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def load_golden(name):
    import torch

    return torch.load(os.path.join(GOLDEN, name + ".pt"), weights_only=False)


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library (built on demand from source when missing)."""
    from vexact_b200 import _lib, build

    build.build()
    return _lib.load()


@pytest.fixture(autouse=True)
def _device_status_word_stays_clean(request):
    """Every GPU test must leave the device status word at zero (no bounded wait expired, no index out of
    range): it is read before and after each test so that a report is pinned to the test that caused it."""
    if request.node.get_closest_marker("gpu") is None:
        yield
        return
    import torch

    if not torch.cuda.is_available():
        yield
        return
    from vexact_b200 import _lib

    before = _lib.read_status()
    assert before[0] == 0, f"status word {before} was left behind by an earlier test"
    yield
    torch.cuda.synchronize()
    after = _lib.read_status()
    assert after[0] == 0, f"{request.node.name} left the device status word at {after} (code, detail, block, -)"
