import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "spiral-s-ml-library_b200")
for p in (ROOT, PKG_DIR):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def sb():
    """The product package, with the CUDA library loaded (fails loudly if it is missing)."""
    import spiral_b200
    from spiral_b200 import _lib
    _lib.load()
    return spiral_b200


@pytest.fixture(scope="session")
def gpu(sb):
    if sb.device_count() < 1:
        pytest.fail("a test marked gpu ran without a CUDA device")
    sb.set_device(0)
    return sb


@pytest.fixture(autouse=True)
def _healthy_device(request):
    """After every GPU test the device status word must still be clean."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        import spiral_b200
        site, count = spiral_b200.device_status(clear=True)
        assert (site, count) == (0, 0), "a bounded device-side wait expired (site %d, %d times)" % (site, count)
