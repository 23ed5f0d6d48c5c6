import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def runtime():
    """The process-wide device runtime (4 GiB arena) for GPU tests."""
    import attention_superoptimizer_b200 as mg
    rt = mg.Runtime.get(device=0, arena_bytes=4 << 30)
    yield rt


@pytest.fixture()
def planning_runtime():
    """A runtime without a device: graphs can be built and lowered, nothing can be launched."""
    import attention_superoptimizer_b200 as mg
    assert mg.Runtime._instance is None, "one runtime per process"
    rt = mg.Runtime(device=-1, arena_bytes=1 << 30)
    yield rt
    mg._abi.check(rt.lib.mg_runtime_destroy(rt.handle))
