import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o

    o.build()
    return o


@pytest.fixture(scope="session")
def fso():
    import fish_scales_ops_b200 as pkg

    pkg.build()
    return pkg


@pytest.fixture()
def device_ok(fso):
    """After a GPU test: no kernel wait ran out (the device-side status word is still zero)."""
    yield
    from fish_scales_ops_b200 import _ops

    assert _ops.device_status() == 0
