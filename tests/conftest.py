import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle_backend import OracleBackend
    return OracleBackend()


@pytest.fixture(scope="session")
def gpu():
    """The CUDA backend; the library must be present and a device must answer."""
    from npu_plugin_b200.const import CudaBackend
    return CudaBackend(0)


@pytest.fixture(params=["oracle", pytest.param("b200", marks=pytest.mark.gpu)])
def backend(request):
    """Known-answer tests run against the CPU oracle here and against the CUDA library on the GPU box."""
    return request.getfixturevalue("oracle" if request.param == "oracle" else "gpu")
