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
def built_library():
    """Builds librocfft.so in-tree if it is missing; the tests never fall back
    to anything else."""
    import rocfft_b200 as rf
    if not os.path.exists(rf.LIB_PATH):
        from rocfft_b200 import build
        build.build()
    return rf.lib()


@pytest.fixture(scope="session")
def gpu(built_library):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    import rocfft_b200 as rf
    assert rf.rocfft_setup() == rf.rocfft_status_success
    yield torch
    rf.rocfft_cleanup()
