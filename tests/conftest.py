import ctypes
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def _oracle_cdll():
    so = os.path.join(ROOT, "oracle", "_build", "libndarray_ref.so")
    if not os.path.exists(so):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True, capture_output=True)
    return ctypes.CDLL(so)


@pytest.fixture(scope="session")
def oracle():
    """The CPU restatement of the reference ndarray backend, behind the same host wrapper as the GPU library."""
    import catgrad_b200 as cb
    return cb.Backend(_cdll=_oracle_cdll(), _prefix="ref_")


@pytest.fixture(scope="session")
def gpu():
    """The shipped CUDA backend on device 0.  Raises (does not skip) when the library or the GPU is missing."""
    import catgrad_b200 as cb
    return cb.Backend(0)
