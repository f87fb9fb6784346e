import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def dev():
    """One Device for the whole GPU session; fails loudly when the library or GPU is absent."""
    from vkgrad_b200 import vk
    d = vk.Device()
    yield d
    d.destroy()
