import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # tests/test_zz_* files are collected last by name; keep pytest's default (alphabetical) order.
    pass


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O

    O.build()
    return O
