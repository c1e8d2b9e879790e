import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100); run with -m gpu on a B200")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure); builds oracle/liboracle.so on first use."""
    import oracle as O

    O.load()
    return O


@pytest.fixture(scope="session")
def cb():
    """The package under test; building the library first if this checkout has none yet."""
    from cudaintro_b200 import build

    build.build()
    import cudaintro_b200

    return cudaintro_b200


@pytest.fixture(scope="session")
def device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def reference_tree():
    """Root of a checkout of the reference project (CUDAINTRO_REFERENCE_TREE, or a directory called
    `reference` beside the repository); tests that need it skip where there is none."""
    from __graft_entry__ import reference_tree as find

    tree = find()
    if tree is None:
        pytest.skip("no checkout of the reference project on this machine")
    return tree
