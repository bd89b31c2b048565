import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def vo():
    from oracle import voxoracle
    return voxoracle


@pytest.fixture(scope="session")
def oracle(vo):
    return vo.Oracle()


@pytest.fixture(scope="session")
def ref(vo):
    if not vo.RefGgml.available():
        pytest.skip("oracle/_ref (the reference's ggml CPU backend) was not built on this machine")
    return vo.RefGgml()


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "attn_golden.npz"))


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as entry
    return entry.import_package()


@pytest.fixture(scope="session")
def engine(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    pkg.lib()  # the GPU tests must run the built library: raises if it is missing
    eng = pkg.Engine(0)
    yield eng
    eng.close()
