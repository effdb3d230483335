import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def orc():
    """The plain-C oracle (oracle/dcgan_oracle.c)."""
    import oracle
    return oracle.port()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU code compiled from its sources, or skip."""
    import oracle
    r = oracle.reference()
    if r is None:
        pytest.skip("reference-compiled oracle (oracle/_ref) not available on this machine")
    return r


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_cases.npz"))


@pytest.fixture(scope="session")
def pkg():
    """The product package; building it first if the shared library is missing."""
    import __graft_entry__ as entry
    if not os.path.exists(os.path.join(entry.PKG_DIR, "libdcgan_b200.so")):
        entry.build()
    return entry.load_package()


@pytest.fixture(scope="session")
def dev(pkg):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


def seeded(shape, seed, lo=-1.0, hi=1.0):
    """U(lo, hi) from the reference's xorshift generator (src/utils/xorshift.cu)."""
    import oracle
    o = oracle.port()
    o.xorshift_seed(seed)
    return (o.xorshift_fill(shape) * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)
