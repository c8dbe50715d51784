import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a compute-capability-10.x GPU (run with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    """The ptx.jl_b200 package (imported as ptx_jl_b200) with its library built."""
    import __graft_entry__ as ge
    p = ge.load_package()
    p.build.build()
    return p


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.build_c_oracle()
    return oracle


@pytest.fixture(scope="session")
def gpu(pkg):
    """cuda:0, or fail loudly: GPU tests never fall back to anything else."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    major, _ = torch.cuda.get_device_capability(0)
    assert major == 10, "libptxb200.so holds sm_100a code only"
    torch.cuda.set_device(0)
    pkg.native.lib()
    return torch.device("cuda", 0)
