import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle_mod():
    from oracle import srf_oracle
    srf_oracle.build()
    return srf_oracle


@pytest.fixture(scope="session")
def built_lib():
    """The C-ABI library, rebuilt from the current sources where nvcc exists; otherwise it must already be there."""
    import shutil
    from sphericalrf_b200 import abi
    if shutil.which("nvcc") or Path("/usr/local/cuda/bin/nvcc").exists():
        import __graft_entry__
        __graft_entry__.build()          # incremental: compiles only what is older than its sources
    return abi.load()
