import os
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)


# the front end writes the reference's per-rank log (./logs/<run id>/rank_<r>/checkers.log): keep it out of the tree
import tempfile  # noqa: E402

os.environ.setdefault("CHECKERS_LOG_DIR", tempfile.mkdtemp(prefix="checkers_logs_"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle_lib import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def ref():
    from oracle_lib import RefShim
    if not RefShim.available():
        pytest.skip("oracle/_ref not built (python oracle/build_ref.py needs the reference tree)")
    return RefShim()


@pytest.fixture(scope="session")
def emu():
    from emu_lib import Emu
    return Emu()
