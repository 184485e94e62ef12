import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def ref():
    """The reference project's own kernels compiled into oracle/_ref (bit-exact golden)."""
    from oracle import ref_gpu

    if not ref_gpu.available():
        pytest.skip("oracle/_ref/librisa_ref.so not built (run oracle/build_ref.sh)")
    return ref_gpu
