import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# the reference's OpenMP reductions are order-dependent; one thread keeps the oracle bit-stable
os.environ.setdefault("OMP_NUM_THREADS", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def ref():
    """The compiled reference CPU library (built on the fly where its sources exist)."""
    from oracle import ref_lib
    if not ref_lib.available():
        try:
            ref_lib.build()
        except Exception as ex:  # pragma: no cover
            pytest.skip(f"reference oracle library cannot be built here: {ex}")
    if not ref_lib.available():
        pytest.skip("oracle/_ref/libnocta_ref.so is not present")
    return ref_lib.load()
