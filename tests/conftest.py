import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def pico():
    import numpy as np
    return np.load(ROOT / "tests" / "golden" / "pico_csa.npz")


@pytest.fixture(scope="session")
def pico_ln():
    """The reference's LayerNorm and transformer-block vectors (gpt-pico-ln*, gpt-pico-blk*)."""
    import numpy as np
    return np.load(ROOT / "tests" / "golden" / "pico_ln_blk.npz")
