import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def expert_weights():
    """Layer-0 quantised expert slabs (seed 1000), generated once per session (about 15 s)."""
    from netra_kernel_b200 import synth
    return synth.make_expert_weights(0)


@pytest.fixture(scope="session")
def c_oracle():
    from tests import helpers
    return helpers.load_c_oracle()
