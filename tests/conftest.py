import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(autouse=True)
def _b200_sm_count():
    """Schedules are always built for a 148-SM B200, with or without a GPU."""
    from megakernels_b200.utils import set_sm_count_override

    if torch.cuda.is_available():
        set_sm_count_override(torch.cuda.get_device_properties(0).multi_processor_count)
    else:
        set_sm_count_override(148)
    yield
    set_sm_count_override(None)


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN
