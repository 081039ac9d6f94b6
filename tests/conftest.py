import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# the unmodified reference tree, where a test compares against it (Z2H_REFERENCE overrides)
import os

REFERENCE = Path(os.environ.get("Z2H_REFERENCE", ROOT / "baseline" / "_ref"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def reference_root():
    if not (REFERENCE / "nn").exists():
        pytest.skip("reference tree not available")
    return REFERENCE
