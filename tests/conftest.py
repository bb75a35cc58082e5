import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_dir():
    return ROOT / "tests" / "golden"


def pytest_sessionfinish(session, exitstatus):
    """The labelled long-sum checks record which rule admitted how many elements and both distances to
    the fp64 result; NB2_PARITY_LOG=<file> writes the records there as JSON."""
    import os
    try:
        from tests import tol
        target = os.environ.get("NB2_PARITY_LOG")
        if tol.PARITY_LOG and target:
            import json
            Path(target).write_text(json.dumps(tol.PARITY_LOG, indent=1))
    except Exception:
        pass
