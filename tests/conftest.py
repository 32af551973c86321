"""pytest configuration: registers the ``gpu`` marker and puts the repository root on ``sys.path``."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    def load(name):
        with np.load(GOLDEN / f"{name}.npz") as z:
            return {k: z[k] for k in z.files}
    return load


def pytest_sessionfinish(session, exitstatus):
    """With CDA_PARITY_STATS=<file> every output comparison of the session (elements, elements outside the stated
    tolerance, worst error / bound, cosine) is written to that file as JSON lines."""
    import json
    import os
    path = os.environ.get("CDA_PARITY_STATS")
    if not path:
        return
    try:
        from tests import _cases
    except Exception:
        return
    with open(path, "w") as f:
        for rec in _cases.STATS:
            f.write(json.dumps(rec) + "\n")
