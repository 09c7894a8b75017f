"""Shared test configuration.

Markers: ``gpu`` -- needs a B200 and the built native library (parity tests proper); everything
else runs on CPU.  ``oracle/`` is imported by tests only as the checker.
"""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA GPU (sm_100a) and the built extension")


def pytest_sessionfinish(session, exitstatus):
    """FA_PARITY_LOG=<file>: write every recorded parity comparison (see helpers.PARITY_LOG) as JSON lines."""
    import json
    import os

    path = os.environ.get("FA_PARITY_LOG")
    if not path:
        return
    try:
        import helpers
    except ImportError:
        return
    with open(path, "w") as f:
        for rec in helpers.PARITY_LOG:
            f.write(json.dumps(rec) + "\n")


@pytest.fixture(autouse=True)
def _parity_case_name(request):
    """Prefix the records of helpers.PARITY_LOG with the id of the test that made them."""
    try:
        import helpers
    except ImportError:
        yield
        return
    n0 = len(helpers.PARITY_LOG)
    yield
    for rec in helpers.PARITY_LOG[n0:]:
        rec["name"] = request.node.name + "/" + rec["name"]


@pytest.fixture(scope="session")
def ext():
    """The torch binding; importing it must not silently fall back to anything."""
    from flash_attention_turing_b200 import _ext

    return _ext.load()


@pytest.fixture(autouse=True)
def _check_device_status(request):
    """After every GPU test: no kernel may have recorded a timed-out wait."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        from flash_attention_turing_b200 import _ext

        status = _ext.load().device_status(True)
        assert status == 0, f"device status word = {status} (a bounded wait gave up)"
