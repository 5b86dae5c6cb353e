import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def golden():
    import json
    with open(os.path.join(ROOT, "tests", "golden", "reference_vectors.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def sess():
    """One libzyxb context on cuda:0 for the whole GPU test session."""
    from zyx_b200 import build
    from zyx_b200.ops import Session
    build.build()
    s = Session(device_ids=[0])
    yield s
    s.close()


def pytest_sessionfinish(session, exitstatus):
    """The comparisons that passed only through the float64 attribution of tests/parity.py::assert_parity, with their three
    errors, as a table (tests/parity_fallbacks.md holds the copy of the last full GPU run)."""
    from tests import parity
    if not parity.FALLBACKS:
        return
    out = os.environ.get("ZYXB_PARITY_REPORT")
    if not out:
        return
    with open(out, "w") as f:
        f.write("| test | what | tolerance | floor | gpu vs oracle | gpu vs float64 | oracle vs float64 |\n|---|---|---|---|---|---|---|\n")
        for test, what, tol, floor, e_go, e_ge, e_oe in parity.FALLBACKS:
            f.write("| %s | %s | %g | %g | %.3g | %.3g | %.3g |\n" % (test, what, tol, floor, e_go, e_ge, e_oe))
