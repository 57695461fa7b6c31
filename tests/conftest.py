import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _built_oracle():
    from oracle import build
    build.build_oracle()


def pytest_sessionfinish(session, exitstatus):
    """How much of every forward tensor was held to which bound (oracle/parity.py) goes to a report beside the
    other outputs of a GPU run and, in short, to the terminal."""
    from oracle import parity
    if not parity.REPORT:
        return
    try:
        parity.dump_report(os.path.join(ROOT, os.environ.get("SNNTC_REPORT_DIR", "gpurun_out"), "parity_report.json"))
    except OSError:
        pass
    print("\nparity summary: %s" % (parity.summary(),))
