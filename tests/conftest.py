import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "mindie-sd_b200", ROOT / "tests" / "golden"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

os.environ.setdefault("MINDIE_LOG_TO_FILE", "false")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    # A GPU test on a machine without one is an error of the invocation, not a pass.
    import torch
    if torch.cuda.is_available():
        # A kernel that never returns must not hold the machine: every GPU test gets a time limit (pytest-timeout,
        # where it is installed and no limit was given on the command line).  The "thread" method ends the
        # process even while the main thread sits in a CUDA call that does not return.
        if config.pluginmanager.hasplugin("timeout") and not config.getoption("timeout", None):
            for item in items:
                if "gpu" in item.keywords and item.get_closest_marker("timeout") is None:
                    item.add_marker(pytest.mark.timeout(300, method="thread"))
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
