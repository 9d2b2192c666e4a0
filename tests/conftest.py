import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    """GPU tests fail loudly rather than skip: when tests marked `gpu` are selected and there is no CUDA device,
    the run is stopped with an error before the first test.  With -m "not gpu" they are deselected as usual and
    nothing here looks for a device."""
    markexpr = config.getoption("markexpr", "") or ""
    if "not gpu" in markexpr:
        return
    if any(item.get_closest_marker("gpu") for item in items) and "gpu" in markexpr:
        import torch
        if not torch.cuda.is_available():
            raise pytest.UsageError("tests marked 'gpu' were selected but no CUDA device is available; "
                                    "run them on a B200, or select -m \"not gpu\"")
