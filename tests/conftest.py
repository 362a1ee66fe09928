import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no GPU here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    try:
        from helpers import WORST
    except Exception:
        return
    if terminalreporter.config.getoption("verbose") <= 0:
        worst = {}
        for (dtype, _), frac in WORST.items():
            worst[dtype] = max(worst.get(dtype, 0.0), frac)
        for dtype, frac in sorted(worst.items()):
            terminalreporter.write_line(f"largest error / largest reference value, {dtype}: {frac:.3e}")
        return
    for (dtype, test), frac in sorted(WORST.items()):
        terminalreporter.write_line(f"largest error / largest reference value, {dtype}: {frac:.3e}  {test}")
