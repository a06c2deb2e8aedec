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
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """The worst error of every comparison with the plain implementation, so that the tolerances can be
    read against what was seen."""
    try:
        import helpers
    except Exception:
        return
    if not helpers.WORST:
        return
    terminalreporter.write_line("worst max|diff|/max|ref| against the plain implementation:")
    by_dtype = {}
    for (what, which, dtype), err in sorted(helpers.WORST.items()):
        terminalreporter.write_line(f"  {dtype:9s} {which} {what:40s} {err:.3e}")
        by_dtype[dtype] = max(by_dtype.get(dtype, 0.0), err)
    for dtype, err in by_dtype.items():
        terminalreporter.write_line(f"  worst of all, {dtype}: {err:.3e} (tolerance {helpers.TOL[dtype]:.1e})")
