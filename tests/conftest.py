"""Shared fixtures: the ``gpu`` marker and small helpers."""

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

        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """The largest logit error each family of comparisons showed: what the bounds in ``helpers.py`` rest on."""
    try:
        import helpers
    except Exception:
        return
    for (dtype, family), (err, what) in sorted(helpers.SEEN.items()):
        terminalreporter.write_line(f"largest logit error, {dtype} / {family}: {err:.3e} ({what})")
    for name, text in sorted(helpers.NOTES.items()):
        terminalreporter.write_line(f"{name}: {text}")
