"""Shared fixtures.  GPU tests carry the `gpu` mark and are skipped without a GPU."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# ---------------------------------------------------------------- largest differences
# Tests that compare logits with the plain implementation record the largest |difference| of each case here;
# the table is printed after the run (also when everything passed), so that a drift in rounding shows long
# before it reaches a limit.
_worst: dict = {}


def record_worst(case: str, dtype: str, diff: float, limit: float) -> None:
    old = _worst.get((case, dtype))
    if old is None or diff > old[0]:
        _worst[(case, dtype)] = (diff, limit)


def pytest_terminal_summary(terminalreporter):
    if not _worst:
        return
    terminalreporter.section("largest |difference| of logits from the plain implementation")
    for (case, dtype), (diff, limit) in sorted(_worst.items()):
        terminalreporter.write_line(f"{case:58s} {dtype:9s} {diff:.3e}  (limit {limit:.3e})")
