import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """bfloat16 is measured, not only bounded: the replay tests' agreement with the plain implementation."""
    try:
        import replay
    except Exception:
        return
    if replay.REPORT:
        terminalreporter.write_sep("-", "engine against the plain implementation")
        for line in replay.REPORT:
            terminalreporter.write_line(line)
