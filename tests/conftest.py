"""Test configuration: import paths, the `gpu` marker and golden-vector loading."""
from pathlib import Path
import sys

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
for entry in (ROOT / "ascend-int8-attention_b200", ROOT):
    if str(entry) not in sys.path:
        sys.path.insert(0, str(entry))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_sessionstart(session):
    torch.set_num_threads(4)


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
