"""pytest configuration: import paths and the ``gpu`` marker.

``-m "not gpu"``: oracle vs golden vectors, host logic, C-ABI symbol check (no GPU needed).
``-m gpu``:       parity tests proper, every computation goes through libk2q.so on a B200.
"""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "krea-2_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
