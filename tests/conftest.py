import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")
    config.addinivalue_line("markers", "multigpu: needs 2 or more CUDA devices")


def pytest_collection_modifyitems(config, items):
    import torch

    n_gpus = torch.cuda.device_count() if torch.cuda.is_available() else 0
    skip = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs 2 or more CUDA devices")
    for item in items:
        if "multigpu" in item.keywords and n_gpus < 2:
            item.add_marker(skip_multi)
        elif "gpu" in item.keywords and n_gpus < 1:
            item.add_marker(skip)
