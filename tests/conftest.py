import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


def pytest_collection_modifyitems(config, items):
    # every test that needs several GPUs is also a gpu test
    for item in items:
        if "multigpu" in item.keywords:
            item.add_marker(pytest.mark.gpu)


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def gpus_for_test(at_most: int = 4) -> int:
    """Ranks (one per GPU) a multi-GPU test world uses: the visible GPUs, at most ``at_most``, and at most
    CHB_TEST_MAX_GPUS (default 2: every multi-GPU test spawns its own world of processes, and the suite on two
    ranks is the quick everyday check; export 4 or 8 to widen it).  0 without CUDA."""
    import os

    import torch

    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return min(n, at_most, int(os.environ.get("CHB_TEST_MAX_GPUS", "2")))
