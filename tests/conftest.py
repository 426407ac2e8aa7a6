import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.cpu import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    from oracle.cpu import Reference, reference_available
    if not reference_available():
        pytest.skip("oracle/_ref not built (needs the reference sources; run oracle/build_ref.sh)")
    return Reference()


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
