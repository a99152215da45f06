import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    # The CPU oracle is test infrastructure: compile it on first use (gcc only; seconds).
    oracle_dir = os.path.join(ROOT, "oracle")
    if not os.path.exists(os.path.join(oracle_dir, "libdsmd_oracle.so")):
        subprocess.run(["make", "-C", oracle_dir, "libdsmd_oracle.so"], check=True, stdout=subprocess.DEVNULL)


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return 0
