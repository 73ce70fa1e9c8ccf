import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def registry():
    """All built plugins.  Building is the job of __graft_entry__.build(); a missing kernel
    directory is an error, never a reason to fall back to anything else."""
    import sm120_gemm_b200 as g

    r = g.KernelRegistry()
    if not r.load_dir(g.KERNEL_DIR):
        from sm120_gemm_b200 import build

        build.build_all()
        assert r.load_dir(g.KERNEL_DIR), "no kernel plugins could be built or loaded"
    return r


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    major, _ = torch.cuda.get_device_capability(0)
    assert major == 10, "these kernels are sm_100a only"
    return torch.device("cuda:0")
