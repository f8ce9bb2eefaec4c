import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def nano_sd():
    """Seeded Vui-Nano-shaped weights (bf16 values) from the oracle's generator."""
    import torch
    from oracle.vui_oracle import OracleConfig, init_weights

    return init_weights(OracleConfig(), seed=0, dtype=torch.bfloat16)


@pytest.fixture(scope="session")
def nano_model(nano_sd):
    """The same weights loaded into the product's container on the GPU."""
    import torch
    from vui_b200 import VuiB200, VuiShape

    if not torch.cuda.is_available():
        pytest.skip("needs CUDA")
    return VuiB200(VuiShape(), nano_sd, device="cuda")
