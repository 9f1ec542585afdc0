import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "knet.jl_b200"), os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def ko():
    """The CPU checker (oracle/knet_oracle.py), built on demand."""
    import knet_oracle
    knet_oracle.build()
    return knet_oracle


@pytest.fixture(scope="session")
def K():
    """The product package; its import fails if libknet_sm100.so is missing."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import knet_sm100
    return knet_sm100
