"""Shared pytest setup: marker registration, repo root on sys.path, build-once fixture."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def built_library():
    """Path of the C-ABI shared library, building it first if it is not there yet."""
    from nano_vllm_ninetoothed_b200 import build as b
    return b.build()


@pytest.fixture(scope="session")
def mops(built_library):
    """The drop-in operator module.  GPU tests fail loudly if CUDA or the library is missing."""
    import torch
    assert torch.cuda.is_available(), "GPU test selected but no CUDA device is visible"
    from nano_vllm_ninetoothed_b200 import mops as m
    from nano_vllm_ninetoothed_b200 import _cabi
    assert _cabi.lib.b200mops_device_supported(torch.cuda.current_device()) == 0, \
        "the library contains sm_100a code only"
    m.reset_device_status()
    return m


@pytest.fixture()
def oracle():
    from oracle import mops_oracle
    return mops_oracle
