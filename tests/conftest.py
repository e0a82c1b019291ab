"""Shared fixtures.  Tests marked ``gpu`` need a B200 and call the CUDA path through the C ABI;
everything else runs on CPU (oracle, host logic, symbol checks, gloo ranks)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def built(pkg):
    entry.build()
    return pkg


@pytest.fixture(scope="session")
def ob():
    import oracle_binding
    oracle_binding.oracle()
    return oracle_binding


@pytest.fixture(scope="session")
def params0(pkg):
    return pkg.synth.synth_params(0)


@pytest.fixture(scope="session")
def data64(pkg):
    return pkg.synth.synth_images(11, 64)


@pytest.fixture(scope="session")
def cuda(built):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch


def rel_err(a, b, floor=0.0):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), floor))) if a.size else 0.0


def scaled_err(a, b):
    """max |a-b| / max |b|: for signed quantities that pass through zero."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    if a.size == 0:
        return 0.0
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))
