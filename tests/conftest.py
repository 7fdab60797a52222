import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "ref_vectors.npz"))


@pytest.fixture(scope="session")
def oracle():
    from oracle import pet_oracle
    pet_oracle.lib()  # builds libpet_oracle.so on first use
    return pet_oracle


@pytest.fixture(scope="session")
def ctx():
    """One C-ABI context on cuda:0 for the whole GPU session.  Fails (does not skip) if the library is missing."""
    from pet_b200.ops import Context
    c = Context(0)
    yield c
    c.close()


def contract_err(a, b):
    """The parity metric of the floating-point operators, stated once for every test:
        max_i |a_i - b_i| / max(|b_i|, 1e-3 * max_j |b_j|)
    i.e. elementwise relative error against the reference value b, where outputs smaller than a thousandth of the
    tensor's largest magnitude are judged against that floor (an output that cancels to ~0 has no meaningful relative
    error of its own).  Bound: 1e-3."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    floor = max(1e-3 * float(np.max(np.abs(b))), 1e-30)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), floor)))


rel_err = contract_err  # every `rel_err(...) <= TOL` in the tests asserts the contract metric


def rms_rel_err(a, b):
    """A looser companion figure, reported only: the same ratio with the tensor's RMS as the floor."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    floor = max(float(np.sqrt(np.mean(b * b))), 1e-30)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), floor)))


def scale_err(a, b):
    """max |a-b| / max |b| — used for the tighter accuracy statement of the 3xTF32 kernels."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / max(float(np.max(np.abs(b))), 1e-30))
