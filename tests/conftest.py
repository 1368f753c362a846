import importlib
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def package():
    """The product package (its directory name carries a hyphen)."""
    return importlib.import_module("kanso-infer_b200")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def kb():
    return package().backend


@pytest.fixture(scope="session")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    return torch


@pytest.fixture(scope="session")
def ctx(kb, torch_cuda):
    """A context on a torch stream made current for the session, so torch tensors, copies
    and events are ordered with the library's kernels."""
    stream = torch_cuda.cuda.Stream()
    torch_cuda.cuda.set_stream(stream)
    c = kb.Context(0, stream)
    yield c
    c.close()


def golden(name):
    return np.load(os.path.join(GOLDEN, name))


def rel_err(a, b):
    """Scale-relative error the reference's own tests use (tests/test_quantized_weights.rs:375-397)."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))
