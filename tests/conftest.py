import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def orc():
    import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "ref_decoder_vectors.npz"))


@pytest.fixture(scope="session")
def dev():
    """One Device for the GPU tests. Fails (never skips) if the CUDA library cannot open a B200."""
    from jitllm_b200 import Device
    d = Device(0)
    yield d
    d.Close()


def parity_err(got: np.ndarray, ref: np.ndarray) -> float:
    """max_i |got - ref| / max(|ref_i|, rms(ref)): the output-parity measure (bar 2e-3)."""
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    rms = float(np.sqrt(np.mean(ref * ref)))
    den = np.maximum(np.abs(ref), rms if rms > 0 else 1.0)
    return float(np.max(np.abs(got - ref) / den))


def nmse(got: np.ndarray, ref: np.ndarray) -> float:
    got = np.asarray(got, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    return float(np.sum((got - ref) ** 2) / max(np.sum(ref * ref), 1e-300))
