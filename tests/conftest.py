import os
import sys

import numpy as np
import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

GOLDEN = os.path.join(REPO, "tests", "golden")

# fp32 parity bar of the path: |a - b| <= ATOL + RTOL * |b|
RTOL = 1e-5
ATOL = 1e-5


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def assert_close(actual, expected, what="", scale=None):
    """Relative/absolute 1e-5 check.  `scale` (a positive float) widens the absolute
    term to ATOL*scale for quantities whose magnitude is far from 1 (sums over many nodes)."""
    actual = np.asarray(actual, np.float64)
    expected = np.asarray(expected, np.float64)
    assert actual.shape == expected.shape, f"{what}: shape {actual.shape} != {expected.shape}"
    atol = ATOL * (scale if scale else 1.0)
    err = np.abs(actual - expected)
    tol = atol + RTOL * np.abs(expected)
    bad = err > tol
    if bad.any():
        i = np.unravel_index(np.argmax(err - tol), err.shape)
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} elements outside rel {RTOL} / abs {atol}; "
                             f"worst at {i}: got {actual[i]!r}, want {expected[i]!r}")


@pytest.fixture(scope="session")
def oracle_lib():
    """Builds the C restatement (and the reference build when a checkout is present)."""
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import build as oracle_build
    oracle_build.build_oracle()
    oracle_build.build_ref()
    from oracle import bindings
    return bindings


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(os.path.join(GOLDEN, name))
    return load


@pytest.fixture(scope="session")
def gpu_ctx():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    from graphnn_b200 import capi
    ctx = capi.Context(0)
    yield ctx
    ctx.close()
