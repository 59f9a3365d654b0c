"""Shared fixtures.  Tests marked `gpu` need a B200 and call the CUDA library through its C ABI;
everything else runs on CPU (oracle vs golden vectors, host logic, ABI surface)."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import __graft_entry__ as graft  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def pkg():
    return graft.load_package()


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (C restatement of the reference's algorithms)."""
    return graft.oracle_loader().load_oracle()


@pytest.fixture(scope="session")
def ref():
    """The reference's own kernels, when oracle/_ref was built (skips otherwise)."""
    lib = graft.oracle_loader().load_reference()
    if lib is None:
        pytest.skip("oracle/_ref/libck_ref.so not built on this machine")
    return lib


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_outputs.npz"))


@pytest.fixture(scope="session")
def ck(pkg):
    """The CUDA library, initialised on device 0.  Fails (does not skip) if it cannot run."""
    path = pkg.find_lib()
    lib = pkg.load_lib()
    rc = lib.ckb200_init(0)
    assert rc == 0, f"{path}: ckb200_init -> {rc}: {lib.ckb200_last_error_message().decode()}"
    return lib


@pytest.fixture(autouse=True)
def _no_stale_error(request):
    yield
    if "ck" in request.fixturenames:
        lib = request.getfixturevalue("ck")
        code = lib.ckb200_last_error()
        msg = lib.ckb200_last_error_message().decode()
        lib.ckb200_clear_error()
        assert code == 0, f"library recorded error {code}: {msg}"


@pytest.fixture(scope="session")
def golden_boundary():
    """Reference outputs for the fp32-activation GEMMs, contract forms, pairwise RoPE and copies (tests/cases.boundary_outputs)."""
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_boundary_outputs.npz"))


@pytest.fixture(scope="session")
def ref_parity():
    """The reference's ck_test_* wrappers, when oracle/_ref was built (skips otherwise)."""
    lib = graft.oracle_loader().load_reference_parity()
    if lib is None:
        pytest.skip("oracle/_ref/libck_ref_parity.so not built on this machine")
    return lib
