"""pytest configuration: markers, repo root on sys.path, shared fixtures."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import build_oracle
    from oracle.bindings import Oracle

    build_oracle.build()
    return Oracle()


@pytest.fixture(scope="session")
def reference_lib():
    """The reference CPU backend itself, when its prebuilt library is present."""
    from oracle.bindings import REF_LIB, Reference

    if not REF_LIB.exists():
        pytest.skip("oracle/_ref/libmarmot_ref.so not built (needs the reference checkout)")
    ref = Reference()
    yield ref
    ref.close()


@pytest.fixture(scope="session")
def llama_goldens():
    return dict(np.load(GOLDEN_DIR / "llama_goldens.npz"))


@pytest.fixture(scope="session")
def ref_cases():
    return dict(np.load(GOLDEN_DIR / "ref_cases.npz"))
