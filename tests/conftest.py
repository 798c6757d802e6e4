"""Shared fixtures.  Tests marked ``gpu`` need a B200; everything else runs on
a CPU-only machine.  The CPU checkers under ``oracle/`` are test
infrastructure and are only ever used here as the thing to compare against."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.checker import Oracle

    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own scalar code, if its library was built (it needs the
    reference tree at build time; the built file travels with the repository
    snapshot)."""
    from oracle import checker

    if not os.path.exists(checker.REF_SO) and checker.reference_root():
        checker.build(("ref",))
    ref = checker.Reference()
    if not ref.available:
        pytest.skip("oracle/_ref/libfbgemm_ref.so not built")
    return ref


@pytest.fixture(scope="session")
def gpu_ctx():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("gpu test selected but no CUDA device is visible")
    import fbgemm_b200

    return fbgemm_b200.get_context(0)


def bits(a):
    """Bit pattern view for exact float comparison."""
    a = np.ascontiguousarray(a)
    return a.view({2: np.uint16, 4: np.uint32}[a.dtype.itemsize])
