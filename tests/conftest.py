import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def _reference_root():
    from oracle.oracle import reference_root
    return reference_root()


REFERENCE_ROOT = _reference_root()  # QTIP_REFERENCE_ROOT, else the default of oracle/Makefile; may not exist
REFVEC = os.path.join(REFERENCE_ROOT, "tests", "refvec")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (test infrastructure)."""
    from oracle.oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own CPU code compiled in place; skips when the prebuilt files are absent."""
    from oracle.oracle import Reference
    r = Reference()
    if not r.available:
        pytest.skip("oracle/_ref is not built")
    return r


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as g
    return g.load_package()


@pytest.fixture(scope="session")
def gpu(pkg):
    """The package with a CUDA device selected; GPU tests fail (not skip) when the library cannot run."""
    import torch
    assert torch.cuda.is_available(), "a CUDA device is required for -m gpu tests"
    torch.cuda.set_device(0)
    pkg.codec.init()
    return pkg


@pytest.fixture(scope="session")
def refgpu(gpu):
    """The reference's own CUDA kernels for this path, compiled in place for sm_100a; skips when not prebuilt."""
    from oracle.oracle import ReferenceGpu
    r = ReferenceGpu()
    if not r.available:
        pytest.skip("the reference's CUDA kernels are not built (make -C oracle refgpu)")
    r.initialize_tables()
    return r


def golden(name):
    return np.load(os.path.join(GOLDEN, name))


@pytest.fixture(scope="session")
def hyb(oracle):
    """The codebook the golden vectors were made with: (tlut fp16 bits [512,2], 65,536-entry encoder table)."""
    g = golden("viterbi_ref.npz")
    tl = g["tlut_bits"]
    lut, rms = oracle.build_lut(tl)
    return tl, lut, rms
