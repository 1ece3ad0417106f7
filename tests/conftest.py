import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")
    # A fresh checkout has no built library (build products are not tracked): compile it once, where nvcc is present.
    # This is the package's own build step, not a fallback: without the library the package still refuses to load.
    import shutil
    lib = ROOT / "fast_polynomial_transcendentals_b200" / "libfpt_b200.so"
    compat = ROOT / "fast_polynomial_transcendentals_b200" / "libfpt_b200_compat.so"
    if not (lib.exists() and compat.exists()) and (shutil.which("nvcc") or Path("/usr/local/cuda/bin/nvcc").exists()):
        from fast_polynomial_transcendentals_b200 import build
        build.build()


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as module
    module.build()
    return module


@pytest.fixture(scope="session")
def fpt():
    """The loaded C-ABI library (ctypes)."""
    from fast_polynomial_transcendentals_b200 import _lib
    return _lib


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def ref_kernels():
    """The reference's own CUDA kernels compiled by oracle/Makefile (present only where that was run)."""
    import ctypes
    path = ROOT / "oracle" / "_ref" / "libref_spline_kernels.so"
    if not path.exists():
        pytest.skip("oracle/_ref/libref_spline_kernels.so not built")
    return ctypes.CDLL(str(path))
