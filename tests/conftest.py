import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")

# tolerance of every floating-point parity check: max|y - ref| / max|ref| against the fp32 oracle
TOL = 1e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def libffnk():
    """The built C-ABI library (compiled on first use if the .so is missing)."""
    from ffn_kernel_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.lib()


@pytest.fixture(scope="session")
def dev(libffnk):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU fallback to test instead")
    return torch.device("cuda:0")


def bf16_from_u16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.astype(np.uint16).view(np.int16).copy()).view(torch.bfloat16)


def load_golden(name: str) -> dict:
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = {}
    for k in z.files:
        a = z[k]
        if a.dtype == np.uint16:
            out[k] = bf16_from_u16(a)
        elif a.dtype == np.bool_:
            out[k] = torch.from_numpy(a.copy())
        else:
            out[k] = torch.from_numpy(a.astype(np.float32))
    return out


LINEAR_GOLDEN = ("linear_b2_s192_k64_n96", "linear_b1_s200_k128_n192")
FFN_GOLDEN = ("ffn_b2_s160_d64_h160", "ffn_b1_s257_d128_h256")
