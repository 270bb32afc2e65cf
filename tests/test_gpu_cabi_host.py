"""The C ABI from a host that is neither Python nor C++: tests/cabi_host.c (plain C99, cudaMalloc'd
buffers, default stream) routes a mask, runs MaskedLinear forward and the one-call MaskedFFN forward
and checks them against its own float loop."""
import os
import subprocess

import pytest

from ffn_kernel_b200.build import C_HOST, build_c_host

pytestmark = pytest.mark.gpu


def test_plain_c_host_gets_the_same_answers():
    exe = C_HOST if os.path.exists(C_HOST) else build_c_host()
    assert exe and os.path.exists(exe), "tests/cabi_host.c was not built (python -m ffn_kernel_b200.build)"
    res = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "cabi_host: OK" in res.stdout
