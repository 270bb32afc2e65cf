"""``masked_ffn_tp_fused`` on real peers: needs at least two GPUs (skipped otherwise).  The ranks
run as child processes under torch.distributed.run; see ``tp_fused_worker.py``."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

from conftest import TOL

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(nproc, *worker_args, timeout=600):
    env = dict(os.environ, TORCH_SYMM_MEM_DISABLE_MULTICAST="1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(HERE, "tp_fused_worker.py"), *worker_args]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("TP_FUSED ")]
    assert lines, res.stdout[-2000:] + res.stderr[-2000:]
    return json.loads(lines[-1][len("TP_FUSED "):])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("M,d,h,mask", [(1000, 256, 960, "span"), (4100, 512, 1344, "bernoulli")])
def test_two_ranks(M, d, h, mask):
    out = _run(2, "--tokens", str(M), "--dim", str(d), "--hidden", str(h), "--mask-kind", mask)
    assert out["world"] == 2
    assert out["own_rows_equal"]
    assert out["all_ranks_equal"]
    assert out["chunked_equal"]
    assert out["fused_vs_oracle"] < TOL
    assert out["fused_vs_nccl"] < TOL
