"""The reference arm of bench.py on the host cores: one JSON line with the contract's keys, the same
`config` object the GPU arm prints for the same launch, and every host thread in use even when the
launcher exports OMP_NUM_THREADS=1 (as torch.distributed.run does)."""
import json
import os
import subprocess
import sys

from conftest import ROOT


def _run(env_extra, *args):
    env = dict(os.environ, **env_extra)
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--cpu-sample-rows", "64", *args],
                         capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    return lines


def test_reference_arm_line_and_config():
    sys.path.insert(0, ROOT)
    import bench
    lines = _run({"OMP_NUM_THREADS": "1", "WORLD_SIZE": "8", "RANK": "0"}, "--gpus", "8")
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["metric"] == bench.METRIC and d["n_gpus"] == 8
    assert d["cpu_baseline"]["cores"] == bench.host_threads() and d["cpu_baseline"]["kind"] == "port"
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"]
    # the GPU arm builds its config with the same function from the same launch parameters
    visual = float(d["config"]["mask"].split(",")[1].split()[0])
    assert d["config"] == bench.workload_config("c4_ffn_d4096_h11008_m16384", 8, bench.headline_mode(8, "tp"), visual)
    assert d["config"]["parallelism"] == "tp8"


def test_reference_arm_other_ranks_print_nothing():
    assert _run({"WORLD_SIZE": "2", "RANK": "1"}, "--gpus", "2") == []
