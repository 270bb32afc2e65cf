"""Tile-table check: time every kernel variant the library can be forced into on one shape and
print them beside the library's own choice.

The reference searches Triton tile configurations offline and stores the winner in JSON tables
(``find_spec/find.py:18-64``, ``find_spec/bf16_*.py``, ``ffn_kernel/utils.py:3-5``).  Here the tile
table is compiled into the library (``pick_tile``, ``permute_first``, ``gemm_threads_for``,
``pick_group_m`` in csrc); what remains of the search is this script, which re-measures the
alternatives so that the table can be checked when shapes, clocks or drivers change:

    python -m ffn_kernel_b200.tune ffn    --M 16384 --d 4096 --h 11008 [--mask span]
    python -m ffn_kernel_b200.tune linear --M 32768 --K 4096 --N 4096 [--bwd]

Every variant runs in its own process (the overrides are environment variables the library reads
once) through ``ffn_kernel_b200.sweep``, so the numbers are the sweep's: CUDA events on the launching
stream, warm-up first.  Output: one markdown table, times in ms, the fastest entry of each column
in bold, "default" = what the library picks by itself.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

VARIANTS = [
    ("default", {}),
    ("CTA pairs everywhere", {"FFNK_PAIR": "1"}),
    ("single CTAs everywhere", {"FFNK_PAIR": "0"}),
    ("128x64 tiles", {"FFNK_NARROW": "1"}),
    ("128x128 tiles", {"FFNK_NARROW": "2"}),
    ("128x256 tiles only", {"FFNK_NARROW": "0"}),
    ("x copied to routed order first", {"FFNK_PERMUTE": "1"}),
    ("rows gathered in the gate/up GEMM", {"FFNK_PERMUTE": "0"}),
    ("4 epilogue warps", {"FFNK_EPI_WARPS": "4"}),
    ("8 epilogue warps", {"FFNK_EPI_WARPS": "8"}),
    ("super-tile of 8 row tiles", {"FFNK_GROUP_M": "8"}),
    ("super-tile of 16 row tiles", {"FFNK_GROUP_M": "16"}),
    ("super-tile of 48 row tiles", {"FFNK_GROUP_M": "48"}),
    ("weight gradients on single CTAs", {"FFNK_WGRAD_PAIR": "0"}),
    ("no routed-order copies (MaskedLinear)", {"FFNK_LINEAR_COPY": "0"}),
    ("gather4 only (no tiled boxes for runs)", {"FFNK_MAX_RUN_ROWS": "0"}),
]

OVERRIDES = sorted({k for _, env in VARIANTS for k in env})


def run_variant(sweep_args: list[str], env_over: dict[str, str]) -> dict[str, float]:
    env = {k: v for k, v in os.environ.items() if k not in OVERRIDES}
    env.update(env_over)
    res = subprocess.run([sys.executable, "-m", "ffn_kernel_b200.sweep", *sweep_args], env=env, capture_output=True,
                         text=True)
    if res.returncode != 0:
        raise RuntimeError(f"sweep failed with {env_over}: {res.stderr[-2000:]}")
    out = {}
    for line in res.stdout.splitlines():
        try:
            rec = json.loads(line)
        except ValueError:
            continue
        if "kernel" in rec and "ms" in rec:
            out[rec["kernel"]] = float(rec["ms"])
    return out


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["ffn", "linear"])
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--h", type=int, default=11008)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--mask", default="span")
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    sweep_args = [a.what, "--M", str(a.M), "--mask", a.mask, "--iters", str(a.iters)]
    sweep_args += ["--d", str(a.d), "--h", str(a.h)] if a.what == "ffn" else ["--K", str(a.K), "--N", str(a.N)]
    if a.bwd:
        sweep_args.append("--bwd")
    relevant = {"ffn": {"FFNK_PAIR", "FFNK_NARROW", "FFNK_PERMUTE", "FFNK_EPI_WARPS", "FFNK_GROUP_M", "FFNK_WGRAD_PAIR"},
                "linear": {"FFNK_PAIR", "FFNK_NARROW", "FFNK_EPI_WARPS", "FFNK_GROUP_M", "FFNK_WGRAD_PAIR",
                           "FFNK_LINEAR_COPY", "FFNK_MAX_RUN_ROWS"}}[a.what]
    rows = []
    for name, env in VARIANTS:
        if env and not set(env) <= relevant:
            continue
        if "FFNK_WGRAD_PAIR" in env and not a.bwd:
            continue
        rows.append((name, env, run_variant(sweep_args, env)))
    columns = list(rows[0][2])
    best = {c: min(r[2].get(c, float("inf")) for r in rows) for c in columns}
    print("| variant | " + " | ".join(columns) + " |")
    print("|---|" + "---|" * len(columns))
    for name, env, res in rows:
        cells = []
        for c in columns:
            v = res.get(c)
            cells.append("" if v is None else (f"**{v:.4f}**" if v <= best[c] * 1.0005 else f"{v:.4f}"))
        label = name + (" (" + ", ".join(f"{k}={v}" for k, v in env.items()) + ")" if env else "")
        print(f"| {label} | " + " | ".join(cells) + " |")


if __name__ == "__main__":
    main()
