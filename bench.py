#!/usr/bin/env python
"""Benchmark of the routed MaskedFFN forward (d = 4096, h = 11008, M = 16384 tokens) on B200.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference            # the reference's PyTorch module on the host cores

A step is one MaskedFFN forward over one batch of 16384 synthetic tokens: routing scan, gate/up GEMM
with the SwiGLU epilogue, down projection.  ``value`` is routed useful TFLOP/s (6*M*d*h per step: each
token times its own modality's weights only) with inputs resident in HBM; ``e2e`` is the same metric
with the step's activations and mask starting in pinned host memory and the result ending there.
Rank 0 prints one JSON line.

N = 1: the step is ``MaskedFFN.apply``.  The line also carries ``configs``: every other named
workload (d1024/h2048 forward, MaskedLinear d4096 forward / backward / training step, the small-M
sweep at d1024/h2816 by CUDA-graph replay over rotated weight sets, the routing scan) with its time,
rate and fraction of the roofline that bounds it.

N > 1: the batch stays M = 16384 (strong scaling) and the headline is tensor parallel over h, as the
workload is defined: every rank holds h/N of the six weights, x and the mask are replicated, and the
partial outputs are combined so that every rank ends with the full y.  Several implementations of
that combination are timed (NCCL all-reduce; this library's peer-store down projection + barrier +
block sum stored to every rank, whole or in token chunks); the fastest is the headline and all are
listed under ``tp`` together with a parity record (variants against each other and against the CPU
oracle on sampled rows; the run fails above 1e-2).  The same line carries ``dp_strong`` (the same 16384
tokens split by rows over the ranks, replicated weights, no communication), ``dp_weak`` (every rank its
own batch of 16384) and ``configs.c3_dp`` (MaskedLinear d4096 forward + backward token-sharded, with
the weight-gradient all-reduce).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# peer memory is used through plain loads and stores only: keep NVLink multicast objects out of it
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

WORKLOADS = {
    "c4_ffn_d4096_h11008_m16384": dict(M=16384, d=4096, h=11008),
    "c2_ffn_d1024_h2048_m32768": dict(M=32768, d=1024, h=2048),
}
METRIC = "routed_bf16_tflops_maskedffn_fwd"
PARITY_TOL = 1e-2


def measured_traffic():
    """DRAM bytes per launch of the gate/up GEMM from the committed one-pass ncu capture
    (bench_traffic.json: the capture command, its date and the commit it was taken at)."""
    try:
        with open(os.path.join(ROOT, "bench_traffic.json")) as f:
            return json.load(f)
    except Exception:
        return {}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return dict(tflops=float(p["bf16_tflops"]), tflops_sustained=float(p.get("bf16_tflops_sustained", 0)) or None,
                    hbm=float(p["hbm_gbs"]), source="measured")
    except Exception:
        return dict(tflops=1590.0, tflops_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples the SM clock and the clock-event (throttle) reasons while the timed region runs.

    Read-only NVML queries from a thread of this process every few milliseconds (a timed region
    of 20 steps lasts well under 100 ms, less than nvidia-smi needs to print its first line);
    `nvidia-smi -lms` in a child process is the fallback when the NVML binding is missing."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
                   0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.samples = []          # (sm_mhz, reason bit mask, watts)
        self.nvml = None
        self.running = False
        self.source = None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.gpu).uuid)
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu)

    def _poll(self):
        nv, h = self.nvml
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while self.running:
            try:
                self.samples.append((float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), int(reasons_fn(h)),
                                     nv.nvmlDeviceGetPowerUsage(h) / 1000.0))
            except Exception:
                pass
            time.sleep(0.003)

    def start(self):
        try:
            self.nvml = self._nvml_handle()
            self.max_mhz = float(self.nvml[0].nvmlDeviceGetMaxClockInfo(self.nvml[1], self.nvml[0].NVML_CLOCK_SM))
            self.running = True
            self.source = "nvml"
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.source = "nvidia-smi"
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self.running = False
            self.thread.join(timeout=2)
            if not self.samples:
                return dict(sm_mhz=None, sm_max_mhz=self.max_mhz, reasons=["no samples"], source="nvml")
            sm = [v[0] for v in self.samples]
            mask = 0
            for v in self.samples:
                mask |= v[1]
            reasons = sorted(name for bit, name in self.REASON_BITS.items() if mask & bit)
            return dict(sm_mhz=statistics.median(sm), sm_min_mhz=min(sm), sm_max_mhz=self.max_mhz, reasons=reasons,
                        samples=len(sm), watts=statistics.median(v[2] for v in self.samples), source="nvml")
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        busy = [v for v in sm if v > 0.5 * max(sm)] or sm
        return dict(sm_mhz=statistics.median(busy), sm_max_mhz=max(smax), reasons=sorted(reasons), samples=len(sm),
                    source="nvidia-smi")


# ------------------------------------------------------------------------------------------------
# shared by both arms
# ------------------------------------------------------------------------------------------------
def host_threads() -> int:
    """CPU threads this process may use (torchrun exports OMP_NUM_THREADS=1; the affinity mask is the truth)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


def workload_config(workload: str, world: int, mode: str, visual_frac: float) -> dict:
    """The `config` object of the JSON line; the reference arm prints the very same object."""
    wl = WORKLOADS[workload]
    return {"workload": workload, "M": wl["M"], "d": wl["d"], "h": wl["h"],
            "parallelism": f"{mode}{world}",
            "mask": f"image spans of 576 tokens, {visual_frac:.3f} visual",
            "l2": "inputs larger than L2 (activations 128 MiB + weights 516 MiB per step)"
            if workload.startswith("c4") else "inputs larger than L2"}


def headline_mode(world: int, mode_arg: str) -> str:
    return "single" if world == 1 else mode_arg


# ------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's PyTorch module arithmetic on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_reference_rate(case, sample_rows: int, steps: int, warmup: int):
    """bf16 CPU evaluation of the reference module (both branches dense, then mask-select) on the
    first `sample_rows` tokens of the workload.  Returns (useful TFLOP/s, seconds per pass)."""
    from oracle import masked_ref as O
    args = case.apply_args()
    x, mask = args[0][:sample_rows], args[7][:sample_rows]
    d, h = args[1].shape
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.masked_ffn(x, *args[1:7], mask, dtype=torch.bfloat16)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    return 6.0 * sample_rows * d * h / t / 1e12, t


def run_reference(args):
    from ffn_kernel_b200.synth import ffn_case
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cores = args.cpu_threads or host_threads()
    torch.set_num_threads(cores)
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    wl = WORKLOADS[args.workload]
    case = ffn_case(wl["M"], wl["d"], wl["h"], seed=0)
    rows = min(args.cpu_sample_rows, wl["M"])
    tf, sec = cpu_reference_rate(case, rows, max(1, args.steps), max(0, args.warmup))
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.workload, world, headline_mode(world, args.mode),
                                  float(case.mask.float().mean())),
        "tokens_per_s": rows / sec,
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"first {rows} of {wl['M']} tokens per step, full weights; torch CPU bf16 on "
                                   f"{cores} threads, both branches dense then mask-selected as the reference module does"},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
class Bench:
    """State shared by the sections of one run (one rank)."""

    def __init__(self, args):
        import torch.distributed as dist
        self.args = args
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world > 1:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        # host threads: a fair share of the cores for input generation, all of them for rank 0's oracle checks
        self.cores = host_threads()
        torch.set_num_threads(max(1, self.cores // max(1, self.world)))
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.peaks = measured_peaks()

    # -- timing -----------------------------------------------------------------------------------
    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = torch.tensor([v], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def time_steps(self, fn, steps: int, warmup: int, sampler=None) -> float:
        """ms per step: `warmup` untimed calls, then exactly `steps` calls between CUDA events on the
        launching stream, a barrier and a device synchronisation on both sides, maximum over ranks."""
        from ffn_kernel_b200 import check_status
        for _ in range(warmup):
            fn()
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if sampler is not None:
            sampler.samples.clear()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.barrier()
        ms = e0.elapsed_time(e1) / steps
        check_status()
        return self.max_over_ranks(ms)

    def oracle_threads(self):
        """Context: rank 0 uses every host thread while the other ranks wait at a barrier."""
        bench = self

        class _Ctx:
            def __enter__(self):
                self.prev = torch.get_num_threads()
                torch.set_num_threads(bench.cores)

            def __exit__(self, *a):
                torch.set_num_threads(self.prev)
        return _Ctx()


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.float(), b.float()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def graph_replay_ms(fn_list, iters: int = 20, warmup: int = 3) -> float:
    """Time per call of the calls in `fn_list` captured back to back into one CUDA graph (the calls use
    different weight sets so that no call finds its weights in L2) and replayed `iters` times."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for fn in fn_list:
            fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for fn in fn_list:
            fn()
    for _ in range(warmup):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (iters * len(fn_list))


def named_configs(b: Bench) -> dict:
    """Every named workload besides the headline, one GPU: time, rate and roofline fraction each."""
    from ffn_kernel_b200 import MaskedFFN, MaskedLinear, check_status, route
    from ffn_kernel_b200.linear import _bf16_linear_backward, _bf16_linear_forward
    from ffn_kernel_b200.synth import edge_mask, ffn_case, linear_case
    dev, peaks = b.dev, b.peaks
    out = {"peaks": {"bf16_tflops": peaks["tflops"], "hbm_gbs": peaks["hbm"], "source": peaks["source"]},
           "timing": "CUDA events on the launching stream; inputs larger than L2, or (c5, routing at 16384) weight "
                     "sets / masks rotated so that no call finds its operands in L2"}

    def tensor_entry(ms, flops, **extra):
        tf = flops / (ms * 1e-3) / 1e12
        return dict(ms=ms, rate=tf, unit="TFLOP/s", bound="tensor", frac=tf / peaks["tflops"], **extra)

    def hbm_entry(ms, nbytes, **extra):
        gbs = nbytes / (ms * 1e-3) / 1e9
        return dict(ms=ms, rate=gbs, unit="GB/s", bound="hbm", frac=gbs / peaks["hbm"], **extra)

    # C2: MaskedFFN forward d1024 / h2048, M = 32768
    c = ffn_case(32768, 1024, 2048, seed=0).to(dev)
    a = c.apply_args()
    with torch.no_grad():
        ms = b.time_steps(lambda: MaskedFFN.apply(*a), 20, 5)
    out["c2_ffn_fwd"] = tensor_entry(ms, 6.0 * 32768 * 1024 * 2048, tokens_per_s=32768 / (ms * 1e-3))
    del c, a

    # C3: MaskedLinear d4096, M = 32768, 70 % visual in 576 / 2304-token spans
    M, K, N = 32768, 4096, 4096
    lc = linear_case(M, K, N, seed=0, with_grad=True, visual_frac=0.7, image_lens=(576, 2304)).to(dev)
    with torch.no_grad():
        ms_f = b.time_steps(lambda: _bf16_linear_forward(lc.x, lc.wv.T, lc.wt.T, lc.mask), 10, 3)
        ms_b = b.time_steps(lambda: _bf16_linear_backward(lc.g, lc.x, lc.wv.T, lc.wt.T, lc.mask), 10, 3)
    xa = lc.x.clone().requires_grad_(True)
    wv, wt = lc.wv.clone().requires_grad_(True), lc.wt.clone().requires_grad_(True)

    def train_step():
        xa.grad = wv.grad = wt.grad = None
        MaskedLinear.apply(xa, wv.T, wt.T, lc.mask).backward(lc.g)
    ms_t = b.time_steps(train_step, 10, 3)
    vf = float(lc.mask.float().mean())
    out["c3_linear_fwd"] = tensor_entry(ms_f, 2.0 * M * K * N, visual=vf)
    out["c3_linear_bwd"] = tensor_entry(ms_b, 4.0 * M * K * N)
    out["c3_linear_train_step"] = tensor_entry(ms_t, 6.0 * M * K * N, tokens_per_s=M / (ms_t * 1e-3))
    del lc, xa, wv, wt
    torch.cuda.empty_cache()

    # C5: MaskedFFN d1024 / h2816, small and ragged token counts, Bernoulli(0.5) mask.  Five weight sets
    # (173 MB, more than L2) are visited in turn inside one CUDA graph, so every call streams its
    # weights from HBM.  Up to 127 tokens the yardstick is HBM: the weights of every modality present
    # (3*d*h*2 B each) plus the activations in and out.
    d, h, sets = 1024, 2816, 5
    cases = [ffn_case(8, d, h, seed=100 + s).to(dev) for s in range(sets)]
    c5 = {}
    for Mx in (1, 8, 64, 127, 1000, 4099):
        big = ffn_case(Mx, d, h, seed=7, mask=edge_mask(Mx, "bernoulli", seed=Mx))
        x, mask = big.x.to(dev), big.mask.to(dev)
        present = int(bool(mask.any())) + int(bool((~mask).any()))
        with torch.no_grad():
            fns = [(lambda cs=cs: MaskedFFN.apply(x, *cs.apply_args()[1:7], mask)) for cs in cases]
            ms = graph_replay_ms(fns)
        from ffn_kernel_b200.ffn import takes_decode
        path = "one-launch decode kernel" if takes_decode(Mx, d, h) else "routing + row copy, gate/up GEMM, down GEMM"
        if Mx <= 127:
            c5[f"m{Mx}"] = hbm_entry(ms, present * 3.0 * d * h * 2 + 2.0 * Mx * d * 2, modalities_present=present,
                                     path=path)
        else:
            c5[f"m{Mx}"] = tensor_entry(ms, 6.0 * Mx * d * h, path=path)
    out["c5_ffn_fwd_d1024_h2816"] = c5
    del cases

    # routing scan: mask -> two ascending row lists, 5 B per token (1 read + 4 written)
    gen = torch.Generator(device=dev).manual_seed(0)
    masks = [(torch.rand(16384, device=dev, generator=gen) < 0.5) for _ in range(4)]
    with torch.no_grad():
        ms = graph_replay_ms([(lambda m=m: route(m)) for m in masks])
    out["route_m16384"] = hbm_entry(ms, 5.0 * 16384, note="launch bound: 80 KB of traffic")
    big = torch.rand(1 << 26, device=dev, generator=gen) < 0.5
    ms = b.time_steps(lambda: route(big), 5, 2)
    out["route_m67108864"] = hbm_entry(ms, 5.0 * (1 << 26))
    del big
    torch.cuda.empty_cache()
    check_status()
    return out


def bind_to_gpu_cpus(dev_index: int):
    """Run this process on the CPUs NVML lists as local to the GPU, so that pinned buffers allocated
    afterwards land on that NUMA node (first touch).  Returns the CPU count or None if unknown."""
    try:
        import pynvml
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(dev_index).uuid)
        h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(h, 16)
        cpus = {i * 64 + bit for i, w in enumerate(words) for bit in range(64) if (int(w) >> bit) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def run_ours(args):
    from ffn_kernel_b200 import MaskedFFN, MaskedLinear, check_status, tp
    from ffn_kernel_b200 import ffn as ffn_mod
    from ffn_kernel_b200.synth import ffn_case, ffn_tokens, linear_case
    from oracle import masked_ref as O      # the checker: parity records and the CPU baseline only

    b = Bench(args)
    dist, world, rank, dev, peaks = b.dist, b.world, b.rank, b.dev, b.peaks
    wl = WORKLOADS[args.workload]
    M, d, h = wl["M"], wl["d"], wl["h"]
    mode = headline_mode(world, args.mode)
    flops_step = 6.0 * M * d * h
    steps, warmup = args.steps, max(3, args.warmup)

    case_cpu = ffn_case(M, d, h, seed=0)            # the same batch and weights on every rank
    case = case_cpu.to(dev)
    full_args = case.apply_args()
    x, mask = full_args[0], full_args[7]
    weights = full_args[1:7]
    visual_frac = float(case_cpu.mask.float().mean())

    # sampled rows of the oracle: fp32 CPU evaluation of the reference module on bf16-rounded inputs
    g = torch.Generator().manual_seed(1)
    sample_rows = torch.randperm(M, generator=g)[:128].sort().values
    ref_rows = None
    if rank == 0 and not args.skip_parity:
        with b.oracle_threads():
            a_cpu = case_cpu.apply_args()
            ref_rows = O.masked_ffn(a_cpu[0][sample_rows], *a_cpu[1:7], a_cpu[7][sample_rows])

    def vs_oracle(y_rows: torch.Tensor) -> float:
        return rel_err(y_rows.cpu(), ref_rows)

    parity_failures = []
    tp_line = dp_strong = dp_weak = None
    variant_name, kernels_per_step = "MaskedFFN.apply", 4

    # ---- the step of the headline ------------------------------------------------------------------
    if mode == "single":
        def step(xi=x, mi=mask):
            return MaskedFFN.apply(xi, *weights, mi)
    elif mode == "tp":
        w_tp = tp.shard_ffn_weights(*weights, rank, world)      # views of the full weights
        blocks = tp.PeerBlocks(M, d)
        variants = {
            "nccl_all_reduce": (lambda xi=x, mi=mask: tp.masked_ffn_tp(xi, *w_tp, mi), 4,
                                "per-rank MaskedFFN on its h shard, then one NCCL all-reduce of the partial y"),
            "fused_broadcast": (lambda xi=x, mi=mask: tp.masked_ffn_tp_fused(xi, *w_tp, mi, blocks), 7,
                                "down projection stores partial rows into their owner's memory over NVLink; own "
                                "barrier kernel; owner sums in fp32 and stores the rows into every rank's y; barrier"),
            "fused_broadcast_2col": (lambda xi=x, mi=mask: tp.masked_ffn_tp_fused(xi, *w_tp, mi, blocks, col_chunks=2), 9,
                                     "the same with the down projection in two column ranges: barrier, sum and "
                                     "broadcast of a range run on a side stream under the next range's GEMM"),
            "fused_broadcast_4col": (lambda xi=x, mi=mask: tp.masked_ffn_tp_fused(xi, *w_tp, mi, blocks, col_chunks=4), 15,
                                     "the same in four column ranges"),
            "fused_broadcast_2chunks": (lambda xi=x, mi=mask: tp.masked_ffn_tp_fused(xi, *w_tp, mi, blocks, chunks=2),
                                        13, "the same in two token chunks: barrier, sum and broadcast of a chunk "
                                            "run on a side stream under the next chunk's GEMMs"),
            "fused_broadcast_4chunks": (lambda xi=x, mi=mask: tp.masked_ffn_tp_fused(xi, *w_tp, mi, blocks, chunks=4),
                                        25, "the same in four token chunks"),
        }
        tp_steps = max(3, min(steps, 10))
        tp_line = {"scaling": "strong", "steps": tp_steps, "variants": {}}
        results = {}
        with torch.no_grad():
            for name, (fn, nk, what) in variants.items():
                ms = b.time_steps(fn, tp_steps, 3)
                results[name] = fn().clone()
                tp_line["variants"][name] = {"ms_per_step": ms, "value": flops_step / (ms * 1e-3) / 1e12,
                                             "unit": "TFLOP/s", "tokens_per_s": M / (ms * 1e-3), "collective": what}
            # rows left with their owners (no broadcast): what a token-parallel consumer would take
            ms = b.time_steps(lambda: tp.masked_ffn_tp_fused(x, *w_tp, mask, blocks, gather=False), tp_steps, 3)
            rows_own, y_own = tp.masked_ffn_tp_fused(x, *w_tp, mask, blocks, gather=False)
            tp_line["row_sharded_output"] = {"ms_per_step": ms, "value": flops_step / (ms * 1e-3) / 1e12,
                                             "unit": "TFLOP/s", "note": "different result layout: not a candidate"}
        torch.cuda.synchronize()
        check_status()
        # parity: every variant holds the same full y on every rank, within tolerance of each other and the oracle
        par = {}
        base = results["nccl_all_reduce"]
        for name, y in results.items():
            if name != "nccl_all_reduce":
                par[f"{name}_vs_nccl"] = b.max_over_ranks(rel_err(y, base))
        par["row_sharded_vs_fused_rows"] = b.max_over_ranks(rel_err(y_own, results["fused_broadcast"][rows_own]))
        y0 = results["fused_broadcast"].clone()
        dist.broadcast(y0, 0)
        par["fused_ranks_identical"] = b.max_over_ranks(0.0 if torch.equal(y0, results["fused_broadcast"]) else 1.0) == 0.0
        if ref_rows is not None:
            par["nccl_vs_oracle_rows"] = vs_oracle(base[sample_rows.to(dev)])
            par["fused_vs_oracle_rows"] = vs_oracle(results["fused_broadcast"][sample_rows.to(dev)])
            par["fused_2chunks_vs_oracle_rows"] = vs_oracle(results["fused_broadcast_2chunks"][sample_rows.to(dev)])
        par["rows_sampled"] = int(sample_rows.numel())
        par["tolerance"] = PARITY_TOL
        tp_line["parity"] = par
        for k, v in par.items():
            if isinstance(v, float) and k not in ("tolerance",) and not (v < PARITY_TOL):
                parity_failures.append(f"tp.{k} = {v:.3e}")
        if par["fused_ranks_identical"] is False:
            parity_failures.append("tp: ranks hold different results")
        del results, base, y0
        # the fastest implementation that leaves the full y on every rank is the headline
        variant_name = min(tp_line["variants"], key=lambda n: tp_line["variants"][n]["ms_per_step"])
        tp_line["headline_variant"] = variant_name
        step, kernels_per_step, _ = variants[variant_name]
    else:   # dp: the same 16384 tokens split by rows, replicated weights, no communication
        rows = tp.row_shard(M, rank, world)
        xs, ms_ = x[rows].contiguous(), mask[rows].contiguous()

        def step(xi=xs, mi=ms_):
            return MaskedFFN.apply(xi, *weights, mi)
        variant_name = "token-sharded rows, no communication"

    # ---- headline: kernel-resident timing --------------------------------------------------------
    # CUDA events between the phases of the forward are recorded on the launching stream inside the
    # timed region (the library's phase observer; the forward is then launched step by step from
    # Python, the same kernels as the single library call); one step also fills the cycle counters
    # of the CTA-pair kernels.
    rows_dp = tp.row_shard(M, rank, world)
    h_local = h // world if mode == "tp" else h
    probe_rows = (rows_dp.stop - rows_dp.start) if mode == "dp" else M
    chunks_in_step = {"fused_broadcast_2chunks": 2, "fused_broadcast_4chunks": 4}.get(variant_name, 1)
    phase_events = []
    # events made ahead of the timed region: creating one costs the host several microseconds, which shows in
    # a step of 0.8 ms that Python launches kernel by kernel
    event_pool = [torch.cuda.Event(enable_timing=True) for _ in range(8 * steps * chunks_in_step + 8)]

    def hook(name):
        ev = event_pool.pop() if event_pool else torch.cuda.Event(enable_timing=True)
        ev.record()
        phase_events.append((name, ev))

    sampler = ClockSampler(b.local)
    if rank == 0:
        sampler.start()
        if sampler.source != "nvml":
            time.sleep(0.3)
    with torch.no_grad():
        for _ in range(warmup):
            step()
        b.barrier()
        check_status()
        ffn_mod.PHASE_HOOK = hook
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler.samples.clear()            # keep only what is sampled while the timed steps run
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        ffn_mod.PHASE_HOOK = None
        b.barrier()
    ms_per_step = b.max_over_ranks(e0.elapsed_time(e1) / steps)
    clocks = sampler.stop() if rank == 0 else None
    check_status()
    value = flops_step / (ms_per_step * 1e-3) / 1e12
    tokens_per_s = M / (ms_per_step * 1e-3)

    # the SM clock the kernels ran at: cycles counted by the MMA-issuing threads of a CTA-pair kernel
    # over that launch's duration (NVML keeps reporting the granted clock under the power cap)
    in_kernel_mhz = None
    if rank == 0 and mode == "single":
        try:
            from ffn_kernel_b200._lib import lib as _lib
            sms = torch.cuda.get_device_properties(dev).multi_processor_count
            prof = torch.zeros(sms * 8, dtype=torch.int64, device=dev)
            probe = []
            ffn_mod.PHASE_HOOK = lambda name: (probe.append((name, torch.cuda.Event(enable_timing=True))),
                                               probe[-1][1].record())
            _lib().ffnk_debug_profile_buffer(prof.data_ptr())
            with torch.no_grad():
                for _ in range(3):
                    probe.clear()
                    step()
            _lib().ffnk_debug_profile_buffer(None)
            ffn_mod.PHASE_HOOK = None
            torch.cuda.synchronize()
            ev = dict(probe)
            cyc = prof.view(sms, 8)[0::2, 0].double()
            cyc = cyc[cyc > 0]
            dms = ev["down"].elapsed_time(ev["end"])
            if cyc.numel() and dms > 0:
                in_kernel_mhz = float(cyc.mean()) / dms / 1e3
        except Exception as exc:
            if clocks is not None:
                clocks["in_kernel_note"] = f"{type(exc).__name__}: {exc}"[:120]
        finally:
            ffn_mod.PHASE_HOOK = None
    if clocks is not None:
        clocks["sm_mhz_in_kernel"] = in_kernel_mhz

    names = [n for n, _ in phase_events]
    gateup_ms, down_ms, route_ms, permute_ms = [], [], [], []
    for i in range(len(phase_events) - 1):
        n, ev = phase_events[i]
        dt = ev.elapsed_time(phase_events[i + 1][1])
        if n == "gateup" and names[i + 1] == "down":
            gateup_ms.append(dt)
        elif n == "down" and names[i + 1] == "end":
            down_ms.append(dt)
        elif n == "route" and names[i + 1] in ("gateup", "permute"):
            route_ms.append(dt)
        elif n == "permute" and names[i + 1] == "gateup":
            permute_ms.append(dt)
    roofline = None
    if gateup_ms:
        g_ms = statistics.mean(gateup_ms)
        rows_per_launch = probe_rows / chunks_in_step
        achieved = 4.0 * rows_per_launch * d * h_local / (g_ms * 1e-3) / 1e12
        traffic = measured_traffic().get(args.workload) if mode == "single" else None
        roofline = {"bound": "tensor", "kernel": "routed_gemm_kernel, gate/up GEMM with SwiGLU epilogue"
                    + ("" if mode == "single" else f" (one rank's launch: {rows_per_launch:.0f} rows, h shard {h_local})"),
                    "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
                    "peak_source": f"{peaks['source']} burst bf16 (MEASURED_PEAKS.json)",
                    "peak_sustained": peaks["tflops_sustained"],
                    "frac_of_sustained": achieved / peaks["tflops_sustained"] if peaks["tflops_sustained"] else None,
                    "launch_ms": g_ms, "down_launch_ms": statistics.mean(down_ms) if down_ms else None,
                    "route_launch_ms": statistics.mean(route_ms) if route_ms else None,
                    "permute_launch_ms": statistics.mean(permute_ms) if permute_ms else None,
                    "traffic": args.traffic_bytes if args.traffic_bytes is not None
                    else (traffic.get("gateup_dram_bytes") if traffic else None),
                    "traffic_source": None if not traffic else
                    f"one-pass ncu capture of {traffic.get('captured')} at commit {traffic.get('commit')}",
                    "algorithmic_bytes": 2.0 * (rows_per_launch * d + 2 * d * h_local * 2 + rows_per_launch * h_local)}
    # ---- parity of the headline at N = 1 and of the row-sharded mode -----------------------------
    parity = None
    if ref_rows is not None and mode == "single":
        with torch.no_grad():
            y = step()
        parity = {"vs_oracle_rows": vs_oracle(y[sample_rows.to(dev)]), "rows_sampled": int(sample_rows.numel()),
                  "tolerance": PARITY_TOL}
        if not parity["vs_oracle_rows"] < PARITY_TOL:
            parity_failures.append(f"parity.vs_oracle_rows = {parity['vs_oracle_rows']:.3e}")

    # ---- the other sharding of the same batch, and replicas ----------------------------------------
    if world > 1 and not args.skip_modes:
        side_steps = max(3, min(steps, 10))
        rows = tp.row_shard(M, rank, world)
        xs, ms_ = x[rows].contiguous(), mask[rows].contiguous()
        with torch.no_grad():
            ms = b.time_steps(lambda: MaskedFFN.apply(xs, *weights, ms_), side_steps, 3)
            y_shard = MaskedFFN.apply(xs, *weights, ms_)
        dp_strong = {"ms_per_step": ms, "value": flops_step / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                     "tokens_per_s": M / (ms * 1e-3), "scaling": "strong", "steps": side_steps,
                     "what": f"the same {M} tokens, {M // world} rows per rank (tp.row_shard), replicated weights, "
                             "no data-path collective; max over ranks"}
        if ref_rows is not None:
            mine = sample_rows[(sample_rows >= rows.start) & (sample_rows < rows.stop)]
            sel = torch.isin(sample_rows, mine)
            e = rel_err(y_shard[(mine - rows.start).to(dev)].cpu(), ref_rows[sel]) if mine.numel() else 0.0
            dp_strong["parity"] = {"rank0_rows_vs_oracle": e, "rows_sampled": int(mine.numel()), "tolerance": PARITY_TOL}
            if not e < PARITY_TOL:
                parity_failures.append(f"dp_strong.rank0_rows_vs_oracle = {e:.3e}")
        del y_shard
        xw, mw = (x, mask) if rank == 0 else tuple(t.to(dev) for t in ffn_tokens(M, d, seed=rank))
        with torch.no_grad():
            ms = b.time_steps(lambda: MaskedFFN.apply(xw, *weights, mw), side_steps, 3)
        dp_weak = {"ms_per_step": ms, "value": world * flops_step / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                   "tokens_per_s": world * M / (ms * 1e-3), "scaling": "weak", "steps": side_steps,
                   "what": f"every rank its own batch of {M} tokens (replicas of the 1-GPU job)"}
        del xw, mw

    # ---- end to end: inputs start in pinned host memory, the result ends there ---------------------
    e2e = None
    if not args.skip_e2e:
        numa_cpus = bind_to_gpu_cpus(b.local)
        rows = tp.row_shard(M, rank, world)             # at N > 1 every rank feeds and drains its own rows
        n_rows = rows.stop - rows.start
        xh = case_cpu.x[rows].contiguous().pin_memory()
        mh = case_cpu.mask.pin_memory()
        yh = [torch.empty((n_rows, d), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        xd = [torch.empty((M, d), device=dev, dtype=torch.bfloat16) for _ in range(2)]
        md = [torch.empty_like(mask) for _ in range(2)]
        s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def e2e_steps(n, compute=True):
            for i in range(n):
                bb = i & 1
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_done[bb])           # the step that last read this input buffer
                    xd[bb][rows].copy_(xh, non_blocking=True)
                    md[bb].copy_(mh, non_blocking=True)
                    ev_in[bb].record(s_in)
                s_main.wait_event(ev_in[bb])
                if compute:
                    with torch.no_grad():
                        if mode == "tp":
                            # the other ranks' rows of x arrive over NVLink, not from the host
                            dist.all_gather_into_tensor(xd[bb], xd[bb][rows])
                            y = step(xd[bb], md[bb])[rows].clone()    # the full y lives in buffers that are reused
                        elif mode == "dp":
                            y = step(xd[bb][rows], md[bb][rows])
                        else:
                            y = step(xd[bb], md[bb])
                else:
                    y = xd[bb][rows]
                ev_done[bb].record(s_main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[bb])
                    s_out.wait_event(ev_out[bb])           # previous read-back into this host buffer
                    yh[bb].copy_(y, non_blocking=True)
                    ev_out[bb].record(s_out)
                y.record_stream(s_out)

        def timed_e2e(n, compute):
            e2e_steps(max(2, min(warmup, 4)), compute)
            b.barrier()
            t0 = time.perf_counter()
            e2e_steps(n, compute)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            return b.max_over_ranks(time.perf_counter() - t0) / n

        e2e_s = timed_e2e(steps, True)
        floor_s = timed_e2e(max(3, min(steps, 10)), False)
        check_status()
        h2d = int(M * d * 2 + world * M)
        d2h = int(M * d * 2)
        e2e = {"value": flops_step / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_s * 1e3, "tokens_per_s": M / e2e_s,
               "copy_floor_ms": floor_s * 1e3, "compute_ms": ms_per_step,
               "copy_floor_gbs_each_way": max(h2d, d2h) / floor_s / 1e9,
               "frac_of_max_floor_compute": max(floor_s * 1e3, ms_per_step) / (e2e_s * 1e3),
               "cpus_local_to_gpu": numa_cpus,
               "pipeline": "H2D of step i+1, compute of step i and D2H of step i-1 overlap on three streams; "
                           + ("every rank copies its own M/N rows in and out, the rest of x arrives by NVLink all-gather; "
                              if mode == "tp" else "every rank copies its own M/N rows in and out; " if mode == "dp" else "")
                           + "copy_floor_ms is the same loop with the copies only, all ranks at once"}
        del xd, md

    # ---- N = 1: the other named workloads, and the CPU baseline ------------------------------------
    configs = None
    cpu = None
    if world == 1:
        if not args.skip_configs:
            configs = named_configs(b)
        if not args.skip_cpu:
            rows_c = min(args.cpu_sample_rows, M)
            torch.set_num_threads(b.cores)
            tf, sec = cpu_reference_rate(case_cpu, rows_c, steps=5, warmup=1)
            cpu = {"value": tf, "unit": "TFLOP/s", "cores": b.cores, "kind": "port",
                   "sample": f"first {rows_c} of {M} tokens, full weights, median of 5 passes ({sec:.2f} s each); torch CPU "
                             "bf16, both branches dense then mask-selected as the reference module does"}
    elif not args.skip_configs:
        configs = {"c3_dp": c3_token_sharded(b)}
        if "parity_failure" in configs["c3_dp"]:
            parity_failures.append(configs["c3_dp"]["parity_failure"])

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args.workload, world, mode, visual_frac),
            "headline": variant_name, "tokens_per_s": tokens_per_s,
            "frac_of_measured_bf16_peak": value / peaks["tflops"] / world,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks, "parity": parity,
            "tp": tp_line, "dp_strong": dp_strong, "dp_weak": dp_weak, "configs": configs,
            "gpu_launches": kernels_per_step * steps,
        }
        if parity_failures:
            line["parity_failures"] = parity_failures
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if parity_failures:
        raise SystemExit("parity outside tolerance: " + "; ".join(parity_failures))


def c3_token_sharded(b: Bench) -> dict:
    """MaskedLinear forward + backward at d = 4096, M = 32768 (70 % visual), rows split over the ranks:
    no communication on the data path, weight gradients come out as per-rank partial sums; then the
    gradient all-reduce (fp32 buckets over NCCL), plain and overlapped with the dx GEMM."""
    from ffn_kernel_b200 import MaskedLinear, check_status, tp
    from ffn_kernel_b200.linear import _bf16_linear_backward
    from ffn_kernel_b200.synth import linear_case
    dist, world, rank, dev = b.dist, b.world, b.rank, b.dev
    M, K, N = 32768, 4096, 4096
    lc = linear_case(M, K, N, seed=0, with_grad=True, visual_frac=0.7, image_lens=(576, 2304)).to(dev)
    rows = tp.row_shard(M, rank, world)
    xs = lc.x[rows].clone().requires_grad_(True)
    gs, ms_ = lc.g[rows].contiguous(), lc.mask[rows].contiguous()
    wv, wt = lc.wv.clone().requires_grad_(True), lc.wt.clone().requires_grad_(True)

    def train_step():
        xs.grad = wv.grad = wt.grad = None
        MaskedLinear.apply(xs, wv.T, wt.T, ms_).backward(gs)

    n = 10

    def timed(fn, warmup=3):
        # the smaller of two rounds of n steps: a single stall on the host or in the collective library
        # (seen once as 43 ms in a step of 1.7) would otherwise be the figure
        return min(b.time_steps(fn, n, warmup), b.time_steps(fn, n, 1))

    ms = timed(train_step)
    out = {"ms_per_step": ms, "value": 6.0 * M * K * N / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "scaling": "strong",
           "tokens_per_s": M / (ms * 1e-3), "steps": n, "launch": "eager",
           "what": f"MaskedLinear forward + backward, M={M}, K=N={K}, {M // world} rows per rank, no data-path "
                   "collective; max over ranks"}

    # the step followed by the weight-gradient all-reduce, plain (after the backward) ...
    def step_then_allreduce():
        train_step()
        tp.all_reduce_gradients([wv.grad, wt.grad])
    out["with_grad_allreduce_ms"] = timed(step_then_allreduce)

    # ... and launched on a side stream as soon as the weight gradients exist, under the dx GEMM
    sync = tp.GradientSync()

    def step_overlapped():
        xs.grad = wv.grad = wt.grad = None
        with sync:
            MaskedLinear.apply(xs, wv.T, wt.T, ms_).backward(gs)
    out["with_overlapped_grad_allreduce_ms"] = timed(step_overlapped)
    out["allreduce_exposed_ms"] = out["with_overlapped_grad_allreduce_ms"] - ms
    out["allreduce_hidden_ms"] = out["with_grad_allreduce_ms"] - out["with_overlapped_grad_allreduce_ms"]
    # the same with the bf16 gradients all-reduced in place (no fp32 bucket)
    sync_bf16 = tp.GradientSync(reduce_dtype=None)

    def step_overlapped_bf16():
        xs.grad = wv.grad = wt.grad = None
        with sync_bf16:
            MaskedLinear.apply(xs, wv.T, wt.T, ms_).backward(gs)
    out["with_overlapped_bf16_allreduce_ms"] = timed(step_overlapped_bf16)
    step_overlapped_bf16()
    gv16, gt16 = wv.grad.clone(), wt.grad.clone()

    # summed partial gradients against the gradient of the whole batch on one GPU
    step_overlapped()
    gv_sum, gt_sum = wv.grad.clone(), wt.grad.clone()
    dx_shard = xs.grad.clone()
    with torch.no_grad():
        dx_full, gv_full, gt_full = _bf16_linear_backward(lc.g, lc.x, lc.wv.T, lc.wt.T, lc.mask)
    torch.cuda.synchronize()
    check_status()
    err = max(rel_err(gv_sum.T, gv_full), rel_err(gt_sum.T, gt_full))
    out["grad_allreduce_err"] = b.max_over_ranks(err)
    out["grad_allreduce_bf16_err"] = b.max_over_ranks(max(rel_err(gv16.T, gv_full), rel_err(gt16.T, gt_full)))
    out["dx_rows_vs_single_gpu"] = b.max_over_ranks(rel_err(dx_shard, dx_full[rows]))
    if not (out["grad_allreduce_err"] < PARITY_TOL and out["dx_rows_vs_single_gpu"] < PARITY_TOL
            and out["grad_allreduce_bf16_err"] < 2 * PARITY_TOL):
        out["parity_failure"] = (f"c3_dp: grad_allreduce_err {out['grad_allreduce_err']:.3e}, "
                                 f"dx {out['dx_rows_vs_single_gpu']:.3e}")

    # Last, the plain step replayed from a CUDA graph: at 8 GPUs a rank's 4096 rows are 0.35 ms of kernels, about
    # what Python and autograd spend on one call, so the eager figure is host bound and moves with the host's load.
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            train_step()
        gms = timed(graph.replay)
        out.update(eager_ms_per_step=ms, graph_ms_per_step=gms)
        if gms < ms:      # host bound when launched eagerly: the replayed step is the device's time
            out.update(ms_per_step=gms, launch="CUDA graph replay", value=6.0 * M * K * N / (gms * 1e-3) / 1e12,
                       tokens_per_s=M / (gms * 1e-3))
    except Exception as e:  # the capture is a convenience of the measurement, not part of the operator
        out["graph_error"] = f"{type(e).__name__}: {e}"[:200]
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="c4_ffn_d4096_h11008_m16384")
    ap.add_argument("--mode", choices=["tp", "dp"], default="tp",
                    help="headline at N > 1: tensor parallel over h (the workload's definition) or rows split over the ranks")
    ap.add_argument("--cpu-sample-rows", type=int, default=8192,
                    help="tokens per CPU pass (cpu_baseline and --impl reference): about 10-20 s of host work per run")
    ap.add_argument("--cpu-threads", type=int, default=0, help="host threads of --impl reference (0: all the process may use)")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--skip-configs", action="store_true", help="leave out the other named workloads")
    ap.add_argument("--skip-modes", action="store_true", help="N > 1: leave out dp_strong / dp_weak")
    ap.add_argument("--skip-parity", action="store_true", help="leave out the oracle rows (CPU work on rank 0)")
    ap.add_argument("--traffic-bytes", type=float, default=None,
                    help="DRAM bytes per gate/up launch from an ncu capture, overriding bench_traffic.json")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
