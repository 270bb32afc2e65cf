"""Per-kernel timing sweep: the tool behind the tile table and the committed profile summaries.

    python -m ffn_kernel_b200.sweep ffn      --M 16384 --d 4096 --h 11008 [--mask span]
    python -m ffn_kernel_b200.sweep linear   --M 32768 --K 4096 --N 4096 [--mask span] [--bwd]
    python -m ffn_kernel_b200.sweep route    --M 67108864
    python -m ffn_kernel_b200.sweep decode   --M 8 --d 1024 --h 2816 [--mask alternating]
    FFNK_PAIR=1 python -m ffn_kernel_b200.sweep waits --M 16384 --d 4096 --h 11008
        (wait-cycle counters of the CTA-pair GEMM kernels: who waits for whom, and the SM clock)
    python -m ffn_kernel_b200.sweep paths    --d 1024 --h 2816 --tokens 8,32,64,127,256
        (small token counts: the decode kernel, the GEMM path and the GEMM path without its split-K down
         projection, each as one library call replayed from a CUDA graph over rotated weight sets)

Each kernel is launched through the C ABI and timed with CUDA events on the launching stream
(warm-up first, inputs larger than L2 or rotated over several copies).  One JSON line per kernel.
The environment variable FFNK_MAX_RUN_ROWS (0, 4, 8, ..., 128) caps the height of the tiled TMA
boxes used for runs of consecutive tokens; 0 forces gather4 everywhere.  It replaces the reference's
offline search (``find_spec/find.py:18-64``): there is nothing to search, only choices to measure.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import check_status, route
from ._lib import lib
from .ffn import _bf16_ffn_fused_forward
from .linear import _bf16_linear_backward, _bf16_linear_forward
from .route import status_word, stream_ptr
from .synth import edge_mask, ffn_case, linear_case


def timeit(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def emit(**kw):
    kw["max_run_rows"] = os.environ.get("FFNK_MAX_RUN_ROWS", "128")
    print(json.dumps(kw), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["ffn", "linear", "route", "decode", "once", "waits", "paths"])
    ap.add_argument("--tokens", default="8,32,64,127,256", help="paths: token counts, comma separated")
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--d", type=int, default=4096)
    ap.add_argument("--h", type=int, default=11008)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--mask", default="span")
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--decode", action="store_true", help="once: let small token counts take the decode kernel")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda", torch.cuda.current_device())
    L = lib()
    st, sp = status_word(dev).data_ptr(), stream_ptr(dev)

    if a.what == "paths":
        # The table entries for small token counts, measured: every path as the single library call,
        # replayed from a CUDA graph that visits enough weight sets to overflow L2 (so each call streams
        # its weights from HBM), Bernoulli(0.5) mask unless --mask says otherwise.
        d, h = a.d, a.h
        kind = "bernoulli" if a.mask == "span" else a.mask
        sets = max(2, min(6, int(200e6 // (12 * d * h)) + 1))
        capacity = int(L.ffnk_decode_capacity())

        def replay_us(fns):
            for fn in fns:
                fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for fn in fns:
                    fn()
            return timeit(g.replay, a.iters, a.warmup) / len(fns) * 1e3

        def decode_call(cs, M, inter, y):
            L.ffnk_ffn_decode(cs.x.data_ptr(), d, cs.w1.data_ptr(), cs.w2.data_ptr(), cs.w3.data_ptr(), cs.u1.data_ptr(),
                              cs.u2.data_ptr(), cs.u3.data_ptr(), 1, d, 1, h, cs.mask.data_ptr(), inter.data_ptr(),
                              y.data_ptr(), d, M, d, h, st, stream_ptr(dev))   # the stream current now (the capture's)

        for M in [int(t) for t in a.tokens.split(",") if t]:
            cases = [ffn_case(M, d, h, seed=100 + i, mask=edge_mask(M, kind, seed=M)).to(dev) for i in range(sets)]
            row = dict(kernel="ffn_forward paths", M=M, d=d, h=h, mask=kind, weight_sets=sets,
                       table_takes_decode=bool(L.ffnk_ffn_takes_decode(M, d, h)))
            with torch.no_grad():
                if M <= capacity:
                    inter = torch.empty((M, h), device=dev, dtype=torch.bfloat16)
                    y = torch.empty((M, d), device=dev, dtype=torch.bfloat16)
                    row["decode_us"] = replay_us([(lambda cs=cs: decode_call(cs, M, inter, y)) for cs in cases])
                gemm = [(lambda cs=cs: _bf16_ffn_fused_forward(*cs.apply_args(), allow_decode=False)) for cs in cases]
                row["gemm_us"] = replay_us(gemm)
                L.ffnk_tune_override(b"ksplit", 0)
                try:
                    row["gemm_no_splitk_us"] = replay_us(gemm)
                finally:
                    L.ffnk_tune_override(b"ksplit", -1)
            check_status()
            emit(**{k: (round(v, 2) if isinstance(v, float) else v) for k, v in row.items()})
            del cases
        return

    if a.what == "waits" and a.bwd:
        # weight-gradient kernel of the MaskedLinear backward: who waits for whom
        M, K, N = a.M, a.K, a.N
        c = linear_case(M, K, N, seed=0, mask=edge_mask(M, a.mask, 0)).to(dev)
        g = torch.randn((M, N), device=dev, dtype=torch.bfloat16)
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        prof = torch.zeros(sms * 8, dtype=torch.int64, device=dev)
        for _ in range(a.warmup):
            _bf16_linear_backward(g, c.x, c.wv.T, c.wt.T, c.mask)
        torch.cuda.synchronize()
        L.ffnk_debug_profile_buffer(prof.data_ptr())
        ms = timeit(lambda: _bf16_linear_backward(g, c.x, c.wv.T, c.wt.T, c.mask), 1, 0)
        L.ffnk_debug_profile_buffer(None)
        p = prof.view(sms, 8).cpu().double()
        tot = float(p[:, 0].mean())
        emit(kernel="wgrad (inside linear_bwd)", M=M, K=K, N=N, mask=a.mask, bwd_ms=ms, mma_cycles=tot,
             mma_wait_operands_pct=100 * float(p[:, 1].mean()) / tot,
             mma_wait_accumulator_pct=100 * float(p[:, 2].mean()) / tot,
             producer_wait_stage_pct=100 * float(p[:, 3].mean() / p[:, 4].mean()),
             tiles_per_cta=float(p[:, 7].mean()), mma_cycles_min=float(p[:, 0].min()), mma_cycles_max=float(p[:, 0].max()))
        check_status()
        return

    if a.what == "waits":
        M, d, h = a.M, a.d, a.h
        c = ffn_case(M, d, h, seed=0, mask=edge_mask(M, a.mask, 0)).to(dev)
        rt = route(c.mask)
        inter = torch.empty((rt.cap + 512, h), device=dev, dtype=torch.bfloat16)
        y = torch.empty((M, d), device=dev, dtype=torch.bfloat16)
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        prof = torch.zeros(sms * 8, dtype=torch.int64, device=dev)
        xr = torch.empty((rt.cap + 512, d), device=dev, dtype=torch.bfloat16)
        L.ffnk_permute_rows(c.x.data_ptr(), d, rt.perm.data_ptr(), rt.counts.data_ptr(), xr.data_ptr(), d, M, d, sp)
        launches = {
            "ffn_gateup(gather in kernel)": lambda: L.ffnk_ffn_gateup(
                c.x.data_ptr(), d, c.w1.data_ptr(), c.w3.data_ptr(), c.u1.data_ptr(), c.u3.data_ptr(), 1, d,
                rt.perm.data_ptr(), rt.counts.data_ptr(), inter.data_ptr(), h, 0, 1, M, d, h, st, sp),
            "ffn_gateup(routed input)": lambda: L.ffnk_ffn_gateup(
                xr.data_ptr(), d, c.w1.data_ptr(), c.w3.data_ptr(), c.u1.data_ptr(), c.u3.data_ptr(), 1, d,
                rt.perm.data_ptr(), rt.counts.data_ptr(), inter.data_ptr(), h, 1, 1, M, d, h, st, sp),
            "ffn_down": lambda: L.ffnk_ffn_down(
                inter.data_ptr(), h, c.w2.data_ptr(), c.u2.data_ptr(), 1, h, rt.perm.data_ptr(), rt.counts.data_ptr(),
                y.data_ptr(), d, M, d, h, st, sp),
        }
        for name, fn in launches.items():
            for _ in range(a.warmup):
                fn()
            torch.cuda.synchronize()
            prof.zero_()
            L.ffnk_debug_profile_buffer(prof.data_ptr())
            ms = timeit(fn, 1, 0)
            L.ffnk_debug_profile_buffer(None)
            p = prof.view(sms, 8).cpu().double()
            if float(p[1::2, 0].sum()) > 0:
                # single-CTA kernel: every CTA issues MMAs; only the MMA issuer keeps counters
                tot = float(p[:, 0].mean())
                emit(kernel=name + " [single CTA]", M=M, d=d, h=h, mask=a.mask, ms=ms, mma_cycles=tot,
                     sm_mhz=tot / ms / 1e3, mma_wait_operands_pct=100 * float(p[:, 1].mean()) / tot,
                     mma_wait_accumulator_pct=100 * float(p[:, 2].mean()) / tot, tiles_per_cta=float(p[:, 7].mean()))
                continue
            lead = p[0::2]
            tot = float(lead[:, 0].mean())
            emit(kernel=name, M=M, d=d, h=h, mask=a.mask, ms=ms, mma_cycles=tot, sm_mhz=tot / ms / 1e3,
                 mma_wait_operands_pct=100 * float(lead[:, 1].mean()) / tot,
                 mma_wait_accumulator_pct=100 * float(lead[:, 2].mean()) / tot,
                 producer_wait_stage_pct=100 * float(p[:, 3].mean() / p[:, 4].mean()),
                 epilogue_wait_accumulator_pct=100 * float(p[:, 5].mean() / p[:, 6].mean()),
                 tiles_per_pair=float(lead[:, 7].mean()))
        check_status()
        return

    if a.what in ("ffn", "once"):
        M, d, h = a.M, a.d, a.h
        c = ffn_case(M, d, h, seed=0, mask=edge_mask(M, a.mask, 0)).to(dev)
        if a.what == "once":          # a couple of plain forward passes: the command ncu captures
            for _ in range(2):
                _bf16_ffn_fused_forward(*c.apply_args(), allow_decode=a.decode)
            torch.cuda.synchronize()
            check_status()
            return
        rt = route(c.mask)
        inter = torch.empty((rt.cap + 512, h), device=dev, dtype=torch.bfloat16)
        y = torch.empty((M, d), device=dev, dtype=torch.bfloat16)

        def gateup():
            L.ffnk_ffn_gateup(c.x.data_ptr(), d, c.w1.data_ptr(), c.w3.data_ptr(), c.u1.data_ptr(), c.u3.data_ptr(),
                              1, d, rt.perm.data_ptr(), rt.counts.data_ptr(), inter.data_ptr(), h, 0, 1, M, d, h, st, sp)

        def down():
            L.ffnk_ffn_down(inter.data_ptr(), h, c.w2.data_ptr(), c.u2.data_ptr(), 1, h, rt.perm.data_ptr(),
                            rt.counts.data_ptr(), y.data_ptr(), d, M, d, h, st, sp)

        xr = torch.empty((rt.cap + 512, d), device=dev, dtype=torch.bfloat16)

        def permute():
            L.ffnk_permute_rows(c.x.data_ptr(), d, rt.perm.data_ptr(), rt.counts.data_ptr(), xr.data_ptr(), d, M, d, sp)

        def gateup_routed():
            L.ffnk_ffn_gateup(xr.data_ptr(), d, c.w1.data_ptr(), c.w3.data_ptr(), c.u1.data_ptr(), c.u3.data_ptr(),
                              1, d, rt.perm.data_ptr(), rt.counts.data_ptr(), inter.data_ptr(), h, 1, 1, M, d, h, st, sp)

        t = timeit(gateup, a.iters, a.warmup)
        emit(kernel="ffn_gateup(gather in kernel)", M=M, d=d, h=h, mask=a.mask, ms=t, tflops=4 * M * d * h / t / 1e9)
        t = timeit(permute, a.iters, a.warmup)
        emit(kernel="permute_rows", M=M, d=d, mask=a.mask, ms=t, gbs=4 * M * d / t / 1e6)
        t = timeit(gateup_routed, a.iters, a.warmup)
        emit(kernel="ffn_gateup(routed input)", M=M, d=d, h=h, mask=a.mask, ms=t, tflops=4 * M * d * h / t / 1e9)
        t = timeit(down, a.iters, a.warmup)
        emit(kernel="ffn_down", M=M, d=d, h=h, mask=a.mask, ms=t, tflops=2 * M * d * h / t / 1e9)
        t = timeit(lambda: _bf16_ffn_fused_forward(*c.apply_args(), allow_decode=False), a.iters, a.warmup)
        emit(kernel="ffn_forward(Python API, one library call)", M=M, d=d, h=h, mask=a.mask, ms=t,
             tflops=6 * M * d * h / t / 1e9, weight_gbs=6 * d * h * 2 / t / 1e6)
        if a.bwd:
            from .ffn import _bf16_ffn_backward, _bf16_ffn_train_forward
            gy = torch.randn(M, d, device=dev, dtype=torch.bfloat16)
            t = timeit(lambda: _bf16_ffn_train_forward(*c.apply_args()), a.iters, a.warmup)
            emit(kernel="ffn_forward_train(saves t1, t3, hid)", M=M, d=d, h=h, mask=a.mask, ms=t,
                 tflops=6 * M * d * h / t / 1e9)
            _, saved = _bf16_ffn_train_forward(*c.apply_args())
            t = timeit(lambda: _bf16_ffn_backward(gy, saved), max(3, a.iters // 2), a.warmup)
            emit(kernel="ffn_backward(dx + six dW)", M=M, d=d, h=h, mask=a.mask, ms=t,
                 tflops=12 * M * d * h / t / 1e9)
            del saved
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            _bf16_ffn_fused_forward(*c.apply_args(), allow_decode=False)
        t = timeit(g.replay, a.iters, a.warmup)
        emit(kernel="ffn_forward(CUDA graph replay)", M=M, d=d, h=h, mask=a.mask, ms=t,
             tflops=6 * M * d * h / t / 1e9, weight_gbs=6 * d * h * 2 / t / 1e6)
    elif a.what == "linear":
        M, K, N = a.M, a.K, a.N
        c = linear_case(M, K, N, seed=0, mask=edge_mask(M, a.mask, 0), with_grad=True).to(dev)
        rt = route(c.mask)
        t = timeit(lambda: _bf16_linear_forward(c.x, c.wv.T, c.wt.T, c.mask, rt), a.iters, a.warmup)
        emit(kernel="linear_fwd", M=M, K=K, N=N, mask=a.mask, ms=t, tflops=2 * M * K * N / t / 1e9)
        if a.bwd:
            t = timeit(lambda: _bf16_linear_backward(c.g, c.x, c.wv.T, c.wt.T, c.mask, rt), a.iters, a.warmup)
            emit(kernel="linear_bwd(dx+dW)", M=M, K=K, N=N, mask=a.mask, ms=t, tflops=4 * M * K * N / t / 1e9)
            # the whole training step through the operator: routing, forward, backward (the forward's
            # routed-order copy of the activations is reused by the backward)
            from .ops import MaskedLinear
            x = c.x.clone().requires_grad_(True)
            wv, wt = c.wv.clone().requires_grad_(True), c.wt.clone().requires_grad_(True)

            def train_step():
                x.grad = wv.grad = wt.grad = None
                MaskedLinear.apply(x, wv.T, wt.T, c.mask).backward(c.g)

            t = timeit(train_step, a.iters, a.warmup)
            emit(kernel="linear train step (apply + backward)", M=M, K=K, N=N, mask=a.mask, ms=t,
                 tflops=6 * M * K * N / t / 1e9)
    elif a.what == "route":
        m = edge_mask(a.M, "bernoulli" if a.mask == "span" and a.M > (1 << 22) else a.mask, 0).to(dev)
        t = timeit(lambda: route(m), a.iters, a.warmup)
        emit(kernel="route", M=a.M, ms=t, gbs=5 * a.M / t / 1e6)
    elif a.what == "decode":
        M, d, h = a.M, a.d, a.h
        # rotate over enough weight sets that the stream comes from HBM, not from L2
        n_sets = max(2, int(300e6 // (6 * d * h * 2)) + 1)
        cases = [ffn_case(M, d, h, seed=s, mask=edge_mask(M, a.mask, 0)).to(dev) for s in range(n_sets)]
        args = [cs.apply_args() for cs in cases]
        g = torch.cuda.CUDAGraph()
        for ar in args:
            _bf16_ffn_fused_forward(*ar)
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            for ar in args:
                _bf16_ffn_fused_forward(*ar)
        t = timeit(g.replay, a.iters, a.warmup) / n_sets
        present = (1 if bool(cases[0].mask.any()) else 0) + (1 if bool((~cases[0].mask).any()) else 0)
        emit(kernel="ffn_decode(one launch)", M=M, d=d, h=h, mask=a.mask, ms=t, weight_sets=n_sets,
             gbs=present * 3 * d * h * 2 / t / 1e6)
    check_status()


if __name__ == "__main__":
    main()
