"""Host launchers of the routed MaskedFFN kernels.

``_bf16_ffn_forward`` keeps the name, arguments and result of the reference launcher
(``ffn_kernel/ffn.py:527-560``): the SwiGLU intermediate ``silu(x w1) * (x w3)`` (``u1``/``u3``
for text rows) as an [M, h] tensor in token order.  ``_bf16_ffn_fused_forward`` is the whole
``MaskedFFN.forward`` (``ffn_kernel/ops.py:28-32``): it keeps the intermediate in routed
order, so the down projection reads it with plain tiled loads and scatters the result rows
back to token order in its epilogue.
"""
from __future__ import annotations

import os

import torch

from ._lib import check, lib
from .linear import _activation, _check_dims, _mask_route, _weights
from .route import Route, maybe_check, status_word, stream_ptr


def _bf16_ffn_forward(x, w1, w3, u1, u3, mask, rt: Route | None = None):
    """x [M,d]; w1,w3,u1,u3 [d,h]; mask [M] -> [M,h] bf16 in token order."""
    x = _activation(x, "x")
    M, d = x.shape
    h = w1.shape[1] if isinstance(w1, torch.Tensor) and w1.dim() == 2 else -1
    w1, w3, u1, u3 = _weights((w1, w3, u1, u3), ("w1", "w3", "u1", "u3"), d, h)
    _check_dims(d=d, h=h)
    dev = x.device
    with torch.cuda.device(dev):
        out = torch.empty((M, h), device=dev, dtype=torch.bfloat16)
        if M == 0:
            return out
        rt = _mask_route(mask, M, dev, rt)
        check("ffnk_ffn_gateup", lib().ffnk_ffn_gateup(
            x.data_ptr(), x.stride(0), w1.data_ptr(), w3.data_ptr(), u1.data_ptr(), u3.data_ptr(),
            w1.stride(0), w1.stride(1), rt.perm.data_ptr(), rt.counts.data_ptr(), out.data_ptr(), out.stride(0),
            0, 0, M, d, h, status_word(dev).data_ptr(), stream_ptr(dev)))
    maybe_check(dev)
    return out


# Optional observer called with a phase name ("route", "gateup", "down", "end") at the phase
# boundaries of the fused forward, on the launching thread; the benchmark uses it to record
# CUDA events on the launching stream.  None in normal use.
PHASE_HOOK = None


def _phase(name: str) -> None:
    if PHASE_HOOK is not None:
        PHASE_HOOK(name)


def permute_rows_first(M: int, d: int, h: int) -> bool:
    """Tile-table entry of the library for the FFN forward: is x copied into routed order before
    the gate/up GEMM for this shape?  (``ffnk_tune_override("permute", 0/1)`` replaces the choice.)"""
    return bool(lib().ffnk_ffn_permute_first(M, d, h))


def decode_max_tokens() -> int:
    """Largest token count the tile table ever sends to the one-launch decode kernel."""
    return int(lib().ffnk_decode_max_tokens())


def takes_decode(M: int, d: int, h: int) -> bool:
    """Tile-table entry of the library: does a forward of this shape (K-major weights) take the decode kernel?"""
    return bool(lib().ffnk_ffn_takes_decode(M, d, h))


def _bf16_ffn_fused_forward(x, w1, w2, w3, u1, u2, u3, mask, rt: Route | None = None,
                            allow_decode: bool = True):
    """The full forward: y[m] = (silu(x[m] W1) * (x[m] W3)) W2 with the modality's weights.

    Small token counts take the weight-streaming decode kernel, everything else the two
    routed GEMMs.  Argument order follows ``MaskedFFN.apply`` (``ffn_kernel/ops.py:30``)."""
    x = _activation(x, "x")
    M, d = x.shape
    h = w1.shape[1] if isinstance(w1, torch.Tensor) and w1.dim() == 2 else -1
    w1, w3, u1, u3 = _weights((w1, w3, u1, u3), ("w1", "w3", "u1", "u3"), d, h)
    w2, u2 = _weights((w2, u2), ("w2", "u2"), h, d)
    _check_dims(d=d, h=h)
    dev = x.device
    L = lib()
    with torch.cuda.device(dev):
        y = torch.empty((M, d), device=dev, dtype=torch.bfloat16)
        if M == 0:
            return y
        st, sp = status_word(dev).data_ptr(), stream_ptr(dev)
        if rt is None and PHASE_HOOK is None:
            # the normal path: one call into the library does routing, permutation and both GEMMs
            # (or the decode kernel) out of one workspace allocation
            if mask.dim() != 1 or mask.shape[0] != M or mask.device != dev:
                raise RuntimeError(f"mask must have shape [{M}] on {dev}")
            if mask.dtype not in (torch.bool, torch.uint8):
                raise RuntimeError(f"mask must be torch.bool (or uint8), got {mask.dtype}")
            m8 = mask.contiguous()
            nbytes = int(L.ffnk_ffn_workspace_bytes(M, d, h))
            ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
            check("ffnk_ffn_forward", L.ffnk_ffn_forward(
                x.data_ptr(), x.stride(0), w1.data_ptr(), w2.data_ptr(), w3.data_ptr(), u1.data_ptr(),
                u2.data_ptr(), u3.data_ptr(), w1.stride(0), w1.stride(1), w2.stride(0), w2.stride(1),
                m8.data_ptr(), ws.data_ptr(), nbytes, y.data_ptr(), y.stride(0), M, d, h,
                1 if allow_decode else 0, st, sp))
            maybe_check(dev)
            return y
        # step by step (an observer wants the phase boundaries, or the caller brings routing lists)
        if (allow_decode and rt is None and takes_decode(M, d, h) and w1.stride(0) == 1
                and w2.stride(0) == 1):
            if mask.dim() != 1 or mask.shape[0] != M or mask.device != dev:
                raise RuntimeError(f"mask must have shape [{M}] on {dev}")
            m8 = mask.contiguous()
            inter = torch.empty((M, h), device=dev, dtype=torch.bfloat16)
            check("ffnk_ffn_decode", L.ffnk_ffn_decode(
                x.data_ptr(), x.stride(0), w1.data_ptr(), w2.data_ptr(), w3.data_ptr(), u1.data_ptr(),
                u2.data_ptr(), u3.data_ptr(), w1.stride(0), w1.stride(1), w2.stride(0), w2.stride(1),
                m8.data_ptr(), inter.data_ptr(), y.data_ptr(), y.stride(0), M, d, h, st, sp))
            maybe_check(dev)
            return y
        _phase("route")
        rt = _mask_route(mask, M, dev, rt)
        inter = torch.empty((rt.cap + 512, h), device=dev, dtype=torch.bfloat16)
        routed_in = 0
        if permute_rows_first(M, d, h):
            _phase("permute")
            xr = torch.empty((rt.cap + 512, d), device=dev, dtype=torch.bfloat16)
            check("ffnk_permute_rows", L.ffnk_permute_rows(
                x.data_ptr(), x.stride(0), rt.perm.data_ptr(), rt.counts.data_ptr(), xr.data_ptr(), xr.stride(0),
                M, d, sp))
            x, routed_in = xr, 1
        _phase("gateup")
        check("ffnk_ffn_gateup", L.ffnk_ffn_gateup(
            x.data_ptr(), x.stride(0), w1.data_ptr(), w3.data_ptr(), u1.data_ptr(), u3.data_ptr(),
            w1.stride(0), w1.stride(1), rt.perm.data_ptr(), rt.counts.data_ptr(), inter.data_ptr(), inter.stride(0),
            routed_in, 1, M, d, h, st, sp))
        _phase("down")
        check("ffnk_ffn_down", L.ffnk_ffn_down(
            inter.data_ptr(), inter.stride(0), w2.data_ptr(), u2.data_ptr(), w2.stride(0), w2.stride(1),
            rt.perm.data_ptr(), rt.counts.data_ptr(), y.data_ptr(), y.stride(0), M, d, h, st, sp))
        _phase("end")
    maybe_check(dev)
    return y


def _bf16_ffn_train_forward(x, w1, w2, w3, u1, u2, u3, mask):
    """Forward pass that keeps the routed activations for the backward pass.
    Returns ``(y, saved)``; ``saved`` goes to ``_bf16_ffn_backward`` unchanged."""
    x = _activation(x, "x")
    M, d = x.shape
    h = w1.shape[1] if isinstance(w1, torch.Tensor) and w1.dim() == 2 else -1
    w1, w3, u1, u3 = _weights((w1, w3, u1, u3), ("w1", "w3", "u1", "u3"), d, h)
    w2, u2 = _weights((w2, u2), ("w2", "u2"), h, d)
    _check_dims(d=d, h=h)
    dev = x.device
    if not isinstance(mask, torch.Tensor) or mask.dim() != 1 or mask.shape[0] != M or mask.device != dev:
        raise RuntimeError(f"mask must have shape [{M}] on {dev}")
    if mask.dtype not in (torch.bool, torch.uint8):
        raise RuntimeError(f"mask must be torch.bool (or uint8), got {mask.dtype}")
    L = lib()
    with torch.cuda.device(dev):
        y = torch.empty((M, d), device=dev, dtype=torch.bfloat16)
        cap = int(L.ffnk_route_capacity(M))
        rows = cap + 512
        perm = torch.empty(max(2 * cap, 4), dtype=torch.int32, device=dev)
        counts = torch.empty(8, dtype=torch.int32, device=dev)
        xr = torch.empty((rows, d), device=dev, dtype=torch.bfloat16)
        t1, t3, hid = (torch.empty((rows, h), device=dev, dtype=torch.bfloat16) for _ in range(3))
        saved = dict(M=M, d=d, h=h, perm=perm, counts=counts, xr=xr, t1=t1, t3=t3, hid=hid,
                     weights=(w1, w2, w3, u1, u2, u3))
        if M == 0:
            return y, saved
        scan = torch.empty(max(int(L.ffnk_route_workspace_bytes(M)), 4), dtype=torch.uint8, device=dev)
        check("ffnk_ffn_forward_train", L.ffnk_ffn_forward_train(
            x.data_ptr(), x.stride(0), w1.data_ptr(), w2.data_ptr(), w3.data_ptr(), u1.data_ptr(), u2.data_ptr(),
            u3.data_ptr(), w1.stride(0), w1.stride(1), w2.stride(0), w2.stride(1), mask.contiguous().data_ptr(),
            perm.data_ptr(), counts.data_ptr(), scan.data_ptr(), xr.data_ptr(), t1.data_ptr(), t3.data_ptr(),
            hid.data_ptr(), y.data_ptr(), y.stride(0), M, d, h, status_word(dev).data_ptr(), stream_ptr(dev)))
    maybe_check(dev)
    return y, saved


def _bf16_ffn_backward(gy, saved):
    """Gradients ``(dx, dw1, dw2, dw3, du1, du2, du3)``; weight gradients carry their weights' strides."""
    M, d, h = saved["M"], saved["d"], saved["h"]
    w1, w2, w3, u1, u2, u3 = saved["weights"]
    dev = saved["xr"].device
    if tuple(gy.shape) != (M, d):
        raise RuntimeError(f"grad must have shape [{M}, {d}], got {tuple(gy.shape)}")
    gy = _activation(gy, "grad")
    L = lib()
    with torch.cuda.device(dev):
        dx = torch.empty((M, d), device=dev, dtype=torch.bfloat16)
        grads = [torch.empty_strided(w.shape, w.stride(), device=dev, dtype=torch.bfloat16)
                 for w in (w1, w2, w3, u1, u2, u3)]
        if M == 0:
            return (dx, *[g.zero_() for g in grads])
        rows = saved["xr"].shape[0]
        gr = torch.empty((rows, d), device=dev, dtype=torch.bfloat16)
        dt1, dt3 = (torch.empty((rows, h), device=dev, dtype=torch.bfloat16) for _ in range(2))
        check("ffnk_ffn_backward", L.ffnk_ffn_backward(
            gy.data_ptr(), gy.stride(0), saved["xr"].data_ptr(), saved["t1"].data_ptr(), saved["t3"].data_ptr(),
            saved["hid"].data_ptr(), w1.data_ptr(), w2.data_ptr(), w3.data_ptr(), u1.data_ptr(), u2.data_ptr(),
            u3.data_ptr(), w1.stride(0), w1.stride(1), w2.stride(0), w2.stride(1), saved["perm"].data_ptr(),
            saved["counts"].data_ptr(), gr.data_ptr(), dt1.data_ptr(), dt3.data_ptr(), dx.data_ptr(), dx.stride(0),
            *[g.data_ptr() for g in grads], M, d, h, status_word(dev).data_ptr(), stream_ptr(dev)))
    maybe_check(dev)
    return (dx, *grads)
