"""Host launchers of the routed MaskedLinear kernels.

Same names and argument meaning as the reference's launchers
(``ffn_kernel/linear.py:418-452`` ``_bf16_linear_forward``,
``ffn_kernel/linear.py:455-496`` ``_bf16_linear_backward``); the Triton kernels and the
JSON tile table behind them are replaced by calls into libffnk.so (hand-written sm_100a
CUDA).  Tile shapes are fixed per kernel in the library, not looked up from a config.
"""
from __future__ import annotations

import os

import torch

from ._lib import check, lib
from .route import Route, _require_cuda, maybe_check, route, status_word, stream_ptr


def _rows_ok(t: torch.Tensor) -> bool:
    return t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.stride(0) >= t.shape[1] and t.data_ptr() % 16 == 0


def _activation(t: torch.Tensor, name: str) -> torch.Tensor:
    """2-D bf16 CUDA activation with 16-byte aligned rows (copied only if it has to be,
    as the reference does with ``.contiguous()``, ``ffn_kernel/linear.py:430``)."""
    _require_cuda(t, name)
    if t.dim() != 2:
        raise RuntimeError(f"{name} must be 2-D, got shape {tuple(t.shape)}")
    if t.dtype != torch.bfloat16:
        raise RuntimeError(f"{name} must be torch.bfloat16, got {t.dtype}")
    return t if _rows_ok(t) else t.contiguous()


def _weight_ok(w: torch.Tensor) -> bool:
    K, N = w.shape
    if w.data_ptr() % 16:
        return False
    if w.stride(0) == 1 and w.stride(1) >= K and w.stride(1) % 8 == 0:
        return True
    return w.stride(1) == 1 and w.stride(0) >= N and w.stride(0) % 8 == 0


def _weights(ws, names, K, N):
    """Logical [K, N] bf16 weights, either the ``nn.Linear.weight.T`` view (stride_k == 1) or
    contiguous (stride_n == 1); both are multiplied from their own storage, no copy is made.

    The kernels take one pair of strides per call (as the reference's launchers do: they pass the
    first weight's strides for all of them, ``ffn_kernel/linear.py:482``, ``ffn_kernel/ffn.py:551``,
    and compute garbage when the others differ).  Weights of one call that do NOT share a layout,
    or a weight that is neither K-major nor N-major with 16-byte aligned rows, are therefore copied
    to contiguous [K, N] here -- the one place a weight is ever copied, and never on the layouts
    the reference's callers use."""
    for w, n in zip(ws, names):
        _require_cuda(w, n)
        if w.dim() != 2 or tuple(w.shape) != (K, N):
            raise RuntimeError(f"{n} must have shape [{K}, {N}], got {tuple(w.shape)}")
        if w.dtype != torch.bfloat16:
            raise RuntimeError(f"{n} must be torch.bfloat16, got {w.dtype}")
    strides = {tuple(w.stride()) for w in ws}
    if len(strides) != 1 or not all(_weight_ok(w) for w in ws):
        ws = [w.contiguous() for w in ws]
    return list(ws)


def _check_dims(**dims):
    for n, v in dims.items():
        if v < 8 or v % 8:
            raise RuntimeError(f"{n} = {v} must be a positive multiple of 8 (16-byte rows of bf16)")


def _mask_route(mask, M, device, rt: Route | None) -> Route:
    if rt is not None:
        if rt.M != M:
            raise RuntimeError(f"route was built for M = {rt.M}, got M = {M}")
        return rt
    _require_cuda(mask, "mask")
    if mask.dim() != 1 or mask.shape[0] != M:
        raise RuntimeError(f"mask must have shape [{M}], got {tuple(mask.shape)}")
    if mask.device != device:
        raise RuntimeError("mask must be on the same device as the activations")
    return route(mask)


def _copy_scratch(M: int, width: int, dev):
    """Scratch for a routed-order copy of an [M, width] activation, or None for small M.

    The forward fills and reads it only when the routing statistics say the mask is scattered
    (runs of same-modality tokens averaging under max(32, columns / 6) rows); masks made of long
    spans never touch it.  The backward always works from routed-order copies when it gets them.
    FFNK_LINEAR_COPY=0 withholds it (the GEMM then always gathers token rows itself)."""
    if os.environ.get("FFNK_LINEAR_COPY", "1") == "0" or M < 512:
        return None
    cap = int(lib().ffnk_route_capacity(M))
    return torch.empty((cap + 512, width), device=dev, dtype=torch.bfloat16)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _bf16_linear_forward(a, b1, b2, mask, rt: Route | None = None):
    """c[m] = a[m] @ (b1 if mask[m] else b2).  a [M,K], b1/b2 [K,N], mask [M] -> [M,N] bf16."""
    a = _activation(a, "a")
    M, K = a.shape
    N = b1.shape[1] if isinstance(b1, torch.Tensor) and b1.dim() == 2 else -1
    b1, b2 = _weights((b1, b2), ("b1", "b2"), K, N)
    _check_dims(K=K, N=N)
    dev = a.device
    with torch.cuda.device(dev):
        c = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
        if M == 0:
            return c
        rt = _mask_route(mask, M, dev, rt)
        a_copy = _copy_scratch(M, K, dev)
        check("ffnk_linear_fwd", lib().ffnk_linear_fwd(
            a.data_ptr(), a.stride(0), b1.data_ptr(), b2.data_ptr(), b1.stride(0), b1.stride(1),
            rt.perm.data_ptr(), rt.counts.data_ptr(), c.data_ptr(), c.stride(0), _ptr(a_copy), M, N, K,
            status_word(dev).data_ptr(), stream_ptr(dev)))
    maybe_check(dev)
    return c


def _bf16_linear_train_forward(a, b1, b2, mask, rt: Route | None = None):
    """Forward pass for training at M >= 512: copies ``a`` into routed order once, multiplies from
    the copy (the kernel of the FFN down projection: whole tiles of consecutive rows, results
    scattered back to token order) and hands the copy to the backward pass, which would otherwise
    make it again.  Returns ``(c, a_routed)``; ``a_routed`` is None when the ordinary forward ran."""
    a = _activation(a, "a")
    M, K = a.shape
    N = b1.shape[1] if isinstance(b1, torch.Tensor) and b1.dim() == 2 else -1
    b1, b2 = _weights((b1, b2), ("b1", "b2"), K, N)
    _check_dims(K=K, N=N)
    dev = a.device
    with torch.cuda.device(dev):
        a_routed = _copy_scratch(M, K, dev) if M > 0 else None
    if a_routed is None:
        return _bf16_linear_forward(a, b1, b2, mask, rt), None
    L = lib()
    with torch.cuda.device(dev):
        c = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
        rt = _mask_route(mask, M, dev, rt)
        st, sp = status_word(dev).data_ptr(), stream_ptr(dev)
        check("ffnk_permute_rows", L.ffnk_permute_rows(
            a.data_ptr(), a.stride(0), rt.perm.data_ptr(), rt.counts.data_ptr(), a_routed.data_ptr(), K, M, K, sp))
        check("ffnk_ffn_down", L.ffnk_ffn_down(
            a_routed.data_ptr(), K, b1.data_ptr(), b2.data_ptr(), b1.stride(0), b1.stride(1), rt.perm.data_ptr(),
            rt.counts.data_ptr(), c.data_ptr(), c.stride(0), M, N, K, st, sp))
    maybe_check(dev)
    return c, a_routed


# Data-parallel training: when set (``tp.GradientSync`` does), ``_bf16_linear_backward`` computes the
# weight gradients first, calls ``GRAD_HOOK(db1, db2)`` -- which starts their all-reduce on another
# stream and returns a function -- launches the dx GEMM beside it, and calls the returned function,
# which makes the launching stream wait for the reduced gradients.  None in normal use.
GRAD_HOOK = None


def _bf16_linear_backward(gd, a, b1, b2, mask, rt: Route | None = None, a_routed=None):
    """Returns (da, db1, db2); db1/db2 carry the strides of b1/b2 (``empty_like``,
    ``ffn_kernel/linear.py:475``).  ``a_routed``: the routed-order copy of ``a`` a training forward
    left behind (``a`` itself is then not needed and may be None)."""
    if a_routed is not None:
        M, K = int(mask.shape[0]), int(a_routed.shape[1])
    else:
        a = _activation(a, "a")
        M, K = a.shape
    N = b1.shape[1] if isinstance(b1, torch.Tensor) and b1.dim() == 2 else -1
    _require_cuda(gd, "grad")
    if tuple(gd.shape) != (M, N):
        raise RuntimeError(f"grad must have shape [{M}, {N}], got {tuple(gd.shape)}")
    gd = _activation(gd, "grad")
    b1, b2 = _weights((b1, b2), ("b1", "b2"), K, N)
    _check_dims(K=K, N=N)
    dev = gd.device
    with torch.cuda.device(dev):
        da = torch.empty((M, K), device=dev, dtype=torch.bfloat16)
        db1, db2 = torch.empty_like(b1), torch.empty_like(b2)
        if tuple(db1.stride()) != tuple(b1.stride()) or tuple(db2.stride()) != tuple(b1.stride()):
            db1 = torch.empty_strided(b1.shape, b1.stride(), device=dev, dtype=torch.bfloat16)
            db2 = torch.empty_strided(b1.shape, b1.stride(), device=dev, dtype=torch.bfloat16)
        if M == 0:
            return da, db1.zero_(), db2.zero_()
        rt = _mask_route(mask, M, dev, rt)
        if a_routed is not None:
            g_copy, a_copy = torch.empty((a_routed.shape[0], N), device=dev, dtype=torch.bfloat16), a_routed
            a_ptr, a_ld = None, K
        else:
            g_copy, a_copy = _copy_scratch(M, N, dev), _copy_scratch(M, K, dev)
            a_ptr, a_ld = a.data_ptr(), a.stride(0)
        args = (gd.data_ptr(), gd.stride(0), a_ptr, a_ld, b1.data_ptr(), b2.data_ptr(),
                b1.stride(0), b1.stride(1), rt.perm.data_ptr(), rt.counts.data_ptr(),
                da.data_ptr(), da.stride(0), db1.data_ptr(), db2.data_ptr(), _ptr(g_copy), _ptr(a_copy), M, N, K)
        tail = (status_word(dev).data_ptr(), stream_ptr(dev))
        if GRAD_HOOK is None:
            check("ffnk_linear_bwd", lib().ffnk_linear_bwd(*args, *tail))
        else:
            check("ffnk_linear_bwd_parts", lib().ffnk_linear_bwd_parts(*args, 1 | 2, *tail))
            finish = GRAD_HOOK(db1, db2)
            try:
                check("ffnk_linear_bwd_parts", lib().ffnk_linear_bwd_parts(*args, 4, *tail))
            finally:
                finish()
    maybe_check(dev)
    return da, db1, db2
