"""The operator API: ``MaskedLinear`` and ``MaskedFFN``.

Drop-in for ``ffn_kernel/ops.py:9-38``: same ``torch.autograd.Function`` classes, same
argument order and tensor layouts, same gradients returned
(``(da, db1, db2, None)``, ``ffn_kernel/ops.py:24``).  One extension: ``MaskedFFN.backward``, which
the reference leaves raising ``NotImplementedError`` (``ffn_kernel/ops.py:34-38``), is implemented.
"""
from __future__ import annotations

import threading

import torch
from torch.amp import custom_bwd, custom_fwd
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from .ffn import (_bf16_ffn_backward, _bf16_ffn_forward, _bf16_ffn_fused_forward,  # noqa: F401  (re-exported)
                  _bf16_ffn_train_forward)
from .linear import _bf16_linear_backward, _bf16_linear_forward, _bf16_linear_train_forward
from .route import route

__all__ = ["MaskedLinear", "MaskedFFN"]

# Whether gradients were being recorded when MaskedFFN.apply was called.  Inside Function.forward
# grad mode is always off and ctx.needs_input_grad only says which inputs have requires_grad set
# (true for every nn.Parameter, also under torch.no_grad()), so the caller's grad mode is noted
# on the way in: inference under no_grad must not pay for the training forward.
_call = threading.local()


class MaskedLinear(Function):
    """``MaskedLinear.apply(a, b1, b2, mask)``: ``a[m] @ b1`` where ``mask[m]`` else ``a[m] @ b2``."""

    @classmethod
    def apply(cls, *args, **kwargs):
        _call.grad_enabled = torch.is_grad_enabled()
        return super().apply(*args, **kwargs)

    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, a, b1, b2, mask):
        ctx.b1, ctx.b2 = b1, b2
        rt = route(mask) if a.shape[0] > 0 else None
        ctx.route = rt          # the backward pass reuses the routing lists
        if getattr(_call, "grad_enabled", True) and any(ctx.needs_input_grad[:3]):
            # a backward pass will follow: it gets the routed-order copy of a instead of a itself
            c, a_routed = _bf16_linear_train_forward(a, b1, b2, mask, rt)
            if a_routed is not None:
                ctx.save_for_backward(mask, a_routed)
                ctx.routed = True
                return c
            ctx.save_for_backward(a, mask)
            ctx.routed = False
            return c
        ctx.save_for_backward(a, mask)
        ctx.routed = False
        return _bf16_linear_forward(a, b1, b2, mask, rt)

    @staticmethod
    @once_differentiable
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad):
        b1, b2 = ctx.b1, ctx.b2
        if ctx.routed:
            mask, a_routed = ctx.saved_tensors
            da, db1, db2 = _bf16_linear_backward(grad, None, b1, b2, mask, ctx.route, a_routed=a_routed)
        else:
            a, mask = ctx.saved_tensors
            da, db1, db2 = _bf16_linear_backward(grad, a, b1, b2, mask, ctx.route)
        return da, db1, db2, None


class MaskedFFN(Function):
    """``MaskedFFN.apply(a, w1, w2, w3, u1, u2, u3, mask)``: routed SwiGLU FFN.

    The forward pass is the reference's (``ffn_kernel/ops.py:28-32``).  The reference's backward
    raises ``NotImplementedError`` (``ffn_kernel/ops.py:34-38``, its kernels are unfinished); here
    it is implemented after the reference's own formulas (``README.md:159-172``): when any input
    requires a gradient, the forward keeps the routed activations and pre-activations."""

    @classmethod
    def apply(cls, *args, **kwargs):
        _call.grad_enabled = torch.is_grad_enabled()
        return super().apply(*args, **kwargs)

    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, a, w1, w2, w3, u1, u2, u3, mask):
        if getattr(_call, "grad_enabled", True) and any(ctx.needs_input_grad[:7]):
            y, ctx.saved = _bf16_ffn_train_forward(a, w1, w2, w3, u1, u2, u3, mask)
            return y
        ctx.saved = None
        return _bf16_ffn_fused_forward(a, w1, w2, w3, u1, u2, u3, mask)

    @staticmethod
    @once_differentiable
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad):
        if ctx.saved is None:
            raise RuntimeError("MaskedFFN.backward called but the forward pass saw no input that requires grad")
        grads = _bf16_ffn_backward(grad, ctx.saved)
        ctx.saved = None
        return (*grads, None)
