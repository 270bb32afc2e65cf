"""The operator API: ``MaskedLinear`` and ``MaskedFFN``.

Drop-in for ``ffn_kernel/ops.py:9-38``: same ``torch.autograd.Function`` classes, same
argument order and tensor layouts, same gradients returned
(``(da, db1, db2, None)``, ``ffn_kernel/ops.py:24``), and ``MaskedFFN.backward`` raises
``NotImplementedError`` exactly as the reference does (``ffn_kernel/ops.py:34-38``).
"""
from __future__ import annotations

from torch.amp import custom_bwd, custom_fwd
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from .ffn import _bf16_ffn_forward, _bf16_ffn_fused_forward  # noqa: F401  (re-exported)
from .linear import _bf16_linear_backward, _bf16_linear_forward
from .route import route

__all__ = ["MaskedLinear", "MaskedFFN"]


class MaskedLinear(Function):
    """``MaskedLinear.apply(a, b1, b2, mask)``: ``a[m] @ b1`` where ``mask[m]`` else ``a[m] @ b2``."""

    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, a, b1, b2, mask):
        ctx.save_for_backward(a, mask)
        ctx.b1, ctx.b2 = b1, b2
        rt = route(mask) if a.shape[0] > 0 else None
        ctx.route = rt          # the backward pass reuses the routing lists
        return _bf16_linear_forward(a, b1, b2, mask, rt)

    @staticmethod
    @once_differentiable
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad):
        a, mask = ctx.saved_tensors
        b1, b2 = ctx.b1, ctx.b2
        da, db1, db2 = _bf16_linear_backward(grad, a, b1, b2, mask, ctx.route)
        return da, db1, db2, None


class MaskedFFN(Function):
    """``MaskedFFN.apply(a, w1, w2, w3, u1, u2, u3, mask)``: routed SwiGLU FFN, forward only."""

    @staticmethod
    @custom_fwd(device_type="cuda")
    def forward(ctx, a, w1, w2, w3, u1, u2, u3, mask):
        return _bf16_ffn_fused_forward(a, w1, w2, w3, u1, u2, u3, mask)

    @staticmethod
    @once_differentiable
    @custom_bwd(device_type="cuda")
    def backward(ctx, grad):
        raise NotImplementedError
