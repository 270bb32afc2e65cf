"""CPU restatement of the reference's PyTorch modules for the masked path.

TEST INFRASTRUCTURE ONLY: the product never routes through this file.

Parity status: the reference ships no golden vectors, known-answer tests or
tolerances for this path (its ``--check`` mode only prints ``torch.dist``), so
the oracle is pinned against outputs of the reference's own ``Torch`` modules
(``test_linear.py:41-49``, ``test_ffn.py:32-47``) executed on CPU; the vectors
and the script that generated them live in ``tests/golden/``.

What is restated, with the reference lines each function follows:

* ``masked_linear``            -- ``test_linear.py:41-49``: both branches are
  computed densely and selected per token, ``lin_v(x)*m + lin_t(x)*~m``.
  Mask polarity (True selects the first weight set) as in
  ``ffn_kernel/linear.py:137-140``.
* ``masked_linear_backward``   -- autograd through the same module with an
  upstream gradient (``test_linear.py:94-97``), written out in closed form to
  match ``ffn_kernel/linear.py:242-415``: ``dA = where(m, G B1^T, G B2^T)``,
  ``dB1 = A[m]^T G[m]``, ``dB2 = A[~m]^T G[~m]``.
* ``masked_ffn``               -- ``test_ffn.py:32-47``:
  ``w2(silu(w1 x) * w3 x) * m + u2(silu(u1 x) * u3 x) * ~m``.
* ``masked_ffn_backward``      -- autograd through the same expression; the reference states the
  closed form in ``README.md:159-172`` but ships no working kernel for it.
* ``routing``                  -- the compacted per-modality row lists that
  replace the reference's per-tile uniformity test
  (``ffn_kernel/linear.py:132,137``): ``nonzero(mask)`` / ``nonzero(~mask)``.

Weights use the operator API's convention: ``b`` is ``[in, out]`` (the
``weight.T`` view of an ``nn.Linear``), so a branch is ``x @ b``.

``dtype=torch.float32`` gives the parity oracle (inputs are the bf16-rounded
values, arithmetic in fp32); ``dtype=torch.bfloat16`` gives the reference's own
CPU arithmetic, which is what the CPU baseline times.
"""
from __future__ import annotations

import numpy as np
import torch


def routing(mask) -> tuple[np.ndarray, np.ndarray]:
    """Ascending int32 row lists (visual, text) for a 1-D boolean mask."""
    m = np.asarray(mask.detach().cpu().numpy() if isinstance(mask, torch.Tensor) else mask)
    m = m.reshape(-1) != 0
    return (np.flatnonzero(m).astype(np.int32), np.flatnonzero(~m).astype(np.int32))


def _sel(mask: torch.Tensor, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    m = mask.reshape(-1, 1).to(torch.bool)
    return m.to(dtype), (~m).to(dtype)


@torch.no_grad()
def masked_linear(x, b1, b2, mask, dtype=torch.float32) -> torch.Tensor:
    """x [M,K], b1/b2 [K,N], mask [M] -> [M,N]; dense both branches, then select."""
    x, b1, b2 = x.to(dtype), b1.to(dtype), b2.to(dtype)
    mv, mt = _sel(mask, dtype)
    return (x @ b1) * mv + (x @ b2) * mt


@torch.no_grad()
def masked_linear_backward(g, x, b1, b2, mask, dtype=torch.float32):
    """Returns (dx [M,K], db1 [K,N], db2 [K,N]) for upstream gradient g [M,N]."""
    g, x, b1, b2 = g.to(dtype), x.to(dtype), b1.to(dtype), b2.to(dtype)
    mv, mt = _sel(mask, dtype)
    gv, gt = g * mv, g * mt
    dx = gv @ b1.T + gt @ b2.T
    return dx, x.T @ gv, x.T @ gt


@torch.no_grad()
def masked_ffn_gateup(x, w1, w3, u1, u3, mask, dtype=torch.float32) -> torch.Tensor:
    """The SwiGLU intermediate [M,h]: silu(x w1) * (x w3) for visual rows, u1/u3 for text."""
    x = x.to(dtype)
    mv, mt = _sel(mask, dtype)
    pv = torch.nn.functional.silu(x @ w1.to(dtype)) * (x @ w3.to(dtype))
    pt = torch.nn.functional.silu(x @ u1.to(dtype)) * (x @ u3.to(dtype))
    return pv * mv + pt * mt


@torch.no_grad()
def masked_ffn(x, w1, w2, w3, u1, u2, u3, mask, dtype=torch.float32) -> torch.Tensor:
    """Argument order follows ``MaskedFFN.apply`` (``ffn_kernel/ops.py:30``)."""
    x = x.to(dtype)
    mv, mt = _sel(mask, dtype)
    pv = torch.nn.functional.silu(x @ w1.to(dtype)) * (x @ w3.to(dtype))
    pt = torch.nn.functional.silu(x @ u1.to(dtype)) * (x @ u3.to(dtype))
    return (pv @ w2.to(dtype)) * mv + (pt @ u2.to(dtype)) * mt


def masked_ffn_backward(g, x, w1, w2, w3, u1, u2, u3, mask, dtype=torch.float32):
    """Gradients of ``masked_ffn`` for upstream gradient g [M,d], by autograd through the same
    dense-then-select expression as the reference module (``test_ffn.py:41-47``; closed form in
    the reference's ``README.md:159-172``).  Returns (dx, dw1, dw2, dw3, du1, du2, du3), weight
    gradients in the operator's [in, out] orientation."""
    leaves = [t.detach().to(dtype).clone().requires_grad_(True) for t in (x, w1, w2, w3, u1, u2, u3)]
    xx, a1, a2, a3, b1, b2, b3 = leaves
    mv, mt = _sel(mask, dtype)
    pv = torch.nn.functional.silu(xx @ a1) * (xx @ a3)
    pt = torch.nn.functional.silu(xx @ b1) * (xx @ b3)
    y = (pv @ a2) * mv + (pt @ b2) * mt
    return torch.autograd.grad(y, leaves, g.to(dtype))


def max_rel_err(y, ref) -> float:
    """max|y - ref| / max|ref| -- the metric the 1e-2 output tolerance is stated in."""
    y, ref = y.detach().float().cpu(), ref.detach().float().cpu()
    if ref.numel() == 0:
        return 0.0
    denom = float(ref.abs().max())
    return float((y - ref).abs().max()) / (denom if denom > 0 else 1.0)
