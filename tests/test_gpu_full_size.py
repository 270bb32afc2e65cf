"""The named workloads at their own sizes and masks, and scratch that starts out poisoned.

Full-size results cannot be compared element by element with a CPU oracle in reasonable time, so
these tests use what the operators guarantee: rows are independent (sampled rows against the oracle
on those rows alone) and a column block of a weight gradient is one tall-skinny fp32 product."""
import pytest
import torch

from conftest import TOL
from ffn_kernel_b200 import MaskedFFN, MaskedLinear, check_status
from ffn_kernel_b200._lib import lib
from ffn_kernel_b200.synth import edge_mask, ffn_case, linear_case
from oracle import masked_ref as O

pytestmark = pytest.mark.gpu


def _sample(M, n, seed=1):
    return torch.randperm(M, generator=torch.Generator().manual_seed(seed))[:n].sort().values


def test_linear_backward_at_d4096_m32768_70pct_visual(dev):
    """MaskedLinear forward + backward, M = 32768, K = N = 4096, 70 % visual in 576 / 2304-token spans
    (the reference's per-modality contraction, ffn_kernel/linear.py:329-415): out and dx on 192 sampled
    rows, one 256-column block of each weight gradient against an fp32 CPU product over all rows."""
    M, K, N = 32768, 4096, 4096
    c = linear_case(M, K, N, seed=0, with_grad=True, visual_frac=0.7, image_lens=(576, 2304))
    assert 0.6 < float(c.mask.float().mean()) < 0.8
    g = c.to(dev)
    x = g.x.clone().requires_grad_(True)
    wv, wt = g.wv.clone().requires_grad_(True), g.wt.clone().requires_grad_(True)
    out = MaskedLinear.apply(x, wv.T, wt.T, g.mask)
    out.backward(g.g)
    check_status()
    rows = _sample(M, 192)
    ref_out = O.masked_linear(c.x[rows], c.wv.T, c.wt.T, c.mask[rows])
    ref_dx, _, _ = O.masked_linear_backward(c.g[rows], c.x[rows], c.wv.T, c.wt.T, c.mask[rows])
    assert O.max_rel_err(out[rows.to(dev)], ref_out) < TOL
    assert O.max_rel_err(x.grad[rows.to(dev)], ref_dx) < TOL
    cols = slice(1792, 2048)                          # dW[:, cols] = x_g^T @ g_g[:, cols], logical [K, N]
    xf, gf = c.x.float(), c.g[:, cols].float()
    mv = c.mask.view(-1, 1).float()
    ref_v = (xf * mv).T @ gf
    ref_t = (xf * (1 - mv)).T @ gf
    assert O.max_rel_err(wv.grad.T[:, cols], ref_v) < TOL
    assert O.max_rel_err(wt.grad.T[:, cols], ref_t) < TOL
    assert bool(torch.isfinite(wv.grad.float()).all()) and bool(torch.isfinite(wt.grad.float()).all())


def test_ffn_backward_at_d4096_h11008_m16384(dev):
    """MaskedFFN training step at the LLaMA-7B shape: y and dx on 64 sampled rows against the oracle on those
    rows; a 256-column block of dW2/dU2 (= H_g^T dY_g) against a CPU product over all rows, with H from the
    reference module's own bf16 arithmetic (the GPU's intermediate is bf16 as well)."""
    M, d, h = 16384, 4096, 11008
    c = ffn_case(M, d, h, seed=0)
    gy = torch.randn(M, d, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    g = c.to(dev)
    x = g.x.clone().requires_grad_(True)
    leaves = [w.clone().requires_grad_(True) for w in (g.w1, g.w2, g.w3, g.u1, g.u2, g.u3)]
    y = MaskedFFN.apply(x, *(w.T for w in leaves), g.mask)
    y.backward(gy.to(dev))
    check_status()
    rows = _sample(M, 64)
    a = c.apply_args()
    ref = O.masked_ffn_backward(gy[rows], c.x[rows], *a[1:7], c.mask[rows])
    assert O.max_rel_err(y[rows.to(dev)], O.masked_ffn(c.x[rows], *a[1:7], c.mask[rows])) < TOL
    assert O.max_rel_err(x.grad[rows.to(dev)], ref[0]) < TOL
    assert all(bool(torch.isfinite(w.grad.float()).all()) for w in leaves)
    hid = O.masked_ffn_gateup(c.x, a[1], a[3], a[4], a[6], c.mask, dtype=torch.bfloat16).float()   # [M, h]
    cols = slice(1024, 1280)
    mv = c.mask.view(-1, 1).float()
    gf = gy[:, cols].float()
    assert O.max_rel_err(leaves[1].grad.T[:, cols], (hid * mv).T @ gf) < TOL           # dW2, logical [h, d]
    assert O.max_rel_err(leaves[4].grad.T[:, cols], (hid * (1 - mv)).T @ gf) < TOL     # dU2


@pytest.mark.parametrize("M,d,h", [(16384, 4096, 11008), (32768, 1024, 2048)])
@pytest.mark.parametrize("kind", ["bernoulli", "alternating"])
def test_ffn_forward_full_size_scattered_masks(dev, M, d, h, kind):
    # i.i.d. and per-token alternating masks at the two big FFN shapes: every row tile is gathered from
    # scattered tokens (the reference would compute both branches for every tile, ffn_kernel/ffn.py:86-99)
    c = ffn_case(M, d, h, seed=2, mask=edge_mask(M, kind, seed=5))
    y = MaskedFFN.apply(*c.to(dev).apply_args())
    check_status()
    rows = _sample(M, 128, seed=4)
    a = c.apply_args()
    assert O.max_rel_err(y[rows.to(dev)], O.masked_ffn(c.x[rows], *a[1:7], c.mask[rows])) < TOL
    assert bool(torch.isfinite(y.float()).all())


def _poison(dev, shapes):
    """Leave NaN in the memory the next allocations will be served from: a large block, and blocks of
    exactly the scratch shapes, are filled with NaN and handed back to torch's caching allocator."""
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    big = torch.full((96 << 20,), float("nan"), device=dev, dtype=torch.bfloat16)
    exact = [torch.full(s, float("nan"), device=dev, dtype=torch.bfloat16) for s in shapes for _ in range(3)]
    torch.cuda.synchronize()
    del big, exact


@pytest.mark.parametrize("kind", ["span", "bernoulli", "all_visual"])
def test_linear_train_step_with_poisoned_scratch(dev, kind):
    """The routed-order copies of a and g have rows between the visual and the text group that nothing
    writes; the weight-gradient kernels must not contract over them whatever they contain."""
    M, K, N = 3001, 512, 768
    c = linear_case(M, K, N, seed=5, mask=edge_mask(M, kind, seed=2), with_grad=True)
    rdx, rd1, rd2 = O.masked_linear_backward(c.g, c.x, c.wv.T, c.wt.T, c.mask)
    g = c.to(dev)
    x = g.x.clone().requires_grad_(True)
    wv, wt = g.wv.clone().requires_grad_(True), g.wt.clone().requires_grad_(True)
    cap = int(lib().ffnk_route_capacity(M))
    _poison(dev, [(cap + 512, K), (cap + 512, N), (M, N), (M, K)])
    out = MaskedLinear.apply(x, wv.T, wt.T, g.mask)
    _poison(dev, [(cap + 512, K), (cap + 512, N), (M, N), (M, K)])
    out.backward(g.g)
    check_status()
    for got, ref in ((x.grad, rdx), (wv.grad.T, rd1), (wt.grad.T, rd2)):
        assert bool(torch.isfinite(got.float()).all())
        assert O.max_rel_err(got, ref) < TOL


@pytest.mark.parametrize("kind", ["span", "bernoulli", "all_text"])
def test_ffn_train_step_with_poisoned_scratch(dev, kind):
    M, d, h = 2500, 256, 520
    c = ffn_case(M, d, h, seed=6, mask=edge_mask(M, kind, seed=3))
    gy = torch.randn(M, d, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16)
    ref = O.masked_ffn_backward(gy, *c.apply_args())
    g = c.to(dev)
    x = g.x.clone().requires_grad_(True)
    leaves = [w.clone().requires_grad_(True) for w in (g.w1, g.w2, g.w3, g.u1, g.u2, g.u3)]
    cap = int(lib().ffnk_route_capacity(M))
    shapes = [(cap + 512, d), (cap + 512, h), (M, d)]
    _poison(dev, shapes)
    y = MaskedFFN.apply(x, *(w.T for w in leaves), g.mask)
    _poison(dev, shapes)
    y.backward(gy.to(dev))
    check_status()
    assert bool(torch.isfinite(x.grad.float()).all()) and O.max_rel_err(x.grad, ref[0]) < TOL
    for w, r in zip(leaves, ref[1:]):
        assert bool(torch.isfinite(w.grad.float()).all())
        assert O.max_rel_err(w.grad.T, r) < TOL
