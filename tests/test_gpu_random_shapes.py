"""Seeded random shapes, masks and weight layouts: tile tails in every dimension (rows per
modality around multiples of 128 and 256, K and N that are multiples of 8 but not of 64),
empty modalities, strided activations.  Every case is checked against the fp32 CPU oracle."""
import os
import random

import pytest
import torch

from conftest import TOL
from ffn_kernel_b200 import MaskedFFN, MaskedLinear, check_status
from ffn_kernel_b200.synth import ffn_case, linear_case
from oracle import masked_ref as O

pytestmark = pytest.mark.gpu

# FFNK_STRESS_SEEDS=N widens the sweep for a one-off soak run
SEEDS = int(os.environ.get("FFNK_STRESS_SEEDS", "24"))


def _random_mask(M, rng):
    kind = rng.choice(["iid", "spans", "short_spans", "all", "none", "one_token"])
    m = torch.zeros(M, dtype=torch.bool)
    if kind == "iid":
        g = torch.Generator().manual_seed(rng.randrange(1 << 30))
        m = torch.rand(M, generator=g) < rng.choice([0.1, 0.5, 0.9])
    elif kind in ("spans", "short_spans"):
        hi = 300 if kind == "spans" else 9
        pos, val = 0, rng.random() < 0.5
        while pos < M:
            n = rng.randint(1, hi)
            m[pos:pos + n] = val
            pos, val = pos + n, not val
    elif kind == "all":
        m[:] = True
    elif kind == "one_token":
        m[rng.randrange(M)] = True
    return m


def _dims(rng):
    M = rng.choice([1, 7, 33, 127, 128, 129, 255, 256, 257, 384, 511, 513, 777, 1025, 2049, 4097, 5000])
    pick = lambda: rng.choice([8, 24, 64, 72, 136, 200, 264, 320, 520])
    return M, pick(), pick()


@pytest.mark.parametrize("seed", range(SEEDS))
def test_linear_forward_backward_random(dev, seed):
    rng = random.Random(1000 + seed)
    M, K, N = _dims(rng)
    mask = _random_mask(M, rng)
    c = linear_case(M, K, N, seed=seed, mask=mask, with_grad=True)
    ref_y = O.masked_linear(c.x, c.wv.T, c.wt.T, c.mask)
    rdx, rd1, rd2 = O.masked_linear_backward(c.g, c.x, c.wv.T, c.wt.T, c.mask)
    g = c.to(dev)
    contiguous = rng.random() < 0.4
    x = g.x.clone().requires_grad_(True)
    if contiguous:
        b1 = g.wv.T.contiguous().requires_grad_(True)
        b2 = g.wt.T.contiguous().requires_grad_(True)
        v1, v2 = b1, b2
    else:
        b1, b2 = g.wv.clone().requires_grad_(True), g.wt.clone().requires_grad_(True)
        v1, v2 = b1.T, b2.T
    y = MaskedLinear.apply(x, v1, v2, g.mask)
    y.backward(g.g)
    check_status()
    d1 = b1.grad if contiguous else b1.grad.T
    d2 = b2.grad if contiguous else b2.grad.T
    tag = f"M={M} K={K} N={N} visual={int(mask.sum())} contiguous={contiguous}"
    assert O.max_rel_err(y, ref_y) < TOL, tag
    assert O.max_rel_err(x.grad, rdx) < TOL, tag
    assert O.max_rel_err(d1, rd1) < TOL and O.max_rel_err(d2, rd2) < TOL, tag


@pytest.mark.parametrize("seed", range(SEEDS))
def test_ffn_forward_backward_random(dev, seed):
    rng = random.Random(2000 + seed)
    M, d, h = _dims(rng)
    mask = _random_mask(M, rng)
    c = ffn_case(M, d, h, seed=seed, mask=mask)
    gy = torch.randn(M, d, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)
    ref_y = O.masked_ffn(*c.apply_args())
    ref_g = O.masked_ffn_backward(gy, *c.apply_args())
    g = c.to(dev)
    tag = f"M={M} d={d} h={h} visual={int(mask.sum())}"
    y_inf = MaskedFFN.apply(*g.apply_args())                      # inference path (decode kernels for small M)
    assert O.max_rel_err(y_inf, ref_y) < TOL, tag
    x = g.x.clone().requires_grad_(True)
    leaves = [w.clone().requires_grad_(True) for w in (g.w1, g.w2, g.w3, g.u1, g.u2, g.u3)]
    y = MaskedFFN.apply(x, *(w.T for w in leaves), g.mask)        # training path
    y.backward(gy.to(dev))
    check_status()
    assert O.max_rel_err(y, ref_y) < TOL, tag
    assert O.max_rel_err(x.grad, ref_g[0]) < TOL, tag
    for leaf, r in zip(leaves, ref_g[1:]):
        assert O.max_rel_err(leaf.grad.T, r) < TOL, tag
