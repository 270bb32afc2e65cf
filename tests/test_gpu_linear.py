"""MaskedLinear forward and backward on the GPU against the fp32 CPU oracle and the golden
vectors of the reference's own module; called the way the reference's wrapper calls it
(test_linear.py:58-65: x flattened to [B*S, K], weights as the .T view)."""
import pytest
import torch

from conftest import LINEAR_GOLDEN, TOL, load_golden
from ffn_kernel_b200 import MaskedLinear, check_status
from ffn_kernel_b200.synth import edge_mask, linear_case
from oracle import masked_ref as O

pytestmark = pytest.mark.gpu


def _weights(c, layout):
    if layout == "T":                                   # nn.Linear.weight.T views
        return c.wv.T, c.wt.T
    return c.wv.T.contiguous(), c.wt.T.contiguous()    # plain contiguous [K, N]


@pytest.mark.parametrize("name", LINEAR_GOLDEN)
def test_forward_backward_golden(dev, name):
    z = load_golden(name)
    x = z["x"].flatten(0, 1).to(dev).requires_grad_(True)
    wv = z["wv"].to(dev).requires_grad_(True)
    wt = z["wt"].to(dev).requires_grad_(True)
    mask = z["mask"].flatten().to(dev)
    y = MaskedLinear.apply(x, wv.T, wt.T, mask)
    y.backward(z["g"].flatten(0, 1).to(dev))
    check_status()
    assert y.dtype == torch.bfloat16 and y.is_contiguous()
    assert O.max_rel_err(y, z["y_f32"].flatten(0, 1)) < TOL
    assert O.max_rel_err(x.grad, z["dx_f32"].flatten(0, 1)) < TOL
    assert O.max_rel_err(wv.grad, z["dwv_f32"]) < TOL          # gradient w.r.t. the [N, K] storage
    assert O.max_rel_err(wt.grad, z["dwt_f32"]) < TOL


@pytest.mark.parametrize("M,K,N", [(1, 64, 64), (8, 64, 256), (127, 128, 192), (128, 64, 512), (129, 264, 328),
                                   (1000, 1024, 1024), (4099, 512, 1000), (4096, 1024, 1024)])
@pytest.mark.parametrize("layout", ["T", "C"])
@pytest.mark.parametrize("kind", ["bernoulli", "span"])
def test_forward_parity(dev, M, K, N, layout, kind):
    c = linear_case(M, K, N, seed=M + K, mask=edge_mask(M, kind, seed=N))
    ref = O.masked_linear(c.x, c.wv.T, c.wt.T, c.mask)
    g = c.to(dev)
    y = MaskedLinear.apply(g.x, *_weights(g, layout), g.mask)
    check_status()
    assert y.shape == (M, N)
    assert O.max_rel_err(y, ref) < TOL


@pytest.mark.parametrize("kind", ["all_visual", "all_text", "alternating"])
def test_forward_edge_masks(dev, kind):
    M, K, N = 1000, 256, 264
    c = linear_case(M, K, N, seed=5, mask=edge_mask(M, kind))
    ref = O.masked_linear(c.x, c.wv.T, c.wt.T, c.mask)
    g = c.to(dev)
    y = MaskedLinear.apply(g.x, g.wv.T, g.wt.T, g.mask)
    check_status()
    assert O.max_rel_err(y, ref) < TOL


def test_forward_writes_every_row_exactly(dev):
    # rows must equal the single-branch product of their own modality, bit for bit across calls
    M, K, N = 3000, 512, 512
    c = linear_case(M, K, N, seed=9, mask=edge_mask(M, "bernoulli", 1)).to(dev)
    y1 = MaskedLinear.apply(c.x, c.wv.T, c.wt.T, c.mask)
    y2 = MaskedLinear.apply(c.x, c.wv.T, c.wt.T, c.mask)
    allv = MaskedLinear.apply(c.x, c.wv.T, c.wt.T, torch.ones_like(c.mask))
    allt = MaskedLinear.apply(c.x, c.wv.T, c.wt.T, torch.zeros_like(c.mask))
    check_status()
    assert torch.equal(y1, y2)
    assert torch.equal(y1[c.mask], allv[c.mask]) and torch.equal(y1[~c.mask], allt[~c.mask])


@pytest.mark.parametrize("M,K,N", [(1, 64, 64), (127, 128, 192), (300, 264, 328), (1000, 512, 1000),
                                   (4096, 1024, 1024)])
@pytest.mark.parametrize("layout", ["T", "C"])
@pytest.mark.parametrize("kind", ["bernoulli", "span", "all_visual", "all_text"])
def test_backward_parity(dev, M, K, N, layout, kind):
    c = linear_case(M, K, N, seed=M + N, mask=edge_mask(M, kind, seed=K), with_grad=True)
    rdx, rdb1, rdb2 = O.masked_linear_backward(c.g, c.x, c.wv.T, c.wt.T, c.mask)
    g = c.to(dev)
    b1, b2 = _weights(g, layout)
    x = g.x.clone().requires_grad_(True)
    b1 = b1.detach().requires_grad_(True) if layout == "C" else b1
    b2 = b2.detach().requires_grad_(True) if layout == "C" else b2
    if layout == "T":
        wv, wt = g.wv.clone().requires_grad_(True), g.wt.clone().requires_grad_(True)
        b1, b2 = wv.T, wt.T
    y = MaskedLinear.apply(x, b1, b2, g.mask)
    y.backward(g.g)
    check_status()
    db1 = wv.grad.T if layout == "T" else b1.grad
    db2 = wt.grad.T if layout == "T" else b2.grad
    assert O.max_rel_err(x.grad, rdx) < TOL
    assert O.max_rel_err(db1, rdb1) < TOL
    assert O.max_rel_err(db2, rdb2) < TOL


def test_backward_gradient_strides_follow_the_weights(dev):
    from ffn_kernel_b200.linear import _bf16_linear_backward
    c = linear_case(256, 64, 96, seed=3, with_grad=True).to(dev)
    for b1, b2 in ((c.wv.T, c.wt.T), (c.wv.T.contiguous(), c.wt.T.contiguous())):
        da, db1, db2 = _bf16_linear_backward(c.g, c.x, b1, b2, c.mask)
        assert db1.stride() == b1.stride() and db2.stride() == b2.stride() and da.shape == c.x.shape


def test_sum_backward_like_the_reference_check(dev):
    # test_linear.py:94-97 calls .sum().backward(): the upstream gradient is an expanded scalar
    c = linear_case(512, 128, 128, seed=4).to(dev)
    x = c.x.clone().requires_grad_(True)
    wv = c.wv.clone().requires_grad_(True)
    wt = c.wt.clone().requires_grad_(True)
    MaskedLinear.apply(x, wv.T, wt.T, c.mask).sum().backward()
    check_status()
    ones = torch.ones(512, 128, dtype=torch.bfloat16)
    rdx, rdb1, rdb2 = O.masked_linear_backward(ones, c.x.cpu(), c.wv.T.cpu(), c.wt.T.cpu(), c.mask.cpu())
    assert O.max_rel_err(x.grad, rdx) < TOL
    assert O.max_rel_err(wv.grad.T, rdb1) < TOL and O.max_rel_err(wt.grad.T, rdb2) < TOL


def test_non_contiguous_activation_is_accepted(dev):
    c = linear_case(300, 128, 136, seed=6).to(dev)
    wide = torch.zeros(300, 200, dtype=torch.bfloat16, device=dev)
    wide[:, 3:131] = c.x                                # row stride 200, column offset 3: misaligned rows
    y = MaskedLinear.apply(wide[:, 3:131], c.wv.T, c.wt.T, c.mask)
    ref = O.masked_linear(c.x.cpu(), c.wv.T.cpu(), c.wt.T.cpu(), c.mask.cpu())
    assert O.max_rel_err(y, ref) < TOL


def test_bad_arguments_raise_before_launch(dev):
    c = linear_case(64, 64, 64, seed=1).to(dev)
    with pytest.raises(RuntimeError):
        MaskedLinear.apply(c.x.float(), c.wv.T, c.wt.T, c.mask)            # dtype
    with pytest.raises(RuntimeError):
        MaskedLinear.apply(c.x, c.wv.T[:, :32], c.wt.T, c.mask)            # mismatched N
    with pytest.raises(RuntimeError):
        MaskedLinear.apply(c.x, c.wv.T, c.wt.T, c.mask[:10])               # mask length
    with pytest.raises(RuntimeError):
        MaskedLinear.apply(c.x[:, :60], c.wv.T[:60], c.wt.T[:60], c.mask)  # K not a multiple of 8


def test_full_size_rows_sampled(dev):
    # d = 4096 benchmark shape: compare 192 sampled rows with the oracle evaluated on those rows only
    M, K, N = 32768, 4096, 4096
    c = linear_case(M, K, N, seed=0, visual_frac=0.7, image_lens=(576, 2304))
    g = c.to(dev)
    y = MaskedLinear.apply(g.x, g.wv.T, g.wt.T, g.mask)
    check_status()
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(1))[:192]
    ref = O.masked_linear(c.x[rows], c.wv.T, c.wt.T, c.mask[rows])
    assert O.max_rel_err(y[rows.to(dev)], ref) < TOL
    assert bool(torch.isfinite(y.float()).all())


@pytest.mark.parametrize("kind", ["bernoulli", "alternating", "span"])
def test_scattered_masks_with_and_without_the_routed_copy(dev, kind, monkeypatch):
    # with the scratch the library copies rows into routed order for scattered masks only; without
    # it the GEMMs gather every row themselves: both must give the same gradients and outputs
    from ffn_kernel_b200.linear import _bf16_linear_backward, _bf16_linear_forward
    M, K, N = 2000, 264, 328
    c = linear_case(M, K, N, seed=11, mask=edge_mask(M, kind, seed=5), with_grad=True)
    ref_y = O.masked_linear(c.x, c.wv.T, c.wt.T, c.mask)
    ref_g = O.masked_linear_backward(c.g, c.x, c.wv.T, c.wt.T, c.mask)
    g = c.to(dev)
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("FFNK_LINEAR_COPY", flag)
        y = _bf16_linear_forward(g.x, g.wv.T, g.wt.T, g.mask)
        grads = _bf16_linear_backward(g.g, g.x, g.wv.T, g.wt.T, g.mask)
        check_status()
        assert O.max_rel_err(y, ref_y) < TOL
        for got, ref in zip(grads, ref_g):
            assert O.max_rel_err(got, ref) < TOL
        outs.append((y, *grads))
    assert torch.equal(outs[0][0], outs[1][0])        # forward rows are the same sums either way


@pytest.mark.parametrize("M", [600, 4200])
def test_training_forward_hands_its_routed_copy_to_the_backward(dev, M):
    # through .apply with gradients on, the forward multiplies from a routed-order copy of a and the
    # backward reuses it; the launcher called directly with a itself must give the same gradients
    from ffn_kernel_b200.linear import _bf16_linear_backward, _bf16_linear_forward
    c = linear_case(M, 264, 328, seed=M, mask=edge_mask(M, "span", seed=1), with_grad=True).to(dev)
    x = c.x.clone().requires_grad_(True)
    b1, b2 = c.wv.clone().requires_grad_(True), c.wt.clone().requires_grad_(True)
    y = MaskedLinear.apply(x, b1.T, b2.T, c.mask)
    y.backward(c.g)
    y_inf = _bf16_linear_forward(c.x, c.wv.T, c.wt.T, c.mask)
    da, db1, db2 = _bf16_linear_backward(c.g, c.x, c.wv.T, c.wt.T, c.mask)
    check_status()
    assert torch.equal(y.detach(), y_inf)
    assert torch.equal(x.grad, da) and torch.equal(b1.grad.T, db1) and torch.equal(b2.grad.T, db2)
    with torch.no_grad():
        assert not MaskedLinear.apply(x, b1.T, b2.T, c.mask).requires_grad
