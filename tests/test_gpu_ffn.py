"""MaskedFFN forward on the GPU against the fp32 CPU oracle and the golden vectors of the
reference's own module; called the way the reference's wrapper calls it (test_ffn.py:61-72)."""
import pytest
import torch

from conftest import FFN_GOLDEN, TOL, load_golden
from ffn_kernel_b200 import MaskedFFN, check_status
from ffn_kernel_b200.ffn import _bf16_ffn_forward, _bf16_ffn_fused_forward, decode_max_tokens
from ffn_kernel_b200.synth import edge_mask, ffn_case
from oracle import masked_ref as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", FFN_GOLDEN)
def test_forward_golden(dev, name):
    z = load_golden(name)
    B = z["x"].shape[0]
    g = {k: v.to(dev) for k, v in z.items() if k in ("x", "mask", "w1", "w2", "w3", "u1", "u2", "u3")}
    y = MaskedFFN.apply(g["x"].flatten(0, 1), g["w1"].T, g["w2"].T, g["w3"].T, g["u1"].T, g["u2"].T, g["u3"].T,
                        g["mask"].flatten(0, 1)).unflatten(0, (B, -1))
    check_status()
    assert y.dtype == torch.bfloat16
    assert O.max_rel_err(y, z["y_f32"]) < TOL


@pytest.mark.parametrize("M,d,h", [(9, 64, 160), (127, 128, 256), (300, 128, 328), (1000, 1024, 2816),
                                   (4099, 1024, 2816), (4096, 1024, 2048)])
@pytest.mark.parametrize("kind", ["bernoulli", "span"])
def test_forward_parity(dev, M, d, h, kind):
    c = ffn_case(M, d, h, seed=M, mask=edge_mask(M, kind, seed=h))
    ref = O.masked_ffn(*c.apply_args())
    y = MaskedFFN.apply(*c.to(dev).apply_args())
    check_status()
    assert y.shape == (M, d) and y.is_contiguous()
    assert O.max_rel_err(y, ref) < TOL


@pytest.mark.parametrize("M", [1, 8, 64, 127, 1000, 4099])
@pytest.mark.parametrize("kind", ["all_visual", "all_text", "alternating", "bernoulli"])
def test_edge_and_decode_sweep(dev, M, kind):
    # d = 1024, h = 2816 with every mask of the edge sweep, token counts around the tile size
    c = ffn_case(M, 1024, 2816, seed=M, mask=edge_mask(M, kind, seed=1))
    ref = O.masked_ffn(*c.apply_args())
    y = MaskedFFN.apply(*c.to(dev).apply_args())
    check_status()
    assert O.max_rel_err(y, ref) < TOL


@pytest.mark.parametrize("M", [9, 16, 17, 24, 25, 32, 33, 47, 64, 80])
@pytest.mark.parametrize("kind", ["all_visual", "all_text", "alternating", "bernoulli"])
def test_decode_kernels_token_groups(dev, M, kind):
    # several groups of sixteen tokens per modality, partly filled last group
    assert M <= decode_max_tokens()
    c = ffn_case(M, 264, 520, seed=M, mask=edge_mask(M, kind, seed=2))
    ref = O.masked_ffn(*c.apply_args())
    y = _bf16_ffn_fused_forward(*c.to(dev).apply_args())
    check_status()
    assert O.max_rel_err(y, ref) < TOL


@pytest.mark.parametrize("M", [33, 48, 64, 65, 80, 96, 127])
@pytest.mark.parametrize("kind", ["all_visual", "all_text", "alternating", "bernoulli"])
@pytest.mark.parametrize("d,h", [(264, 520), (1024, 2816)])
def test_decode_kernel_up_to_its_capacity(dev, M, kind, d, h):
    # the one-launch kernel through the C ABI beyond the table's threshold: up to 127 tokens, more than
    # four groups of sixteen in one modality (a second pass over the weights), ragged last groups;
    # two calls in a row give the same bits (fixed summation order)
    from ffn_kernel_b200._lib import lib
    from ffn_kernel_b200.route import status_word, stream_ptr
    L = lib()
    assert M <= L.ffnk_decode_capacity()
    c = ffn_case(M, d, h, seed=M + d, mask=edge_mask(M, kind, seed=3))
    ref = O.masked_ffn(*c.apply_args())
    g = c.to(dev)
    ys = []
    for _ in range(2):
        inter = torch.full((M, h), float("nan"), device=dev, dtype=torch.bfloat16)
        y = torch.full((M, d), float("nan"), device=dev, dtype=torch.bfloat16)
        assert L.ffnk_ffn_decode(g.x.data_ptr(), d, g.w1.data_ptr(), g.w2.data_ptr(), g.w3.data_ptr(), g.u1.data_ptr(),
                                 g.u2.data_ptr(), g.u3.data_ptr(), 1, d, 1, h, g.mask.data_ptr(), inter.data_ptr(),
                                 y.data_ptr(), d, M, d, h, status_word(dev).data_ptr(), stream_ptr(dev)) == 0
        ys.append(y)
    check_status()
    assert O.max_rel_err(ys[0], ref) < TOL
    assert torch.equal(ys[0], ys[1])


@pytest.mark.parametrize("M", [1, 3, 8, 20, 32, 50, 80])
def test_decode_and_gemm_paths_agree(dev, M):
    assert M <= decode_max_tokens()
    c = ffn_case(M, 256, 520, seed=M, mask=edge_mask(M, "alternating")).to(dev)
    y_dec = _bf16_ffn_fused_forward(*c.apply_args())
    y_gemm = _bf16_ffn_fused_forward(*c.apply_args(), allow_decode=False)
    check_status()
    assert O.max_rel_err(y_dec, y_gemm.float()) < TOL


@pytest.mark.parametrize("layout", ["T", "C"])
def test_gateup_token_order_matches_reference_launcher(dev, layout):
    # _bf16_ffn_forward (ffn_kernel/ffn.py:527-560) returns the [M, h] intermediate in token order
    M, d, h = 700, 256, 392
    c = ffn_case(M, d, h, seed=2, mask=edge_mask(M, "bernoulli", 2))
    ref = O.masked_ffn_gateup(c.x, c.w1.T, c.w3.T, c.u1.T, c.u3.T, c.mask)
    g = c.to(dev)
    ws = [g.w1.T, g.w3.T, g.u1.T, g.u3.T]
    if layout == "C":
        ws = [w.contiguous() for w in ws]
    out = _bf16_ffn_forward(g.x, *ws, g.mask)
    check_status()
    assert out.shape == (M, h)
    assert O.max_rel_err(out, ref) < TOL


def test_contiguous_weights(dev):
    M, d, h = 600, 256, 392
    c = ffn_case(M, d, h, seed=8, mask=edge_mask(M, "span", 1))
    ref = O.masked_ffn(*c.apply_args())
    g = c.to(dev)
    args = [g.x] + [w.T.contiguous() for w in (g.w1, g.w2, g.w3, g.u1, g.u2, g.u3)] + [g.mask]
    y = MaskedFFN.apply(*args)
    check_status()
    assert O.max_rel_err(y, ref) < TOL


def test_tensor_parallel_slices_of_the_weight_views(dev):
    # column slices of the [d, h] views and row slices of the [h, d] views are passed without copies;
    # the partial results of the slices sum to the full result
    M, d, h, P = 512, 256, 512, 4
    c = ffn_case(M, d, h, seed=3)
    ref = O.masked_ffn(*c.apply_args())
    g = c.to(dev)
    acc = torch.zeros(M, d, dtype=torch.float32, device=dev)
    for r in range(P):
        sl = slice(r * h // P, (r + 1) * h // P)
        acc += MaskedFFN.apply(g.x, g.w1.T[:, sl], g.w2.T[sl, :], g.w3.T[:, sl], g.u1.T[:, sl], g.u2.T[sl, :],
                               g.u3.T[:, sl], g.mask).float()
    check_status()
    assert O.max_rel_err(acc, ref) < TOL


def _ffn_grads(g, layout="T"):
    """Run MaskedFFN forward + backward on the GPU case g; returns (y, dx, [dw in operator orientation])."""
    x = g.x.clone().requires_grad_(True)
    if layout == "T":       # leaves are the nn.Linear storages, the operator sees their .T views
        leaves = [w.clone().requires_grad_(True) for w in (g.w1, g.w2, g.w3, g.u1, g.u2, g.u3)]
        views = [w.T for w in leaves]
    else:                   # contiguous [in, out] leaves
        leaves = [w.T.contiguous().requires_grad_(True) for w in (g.w1, g.w2, g.w3, g.u1, g.u2, g.u3)]
        views = leaves
    y = MaskedFFN.apply(x, *views, g.mask)
    return x, leaves, y


@pytest.mark.parametrize("M,d,h", [(1, 64, 64), (9, 64, 160), (300, 128, 328), (1000, 256, 520), (4099, 256, 512)])
@pytest.mark.parametrize("layout", ["T", "C"])
@pytest.mark.parametrize("kind", ["bernoulli", "span", "all_visual", "all_text"])
def test_backward_parity(dev, M, d, h, layout, kind):
    # the reference leaves MaskedFFN.backward unimplemented (ffn_kernel/ops.py:34-38); the oracle
    # differentiates the reference module's expression (formulas: reference README.md:159-172)
    c = ffn_case(M, d, h, seed=M + h, mask=edge_mask(M, kind, seed=d))
    gy = (torch.randn(M, d, generator=torch.Generator().manual_seed(7))).to(torch.bfloat16)
    ref = O.masked_ffn_backward(gy, *c.apply_args())
    x, leaves, y = _ffn_grads(c.to(dev), layout)
    y.backward(gy.to(dev))
    check_status()
    assert O.max_rel_err(y, O.masked_ffn(*c.apply_args())) < TOL
    assert O.max_rel_err(x.grad, ref[0]) < TOL
    for leaf, r, name in zip(leaves, ref[1:], ("w1", "w2", "w3", "u1", "u2", "u3")):
        got = leaf.grad.T if layout == "T" else leaf.grad
        assert got.shape == r.shape
        assert O.max_rel_err(got, r) < TOL, name


def test_backward_golden(dev):
    z = load_golden(FFN_GOLDEN[0])
    names = ("w1", "w2", "w3", "u1", "u2", "u3")
    x = z["x"].flatten(0, 1).to(dev).requires_grad_(True)
    leaves = [z[n].to(dev).requires_grad_(True) for n in names]
    y = MaskedFFN.apply(x, *(w.T for w in leaves), z["mask"].flatten().to(dev))
    y.backward(z["g"].flatten(0, 1).to(dev))
    check_status()
    assert O.max_rel_err(x.grad, z["dx_f32"].flatten(0, 1)) < TOL
    for leaf, n in zip(leaves, names):
        assert O.max_rel_err(leaf.grad, z[f"d{n}_f32"]) < TOL, n


@pytest.mark.parametrize("M,d,h", [(300, 128, 328), (4099, 1024, 2816)])
def test_training_forward_equals_inference_forward(dev, M, d, h):
    # the forward that keeps the pre-activations forms H from the same fp32 accumulators
    c = ffn_case(M, d, h, seed=M, mask=edge_mask(M, "span", seed=d)).to(dev)
    y_inf = MaskedFFN.apply(*c.apply_args())
    args = list(c.apply_args())
    args[0] = args[0].clone().requires_grad_(True)
    y_train = MaskedFFN.apply(*args)
    check_status()
    assert y_train.requires_grad and torch.equal(y_train.detach(), y_inf)


def test_backward_only_when_asked_for(dev):
    c = ffn_case(64, 64, 64, seed=1).to(dev)
    y = MaskedFFN.apply(*c.apply_args())            # nothing requires grad: inference path
    assert not y.requires_grad


def test_no_grad_takes_the_inference_path_even_with_parameters(dev, monkeypatch):
    # nn.Parameter weights have requires_grad set also under torch.no_grad(); the forward that keeps
    # activations for a backward pass must not run then
    import ffn_kernel_b200.ops as ops
    called = []
    real = ops._bf16_ffn_train_forward
    monkeypatch.setattr(ops, "_bf16_ffn_train_forward", lambda *a: (called.append(1), real(*a))[1])
    c = ffn_case(64, 64, 64, seed=1).to(dev)
    args = list(c.apply_args())
    args[1:7] = [w.detach().clone().requires_grad_(True) for w in args[1:7]]
    with torch.no_grad():
        y = MaskedFFN.apply(*args)
    assert not called and not y.requires_grad
    y = MaskedFFN.apply(*args)
    assert called and y.requires_grad
    check_status()


def test_backward_full_size_rows_sampled(dev):
    # d = 1024 / h = 2048, M = 32768: dx on sampled rows (row independence) and a column block of dW
    M, d, h = 32768, 1024, 2048
    c = ffn_case(M, d, h, seed=0)
    gy = torch.randn(M, d, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    x, leaves, y = _ffn_grads(c.to(dev), "T")
    y.backward(gy.to(dev))
    check_status()
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(1))[:96]
    ref = O.masked_ffn_backward(gy[rows], c.x[rows], *c.apply_args()[1:7], c.mask[rows])
    assert O.max_rel_err(x.grad[rows.to(dev)], ref[0]) < TOL
    assert all(bool(torch.isfinite(l.grad.float()).all()) for l in leaves)
    # dW2 (visual) = H_v^T G_v: check against the oracle's intermediate on all rows, fp32 on CPU
    hv = O.masked_ffn_gateup(c.x, c.w1.T, c.w3.T, c.u1.T, c.u3.T, c.mask)
    mv = c.mask.view(-1, 1).float()
    dw2_ref = (hv * mv).T @ gy.float()              # [h, d]
    assert O.max_rel_err(leaves[1].grad.T, dw2_ref) < TOL


def test_empty_input(dev):
    c = ffn_case(8, 64, 64, seed=1).to(dev)
    y = MaskedFFN.apply(c.x[:0], *c.apply_args()[1:7], c.mask[:0])
    assert y.shape == (0, 64)


def test_full_size_rows_sampled(dev):
    # d = 4096 / h = 11008, M = 16384: 128 sampled rows against the oracle on those rows,
    # plus row independence: the same rows computed alone give the same bits
    M, d, h = 16384, 4096, 11008
    c = ffn_case(M, d, h, seed=0)
    g = c.to(dev)
    y = MaskedFFN.apply(*g.apply_args())
    check_status()
    rows = torch.randperm(M, generator=torch.Generator().manual_seed(1))[:128]
    ref = O.masked_ffn(c.x[rows], *c.apply_args()[1:7], c.mask[rows])
    assert O.max_rel_err(y[rows.to(dev)], ref) < TOL
    assert bool(torch.isfinite(y.float()).all())
    sub = MaskedFFN.apply(g.x[rows.to(dev)], *g.apply_args()[1:7], g.mask[rows.to(dev)])
    assert O.max_rel_err(sub, y[rows.to(dev)].float()) < 1e-2


@pytest.mark.parametrize("M", [5, 300, 4099])
def test_single_call_and_step_by_step_paths_agree(dev, M):
    from ffn_kernel_b200 import route
    c = ffn_case(M, 256, 520, seed=M, mask=edge_mask(M, "bernoulli", 4)).to(dev)
    from ffn_kernel_b200._lib import lib
    L = lib()
    # the single call may split the down projection's contraction (another summation order): switched off, the
    # two paths launch the same kernels and give the same bits; switched on, they agree to rounding
    assert L.ffnk_tune_override(b"ksplit", 0) == 0
    try:
        y_one = _bf16_ffn_fused_forward(*c.apply_args(), allow_decode=False)
    finally:
        assert L.ffnk_tune_override(b"ksplit", -1) == 0
    y_steps = _bf16_ffn_fused_forward(*c.apply_args(), rt=route(c.mask), allow_decode=False)
    y_auto = _bf16_ffn_fused_forward(*c.apply_args(), allow_decode=False)
    check_status()
    assert torch.equal(y_one, y_steps)
    assert O.max_rel_err(y_auto, y_steps.float().cpu()) < 5e-3


@pytest.mark.parametrize("M", [1, 8])
def test_small_token_counts_with_contiguous_weights(dev, M):
    # the decode kernels stream K-major rows only; other layouts take the GEMM path
    c = ffn_case(M, 256, 520, seed=M, mask=edge_mask(M, "alternating"))
    ref = O.masked_ffn(*c.apply_args())
    g = c.to(dev)
    args = [g.x] + [w.T.contiguous() for w in (g.w1, g.w2, g.w3, g.u1, g.u2, g.u3)] + [g.mask]
    y = MaskedFFN.apply(*args)
    check_status()
    assert O.max_rel_err(y, ref) < TOL


def test_single_call_rejects_a_short_workspace(dev):
    from ffn_kernel_b200._lib import lib
    from ffn_kernel_b200.route import status_word, stream_ptr
    L = lib()
    M, d, h = 300, 256, 520
    c = ffn_case(M, d, h, seed=1).to(dev)
    need = int(L.ffnk_ffn_workspace_bytes(M, d, h))
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    y = torch.empty(M, d, dtype=torch.bfloat16, device=dev)
    rc = L.ffnk_ffn_forward(c.x.data_ptr(), d, c.w1.data_ptr(), c.w2.data_ptr(), c.w3.data_ptr(), c.u1.data_ptr(),
                            c.u2.data_ptr(), c.u3.data_ptr(), 1, d, 1, h, c.mask.data_ptr(), ws.data_ptr(), need - 256,
                            y.data_ptr(), d, M, d, h, 1, status_word(dev).data_ptr(), stream_ptr(dev))
    assert rc == -8


@pytest.mark.parametrize("M", [81, 127, 129, 1000, 2047])
@pytest.mark.parametrize("kind", ["all_visual", "alternating", "bernoulli", "span"])
@pytest.mark.parametrize("splits", [0, 2, 4])
def test_down_projection_split_over_the_contraction(dev, M, kind, splits):
    # few row tiles: the single-call forward may cut the down projection's contraction into ranges whose
    # fp32 partial tiles are added in a fixed order by the last range to finish; forced off (0) and on
    # (2, 8) here: every choice agrees with the oracle and gives the same bits twice
    from ffn_kernel_b200._lib import lib
    L = lib()
    d, h = 1024, 2816
    c = ffn_case(M, d, h, seed=M, mask=edge_mask(M, kind, seed=M))
    ref = O.masked_ffn(*c.apply_args())
    g = c.to(dev)
    assert L.ffnk_tune_override(b"ksplit", splits) == 0
    try:
        with torch.no_grad():
            y = MaskedFFN.apply(*g.apply_args())
            y2 = MaskedFFN.apply(*g.apply_args())
        check_status()
    finally:
        assert L.ffnk_tune_override(b"ksplit", -1) == 0
    assert O.max_rel_err(y, ref) < TOL
    assert torch.equal(y, y2)


def test_down_projection_split_ragged_shape(dev):
    from ffn_kernel_b200._lib import lib
    L = lib()
    M, d, h = 300, 264, 1096            # d not a multiple of a column tile, h not a multiple of a k-step
    c = ffn_case(M, d, h, seed=3, mask=edge_mask(M, "bernoulli", seed=5))
    ref = O.masked_ffn(*c.apply_args())
    g = c.to(dev)
    for splits in (0, 4):
        assert L.ffnk_tune_override(b"ksplit", splits) == 0
        try:
            with torch.no_grad():
                y = MaskedFFN.apply(*g.apply_args())
            check_status()
        finally:
            assert L.ffnk_tune_override(b"ksplit", -1) == 0
        assert O.max_rel_err(y, ref) < TOL
