"""The packaged nn.Module wrappers against the reference's own module definitions
(test_linear.py:41-65, test_ffn.py:32-72), restated by the oracle."""
import pytest
import torch

from conftest import TOL
from ffn_kernel_b200 import MaskedFFNModule, MaskedLinearModule, check_status
from ffn_kernel_b200.synth import span_mask
from oracle import masked_ref as O

pytestmark = pytest.mark.gpu


def test_linear_module_forward_backward(dev):
    torch.manual_seed(0)
    mod = MaskedLinearModule(128, 192, device=dev)
    B, S = 2, 300
    x = torch.randn(B, S, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    mask = span_mask(B * S, 3, image_lens=(50,), text_min=10).view(B, S).to(dev)
    y = mod(x, mask)
    y.sum().backward()
    check_status()
    assert y.shape == (B, S, 192)
    wv, wt = mod.linear_v.weight.detach().cpu(), mod.linear_t.weight.detach().cpu()
    ref = O.masked_linear(x.detach().cpu().flatten(0, 1), wv.T, wt.T, mask.cpu().flatten())
    assert O.max_rel_err(y.flatten(0, 1), ref) < TOL
    ones = torch.ones(B * S, 192, dtype=torch.bfloat16)
    rdx, rd1, rd2 = O.masked_linear_backward(ones, x.detach().cpu().flatten(0, 1), wv.T, wt.T, mask.cpu().flatten())
    assert O.max_rel_err(x.grad.flatten(0, 1), rdx) < TOL
    assert O.max_rel_err(mod.linear_v.weight.grad.T, rd1) < TOL
    assert O.max_rel_err(mod.linear_t.weight.grad.T, rd2) < TOL


def test_ffn_module_forward_and_state_dict_names(dev):
    torch.manual_seed(1)
    mod = MaskedFFNModule(128, 264, device=dev)
    assert set(mod.state_dict()) == {f"{n}.weight" for n in ("w1", "w2", "w3", "u1", "u2", "u3")}
    B, S = 3, 200
    x = torch.randn(B, S, 128, device=dev, dtype=torch.bfloat16)
    mask = span_mask(B * S, 5, image_lens=(64,), text_min=8).view(B, S).to(dev)
    with torch.no_grad():
        y = mod(x, mask)
    check_status()
    ws = [getattr(mod, n).weight.detach().cpu().T for n in ("w1", "w2", "w3", "u1", "u2", "u3")]
    ref = O.masked_ffn(x.cpu().flatten(0, 1), *ws, mask.cpu().flatten())
    assert y.shape == (B, S, 128)
    assert O.max_rel_err(y.flatten(0, 1), ref) < TOL


@pytest.mark.parametrize("tokens", [8, 300])
def test_graphed_ffn_replays_match_eager(dev, tokens):
    # decode-sized and GEMM-sized token counts; every replay must equal the eager forward on the same inputs
    from ffn_kernel_b200 import GraphedMaskedFFN
    torch.manual_seed(3)
    mod = MaskedFFNModule(256, 520, device=dev)
    graphed = GraphedMaskedFFN(mod, tokens)
    for seed in range(3):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(tokens, 256, generator=g).to(torch.bfloat16).to(dev)
        mask = (torch.rand(tokens, generator=g) < 0.5).to(dev)
        y_graph = graphed(x, mask).clone()
        with torch.no_grad():
            y_eager = mod(x, mask)
        check_status()
        assert torch.equal(y_graph, y_eager)
    with pytest.raises(RuntimeError):
        graphed(torch.zeros(tokens + 1, 256, device=dev, dtype=torch.bfloat16),
                torch.zeros(tokens + 1, device=dev, dtype=torch.bool))


def test_sweep_paths_tool_runs(dev, monkeypatch, capsys):
    # the tool behind the decode table entry: one JSON line per token count with the three paths' times
    import json
    import sys
    from ffn_kernel_b200 import sweep
    monkeypatch.setattr(sys, "argv", ["sweep", "paths", "--d", "256", "--h", "520", "--tokens", "8,200", "--iters", "2",
                                      "--warmup", "1"])
    sweep.main()
    rows = [json.loads(ln) for ln in capsys.readouterr().out.strip().splitlines()]
    assert [r["M"] for r in rows] == [8, 200]
    assert rows[0]["decode_us"] > 0 and rows[0]["gemm_us"] > 0 and rows[0]["gemm_no_splitk_us"] > 0
    assert "decode_us" not in rows[1] and rows[1]["gemm_us"] > 0        # beyond the decode kernel's capacity
