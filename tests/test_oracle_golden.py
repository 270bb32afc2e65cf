"""The CPU oracle against the golden vectors produced by the reference's own modules
(tests/golden/make_golden.py; reference test_linear.py:41-49, test_ffn.py:32-47)."""
import numpy as np
import pytest
import torch

from conftest import FFN_GOLDEN, LINEAR_GOLDEN, load_golden
from oracle import masked_ref as O


@pytest.mark.parametrize("name", LINEAR_GOLDEN)
def test_linear_forward_fp32_matches_reference_module(name):
    z = load_golden(name)
    x, mask = z["x"].flatten(0, 1), z["mask"].flatten()
    y = O.masked_linear(x, z["wv"].T, z["wt"].T, mask)
    assert O.max_rel_err(y, z["y_f32"].flatten(0, 1)) < 1e-5


@pytest.mark.parametrize("name", LINEAR_GOLDEN)
def test_linear_backward_fp32_matches_reference_autograd(name):
    z = load_golden(name)
    x, g, mask = z["x"].flatten(0, 1), z["g"].flatten(0, 1), z["mask"].flatten()
    dx, db1, db2 = O.masked_linear_backward(g, x, z["wv"].T, z["wt"].T, mask)
    assert O.max_rel_err(dx, z["dx_f32"].flatten(0, 1)) < 1e-5
    # the golden weight gradients are in nn.Linear storage order [N, K]; the oracle's are [K, N]
    assert O.max_rel_err(db1.T, z["dwv_f32"]) < 1e-5
    assert O.max_rel_err(db2.T, z["dwt_f32"]) < 1e-5


@pytest.mark.parametrize("name", LINEAR_GOLDEN)
def test_linear_bf16_arithmetic_matches_reference_bf16_run(name):
    z = load_golden(name)
    x, mask = z["x"].flatten(0, 1), z["mask"].flatten()
    y = O.masked_linear(x, z["wv"].T, z["wt"].T, mask, dtype=torch.bfloat16)
    assert O.max_rel_err(y, z["y_bf16"].flatten(0, 1).float()) < 1e-2


@pytest.mark.parametrize("name", FFN_GOLDEN)
def test_ffn_fp32_matches_reference_module(name):
    z = load_golden(name)
    x, mask = z["x"].flatten(0, 1), z["mask"].flatten()
    y = O.masked_ffn(x, z["w1"].T, z["w2"].T, z["w3"].T, z["u1"].T, z["u2"].T, z["u3"].T, mask)
    assert O.max_rel_err(y, z["y_f32"].flatten(0, 1)) < 1e-5


@pytest.mark.parametrize("name", FFN_GOLDEN)
def test_ffn_bf16_reference_run_is_within_stated_tolerance_of_fp32(name):
    # shows that the 1e-2 max-norm tolerance is attainable by bf16 arithmetic at all
    z = load_golden(name)
    assert O.max_rel_err(z["y_bf16"].float(), z["y_f32"]) < 1e-2


def test_ffn_backward_fp32_matches_reference_autograd():
    z = load_golden(FFN_GOLDEN[0])
    x, g, mask = z["x"].flatten(0, 1), z["g"].flatten(0, 1), z["mask"].flatten()
    names = ("w1", "w2", "w3", "u1", "u2", "u3")
    grads = O.masked_ffn_backward(g, x, *(z[n].T for n in names), mask)
    assert O.max_rel_err(grads[0], z["dx_f32"].flatten(0, 1)) < 1e-5
    for gr, n in zip(grads[1:], names):
        assert O.max_rel_err(gr.T, z[f"d{n}_f32"]) < 1e-5, n       # golden gradients are in [out, in] storage order


def test_ffn_composes_gateup_and_linear():
    z = load_golden(FFN_GOLDEN[0])
    x, mask = z["x"].flatten(0, 1), z["mask"].flatten()
    inter = O.masked_ffn_gateup(x, z["w1"].T, z["w3"].T, z["u1"].T, z["u3"].T, mask)
    y = O.masked_linear(inter, z["w2"].T, z["u2"].T, mask)
    assert O.max_rel_err(y, z["y_f32"].flatten(0, 1)) < 1e-5


@pytest.mark.parametrize("M", [0, 1, 7, 128, 1000])
def test_routing_oracle_matches_a_plain_loop(M):
    rng = np.random.default_rng(M)
    mask = rng.random(M) < 0.4
    v, t = O.routing(mask)
    assert v.dtype == np.int32 and t.dtype == np.int32
    assert v.tolist() == [i for i in range(M) if mask[i]]
    assert t.tolist() == [i for i in range(M) if not mask[i]]
    assert v.tolist() == torch.nonzero(torch.from_numpy(mask)).flatten().tolist()
