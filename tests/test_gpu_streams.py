"""Stream plumbing: the operators launch on torch's current stream and never synchronise with the
host, so they work on side streams and inside CUDA graph capture."""
import pytest
import torch

from conftest import TOL
from ffn_kernel_b200 import MaskedFFN, MaskedLinear, check_status
from ffn_kernel_b200.synth import edge_mask, ffn_case, linear_case
from oracle import masked_ref as O

pytestmark = pytest.mark.gpu


def test_operators_on_a_side_stream(dev):
    c = ffn_case(700, 128, 264, seed=1, mask=edge_mask(700, "span", seed=2))
    lc = linear_case(700, 136, 200, seed=3, mask=edge_mask(700, "bernoulli", seed=4))
    ref_f = O.masked_ffn(*c.apply_args())
    ref_l = O.masked_linear(lc.x, lc.wv.T, lc.wt.T, lc.mask)
    g, gl = c.to(dev), lc.to(dev)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        y = MaskedFFN.apply(*g.apply_args())
        z = MaskedLinear.apply(gl.x, gl.wv.T, gl.wt.T, gl.mask)
        done = torch.cuda.Event()
        done.record(side)
    done.synchronize()                       # only the side stream is waited for
    assert O.max_rel_err(y, ref_f) < TOL
    assert O.max_rel_err(z, ref_l) < TOL
    check_status()


@pytest.mark.parametrize("M", [600, 5000])
def test_masked_linear_forward_in_a_cuda_graph(dev, M):
    # both forward variants: rows gathered in the kernel, and (scattered mask) the device-decided routed copy
    for kind in ("span", "bernoulli"):
        lc = linear_case(M, 264, 328, seed=M, mask=edge_mask(M, kind, seed=1)).to(dev)
        for _ in range(2):
            eager = MaskedLinear.apply(lc.x, lc.wv.T, lc.wt.T, lc.mask)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            captured = MaskedLinear.apply(lc.x, lc.wv.T, lc.wt.T, lc.mask)
        for _ in range(2):
            graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(captured, eager)
    check_status()
