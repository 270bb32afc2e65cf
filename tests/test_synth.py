import torch

from ffn_kernel_b200.synth import CONFIGS, edge_mask, ffn_case, linear_case, span_mask


def test_span_mask_is_seeded_and_near_the_requested_fraction():
    a, b = span_mask(32768, 0), span_mask(32768, 0)
    assert torch.equal(a, b)
    assert not torch.equal(a, span_mask(32768, 1))
    assert 0.40 < a.float().mean() < 0.60
    m70 = span_mask(32768, 0, image_lens=(576, 2304), visual_frac=0.7)
    assert 0.60 < m70.float().mean() < 0.80
    # image spans are contiguous runs at least one span long somewhere
    runs = torch.diff(torch.nonzero(torch.diff(a.int()) != 0).flatten())
    assert int(runs.max()) >= 576


def test_edge_masks():
    assert edge_mask(9, "all_visual").all() and not edge_mask(9, "all_text").any()
    assert edge_mask(4, "alternating").tolist() == [True, False, True, False]
    assert torch.equal(edge_mask(100, "bernoulli", 3), edge_mask(100, "bernoulli", 3))


def test_cases_have_reference_layouts():
    c = linear_case(64, 32, 48, seed=1, with_grad=True)
    assert c.x.shape == (64, 32) and c.wv.shape == (48, 32) and c.g.shape == (64, 48)
    assert c.wv.T.stride() == (1, 32)          # the weight.T view the operators receive
    f = ffn_case(64, 32, 80, seed=1)
    args = f.apply_args()
    assert [tuple(a.shape) for a in args[1:7]] == [(32, 80), (80, 32), (32, 80)] * 2
    assert all(a.dtype == torch.bfloat16 for a in args[:7]) and args[7].dtype == torch.bool
    assert set(CONFIGS) >= {"c2_ffn_d1024_h2048_m32768", "c4_ffn_d4096_h11008_m16384"}
