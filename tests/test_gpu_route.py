"""Routing kernel: bit-exact with nonzero(mask) / nonzero(~mask), through the C ABI."""
import numpy as np
import pytest
import torch

from ffn_kernel_b200 import check_status, route
from ffn_kernel_b200.synth import edge_mask, span_mask
from oracle import masked_ref as O

pytestmark = pytest.mark.gpu


def _check(mask_cpu, dev):
    rt = route(mask_cpu.to(dev))
    check_status()
    v, t = rt.lists()
    ov, ot = O.routing(mask_cpu)
    assert v.dtype == torch.int32 and t.dtype == torch.int32
    assert np.array_equal(v.cpu().numpy(), ov)
    assert np.array_equal(t.cpu().numpy(), ot)
    m = np.asarray(mask_cpu.numpy() != 0)
    runs = int(m.size > 0) + int(np.count_nonzero(m[1:] != m[:-1]))
    assert rt.counts.tolist()[:5] == [len(ov), len(ot), rt.cap, mask_cpu.numel(), runs]


@pytest.mark.parametrize("M", [1, 2, 15, 16, 17, 127, 128, 129, 1000, 4095, 4096, 4097, 4099, 8192, 65537, 1 << 20,
                               (1 << 20) + 1, 3000001])   # the last two: more than 128 tiles, the one-launch resident kernel
@pytest.mark.parametrize("kind", ["bernoulli", "all_visual", "all_text", "alternating", "span"])
def test_route_bit_exact(dev, M, kind):
    _check(edge_mask(M, kind, seed=M), dev)


@pytest.mark.parametrize("M", [(1 << 20) + 1, 3000001, (1 << 22) + 8192 * 3 + 5])
@pytest.mark.parametrize("kind", ["bernoulli", "all_visual", "alternating", "span"])
def test_route_count_and_scatter_kernels(dev, M, kind):
    # the path of masks too long for the resident kernel (count, then scatter), forced at sizes a test can afford
    from ffn_kernel_b200._lib import lib
    L = lib()
    assert L.ffnk_tune_override(b"route_resident", 0) == 0
    try:
        _check(edge_mask(M, kind, seed=M), dev)
    finally:
        assert L.ffnk_tune_override(b"route_resident", -1) == 0


def test_route_uint8_mask_nonzero_is_visual(dev):
    g = torch.Generator().manual_seed(0)
    m = torch.randint(0, 4, (5000,), generator=g, dtype=torch.uint8)     # any non-zero byte selects
    rt = route(m.to(dev))
    v, t = rt.lists()
    assert np.array_equal(v.cpu().numpy(), np.flatnonzero(m.numpy() != 0))
    assert np.array_equal(t.cpu().numpy(), np.flatnonzero(m.numpy() == 0))


def test_route_unaligned_view(dev):
    base = edge_mask(10001, "bernoulli", 7)
    view = base.to(dev)[1:]                       # data pointer not 16-byte aligned
    rt = route(view)
    v, t = rt.lists()
    ov, ot = O.routing(base[1:])
    assert np.array_equal(v.cpu().numpy(), ov) and np.array_equal(t.cpu().numpy(), ot)


def test_route_empty(dev):
    rt = route(torch.zeros(0, dtype=torch.bool, device=dev))
    assert rt.counts.tolist()[:2] == [0, 0]


def test_route_full_size_properties(dev):
    # at benchmark sizes: the two lists are ascending, disjoint, and together a permutation
    for M, seed in ((32768, 0), (16384, 0), (1 << 24, 1)):
        m = (span_mask(M, seed) if M < (1 << 20) else edge_mask(M, "bernoulli", seed)).to(dev)
        rt = route(m)
        v, t = rt.lists()
        assert bool((v[1:] > v[:-1]).all()) and bool((t[1:] > t[:-1]).all())
        assert v.numel() + t.numel() == M
        assert bool(m[v.long()].all()) and not bool(m[t.long()].any())
        assert int(v.sum(dtype=torch.int64) + t.sum(dtype=torch.int64)) == M * (M - 1) // 2
    check_status()


def test_route_rejects_bad_arguments(dev):
    with pytest.raises(RuntimeError):
        route(torch.zeros(4, 4, dtype=torch.bool, device=dev))
    with pytest.raises(RuntimeError):
        route(torch.zeros(4, dtype=torch.float32, device=dev))


@pytest.mark.parametrize("M", [1, 7, 127, 129, 1000, 4099, 8191, 8192])
@pytest.mark.parametrize("kind", ["bernoulli", "all_visual", "all_text", "alternating", "span"])
def test_route_and_row_copy_in_one_launch(dev, M, kind):
    # ffnk_route_permute_rows against ffnk_route followed by ffnk_permute_rows: same lists, counts and rows
    from ffn_kernel_b200 import check_status
    from ffn_kernel_b200._lib import lib
    from ffn_kernel_b200.route import stream_ptr
    L = lib()
    d = 264
    mask = edge_mask(M, kind, seed=M).to(dev)
    x = torch.randn((M, d), generator=torch.Generator().manual_seed(M)).to(torch.bfloat16).to(dev)
    rt = route(mask)
    rows = rt.cap + 512
    ref = torch.full((rows, d), 7.0, device=dev, dtype=torch.bfloat16)
    got = ref.clone()
    assert L.ffnk_permute_rows(x.data_ptr(), d, rt.perm.data_ptr(), rt.counts.data_ptr(), ref.data_ptr(), d, M, d,
                               stream_ptr(dev)) == 0
    perm = torch.full_like(rt.perm, -1)
    counts = torch.full_like(rt.counts, -1)
    assert L.ffnk_route_permute_rows(mask.data_ptr(), M, x.data_ptr(), d, d, perm.data_ptr(), counts.data_ptr(),
                                     got.data_ptr(), d, stream_ptr(dev)) == 0
    torch.cuda.synchronize()
    check_status()
    assert counts.tolist()[:5] == rt.counts.tolist()[:5]
    mv, mt = counts.tolist()[:2]
    assert torch.equal(perm[:mv], rt.perm[:mv]) and torch.equal(perm[rt.cap:rt.cap + mt], rt.perm[rt.cap:rt.cap + mt])
    assert torch.equal(got, ref)          # the rows between and after the groups keep their fill


def test_route_and_row_copy_arguments(dev):
    from ffn_kernel_b200._lib import lib
    from ffn_kernel_b200.route import stream_ptr
    L = lib()
    assert L.ffnk_route_permute_max_tokens() == 8192
    buf = torch.zeros(4096, device=dev, dtype=torch.int32)
    p = buf.data_ptr()
    assert L.ffnk_route_permute_rows(p, 8193, p, 8, 8, p, p, p, 8, stream_ptr(dev)) < 0      # more than one tile
    assert L.ffnk_route_permute_rows(p, 16, p, 8, 12, p, p, p, 16, stream_ptr(dev)) < 0      # d not a multiple of 8
    assert L.ffnk_route_permute_rows(None, 16, p, 8, 8, p, p, p, 8, stream_ptr(dev)) < 0
    assert L.ffnk_route_permute_rows(p, 0, None, 8, 8, None, p, None, 8, stream_ptr(dev)) == 0   # empty mask: counts only
    torch.cuda.synchronize()
    assert buf[:5].tolist() == [0, 0, 0, 0, 0]
