"""ffnk_route_noalloc: routing for hosts that cannot hand us scratch memory (a runtime plugin
whose execute callback may not allocate, a serving loop that keeps away from cudaMalloc).  Its
scan state is a fixed array inside the library, shared by every call, so the thing to prove is
that back-to-back calls do not see each other's leftovers: two calls in a row, the second on a
shorter mask, each compared bit for bit with the ordinary ffnk_route entry point."""
import pytest
import torch

from ffn_kernel_b200._lib import lib
from ffn_kernel_b200.route import check_status, status_word, stream_ptr
from ffn_kernel_b200.synth import edge_mask

pytestmark = pytest.mark.gpu

MAX_TOKENS = 1 << 24


def _route_both(mask, dev):
    """(perm, counts) from the allocation-free entry point and from ffnk_route, same mask."""
    L = lib()
    M = mask.numel()
    cap = int(L.ffnk_route_capacity(M))
    st, sp = status_word(dev).data_ptr(), stream_ptr(dev)
    out = []
    for which in ("noalloc", "plain"):
        perm = torch.full((max(2 * cap, 4),), -7, dtype=torch.int32, device=dev)
        counts = torch.full((8,), -7, dtype=torch.int32, device=dev)
        if which == "noalloc":
            rc = L.ffnk_route_noalloc(mask.data_ptr(), M, perm.data_ptr(), counts.data_ptr(), st, sp)
        else:
            ws = torch.empty(int(L.ffnk_route_workspace_bytes(M)), dtype=torch.uint8, device=dev)
            rc = L.ffnk_route(mask.data_ptr(), M, perm.data_ptr(), counts.data_ptr(), ws.data_ptr(), st, sp)
        assert rc == 0
        out.append((perm, counts))
    check_status()
    return out


def test_two_calls_in_a_row_match_the_ordinary_entry_point(dev):
    for M, kind in ((70001, "bernoulli"), (5003, "span")):        # second call: fewer tiles than the first
        mask = edge_mask(M, kind, seed=M).to(dev)
        (perm_a, counts_a), (perm_b, counts_b) = _route_both(mask, dev)
        assert torch.equal(counts_a, counts_b)
        mv, mt, cap, m = counts_a.tolist()[:4]
        assert m == M and mv + mt == M
        assert torch.equal(perm_a[:mv], perm_b[:mv])
        assert torch.equal(perm_a[cap:cap + mt], perm_b[cap:cap + mt])
        assert torch.equal(perm_a[:mv].long(), torch.nonzero(mask).flatten())


def test_full_capacity_then_a_short_mask(dev):
    """The longest mask the fixed array can serve (2^24 tokens: the two-kernel count + scatter path, which
    uses every word of the array), immediately followed by a short multi-tile mask on the same stream."""
    for M, kind in ((MAX_TOKENS, "bernoulli"), (70001, "bernoulli")):
        mask = edge_mask(M, kind, seed=3).to(dev)
        (perm_a, counts_a), (perm_b, counts_b) = _route_both(mask, dev)
        assert torch.equal(counts_a, counts_b)
        mv, mt, cap, m = counts_a.tolist()[:4]
        assert m == M and mv + mt == M
        assert torch.equal(perm_a[:mv], perm_b[:mv])
        assert torch.equal(perm_a[cap:cap + mt], perm_b[cap:cap + mt])
        assert int(perm_a[:mv].long().sum()) == int(torch.nonzero(mask).flatten().sum())


def test_capacity_and_argument_errors(dev):
    L = lib()
    st, sp = status_word(dev).data_ptr(), stream_ptr(dev)
    buf = torch.zeros(64, dtype=torch.int32, device=dev)
    assert L.ffnk_route_noalloc(buf.data_ptr(), MAX_TOKENS + 1, buf.data_ptr(), buf.data_ptr(), st, sp) == -8
    assert b"capacity" in L.ffnk_status_string(-8)
    assert L.ffnk_route_noalloc(None, 16, buf.data_ptr(), buf.data_ptr(), st, sp) == -1
    assert L.ffnk_route_noalloc(buf.data_ptr(), -1, buf.data_ptr(), buf.data_ptr(), st, sp) == -2
    counts = torch.full((8,), -7, dtype=torch.int32, device=dev)
    assert L.ffnk_route_noalloc(None, 0, None, counts.data_ptr(), st, sp) == 0       # empty mask
    assert counts.tolist()[:2] == [0, 0]
    check_status()
