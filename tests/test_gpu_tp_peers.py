"""Down projection that stores partial rows into their owner's block buffer, and the block sum:
the two halves of the tensor-parallel reduce-scatter, exercised with all ranks emulated on ONE
device (each "peer" buffer is just another allocation of the same GPU, the ranks run one after
the other).  The result must equal the fp32 oracle of the unsharded MaskedFFN."""
import ctypes

import pytest
import torch

from conftest import TOL
from ffn_kernel_b200 import check_status, tp
from ffn_kernel_b200._lib import lib
from ffn_kernel_b200.route import route, status_word, stream_ptr
from ffn_kernel_b200.synth import edge_mask, ffn_case
from oracle import masked_ref as O

pytestmark = pytest.mark.gpu


def _emulated_tp_forward(c, world, dev):
    """All ranks on one device: returns y [M, d] assembled from the owners' summed blocks."""
    L = lib()
    x, w1, w2, w3, u1, u2, u3, mask = c.apply_args()
    M, d = x.shape
    rows = max(1, -(-M // world))
    bufs = [torch.full((world * rows, d), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    rt = route(mask)
    st, sp = status_word(dev).data_ptr(), stream_ptr(dev)
    for rank in range(world):
        s1, s2, s3, t1, t2, t3 = tp.shard_ffn_weights(w1, w2, w3, u1, u2, u3, rank, world)
        hs = s1.shape[1]
        inter = torch.empty((rt.cap + 512, hs), device=dev, dtype=torch.bfloat16)
        assert L.ffnk_ffn_gateup(x.data_ptr(), x.stride(0), s1.data_ptr(), s3.data_ptr(), t1.data_ptr(), t3.data_ptr(),
                                 s1.stride(0), s1.stride(1), rt.perm.data_ptr(), rt.counts.data_ptr(), inter.data_ptr(),
                                 inter.stride(0), 0, 1, M, d, hs, st, sp) == 0
        assert L.ffnk_ffn_down_to_peers(inter.data_ptr(), inter.stride(0), s2.data_ptr(), t2.data_ptr(), s2.stride(0),
                                        s2.stride(1), rt.perm.data_ptr(), rt.counts.data_ptr(), ptrs, world, rank, rows,
                                        d, M, d, hs, st, sp) == 0
    y = torch.empty((world * rows, d), device=dev, dtype=torch.bfloat16)
    for owner in range(world):
        out = y[owner * rows:(owner + 1) * rows]
        assert L.ffnk_sum_row_blocks(bufs[owner].data_ptr(), world, rows, d, d, out.data_ptr(), d, sp) == 0
    check_status()
    # rows past M of the last owner were never written by anybody
    return y[:M], bufs, rows


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("M,d,h", [(257, 264, 384), (1000, 256, 960), (4100, 512, 1344)])
@pytest.mark.parametrize("kind", ["bernoulli", "span"])
def test_emulated_ranks_match_oracle(dev, world, M, d, h, kind):
    c = ffn_case(M, d, h, seed=M + world, mask=edge_mask(M, kind, seed=world))
    ref = O.masked_ffn(*c.apply_args())
    y, _, _ = _emulated_tp_forward(c.to(dev), world, dev)
    assert O.max_rel_err(y, ref) < TOL


def test_wide_single_cta_tiles(dev):
    # enough 256-column tiles to fill the SMs but fewer than 4096 rows: the single-CTA 128 x 256 kernel
    M, d, h, world = 2000, 2560, 384, 2
    c = ffn_case(M, d, h, seed=11, mask=edge_mask(M, "span", seed=3))
    ref = O.masked_ffn(*c.apply_args())
    y, _, _ = _emulated_tp_forward(c.to(dev), world, dev)
    assert O.max_rel_err(y, ref) < TOL


def test_every_owned_row_is_written_exactly_where_expected(dev):
    # after one pass, the NaN fill survives only in rows no token maps to (beyond M)
    M, d, h, world = 1001, 136, 320, 4
    c = ffn_case(M, d, h, seed=5, mask=edge_mask(M, "alternating")).to(dev)
    _, bufs, rows = _emulated_tp_forward(c, world, dev)
    for owner, b in enumerate(bufs):
        blocks = b.view(world, rows, d)
        n_owned = max(0, min(M, (owner + 1) * rows) - owner * rows)
        assert not torch.isnan(blocks[:, :n_owned].float()).any()
        if n_owned < rows:
            assert torch.isnan(blocks[:, n_owned:].float()).all()


def test_argument_checks(dev):
    L = lib()
    M, d, h = 64, 64, 64
    c = ffn_case(M, d, h, seed=1).to(dev)
    rt = route(c.mask)
    inter = torch.zeros((rt.cap + 512, h), device=dev, dtype=torch.bfloat16)
    buf = torch.zeros((2 * 32, d), device=dev, dtype=torch.bfloat16)
    w2, u2 = c.apply_args()[2], c.apply_args()[5]
    st, sp = status_word(dev).data_ptr(), stream_ptr(dev)

    def call(world, rank, rows, ptrs):
        return L.ffnk_ffn_down_to_peers(inter.data_ptr(), inter.stride(0), w2.data_ptr(), u2.data_ptr(), w2.stride(0),
                                        w2.stride(1), rt.perm.data_ptr(), rt.counts.data_ptr(), ptrs, world, rank, rows,
                                        d, M, d, h, st, sp)

    two = (ctypes.c_void_p * 2)(buf.data_ptr(), buf.data_ptr())
    assert call(2, 2, 32, two) < 0            # rank outside the world
    assert call(9, 0, 32, two) < 0            # more than eight peers
    assert call(2, 0, 31, two) < 0            # blocks too small for M
    hole = (ctypes.c_void_p * 2)(buf.data_ptr(), None)
    assert call(2, 0, 32, hole) < 0           # a missing peer pointer
    assert L.ffnk_sum_row_blocks(buf.data_ptr(), 0, 32, d, d, buf.data_ptr(), d, sp) < 0
    assert L.ffnk_sum_row_blocks(buf.data_ptr(), 2, 32, d + 4, d + 4, buf.data_ptr(), d + 4, sp) < 0
    torch.cuda.synchronize()
    check_status()


def test_sum_to_peers_fills_every_ranks_output(dev):
    """The owner's block sum stored into the output of every rank (here: `world` allocations of one GPU),
    owner after owner; every output must end up equal to the oracle, rows beyond M untouched."""
    L = lib()
    world, M, d, h = 4, 1001, 136, 320
    c = ffn_case(M, d, h, seed=9, mask=edge_mask(M, "bernoulli", seed=2))
    ref = O.masked_ffn(*c.apply_args())
    _, bufs, rows = _emulated_tp_forward(c.to(dev), world, dev)
    outs = [torch.full((world * rows, d), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(world)]
    optrs = (ctypes.c_void_p * world)(*[o.data_ptr() for o in outs])
    sp = stream_ptr(dev)
    for owner in range(world):
        n_own = max(0, min(rows, M - owner * rows))
        assert L.ffnk_sum_row_blocks_to_peers(bufs[owner].data_ptr(), world, rows, n_own, d, d, optrs, world,
                                              owner * rows, d, 0 if owner % 2 else 3, sp) == 0     # also with a capped grid
    check_status()
    for o in outs:
        assert O.max_rel_err(o[:M], ref) < TOL
        assert torch.equal(o[:M], outs[0][:M])
        assert torch.isnan(o[M:].float()).all()
    assert L.ffnk_sum_row_blocks_to_peers(bufs[0].data_ptr(), 9, rows, rows, d, d, optrs, world, 0, d, 0, sp) < 0
    assert L.ffnk_sum_row_blocks_to_peers(bufs[0].data_ptr(), world, rows, rows, d, d, optrs, 0, 0, d, 0, sp) < 0
    assert L.ffnk_sum_row_blocks_to_peers(bufs[0].data_ptr(), world, rows, rows + 1, d, d, optrs, world, 0, d, 0, sp) < 0


def test_peer_barrier_alone_and_with_a_missing_rank(dev):
    """One rank: the barrier passes on its own flag.  Two ranks of which one never arrives (its flag is
    simply never written): the wait gives up after its budget, reports a status code, and the
    context stays usable.  An arrival written by the host beforehand lets the wait pass."""
    from ffn_kernel_b200._lib import FfnkError
    L = lib()
    st, sp = status_word(dev).data_ptr(), stream_ptr(dev)
    mine = torch.zeros(8, dtype=torch.int32, device=dev)
    other = torch.zeros(8, dtype=torch.int32, device=dev)
    one = (ctypes.c_void_p * 1)(mine.data_ptr())
    for epoch in (1, 2, 3):
        assert L.ffnk_peer_barrier(one, 1, 0, epoch, 0, st, sp) == 0
    check_status()
    assert mine[0].item() == 3
    two = (ctypes.c_void_p * 2)(mine.data_ptr(), other.data_ptr())
    mine.zero_()
    mine[1] = 5                                    # "rank 1 has reached barrier 5 already"
    assert L.ffnk_peer_barrier(two, 2, 0, 5, 1000, st, sp) == 0
    check_status()
    assert other[0].item() == 5                    # and rank 1 was told that rank 0 arrived
    assert L.ffnk_peer_barrier(two, 2, 0, 6, 1000, st, sp) == 0     # nobody writes mine[1] = 6: 1 ms budget
    with pytest.raises(FfnkError) as err:
        check_status()
    assert "rank" in str(err.value)
    check_status()                                  # the status word was cleared, the device still works
    assert (torch.ones(4, device=dev) * 2).sum().item() == 8
    assert L.ffnk_peer_barrier(two, 9, 0, 1, 0, st, sp) < 0      # more than eight ranks
    assert L.ffnk_peer_barrier(two, 2, 2, 1, 0, st, sp) < 0      # rank outside the world
    assert L.ffnk_peer_barrier(None, 1, 0, 1, 0, st, sp) < 0
