"""Host logic of the two multi-GPU modes with two CPU ranks over gloo.  The CUDA operator is
replaced by the CPU oracle here (there is no GPU in this test); what is under test is the
sharding arithmetic, the chunked all-reduce and the error paths."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ffn_kernel_b200 import tp
from ffn_kernel_b200.synth import ffn_case, linear_case
from oracle import masked_ref as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_ffn(x, w1, w2, w3, u1, u2, u3, mask):
    return O.masked_ffn(x, w1, w2, w3, u1, u2, u3, mask)      # fp32


def _worker(rank, world, port, chunks, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c = ffn_case(300, 64, 128, seed=5)
        args = c.apply_args()
        shards = tp.shard_ffn_weights(*args[1:7], rank, world)
        y = tp.masked_ffn_tp(c.x, *shards, c.mask, chunks=chunks, ffn_fn=_oracle_ffn, reduce_dtype=torch.float32)
        ref = O.masked_ffn(*args)
        err_tp = O.max_rel_err(y, ref)
        lc = linear_case(301, 64, 72, seed=6)
        rows, part = tp.masked_linear_dp(lc.x, lc.wv.T, lc.wt.T, lc.mask, rank, world,
                                         linear_fn=lambda a, b1, b2, m: O.masked_linear(a, b1, b2, m))
        full = O.masked_linear(lc.x, lc.wv.T, lc.wt.T, lc.mask)
        err_dp = O.max_rel_err(part, full[rows])
        counts = [None] * world
        dist.all_gather_object(counts, (rows.start, rows.stop))
        # a world-size mismatch in the row count is refused before any collective
        try:
            tp.masked_ffn_tp_reduce_scatter(c.x[:299], *shards, c.mask[:299], ffn_fn=_oracle_ffn)
            refused = False
        except ValueError:
            refused = True
        # data-parallel gradient sum: each rank's partial dW over its own rows adds up to the full dW
        lg = linear_case(200, 32, 40, seed=7, with_grad=True)
        rr = tp.row_shard(200, rank, world)
        _, d1, d2 = O.masked_linear_backward(lg.g[rr], lg.x[rr], lg.wv.T, lg.wt.T, lg.mask[rr])
        d1 = d1.T.contiguous().T                                # a transposed-stride gradient, like weight.T views
        tp.all_reduce_gradients([d1, None, d2], bucket_bytes=1024)
        _, f1, f2 = O.masked_linear_backward(lg.g, lg.x, lg.wv.T, lg.wt.T, lg.mask)
        err_grad = max(O.max_rel_err(d1, f1), O.max_rel_err(d2, f2))
        if rank == 0:
            out.put((err_tp, err_dp, counts, refused, err_grad))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("chunks", [1, 3])
def test_tp_and_dp_two_ranks(chunks):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, chunks, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    err_tp, err_dp, counts, refused, err_grad = q.get()
    assert refused and err_grad < 1e-5
    assert err_tp < 5e-3 and err_dp < 1e-6          # y is returned in bf16 (one rounding)
    assert counts == [(0, 151), (151, 301)]          # contiguous, disjoint, covering


def test_row_shard_covers_everything():
    for M in (0, 1, 7, 8, 16384, 32769):
        for world in (1, 2, 4, 8):
            parts = [tp.row_shard(M, r, world) for r in range(world)]
            assert parts[0].start == 0 and parts[-1].stop == M
            assert all(a.stop == b.start for a, b in zip(parts, parts[1:]))
            sizes = [p.stop - p.start for p in parts]
            assert max(sizes) - min(sizes) <= 1


def test_peer_owned_rows_partition_the_tokens():
    # ownership in the fused tensor-parallel path: equal blocks of ceil(M / world) tokens, trailing ranks may be empty
    for M in (0, 1, 7, 8, 9, 1000, 16384):
        for world in (1, 2, 3, 8):
            rows = tp.peer_block_rows(M, world)
            assert rows >= 1 and rows * world >= M
            parts = [tp.peer_owned_rows(M, r, world) for r in range(world)]
            assert parts[0].start == 0 and parts[-1].stop == M
            assert all(a.stop == b.start for a, b in zip(parts, parts[1:]))
            assert all(p.start == min(M, r * rows) for r, p in enumerate(parts))
    with pytest.raises(ValueError):
        tp.peer_owned_rows(10, 3, 3)


def test_h_shard_alignment_and_errors():
    assert tp.h_shard(11008, 7, 8) == slice(9632, 11008)
    assert all(tp.h_shard(11008, r, 8).start % 8 == 0 for r in range(8))
    with pytest.raises(ValueError):
        tp.h_shard(100, 0, 8)
    with pytest.raises(ValueError):
        tp.row_shard(10, 2, 2)


def test_weight_shards_are_views():
    c = ffn_case(8, 64, 128, seed=0)
    args = c.apply_args()
    sh = tp.shard_ffn_weights(*args[1:7], 1, 2)
    assert sh[0].shape == (64, 64) and sh[1].shape == (64, 64)
    assert sh[0].untyped_storage().data_ptr() == c.w1.untyped_storage().data_ptr()
    assert sh[1].untyped_storage().data_ptr() == c.w2.untyped_storage().data_ptr()


def test_storage_order_view_of_weight_gradients():
    # a weight gradient carries its weight's strides (the transposed view of [out, in] storage): packing
    # it for the all-reduce must be a flat view of the memory, not a transposing copy
    g = torch.arange(12.0).reshape(3, 4).T                     # logical [4, 3], memory order [3, 4]
    v = tp._storage_order_view(g)
    assert v.is_contiguous() and v.data_ptr() == g.data_ptr() and v.shape == (3, 4)
    assert v.reshape(-1).data_ptr() == g.data_ptr()            # flattening is free
    c = torch.zeros(4, 3)
    assert tp._storage_order_view(c) is c


def test_gradient_sync_hook_is_installed_and_removed():
    from ffn_kernel_b200 import linear
    assert linear.GRAD_HOOK is None
    with tp.GradientSync() as outer:
        assert linear.GRAD_HOOK == outer._hook
        with tp.GradientSync(reduce_dtype=None) as inner:
            assert linear.GRAD_HOOK == inner._hook
        assert linear.GRAD_HOOK == outer._hook
    assert linear.GRAD_HOOK is None
    # without a process group (one rank) the hook starts nothing and hands back a no-op
    done = tp.GradientSync()._hook(torch.zeros(2, 2))
    done()


def test_chunk_regions_fit_the_block_buffers():
    # chunked calls place each chunk's world * ceil(Mc / world) block rows one after the other; the buffers
    # are allocated with MAX_CHUNKS spare rows per block
    for M in (1, 9, 1000, 16384, 16385):
        for world in (2, 3, 8):
            rows = tp.peer_block_rows(M, world)
            total = world * (rows + tp.PeerBlocks.MAX_CHUNKS)
            for chunks in range(1, tp.PeerBlocks.MAX_CHUNKS + 1):
                used = 0
                for c in range(min(chunks, M)):
                    tok = tp.row_shard(M, c, min(chunks, M))
                    used += world * tp.peer_block_rows(tok.stop - tok.start, world)
                assert used <= total, (M, world, chunks)
