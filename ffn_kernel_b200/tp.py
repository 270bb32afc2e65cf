"""Multi-GPU use of the routed operators on one node: one process per GPU.

The reference is single-device (``test_linear.py:74`` ``torch.cuda.set_device(0)``); these two
modes are additions around the unchanged operator API:

* token-sharded data parallel -- rows of ``x``/``mask`` are split contiguously over the ranks,
  weights are replicated, nothing is communicated (``row_shard``);
* tensor parallel over the intermediate dimension ``h`` -- rank ``r`` holds columns
  ``[r*h/P, (r+1)*h/P)`` of the gate/up weights and the matching rows of the down weights as
  *views* of the full weights (no copies), computes a partial ``y`` with the ordinary
  ``MaskedFFN.apply`` and the partials are summed by one all-reduce per token chunk (or one
  reduce-scatter, leaving every rank with its block of rows).  With more than one chunk the
  collective of chunk ``i`` overlaps the GEMMs of chunk ``i+1``; on 2 and 8 B200s one chunk was
  fastest (the chunked GEMMs lose more than the overlap gains).
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist


def row_shard(M: int, rank: int, world: int) -> slice:
    """Contiguous row range of rank ``rank``; the first ``M % world`` ranks get one extra row."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(M, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def h_shard(h: int, rank: int, world: int) -> slice:
    """Slice of the intermediate dimension owned by ``rank``; slices start on multiples of 8
    so that every sliced weight view keeps 16-byte aligned rows."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if h % (8 * world):
        raise ValueError(f"h = {h} must be a multiple of 8 * world_size = {8 * world}")
    step = h // world
    return slice(rank * step, (rank + 1) * step)


def shard_ffn_weights(w1, w2, w3, u1, u2, u3, rank: int, world: int):
    """Views of the ``MaskedFFN.apply`` weights ([d,h], [h,d], [d,h], ...) for one TP rank."""
    sl = h_shard(w1.shape[1], rank, world)
    return w1[:, sl], w2[sl, :], w3[:, sl], u1[:, sl], u2[sl, :], u3[:, sl]


def masked_ffn_tp(x, w1, w2, w3, u1, u2, u3, mask, group=None, chunks: int = 1,
                  ffn_fn: Callable | None = None, reduce_dtype: torch.dtype | None = None, sm_margin: int = 16):
    """Tensor-parallel MaskedFFN forward.  The weights are this rank's shards (see
    ``shard_ffn_weights``); ``x`` and ``mask`` are replicated.  Returns the full ``y`` on every rank.

    ``chunks`` splits the tokens into that many row blocks, each reduced as soon as it is
    computed.  While chunks are in flight the persistent GEMM grids leave ``sm_margin`` SMs free so
    that the collective's kernels can run beside them instead of queueing behind them.
    ``ffn_fn`` defaults to ``MaskedFFN.apply``; tests on CPU ranks pass a stand-in."""
    set_margin = None
    if ffn_fn is None:
        from ._lib import lib
        from .ops import MaskedFFN
        ffn_fn = MaskedFFN.apply
        set_margin = lib().ffnk_set_sm_margin
    M = x.shape[0]
    chunks = max(1, min(chunks, max(1, M)))
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    bounds = [row_shard(M, c, chunks) for c in range(chunks)]
    y = torch.empty((M, w2.shape[1]), dtype=reduce_dtype or x.dtype, device=x.device)
    works = []
    overlap = set_margin is not None and world > 1 and chunks > 1 and sm_margin > 0
    if overlap:
        set_margin(sm_margin)
    try:
        for b in bounds:
            part = ffn_fn(x[b], w1, w2, w3, u1, u2, u3, mask[b])
            y[b] = part                              # cast to the reduction dtype if one was asked for
            if world > 1:
                works.append(dist.all_reduce(y[b], op=dist.ReduceOp.SUM, group=group, async_op=True))
    finally:
        if overlap:
            set_margin(0)
    for w in works:
        w.wait()
    return y if y.dtype == x.dtype else y.to(x.dtype)


def masked_ffn_tp_reduce_scatter(x, w1, w2, w3, u1, u2, u3, mask, group=None, ffn_fn: Callable | None = None):
    """Tensor-parallel MaskedFFN forward that leaves the output row-sharded: rank ``r`` returns
    ``(rows, y[rows])`` with ``rows = row_shard(M, r, world)``.  Half the traffic of the all-reduce;
    for callers whose next operator is token-parallel.  ``M`` must be a multiple of the world size."""
    if ffn_fn is None:
        from .ops import MaskedFFN
        ffn_fn = MaskedFFN.apply
    M = x.shape[0]
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if M % world:
        raise ValueError(f"M = {M} must be a multiple of the world size {world} for reduce-scatter")
    part = ffn_fn(x, w1, w2, w3, u1, u2, u3, mask)
    rows = row_shard(M, rank, world)
    if world == 1:
        return rows, part
    out = torch.empty((M // world, part.shape[1]), dtype=part.dtype, device=part.device)
    dist.reduce_scatter_tensor(out, part.contiguous(), op=dist.ReduceOp.SUM, group=group)
    return rows, out


def masked_linear_dp(a, b1, b2, mask, rank: int, world: int, linear_fn: Callable | None = None):
    """Token-sharded MaskedLinear forward: this rank's rows only, no communication."""
    if linear_fn is None:
        from .ops import MaskedLinear
        linear_fn = MaskedLinear.apply
    rows = row_shard(a.shape[0], rank, world)
    return rows, linear_fn(a[rows], b1, b2, mask[rows])


def all_reduce_gradients(tensors: Sequence[torch.Tensor], group=None, bucket_bytes: int = 256 << 20,
                         average: bool = False) -> None:
    """Data-parallel training: sum (or average) the per-rank weight gradients in place.

    In token-sharded mode every rank's ``MaskedLinear`` / ``MaskedFFN`` backward yields the partial
    weight gradient of its own tokens (the reference has no distributed path; its
    ``_bf16_linear_backward``, ``ffn_kernel/linear.py:455-496``, is the single-device partial).
    Gradients are packed into flat fp32 buckets so that a few large NCCL all-reduces run instead
    of one per tensor, and the sum over ranks is taken in fp32."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    world = dist.get_world_size(group)
    bucket, size = [], 0

    def flush():
        nonlocal bucket, size
        if not bucket:
            return
        flat = torch.cat([t.reshape(-1).float() for t in bucket])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            flat /= world
        off = 0
        for t in bucket:
            n = t.numel()
            t.copy_(flat[off:off + n].view(t.shape))       # copy_ honours the (possibly transposed) strides
            off += n
        bucket, size = [], 0

    for t in tensors:
        if t is None:
            continue
        bucket.append(t)
        size += t.numel() * 4
        if size >= bucket_bytes:
            flush()
    flush()


def _storage_order_view(t: torch.Tensor) -> torch.Tensor:
    """A view of ``t`` whose logical order is its memory order when ``t`` is a transposed dense matrix
    (so that flattening it is free); ``t`` itself otherwise."""
    if t.dim() == 2 and not t.is_contiguous() and t.T.is_contiguous():
        return t.T
    return t


class GradientSync:
    """Data-parallel training: all-reduce the weight gradients of every ``MaskedLinear`` backward inside
    the ``with`` block while that backward's dx GEMM runs.

    The backward computes the weight gradients first; the hook packs them into one fp32 bucket and starts
    the NCCL all-reduce on a side stream; the dx GEMM is launched on the compute stream beside it, leaving
    ``sm_margin`` SMs to the collective's kernels; before the backward returns, the compute stream is made
    to wait for the reduced gradients (written back in place), so autograd only ever sees the sums.  What
    the dx GEMM does not cover of the all-reduce is exposed.  ``reduce_dtype=torch.float32`` (default) sums
    over ranks in fp32 through one packed bucket; ``reduce_dtype=None`` all-reduces the bf16 gradients in
    place (no packing pass, half the bytes, bf16 additions).  The reference has no distributed path
    (``ffn_kernel/linear.py:455-496`` is the single-device partial)."""

    def __init__(self, group=None, average: bool = False, sm_margin: int = 16, reduce_dtype=torch.float32):
        self.group, self.average, self.sm_margin, self.reduce_dtype = group, average, sm_margin, reduce_dtype
        self._stream = None
        self._prev = None

    def __enter__(self):
        from . import linear
        self._prev = linear.GRAD_HOOK
        linear.GRAD_HOOK = self._hook
        return self

    def __exit__(self, *exc):
        from . import linear
        linear.GRAD_HOOK = self._prev
        return False

    def _hook(self, *grads):
        if not dist.is_initialized() or dist.get_world_size(self.group) == 1:
            return lambda: None
        from ._lib import lib
        dev = grads[0].device
        if self._stream is None or self._stream.device != dev:
            self._stream = torch.cuda.Stream(device=dev)
        main = torch.cuda.current_stream(dev)
        ready = torch.cuda.Event()
        ready.record(main)
        side = self._stream
        side.wait_event(ready)
        world = dist.get_world_size(self.group)
        with torch.cuda.stream(side):
            # gradients are packed in the order of their storage (a weight gradient carries its weight's
            # strides, usually the transposed view of [out, in] storage): a flat view, not a transposing copy
            views = [_storage_order_view(g) for g in grads]
            if self.reduce_dtype is None:
                # in place, in the gradients' own dtype: no packing pass, half the bytes of an fp32 bucket
                flat = None
                for v in views:
                    work = dist.all_reduce(v, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
                    work.wait()
                    if self.average:
                        v /= world
            else:
                flat = torch.cat([v.reshape(-1).to(self.reduce_dtype) for v in views])
                work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
                work.wait()                             # stream-level: the side stream waits, the host does not
                if self.average:
                    flat /= world
                off = 0
                for v in views:
                    n = v.numel()
                    v.copy_(flat[off:off + n].view(v.shape))
                    off += n
            done = torch.cuda.Event()
            done.record(side)
        lib().ffnk_set_sm_margin(self.sm_margin)        # the dx GEMM launched next leaves SMs to the collective

        def finish(flat=flat, grads=grads):
            lib().ffnk_set_sm_margin(0)
            main.wait_event(done)
            if flat is not None:
                flat.record_stream(main)
        return finish


def peer_block_rows(M: int, world: int) -> int:
    """Rows per owner in the fused tensor-parallel path: token ``t`` belongs to rank ``t // rows``."""
    if world < 1:
        raise ValueError("world must be positive")
    return max(1, -(-M // world))


def peer_owned_rows(M: int, rank: int, world: int) -> slice:
    """Token range owned by ``rank`` (empty for trailing ranks when ``M`` is small)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    rows = peer_block_rows(M, world)
    return slice(min(M, rank * rows), min(M, (rank + 1) * rows))


class PeerBlocks:
    """Peer-mapped buffers of one tensor-parallel group for ``masked_ffn_tp_fused``.

    Rank ``r`` owns tokens ``[r * rows, (r + 1) * rows)`` with ``rows = ceil(M / world)`` (per token
    chunk when the call is chunked).  Every rank holds, in symmetric memory mapped into all ranks:

    * block buffers: ``world`` row blocks, block ``s`` receiving rank ``s``'s partial result for the
      owner's rows (written by the peers' down projections);
    * output matrices ``[M, d]``: every owner stores its summed rows into the output of every rank;
    * one flag array for ``barrier()``.

    Two block buffers and two outputs alternate from call to call: the result of a call stays valid
    until the call after the next one on the same group.  Construction is collective: every rank of
    ``group`` must create it, in the same order.
    """

    MAX_CHUNKS = 8

    def __init__(self, M: int, d: int, group=None, device=None, buffers: int = 2):
        import ctypes

        import torch.distributed._symmetric_memory as symm

        if not dist.is_initialized():
            raise RuntimeError("PeerBlocks needs an initialised torch.distributed process group")
        group = group or dist.group.WORLD
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one NVLink domain)")
        if d % 8:
            raise ValueError("d must be a multiple of 8")
        self.M, self.d = M, d
        self.rows = peer_block_rows(M, self.world)
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.device = device
        self._handles = []

        def mapped(numel, dtype):
            t = symm.empty(numel, dtype=dtype, device=device)
            hdl = symm.rendezvous(t, group)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            if len(ptrs) != self.world or ptrs[self.rank] != t.data_ptr():
                raise RuntimeError("symmetric memory rendezvous returned unexpected buffer pointers")
            self._handles.append(hdl)
            return t, ptrs

        # chunked calls round each chunk's rows per owner up: room for MAX_CHUNKS extra rows per block
        self.block_rows_total = self.world * (self.rows + self.MAX_CHUNKS)
        self.buffers, self.buffer_ptrs, self.outs, self.out_ptrs = [], [], [], []
        for _ in range(buffers):
            t, ptrs = mapped(self.block_rows_total * d, torch.bfloat16)
            self.buffers.append(t.view(self.block_rows_total, d))
            self.buffer_ptrs.append(ptrs)
            y, yptrs = mapped(max(M, 1) * d, torch.bfloat16)
            self.outs.append(y.view(max(M, 1), d))
            self.out_ptrs.append((ctypes.c_void_p * self.world)(*yptrs))
            self._out_ptr_values = getattr(self, "_out_ptr_values", []) + [yptrs]
        self.pointers = [(ctypes.c_void_p * self.world)(*p) for p in self.buffer_ptrs]
        flags, fptrs = mapped(64, torch.int32)
        flags.zero_()
        self._flags = flags
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*fptrs)
        self._epoch = 0
        self._turn = 0
        self._side = torch.cuda.Stream(device=device)
        self._ptr_cache = {}
        # nobody may signal before every rank's flags are zero
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def next(self):
        """(block buffer, its peer pointers, output matrix, its peer pointers) of this call."""
        i = self._turn
        self._turn = (i + 1) % len(self.buffers)
        return i, self.buffers[i], self.pointers[i], self.outs[i], self.out_ptrs[i]

    def block_pointers(self, i: int, row_offset: int, col: int = 0):
        """Peer pointers of block buffer ``i`` advanced by ``row_offset`` rows (one chunk's region) and
        ``col`` columns (one column range of the output)."""
        import ctypes
        key = ("b", i, row_offset, col)
        p = self._ptr_cache.get(key)
        if p is None:
            off = (row_offset * self.d + col) * 2
            p = (ctypes.c_void_p * self.world)(*[q + off for q in self.buffer_ptrs[i]])
            self._ptr_cache[key] = p
        return p

    def out_pointers(self, i: int, col: int = 0):
        """Peer pointers of output matrix ``i`` advanced by ``col`` columns."""
        import ctypes
        if col == 0:
            return self.out_ptrs[i]
        key = ("o", i, col)
        p = self._ptr_cache.get(key)
        if p is None:
            p = (ctypes.c_void_p * self.world)(*[int(q) + col * 2 for q in self._out_ptr_values[i]])
            self._ptr_cache[key] = p
        return p

    def barrier(self, budget_us: int = 0) -> None:
        """Stream-ordered barrier on the current stream (``ffnk_peer_barrier``): returns, on the stream,
        once every rank's earlier work on its stream has completed.  Every rank must call the barriers
        of one ``PeerBlocks`` in the same order.  A rank that never arrives makes the others give up
        after ``budget_us`` (default 2 s) with a device status code (``check_status`` raises)."""
        from ._lib import check, lib
        from .route import status_word, stream_ptr
        self._epoch += 1
        check("ffnk_peer_barrier", lib().ffnk_peer_barrier(
            self._flag_ptrs, self.world, self.rank, self._epoch, budget_us, status_word(self.device).data_ptr(),
            stream_ptr(self.device)))

    def owned_rows(self) -> slice:
        return peer_owned_rows(self.M, self.rank, self.world)


def masked_ffn_tp_fused(x, w1, w2, w3, u1, u2, u3, mask, blocks: PeerBlocks, gather: bool = True, chunks: int = 1,
                        col_chunks: int = 1):
    """Tensor-parallel MaskedFFN forward whose communication is done by this library's own kernels
    over NVLink peer memory; no collective library call is on the path.

    The down projection writes its partial rows straight into the memory of the rank that owns them
    (peer stores from the GEMM epilogue, ``ffnk_ffn_down_to_peers``: the reduce-scatter's traffic
    flows while the GEMM computes); after one barrier (``ffnk_peer_barrier``) every owner sums the
    ``world`` partials in fp32 and stores the bf16 rows into the output of every rank
    (``ffnk_sum_row_blocks_to_peers``); a second barrier completes the output everywhere.

    ``gather=True`` returns the full ``y`` on every rank: a view of symmetric memory owned by
    ``blocks``, valid until the call after the next one.  ``gather=False`` returns
    ``(rows, y[rows])`` with ``rows = blocks.owned_rows()`` and skips the broadcast.
    ``chunks > 1`` (``gather=True`` only) splits the tokens into that many row ranges; the barrier,
    sum and broadcast of one chunk run on a side stream under the GEMMs of the next.
    ``col_chunks > 1`` (``gather=True``, ``chunks == 1``) splits only the down projection, by output
    columns: gate/up runs once over all tokens, and the barrier, sum and broadcast of one column range
    run on a side stream under the down projection of the next, so that half of the broadcast crosses
    the link while the GEMM still computes.
    The weights are this rank's shards (``shard_ffn_weights``); ``x`` and ``mask`` are replicated."""
    from ._lib import check, lib
    from .ffn import _phase, permute_rows_first
    from .linear import _activation, _check_dims, _mask_route, _weights
    from .route import maybe_check, status_word, stream_ptr

    x = _activation(x, "x")
    M, d = x.shape
    h = w1.shape[1] if isinstance(w1, torch.Tensor) and w1.dim() == 2 else -1
    w1, w3, u1, u3 = _weights((w1, w3, u1, u3), ("w1", "w3", "u1", "u3"), d, h)
    w2, u2 = _weights((w2, u2), ("w2", "u2"), h, d)
    _check_dims(d=d, h=h)
    if (M, d) != (blocks.M, blocks.d) or x.device != blocks.device:
        raise RuntimeError(f"PeerBlocks were made for [{blocks.M}, {blocks.d}] on {blocks.device}")
    chunks = max(1, min(int(chunks), blocks.MAX_CHUNKS, max(1, M)))
    if chunks > 1 and not gather:
        raise ValueError("chunks > 1 needs gather=True (owned rows are interleaved by chunk)")
    col_chunks = max(1, min(int(col_chunks), 8, d // 256)) if (gather and chunks == 1 and d % 8 == 0) else 1
    dev = x.device
    L = lib()
    world, rank = blocks.world, blocks.rank
    with torch.cuda.device(dev):
        st = status_word(dev).data_ptr()
        main = torch.cuda.current_stream(dev)
        turn, buf, _, y, y_ptrs = blocks.next()

        def gate_up(tok: slice):
            """route, (permute,) gate/up of one token range -> (routing lists, routed intermediate)"""
            Mc = tok.stop - tok.start
            sp = stream_ptr(dev)
            xc, mc = x[tok], mask[tok]
            _phase("route")
            rt = _mask_route(mc, Mc, dev, None)
            inter = torch.empty((rt.cap + 512, h), device=dev, dtype=torch.bfloat16)
            xin, routed_in = xc, 0
            if permute_rows_first(Mc, d, h):
                _phase("permute")
                xin = torch.empty((rt.cap + 512, d), device=dev, dtype=torch.bfloat16)
                check("ffnk_permute_rows", L.ffnk_permute_rows(
                    xc.data_ptr(), xc.stride(0), rt.perm.data_ptr(), rt.counts.data_ptr(), xin.data_ptr(),
                    xin.stride(0), Mc, d, sp))
                routed_in = 1
            _phase("gateup")
            check("ffnk_ffn_gateup", L.ffnk_ffn_gateup(
                xin.data_ptr(), xin.stride(0), w1.data_ptr(), w3.data_ptr(), u1.data_ptr(), u3.data_ptr(),
                w1.stride(0), w1.stride(1), rt.perm.data_ptr(), rt.counts.data_ptr(), inter.data_ptr(),
                inter.stride(0), routed_in, 1, Mc, d, h, st, sp))
            _phase("down")
            return rt, inter

        def down_to_peers(rt, inter, Mc: int, rows_c: int, block_ptrs, col0: int = 0, ncols: int = d):
            """the peer-storing down projection of output columns [col0, col0 + ncols)"""
            wv, wu = w2[:, col0:col0 + ncols], u2[:, col0:col0 + ncols]
            check("ffnk_ffn_down_to_peers", L.ffnk_ffn_down_to_peers(
                inter.data_ptr(), inter.stride(0), wv.data_ptr(), wu.data_ptr(), wv.stride(0), wv.stride(1),
                rt.perm.data_ptr(), rt.counts.data_ptr(), block_ptrs, world, rank, rows_c, d, Mc, ncols, h, st,
                stream_ptr(dev)))

        def compute_chunk(tok: slice, rows_c: int, block_ptrs):
            rt, inter = gate_up(tok)
            down_to_peers(rt, inter, tok.stop - tok.start, rows_c, block_ptrs)
            _phase("end")

        def sum_chunk(tok: slice, rows_c: int, region_row0: int, to_peers: bool, own=None, max_ctas: int = 0,
                      col0: int = 0, ncols: int = d):
            """this rank's rows of one token range: fp32 sum of the world partials, to every rank or locally"""
            Mc = tok.stop - tok.start
            n_own = max(0, min(rows_c, Mc - rank * rows_c))
            if n_own == 0:
                return
            src = buf[region_row0:region_row0 + world * rows_c]
            sp = stream_ptr(dev)
            if to_peers:
                check("ffnk_sum_row_blocks_to_peers", L.ffnk_sum_row_blocks_to_peers(
                    src.data_ptr() + col0 * 2, world, rows_c, n_own, ncols, d, blocks.out_pointers(turn, col0), world,
                    tok.start + rank * rows_c, d, max_ctas, sp))
            else:
                # blocks are rows_c rows apart; only the first n_own rows of each exist
                check("ffnk_sum_row_blocks", L.ffnk_sum_row_blocks(src.data_ptr(), world, rows_c, d, d, own.data_ptr(), d, sp))

        if M == 0:
            if gather:
                return y[:0]
            return blocks.owned_rows(), torch.empty((0, d), device=dev, dtype=torch.bfloat16)

        if chunks == 1 and col_chunks == 1:
            tok, rows_c = slice(0, M), blocks.rows
            compute_chunk(tok, rows_c, blocks.block_pointers(turn, 0))
            blocks.barrier()
            if not gather:
                own = torch.empty((rows_c, d), device=dev, dtype=torch.bfloat16)
                sum_chunk(tok, rows_c, 0, False, own)
                maybe_check(dev)
                r = blocks.owned_rows()
                return r, own[: r.stop - r.start]
            sum_chunk(tok, rows_c, 0, True)
            blocks.barrier()
            maybe_check(dev)
            return y[:M]

        side = blocks._side
        if chunks == 1:
            # one gate/up over all tokens; the down projection in column ranges (multiples of 256 columns),
            # each range's barrier, sum and broadcast on the side stream under the next range's GEMM
            tok, rows_c = slice(0, M), blocks.rows
            rt, inter = gate_up(tok)
            step = -(-(d // 256) // col_chunks) * 256
            col0 = 0
            while col0 < d:
                ncols = min(step, d - col0)
                down_to_peers(rt, inter, M, rows_c, blocks.block_pointers(turn, 0, col0), col0, ncols)
                ev = torch.cuda.Event()
                ev.record(main)
                side.wait_event(ev)
                with torch.cuda.stream(side):
                    blocks.barrier()
                    sum_chunk(tok, rows_c, 0, True, max_ctas=0 if col0 + ncols >= d else 148, col0=col0, ncols=ncols)
                col0 += ncols
            _phase("end")
            with torch.cuda.stream(side):
                blocks.barrier()
                done = torch.cuda.Event()
                done.record(side)
            main.wait_event(done)
            inter.record_stream(main)
            maybe_check(dev)
            return y[:M]

        region = 0
        for c in range(chunks):
            tok = row_shard(M, c, chunks)
            rows_c = peer_block_rows(tok.stop - tok.start, world)
            compute_chunk(tok, rows_c, blocks.block_pointers(turn, region))
            ev = torch.cuda.Event()
            ev.record(main)
            side.wait_event(ev)
            with torch.cuda.stream(side):
                blocks.barrier()
                # the sum runs beside the next chunk's GEMMs: a quarter of the SMs' worth of CTAs is plenty
                # for a kernel that is bound by the NVLink, and leaves the GEMM's epilogue warps their issue slots
                sum_chunk(tok, rows_c, region, True, max_ctas=0 if c == chunks - 1 else 148)
            region += world * rows_c
        with torch.cuda.stream(side):
            blocks.barrier()
            done = torch.cuda.Event()
            done.record(side)
        main.wait_event(done)
        maybe_check(dev)
        return y[:M]
