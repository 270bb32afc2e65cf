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
    """Per-rank block buffers, mapped into every rank, for ``masked_ffn_tp_fused``.

    Rank ``r`` owns tokens ``[r * rows, (r + 1) * rows)`` with ``rows = ceil(M / world)``.  Its buffer
    holds ``world`` row blocks of ``rows x d`` bf16; block ``s`` receives rank ``s``'s partial result
    for the owner's rows.  Two buffers alternate from call to call, so the writes of step ``k + 1``
    never touch what an owner may still be summing from step ``k`` (one barrier per step is
    enough).  Construction is collective: every rank of ``group`` must create it, in the same order.
    """

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
        self.buffers, self.pointers, self._handles = [], [], []
        for _ in range(buffers):
            t = symm.empty(self.world * self.rows * d, dtype=torch.bfloat16, device=device)
            hdl = symm.rendezvous(t, group)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            if len(ptrs) != self.world or ptrs[self.rank] != t.data_ptr():
                raise RuntimeError("symmetric memory rendezvous returned unexpected buffer pointers")
            self.buffers.append(t.view(self.world * self.rows, d))
            self.pointers.append((ctypes.c_void_p * self.world)(*ptrs))
            self._handles.append(hdl)
        self._turn = 0
        self._token = torch.zeros(1, dtype=torch.float32, device=device)

    def next(self):
        i = self._turn
        self._turn = (i + 1) % len(self.buffers)
        return self.buffers[i], self.pointers[i]

    def barrier(self) -> None:
        """Stream-ordered barrier: returns (on the stream) once every rank's earlier work on its
        stream has completed.  A one-element all-reduce: its kernel on each rank starts after that
        rank's earlier kernels and cannot finish before all ranks have contributed."""
        dist.all_reduce(self._token, op=dist.ReduceOp.SUM, group=self.group)

    def owned_rows(self) -> slice:
        return peer_owned_rows(self.M, self.rank, self.world)


def masked_ffn_tp_fused(x, w1, w2, w3, u1, u2, u3, mask, blocks: PeerBlocks, gather: bool = True):
    """Tensor-parallel MaskedFFN forward whose down projection writes its partial rows straight
    into the memory of the rank that owns them (NVLink peer stores from the GEMM epilogue,
    ``ffnk_ffn_down_to_peers``), followed by one barrier and a local fp32 sum of the ``world``
    partials (``ffnk_sum_row_blocks``).  The partial ``y`` never exists in this rank's memory and
    no reduction collective runs.

    ``gather=True`` returns the full ``y`` on every rank (one all-gather of the owned rows);
    ``gather=False`` returns ``(rows, y[rows])`` with ``rows = blocks.owned_rows()``.
    The weights are this rank's shards (``shard_ffn_weights``); ``x`` and ``mask`` are replicated."""
    from ._lib import check, lib
    from .ffn import permute_rows_first
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
    dev = x.device
    L = lib()
    world, rank, rows = blocks.world, blocks.rank, blocks.rows
    with torch.cuda.device(dev):
        st, sp = status_word(dev).data_ptr(), stream_ptr(dev)
        own = torch.empty((rows, d), device=dev, dtype=torch.bfloat16)
        if M > 0:
            rt = _mask_route(mask, M, dev, None)
            inter = torch.empty((rt.cap + 512, h), device=dev, dtype=torch.bfloat16)
            xin, routed_in = x, 0
            if permute_rows_first(M, d, h):
                xin = torch.empty((rt.cap + 512, d), device=dev, dtype=torch.bfloat16)
                check("ffnk_permute_rows", L.ffnk_permute_rows(
                    x.data_ptr(), x.stride(0), rt.perm.data_ptr(), rt.counts.data_ptr(), xin.data_ptr(),
                    xin.stride(0), M, d, sp))
                routed_in = 1
            check("ffnk_ffn_gateup", L.ffnk_ffn_gateup(
                xin.data_ptr(), xin.stride(0), w1.data_ptr(), w3.data_ptr(), u1.data_ptr(), u3.data_ptr(),
                w1.stride(0), w1.stride(1), rt.perm.data_ptr(), rt.counts.data_ptr(), inter.data_ptr(),
                inter.stride(0), routed_in, 1, M, d, h, st, sp))
            buf, ptrs = blocks.next()
            check("ffnk_ffn_down_to_peers", L.ffnk_ffn_down_to_peers(
                inter.data_ptr(), inter.stride(0), w2.data_ptr(), u2.data_ptr(), w2.stride(0), w2.stride(1),
                rt.perm.data_ptr(), rt.counts.data_ptr(), ptrs, world, rank, rows, d, M, d, h, st, sp))
            blocks.barrier()
            check("ffnk_sum_row_blocks", L.ffnk_sum_row_blocks(buf.data_ptr(), world, rows, d, d, own.data_ptr(), d, sp))
        maybe_check(dev)
        if not gather:
            r = blocks.owned_rows()
            return r, own[: r.stop - r.start]
        y = torch.empty((world * rows, d), device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(y, own, group=blocks.group)
        return y[:M]
