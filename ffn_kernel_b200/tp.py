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
