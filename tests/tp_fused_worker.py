"""One rank of the multi-GPU check of ``masked_ffn_tp_fused`` (run under torch.distributed.run by
``test_gpu_tp_fused.py``; not collected by pytest).  Every rank computes the tensor-parallel
MaskedFFN several ways -- fused peer stores with the result broadcast to every rank (whole and in
token chunks) or left row-sharded, and partial outputs summed by an NCCL all-reduce -- and rank 0
compares them with the fp32 oracle.  With
``--time`` it also prints device timings of the variants."""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ffn_kernel_b200 import check_status, tp  # noqa: E402
from ffn_kernel_b200.synth import edge_mask, ffn_case  # noqa: E402


def timed(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / steps], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1000)
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--hidden", type=int, default=960)
    ap.add_argument("--mask-kind", default="span")
    ap.add_argument("--time", action="store_true")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--no-oracle", action="store_true")
    args = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    c = ffn_case(args.tokens, args.dim, args.hidden, seed=3, mask=edge_mask(args.tokens, args.mask_kind, seed=7))
    g = c.to(dev)
    x, mask = g.x, g.mask
    shards = tp.shard_ffn_weights(*g.apply_args()[1:7], rank, world)
    blocks = tp.PeerBlocks(args.tokens, args.dim)

    out = {}
    for rep in range(3):                       # repeated calls alternate the two block buffers
        y_fused = tp.masked_ffn_tp_fused(x, *shards, mask, blocks)
    y_fused = y_fused.clone()                  # the result lives in the group's buffers (valid for two calls)
    rows, y_own = tp.masked_ffn_tp_fused(x, *shards, mask, blocks, gather=False)
    y_nccl = tp.masked_ffn_tp(x, *shards, mask)
    y_chunked = {c: tp.masked_ffn_tp_fused(x, *shards, mask, blocks, chunks=c).clone() for c in (2, 3)}
    y_chunked.update({f"col{c}": tp.masked_ffn_tp_fused(x, *shards, mask, blocks, col_chunks=c).clone() for c in (2, 4)})
    torch.cuda.synchronize()
    check_status()
    out["fused_vs_nccl"] = float((y_fused.float() - y_nccl.float()).abs().max() / y_nccl.float().abs().max())
    out["own_rows_equal"] = bool(torch.equal(y_own, y_fused[rows]))
    # a chunk routes its own token range, so tile boundaries differ from the unchunked call; the sums
    # are the same fp32 sums of the same bf16 partials, hence bit-identical rows
    out["chunked_equal"] = all(bool(torch.equal(v, y_fused)) for v in y_chunked.values())
    # every rank must hold the same full result
    ref_y = y_fused.clone()
    dist.broadcast(ref_y, 0)
    same_y = torch.tensor([1.0 if torch.equal(ref_y, y_fused) else 0.0], device=dev)
    dist.all_reduce(same_y, op=dist.ReduceOp.MIN)
    out["all_ranks_equal"] = bool(same_y.item() == 1.0)
    same = torch.tensor([1.0 if out["own_rows_equal"] else 0.0], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    out["own_rows_equal"] = bool(same.item() == 1.0)
    if not args.no_oracle and rank == 0:
        from oracle import masked_ref as O
        ref = O.masked_ffn(*c.apply_args())
        out["fused_vs_oracle"] = float(O.max_rel_err(y_fused, ref))
        out["nccl_vs_oracle"] = float(O.max_rel_err(y_nccl, ref))
    if args.time:
        flops = 6.0 * args.tokens * args.dim * args.hidden
        for name, fn in (("fused_broadcast", lambda: tp.masked_ffn_tp_fused(x, *shards, mask, blocks)),
                         ("fused_broadcast_2col", lambda: tp.masked_ffn_tp_fused(x, *shards, mask, blocks, col_chunks=2)),
                         ("fused_broadcast_4col", lambda: tp.masked_ffn_tp_fused(x, *shards, mask, blocks, col_chunks=4)),
                         ("fused_broadcast_2chunks", lambda: tp.masked_ffn_tp_fused(x, *shards, mask, blocks, chunks=2)),
                         ("fused_broadcast_4chunks", lambda: tp.masked_ffn_tp_fused(x, *shards, mask, blocks, chunks=4)),
                         ("fused_row_sharded", lambda: tp.masked_ffn_tp_fused(x, *shards, mask, blocks, gather=False)),
                         ("nccl_all_reduce", lambda: tp.masked_ffn_tp(x, *shards, mask)),
                         ("nccl_reduce_scatter", (lambda: tp.masked_ffn_tp_reduce_scatter(x, *shards, mask))
                          if args.tokens % world == 0 else None)):
            if fn is None:
                continue
            ms = timed(fn, args.steps, 5)
            out[name] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12}
        check_status()
    if rank == 0:
        out.update(world=world, M=args.tokens, d=args.dim, h=args.hidden, mask=args.mask_kind)
        print("TP_FUSED " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
