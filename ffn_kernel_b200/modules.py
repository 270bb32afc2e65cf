"""nn.Module wrappers around the operators, shipped in the package.

The reference defines these only in its README and benchmark scripts (``README.md:60-73`` /
``test_linear.py:52-65`` for the linear layer -- the README version forgets to ``return`` --
and ``README.md:101-123`` / ``test_ffn.py:50-72`` for the FFN).  Same parameter names
(``linear_v``/``linear_t``; ``w1,w2,w3,u1,u2,u3``), same call convention
``module(x[B, S, D], mask[B, S])``, weights kept in ``nn.Linear`` storage and handed to the
operators as ``.T`` views, so a reference checkpoint loads with ``load_state_dict``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import tp as _tp
from .ops import MaskedFFN, MaskedLinear


class MaskedLinearModule(nn.Module):
    """Two-modality linear layer: visual tokens (mask True) use ``linear_v``, text tokens ``linear_t``.
    Forward and backward run the routed kernels (``MaskedLinear``)."""

    def __init__(self, in_dim: int, out_dim: int, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.linear_v = nn.Linear(in_dim, out_dim, bias=False, device=device, dtype=dtype)
        self.linear_t = nn.Linear(in_dim, out_dim, bias=False, device=device, dtype=dtype)

    def forward(self, x: torch.Tensor, visual_mask: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        y = MaskedLinear.apply(x.reshape(-1, x.shape[-1]), self.linear_v.weight.T, self.linear_t.weight.T,
                               visual_mask.reshape(-1))
        return y.view(*lead, -1)


class MaskedFFNModule(nn.Module):
    """Two-modality SwiGLU FFN: ``w2(silu(w1 x) * w3 x)`` for visual tokens, ``u*`` for text tokens."""

    def __init__(self, hidden_size: int, intermediate_size: int, device=None, dtype=torch.bfloat16):
        super().__init__()
        mk = lambda i, o: nn.Linear(i, o, bias=False, device=device, dtype=dtype)
        self.w1, self.w2, self.w3 = mk(hidden_size, intermediate_size), mk(intermediate_size, hidden_size), \
            mk(hidden_size, intermediate_size)
        self.u1, self.u2, self.u3 = mk(hidden_size, intermediate_size), mk(intermediate_size, hidden_size), \
            mk(hidden_size, intermediate_size)

    def weight_views(self):
        """The six ``[in, out]`` views in ``MaskedFFN.apply`` order."""
        return tuple(getattr(self, n).weight.T for n in ("w1", "w2", "w3", "u1", "u2", "u3"))

    def forward(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        y = MaskedFFN.apply(x.reshape(-1, x.shape[-1]), *self.weight_views(), mask.reshape(-1))
        return y.view(*lead, -1)


class GraphedMaskedFFN:
    """The inference forward of a ``MaskedFFNModule`` for one fixed token count, captured in a CUDA
    graph: routing, the row permutation and both GEMMs (or the decode kernels) replay as one graph
    launch with none of the per-call host work.  Meant for serving loops at small token counts,
    where the kernels take 12-45 us and the Python call path more than that.

    ``graphed(x, mask)`` copies the inputs into the graph's static buffers, replays, and returns the
    static output tensor (valid until the next call)."""

    def __init__(self, module: MaskedFFNModule, tokens: int, warmup: int = 3):
        from .ffn import _bf16_ffn_fused_forward
        w = module.w1.weight
        if not w.is_cuda:
            raise RuntimeError("the module must live on a CUDA device; this package has no CPU path")
        self.tokens = tokens
        self.x = torch.zeros((tokens, w.shape[1]), device=w.device, dtype=torch.bfloat16)
        self.mask = torch.zeros(tokens, device=w.device, dtype=torch.bool)
        views = tuple(v.detach() for v in module.weight_views())
        side = torch.cuda.Stream(device=w.device)
        side.wait_stream(torch.cuda.current_stream(w.device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):       # allocator warm-up outside the capture
                _bf16_ffn_fused_forward(self.x, *views, self.mask)
        torch.cuda.current_stream(w.device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.y = _bf16_ffn_fused_forward(self.x, *views, self.mask)

    def __call__(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        if x.numel() != self.x.numel() or mask.numel() != self.tokens:
            raise RuntimeError(f"this graph was captured for {self.tokens} tokens of width {self.x.shape[1]}")
        self.x.copy_(x.reshape(self.x.shape))
        self.mask.copy_(mask.reshape(-1))
        self.graph.replay()
        return self.y.view(*x.shape[:-1], -1)


class TensorParallelMaskedFFN(nn.Module):
    """One tensor-parallel rank of a ``MaskedFFNModule``: holds views of columns
    ``[r*h/P, (r+1)*h/P)`` of the gate/up weights and the matching rows of the down weights, and sums
    the partial outputs over ``group`` (see ``tp.masked_ffn_tp``)."""

    def __init__(self, full: MaskedFFNModule, rank: int, world: int, group=None, chunks: int = 1):
        super().__init__()
        self.full = full
        self.rank, self.world, self.group, self.chunks = rank, world, group, chunks

    @torch.no_grad()
    def forward(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        shards = _tp.shard_ffn_weights(*self.full.weight_views(), self.rank, self.world)
        y = _tp.masked_ffn_tp(x.reshape(-1, x.shape[-1]), *shards, mask.reshape(-1), group=self.group,
                              chunks=self.chunks)
        return y.view(*lead, -1)


# the names the reference's README uses for its wrappers
TritonLinear = MaskedLinearModule
TritonFFN = MaskedFFNModule
