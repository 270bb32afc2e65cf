"""Seeded synthetic inputs for the masked linear / FFN workloads.

The reference benchmarks on no public dataset: its scripts draw ``torch.rand``
activations and one image span (``test_ffn.py:12-18,104``).  The workloads here
follow the named benchmark shapes instead: N(0,1) bf16 activations, N(0,0.02)
bf16 weights held in ``nn.Linear`` storage order ``[out, in]`` and handed to the
operators as the ``.T`` view, and a mask made of contiguous image spans
alternating with text spans of random length.
"""
from __future__ import annotations

import random
from dataclasses import dataclass

import torch


def span_mask(M: int, seed: int = 0, image_lens=(576,), visual_frac: float = 0.5,
              text_min: int = 64) -> torch.Tensor:
    """Boolean [M] mask (True = visual token): text span, image span, text span, ...

    Image spans have a length drawn from ``image_lens``; text spans are uniform on
    ``[text_min, text_max]`` with ``text_max`` chosen so that the expected visual
    fraction is ``visual_frac``.
    """
    rng = random.Random(seed)
    mean_img = sum(image_lens) / len(image_lens)
    mean_txt = mean_img * (1.0 - visual_frac) / max(visual_frac, 1e-6)
    text_max = max(text_min, int(round(2 * mean_txt - text_min)))
    mask = torch.zeros(M, dtype=torch.bool)
    pos = 0
    while pos < M:
        pos += rng.randint(text_min, text_max)
        if pos >= M:
            break
        n = rng.choice(list(image_lens))
        mask[pos:min(M, pos + n)] = True
        pos += n
    return mask


def edge_mask(M: int, kind: str, seed: int = 0) -> torch.Tensor:
    """Masks of the edge sweep: all visual, all text, per-token alternating, Bernoulli(0.5)."""
    if kind == "all_visual":
        return torch.ones(M, dtype=torch.bool)
    if kind == "all_text":
        return torch.zeros(M, dtype=torch.bool)
    if kind == "alternating":
        return (torch.arange(M) % 2) == 0
    if kind == "bernoulli":
        g = torch.Generator().manual_seed(seed)
        return torch.rand(M, generator=g) < 0.5
    if kind == "span":
        return span_mask(M, seed)
    raise ValueError(f"unknown mask kind {kind!r}")


def _randn_bf16(shape, std, gen) -> torch.Tensor:
    return (torch.randn(shape, generator=gen, dtype=torch.float32) * std).to(torch.bfloat16)


@dataclass
class LinearCase:
    x: torch.Tensor          # [M, K] bf16
    wv: torch.Tensor         # [N, K] bf16, nn.Linear storage (visual)
    wt: torch.Tensor         # [N, K] bf16 (text)
    mask: torch.Tensor       # [M] bool
    g: torch.Tensor | None   # [M, N] bf16 upstream gradient

    def to(self, device):
        mv = lambda t: None if t is None else t.to(device)
        return LinearCase(mv(self.x), mv(self.wv), mv(self.wt), mv(self.mask), mv(self.g))


@dataclass
class FFNCase:
    x: torch.Tensor      # [M, d] bf16
    w1: torch.Tensor     # [h, d]   visual gate   (nn.Linear storage)
    w2: torch.Tensor     # [d, h]   visual down
    w3: torch.Tensor     # [h, d]   visual up
    u1: torch.Tensor     # text gate
    u2: torch.Tensor     # text down
    u3: torch.Tensor     # text up
    mask: torch.Tensor   # [M] bool

    def to(self, device):
        return FFNCase(*(t.to(device) for t in
                         (self.x, self.w1, self.w2, self.w3, self.u1, self.u2, self.u3, self.mask)))

    def apply_args(self):
        """Arguments in ``MaskedFFN.apply`` order, weights as ``.T`` views."""
        return (self.x, self.w1.T, self.w2.T, self.w3.T, self.u1.T, self.u2.T, self.u3.T, self.mask)


def linear_case(M: int, K: int, N: int, seed: int = 0, mask: torch.Tensor | None = None,
                with_grad: bool = False, visual_frac: float = 0.5, image_lens=(576,)) -> LinearCase:
    gen = torch.Generator().manual_seed(seed)
    x = _randn_bf16((M, K), 1.0, gen)
    wv = _randn_bf16((N, K), 0.02, gen)
    wt = _randn_bf16((N, K), 0.02, gen)
    g = _randn_bf16((M, N), 1.0, gen) if with_grad else None
    if mask is None:
        mask = span_mask(M, seed, image_lens=image_lens, visual_frac=visual_frac)
    return LinearCase(x, wv, wt, mask, g)


def ffn_case(M: int, d: int, h: int, seed: int = 0, mask: torch.Tensor | None = None,
             visual_frac: float = 0.5) -> FFNCase:
    gen = torch.Generator().manual_seed(seed)
    x = _randn_bf16((M, d), 1.0, gen)
    ws = [_randn_bf16(s, 0.02, gen) for s in ((h, d), (d, h), (h, d), (h, d), (d, h), (h, d))]
    if mask is None:
        mask = span_mask(M, seed, visual_frac=visual_frac)
    return FFNCase(x, *ws, mask)


def ffn_tokens(M: int, d: int, seed: int, visual_frac: float = 0.5):
    """One more batch of activations and mask for an existing FFN case (same weights, new tokens)."""
    gen = torch.Generator().manual_seed(1000003 + seed)
    return _randn_bf16((M, d), 1.0, gen), span_mask(M, 1000003 + seed, visual_frac=visual_frac)


# The named benchmark configurations: name -> (kind, dims)
CONFIGS = {
    "c1_linear_d1024_m4096": dict(op="linear", M=4096, K=1024, N=1024, visual_frac=0.5),
    "c2_ffn_d1024_h2048_m32768": dict(op="ffn", M=32768, d=1024, h=2048, visual_frac=0.5),
    "c3_linear_d4096_m32768": dict(op="linear_fwd_bwd", M=32768, K=4096, N=4096, visual_frac=0.7,
                                   image_lens=(576, 2304)),
    "c4_ffn_d4096_h11008_m16384": dict(op="ffn", M=16384, d=4096, h=11008, visual_frac=0.5),
    "c5_ffn_d1024_h2816": dict(op="ffn_sweep", d=1024, h=2816, Ms=(1, 8, 64, 127, 1000, 4099),
                               masks=("all_visual", "all_text", "alternating", "bernoulli")),
}
