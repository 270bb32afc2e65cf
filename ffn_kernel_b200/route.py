"""Routing: the boolean token mask becomes two compacted, ascending row lists.

The reference never materialises such lists; every one of its kernels re-derives, per
128-row tile, whether the tile is all visual, all text or mixed
(``ffn_kernel/linear.py:132-149``, ``ffn_kernel/ffn.py:72-99``) and computes both
products for mixed tiles.  Here the lists are built once per call by a single-pass scan
kernel and every GEMM tile belongs to exactly one modality.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from ._lib import check, lib, FfnkError

_status_words: dict[int, torch.Tensor] = {}


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor; this package has no CPU path")


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def status_word(device) -> torch.Tensor:
    """Per-device int32 word that kernels write a code into when a bounded wait expires."""
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _status_words[idx] = w
    return w


def check_status(device=None) -> None:
    """Synchronise the current stream and raise if any kernel recorded a device-side error."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(device):
        code = lib().ffnk_read_status(status_word(device).data_ptr(), 1, stream_ptr(device))
    if code != 0:
        raise FfnkError("device status", code)


def maybe_check(device) -> None:
    if os.environ.get("FFNK_DEBUG_SYNC") == "1":
        check_status(device)


@dataclass
class Route:
    """Device-resident routing lists for one mask (see ``include/ffnk.h``, ffnk_route)."""
    perm: torch.Tensor     # int32 [2 * cap]
    counts: torch.Tensor   # int32 [8] = Mv, Mt, cap, M, runs, (unused)
    M: int
    cap: int

    def lists(self) -> tuple[torch.Tensor, torch.Tensor]:
        """(visual rows, text rows) as int32 tensors; synchronises to read the counts."""
        mv, mt = (int(v) for v in self.counts[:2].tolist())
        return self.perm[:mv], self.perm[self.cap:self.cap + mt]


def route(mask: torch.Tensor) -> Route:
    """mask: bool/uint8 [M] on a CUDA device -> Route.  No host synchronisation."""
    _require_cuda(mask, "mask")
    if mask.dim() != 1:
        raise RuntimeError(f"mask must be 1-D [M], got shape {tuple(mask.shape)}")
    if mask.dtype not in (torch.bool, torch.uint8):
        raise RuntimeError(f"mask must be torch.bool (or uint8), got {mask.dtype}")
    mask = mask.contiguous()
    M = mask.shape[0]
    L = lib()
    dev = mask.device
    cap = int(L.ffnk_route_capacity(M))
    with torch.cuda.device(dev):
        perm = torch.empty(max(2 * cap, 4), dtype=torch.int32, device=dev)
        counts = torch.empty(8, dtype=torch.int32, device=dev)
        ws = torch.empty(max(int(L.ffnk_route_workspace_bytes(M)), 4), dtype=torch.uint8, device=dev)
        check("ffnk_route", L.ffnk_route(mask.data_ptr(), M, perm.data_ptr(), counts.data_ptr(), ws.data_ptr(),
                                         status_word(dev).data_ptr(), stream_ptr(dev)))
    maybe_check(dev)
    return Route(perm, counts, M, cap)
