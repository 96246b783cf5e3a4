"""Debug helpers: NVTX ranges and per-rank tensor dumps for A/B comparison
(reference ``kareus/utils/debug.py:7-28``)."""
from __future__ import annotations

import contextlib
import os
from pathlib import Path

import torch


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool = True, sync: bool = False):
    """NVTX range around a block; ``sync`` adds a device synchronisation at the end (the reference
    synchronises after each debug range so ranges do not overlap on the timeline)."""
    on = enabled and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            if sync:
                torch.cuda.synchronize()
            torch.cuda.nvtx.range_pop()


def save_tensors(tensors: dict, out_dir, tp_rank: int = 0, pp_rank: int = 0, tag: str = "tensors") -> Path:
    """Write ``{name: tensor}`` to ``<out_dir>/<tag>_tp<r>_pp<r>.pt`` (CPU copies)."""
    d = Path(out_dir)
    d.mkdir(parents=True, exist_ok=True)
    path = d / f"{tag}_tp{tp_rank}_pp{pp_rank}.pt"
    torch.save({k: v.detach().cpu() for k, v in tensors.items()}, path)
    return path
