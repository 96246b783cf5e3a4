"""Debug helpers: NVTX ranges, a profiler capture window by training step and per-rank tensor dumps
for A/B comparison (reference ``kareus/utils/debug.py:7-28``; step window:
``3rdparty/NeMo/nemo/core/classes/modelPT.py:1835-1881``, ``nsys_profile.{start_step,end_step,ranks}``)."""
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


class ProfilerStepWindow:
    """Trainer hook that opens the CUDA profiler's capture range at ``start_step`` and closes it after
    ``end_step`` on the listed ranks (``cudaProfilerStart`` / ``cudaProfilerStop``), so that
    ``nsys profile --capture-range=cudaProfilerApi`` or ``ncu --profile-from-start off`` records only
    those steps.  Every instruction inside the window gets an NVTX range."""

    def __init__(self, start_step: int = 10, end_step: int = 10, ranks=(0,), rank: int = 0, start_fn=None,
                 stop_fn=None):
        if end_step < start_step:
            raise ValueError("end_step must not be before start_step")
        self.start_step, self.end_step = int(start_step), int(end_step)
        self.enabled = rank in set(ranks)
        self.step = 0
        self.open = False
        self._start = start_fn or (lambda: torch.cuda.profiler.start())
        self._stop = stop_fn or (lambda: torch.cuda.profiler.stop())

    def on_step_begin(self):
        if self.enabled and self.step == self.start_step and not self.open:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self._start()
            self.open = True

    def on_instruction_begin(self, name: str):
        if self.open and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(f"step{self.step}/{name}")

    def on_instruction_end(self, name: str):
        if self.open and torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()

    def on_step_end(self):
        if self.open and self.step == self.end_step:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self._stop()
            self.open = False
        self.step += 1
