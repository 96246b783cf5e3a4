"""Instruction timers with CSV export (the input of the frequency-only baseline profile).

Reference: Megatron ``Timers`` as patched by Kareus (``3rdparty/Megatron-LM/megatron/core/
timers.py:220-258,449-462``): ``forward-compute`` / ``backward-compute`` record wall-clock start and
end lists (each start/stop synchronises the device) and are written to
``timers/instructions-<global rank>-<local rank>.csv``.  As a trainer hook it times every pipeline
instruction.
"""
from __future__ import annotations

import csv
import time
from pathlib import Path
from typing import Dict, List, Tuple

import torch


class Timers:
    def __init__(self, sync: bool = True):
        self.sync = sync
        self.records: Dict[str, List[Tuple[float, float]]] = {}
        self._open: Dict[str, float] = {}

    def _now(self) -> float:
        if self.sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        return time.time()

    def start(self, name: str) -> None:
        if name in self._open:
            raise RuntimeError(f"timer {name!r} already started")
        self._open[name] = self._now()

    def stop(self, name: str) -> float:
        t0 = self._open.pop(name)
        t1 = self._now()
        self.records.setdefault(name, []).append((t0, t1))
        return t1 - t0

    # trainer hook interface ---------------------------------------------------
    def on_step_begin(self):
        pass

    def on_instruction_begin(self, name: str):
        self.start(f"{name}-compute")

    def on_instruction_end(self, name: str):
        self.stop(f"{name}-compute")

    def on_step_end(self):
        pass

    def export(self, out_dir, global_rank: int = 0, local_rank: int = 0) -> Path:
        d = Path(out_dir) / "timers"
        d.mkdir(parents=True, exist_ok=True)
        p = d / f"instructions-{global_rank}-{local_rank}.csv"
        with p.open("w", newline="") as f:
            w = csv.writer(f)
            # columns of the reference's file (tests/perseus/generate_profile_csv.py:203-212 reads
            # instruction, start, end in this order)
            w.writerow(["instruction", "start", "end"])
            rows = [(a, name, b) for name, recs in self.records.items() for a, b in recs]
            for a, name, b in sorted(rows):
                w.writerow([name, a, b])
        return p
