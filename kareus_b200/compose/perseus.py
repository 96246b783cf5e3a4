"""Baseline planners: frequency-only profiles for "Megatron+Perseus" and "Nanobatching+Perseus".

The reference sweeps whole-iteration clocks with ``nvidia-smi --lock-gpu-clocks``, reads the
``forward-compute`` / ``backward-compute`` timers and the energy poller CSVs and produces a
``stage,instruction,frequency,time,energy`` table (``tests/perseus/generate_profile_csv.py``,
``tests/artifact/megatron_perseus_run_profiling.sh``).  Here the table is built from per-instruction
measurements ``(stage, kind, frequency) -> [(time, energy), ...]`` collected by the trainer's
instruction hooks; the same solver then runs with the frequency as the only knob.
"""
from __future__ import annotations

import csv
from pathlib import Path
from typing import Dict, List, Sequence, Tuple


class InstructionRecorder:
    """Trainer hook that measures every pipeline instruction with an :class:`EnergyMonitor`."""

    def __init__(self, monitor, stage: int, frequency: int):
        self.monitor, self.stage, self.frequency = monitor, stage, frequency
        self.samples: Dict[Tuple[int, str, int], List[Tuple[float, float]]] = {}
        self._n = 0

    def on_step_begin(self):
        pass

    def on_instruction_begin(self, name):
        self.monitor.begin_window(f"__inst_{self._n}")

    def on_instruction_end(self, name):
        m = self.monitor.end_window(f"__inst_{self._n}", cancel=True)
        self._n += 1
        self.samples.setdefault((self.stage, name, self.frequency), []).append((m.time, m.total_energy))

    def on_step_end(self):
        pass


def write_frequency_profile(path, samples: Dict[Tuple[int, str, int], Sequence[Tuple[float, float]]],
                            skip: int = 0) -> Path:
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    with p.open("w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["stage", "instruction", "frequency", "time", "energy"])
        for (stage, kind, freq), vals in sorted(samples.items()):
            vals = list(vals)[skip:] or list(vals)
            t = sum(v[0] for v in vals) / len(vals)
            e = sum(v[1] for v in vals) / len(vals)
            w.writerow([stage, kind, freq, t, e])
    return p
