"""Baseline planners: frequency-only profiles for "Megatron+Perseus" and "Nanobatching+Perseus".

The reference sweeps whole-iteration clocks with ``nvidia-smi --lock-gpu-clocks``, reads the
``forward-compute`` / ``backward-compute`` timers and the energy poller CSVs and produces a
``stage,instruction,frequency,time,energy`` table (``tests/perseus/generate_profile_csv.py``,
``tests/artifact/megatron_perseus_run_profiling.sh``).  Two routes to that table exist here:

* :func:`profile_from_timer_files` — the reference's route: per frequency directory, every rank's
  ``timers/time-energy-G-L.csv`` (energy-counter poller) becomes a piecewise-linear energy curve
  that is evaluated at the start and end stamps of each ``forward-compute`` / ``backward-compute``
  row of ``timers/instructions-G-L.csv``; warm-up iterations are skipped, per-rank means are taken,
  a stage's time is the maximum over its ranks and its energy the mean per rank.
* :class:`InstructionRecorder` — a measurement window per instruction taken by the trainer's hooks
  (a synchronisation at every instruction edge), for runs without the pollers.

The same solver then runs with the frequency as the only knob.
"""
from __future__ import annotations

import csv
import bisect
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple


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


class PiecewiseLinearEnergy:
    """Cumulative energy as a function of time, linear between the poller's samples."""

    def __init__(self, times: Sequence[float], energies: Sequence[float]):
        if len(times) != len(energies) or len(times) < 2:
            raise ValueError("need at least two (time, energy) samples")
        if any(b < a for a, b in zip(times, times[1:])):
            raise ValueError("sample times must be sorted")
        if any(b < a for a, b in zip(energies, energies[1:])):
            raise ValueError("the energy counter must not decrease")
        self.t, self.e = list(map(float, times)), list(map(float, energies))

    def __call__(self, x: float) -> float:
        t, e = self.t, self.e
        if x < t[0] or x > t[-1]:
            raise ValueError(f"time {x} is outside the polled range [{t[0]}, {t[-1]}]")
        i = bisect.bisect_right(t, x)
        if i >= len(t):
            return e[-1]
        t0, t1 = t[i - 1], t[i]
        return e[i - 1] if t1 == t0 else e[i - 1] + (e[i] - e[i - 1]) * (x - t0) / (t1 - t0)

    def between(self, start: float, end: float) -> float:
        return self(end) - self(start)

    @classmethod
    def from_csv(cls, path) -> "PiecewiseLinearEnergy":
        ts, es = [], []
        with Path(path).open() as f:
            for row in csv.DictReader(f):
                ts.append(float(row["time"]))
                es.append(float(row["energy"]))
        return cls(ts, es)


def _rank_of(path: Path) -> Optional[int]:
    tok = path.stem.rsplit("-", 2)            # <prefix>-<global rank>-<local rank>
    if len(tok) != 3:
        return None
    try:
        return int(tok[1])
    except ValueError:
        return None


def _read_instructions(path: Path) -> List[Tuple[str, float, float]]:
    with path.open() as f:
        return [(r["instruction"], float(r["start"]), float(r["end"])) for r in csv.DictReader(f)]


def profile_from_timer_files(profile_dir, num_microbatches: int = 8, prof_iters: int = 20, warmup_iters: int = 10,
                             ranks_per_stage: int = 8, out: Optional[str] = None) -> Path:
    """Build ``profile.csv`` from a frequency sweep's timer and poller files.

    Layout: ``<profile_dir>/node*/<frequency MHz>/timers/{instructions,time-energy}-G-L.csv`` (the
    ``node*`` level may be absent on one machine)."""
    root = Path(profile_dir)
    nodes = sorted(p for p in root.glob("node*") if p.is_dir()) or [root]
    freqs = sorted((int(p.name) for p in nodes[0].iterdir() if p.is_dir() and p.name.isdigit()))
    if not freqs:
        raise RuntimeError(f"no frequency directories under {nodes[0]}")
    rows = []
    for freq in freqs:
        models: Dict[int, PiecewiseLinearEnergy] = {}
        insts: Dict[int, List[Tuple[str, float, float]]] = {}
        for node in nodes:
            for f in sorted((node / str(freq) / "timers").glob("time-energy-*.csv")):
                r = _rank_of(f)
                if r is not None and r not in models:
                    models[r] = PiecewiseLinearEnergy.from_csv(f)
            for f in sorted((node / str(freq) / "timers").glob("instructions-*.csv")):
                r = _rank_of(f)
                if r is not None and r not in insts:
                    insts[r] = _read_instructions(f)
        ranks = sorted(models)
        if not ranks or sorted(insts) != ranks:
            raise RuntimeError(f"frequency {freq}: energy files for ranks {ranks}, instruction files for {sorted(insts)}")
        if len(ranks) % ranks_per_stage:
            raise RuntimeError(f"{len(ranks)} ranks are not a multiple of {ranks_per_stage} ranks per stage")
        t_max: Dict[Tuple[int, str], float] = {}
        e_sum: Dict[Tuple[int, str], float] = {}
        lo, hi = warmup_iters * num_microbatches, (warmup_iters + prof_iters) * num_microbatches
        for idx, r in enumerate(ranks):
            stage = idx // ranks_per_stage
            for timer, name in (("forward-compute", "forward"), ("backward-compute", "backward")):
                recs = [(a, b) for n, a, b in insts[r] if n == timer][lo:hi]
                if not recs:
                    continue
                if len(recs) != hi - lo:
                    raise RuntimeError(f"rank {r} at {freq} MHz: {len(recs)} {timer} rows, expected {hi - lo}")
                t = sum(b - a for a, b in recs) / len(recs)
                e = sum(models[r].between(a, b) for a, b in recs) / len(recs)
                t_max[(stage, name)] = max(t_max.get((stage, name), 0.0), t)
                e_sum[(stage, name)] = e_sum.get((stage, name), 0.0) + e
        for stage in range(len(ranks) // ranks_per_stage):
            for name in ("forward", "backward"):
                rows.append((stage, name, freq, t_max.get((stage, name), 0.0),
                             e_sum.get((stage, name), 0.0) / ranks_per_stage))
    p = Path(out) if out else root / "profile.csv"
    with p.open("w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["stage", "instruction", "frequency", "time", "energy"])
        w.writerows(rows)
    return p
