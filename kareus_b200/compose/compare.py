"""Result comparison across methods (reference ``tests/artifact/compare_method.py:72-116,227-302``).

A run directory holds one ``zeus_monitor_global_rank-G_local_rank-L.txt`` per rank.  For the window
``training_step_fwd_bwd_step_call``: skip the first 10 iterations, take the next 20; iteration time
is the max over ranks, iteration energy the sum over ranks; report the means.  Frontier mode
compares two time–energy frontiers at equal time (energy reduction) and at equal energy (time
reduction) by linear interpolation.
"""
from __future__ import annotations

import csv
import re
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

WINDOW = "training_step_fwd_bwd_step_call"


def read_monitor_file(path, window: str = WINDOW) -> List[Tuple[float, float]]:
    """``[(elapsed_time, energy summed over the file's gpu columns), ...]`` for one rank."""
    out = []
    with open(path, newline="") as f:
        for row in csv.DictReader(f):
            if row.get("window_name") != window:
                continue
            e = sum(float(v) for k, v in row.items() if re.fullmatch(r"gpu\d+_energy", k or ""))
            out.append((float(row["elapsed_time"]), e))
    return out


def summarize_run(run_dir, skip: int = 10, take: int = 20, window: str = WINDOW) -> Dict[str, float]:
    files = sorted(Path(run_dir).glob("zeus_monitor_global_rank-*_local_rank-*.txt"))
    if not files:
        raise FileNotFoundError(f"no zeus_monitor_*.txt under {run_dir}")
    per_rank = [read_monitor_file(f, window) for f in files]
    n = min(len(r) for r in per_rank)
    lo, hi = min(skip, max(n - 1, 0)), min(n, skip + take)
    if hi <= lo:
        raise RuntimeError(f"{run_dir}: only {n} iterations recorded, cannot skip {skip}")
    times = [max(r[i][0] for r in per_rank) for i in range(lo, hi)]
    energies = [sum(r[i][1] for r in per_rank) for i in range(lo, hi)]
    return {"time_s": sum(times) / len(times), "energy_j": sum(energies) / len(energies),
            "iterations": hi - lo, "ranks": len(files)}


def reduction(base: Dict[str, float], other: Dict[str, float]) -> Dict[str, float]:
    return {"time_reduction_pct": 100.0 * (1 - other["time_s"] / base["time_s"]),
            "energy_reduction_pct": 100.0 * (1 - other["energy_j"] / base["energy_j"])}


def _interp(points: Sequence[Tuple[float, float]], x: float) -> Optional[float]:
    pts = sorted(points)
    if not pts or x < pts[0][0] or x > pts[-1][0]:
        return None
    for (x0, y0), (x1, y1) in zip(pts, pts[1:]):
        if x0 <= x <= x1:
            return y0 if x1 == x0 else y0 + (y1 - y0) * (x - x0) / (x1 - x0)
    return pts[-1][1]


def compare_frontiers(ours: Sequence[Tuple[float, float]], base: Sequence[Tuple[float, float]]) -> Dict[str, float]:
    """Points are ``(time, energy)``.  Mean energy reduction at the baseline's times that our
    frontier covers, and mean time reduction at the baseline's energies."""
    iso_t = [(1 - _interp(ours, t) / e) * 100 for t, e in base if _interp(ours, t) is not None]
    flip_o = [(e, t) for t, e in ours]
    iso_e = [(1 - _interp(flip_o, e) / t) * 100 for t, e in base if _interp(flip_o, e) is not None]
    return {"iso_time_energy_reduction_pct": sum(iso_t) / len(iso_t) if iso_t else float("nan"),
            "iso_energy_time_reduction_pct": sum(iso_e) / len(iso_e) if iso_e else float("nan"),
            "min_time_ours": min(t for t, _ in ours), "min_time_base": min(t for t, _ in base),
            "min_energy_ours": min(e for _, e in ours), "min_energy_base": min(e for _, e in base)}


def dominates(ours: Sequence[Tuple[float, float]], base: Sequence[Tuple[float, float]], tol: float = 1e-9) -> bool:
    """True if at every baseline time covered by our frontier we use no more energy."""
    ok = True
    for t, e in base:
        v = _interp(ours, t)
        if v is not None and v > e + tol:
            ok = False
    return ok


def frontier_from_plans(plan_dir, num_stages: int, p2p_power: float, pattern: str = "freqs_pipeline_*.py"):
    """``[(T seconds, real energy J)]`` from plan trailers: ``T = (with_p2p − cost) / (stages·P_p2p)``."""
    from ..plan.schedule import read_trailer
    out = []
    for p in sorted(Path(plan_dir).glob(pattern)):
        tr = read_trailer(p.read_text())
        if "total_cost" in tr and "total_cost_p2p" in tr:
            out.append(((tr["total_cost_p2p"] - tr["total_cost"]) / (num_stages * p2p_power), tr["total_cost_p2p"]))
    return out
