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


# ----------------------------------------------------------------------------- measured frontiers, result tables
# What the reference's comparison script prints over a whole results tree
# (``tests/artifact/compare_method.py:119-155`` frontier points, ``:164-182`` configuration discovery,
# ``:191-302`` rows): per configuration the time / energy reduction of every method against the
# one-nanobatch baseline, and in frontier mode two numbers per method against the measured frontier of the
# frequency-only method.

BASELINE_METHOD = "megatron"
TABLE_METHODS = ("perseus", "nanobatch_perseus", "kareus")
FRONTIER_REFERENCE = "perseus"
FRONTIER_METHODS = ("nanobatch_perseus", "kareus")


def load_frontier_runs(method_dir, skip: int = 10, take: int = 20,
                       expected: Optional[int] = None) -> List[Tuple[str, float, float]]:
    """``[(plan tag, time_s, energy_j), ...]`` of the runs under ``<method_dir>/frontier/pipeline_*``."""
    fdir = Path(method_dir) / "frontier"
    runs = sorted(d for d in fdir.glob("pipeline_*") if d.is_dir()) if fdir.is_dir() else []
    if not runs:
        raise FileNotFoundError(f"no frontier/pipeline_* runs under {method_dir}")
    if expected is not None and len(runs) != expected:
        raise ValueError(f"{fdir}: expected {expected} pipeline_* directories, found {len(runs)}")
    out = []
    for d in runs:
        s = summarize_run(d, skip, take)
        out.append((d.name, s["time_s"], s["energy_j"]))
    return out


def iso_reductions(method: Sequence[Tuple[str, float, float]], reference: Sequence[Tuple[str, float, float]],
                   eps: float = 1e-12) -> Dict[str, Optional[float]]:
    """Against a measured reference frontier: energy saved by the method's best run that is at least as fast
    as the reference's fastest run, and time saved by its best run that uses no more energy than the
    reference's most frugal run (``None`` where no run qualifies)."""
    ref_fast = min(reference, key=lambda p: (p[1], p[2], p[0]))
    ref_frugal = min(reference, key=lambda p: (p[2], p[1], p[0]))
    fast_enough = [p for p in method if p[1] <= ref_fast[1] + eps]
    frugal_enough = [p for p in method if p[2] <= ref_frugal[2] + eps]
    iso_t = min(fast_enough, key=lambda p: (p[2], p[1], p[0])) if fast_enough else None
    iso_e = min(frugal_enough, key=lambda p: (p[1], p[2], p[0])) if frugal_enough else None
    return {"iso_time_energy_reduction_pct": None if iso_t is None else 100.0 * (ref_fast[2] - iso_t[2]) / ref_fast[2],
            "iso_energy_time_reduction_pct": None if iso_e is None else 100.0 * (ref_frugal[1] - iso_e[1]) / ref_frugal[1]}


def discover_configs(root) -> List[Tuple[str, str]]:
    """``[(model, layout tag), ...]`` for every ``<root>/<model>/cp*_tp*_mbs*_seq*`` directory."""
    out = []
    for model_dir in sorted(p for p in Path(root).iterdir() if p.is_dir()):
        for cfg in sorted(p for p in model_dir.iterdir() if p.is_dir()):
            if re.fullmatch(r"cp\d+_tp\d+_mbs\d+_seq\d+", cfg.name):
                out.append((model_dir.name, cfg.name))
    return out


def _pct(v: Optional[float]) -> str:
    return "n/a" if v is None else f"{v:+.1f}%"


def results_table(root, skip: int = 10, take: int = 20, frontier: bool = False,
                  expected_frontier: Optional[int] = None) -> List[List[str]]:
    """Header row + one row per configuration found under ``root``.  Normal mode: time and energy reduction
    of each method against the baseline run; frontier mode: iso-time energy and iso-energy time reduction of
    each method's measured frontier against the frequency-only method's."""
    if frontier:
        header = ["model", "layout"] + [f"{m} iso-time energy" for m in FRONTIER_METHODS] + \
                 [f"{m} iso-energy time" for m in FRONTIER_METHODS]
    else:
        header = ["model", "layout"] + [f"{m} time" for m in TABLE_METHODS] + [f"{m} energy" for m in TABLE_METHODS]
    rows = [header]
    for model, tag in discover_configs(root):
        cfg = Path(root) / model / tag
        try:
            if frontier:
                ref = load_frontier_runs(cfg / FRONTIER_REFERENCE, skip, take, expected_frontier)
            else:
                base = summarize_run(cfg / BASELINE_METHOD, skip, take)
        except (FileNotFoundError, ValueError, RuntimeError):
            continue                                   # nothing to compare against in this configuration
        a, b = [], []
        for m in (FRONTIER_METHODS if frontier else TABLE_METHODS):
            try:
                if frontier:
                    r = iso_reductions(load_frontier_runs(cfg / m, skip, take, expected_frontier), ref)
                    a.append(_pct(r["iso_time_energy_reduction_pct"]))
                    b.append(_pct(r["iso_energy_time_reduction_pct"]))
                else:
                    r = reduction(base, summarize_run(cfg / m, skip, take))
                    a.append(_pct(r["time_reduction_pct"]))
                    b.append(_pct(r["energy_reduction_pct"]))
            except (FileNotFoundError, ValueError, RuntimeError):
                a.append("n/a")
                b.append("n/a")
        rows.append([model, tag] + a + b)
    return rows


def format_table(rows: Sequence[Sequence[str]]) -> str:
    """Markdown table."""
    if not rows:
        return ""
    lines = ["| " + " | ".join(rows[0]) + " |", "|" + "---|" * len(rows[0])]
    lines += ["| " + " | ".join(r) + " |" for r in rows[1:]]
    return "\n".join(lines)
