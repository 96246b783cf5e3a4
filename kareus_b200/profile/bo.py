"""Bayesian search over one partition's configurations: orchestration and runner.

Loop (reference ``tests/bayesian/common/runner.py:158-348``, ``orchestration.py:32-611``):
measure ``n_init`` random configs; then ``batches`` times: fit surrogates on (effective energy,
time), score every unevaluated grid point, pick ``acq_batch`` points — 40 % by hypervolume gain on
(real energy, time), 20 % on (effective energy, time), 20 % fastest predicted, the rest most
uncertain — measure them and append to ``eval_results.jsonl``.  Everything measured is cached in
that JSONL file; a restarted search skips what is already there.  At the end it writes
``results_pareto_frontier_{effective,real}.csv``, ``results_all.csv`` and ``bo_timing.csv``.

``E_eff = E − P_p2p·t``: the part of a GPU's energy that is not the static power it would draw
anyway while blocked, which is what the planner trades against time.
"""
from __future__ import annotations

import csv
import json
import random
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from .space import Config, SearchSpace
from .surrogates import Surrogates, hv_improvement, pareto_mask

Evaluator = Callable[[Sequence[Config]], List[Tuple[float, float]]]   # configs -> [(time_s, energy_j)]

RESULTS_HEADER = ["frequency", "overlap_start", "overlap_end", "comm_sm_number", "comm_block_size", "time_s",
                  "avg_energy_J", "effect_energy_J"]


def effective_energy(energy_j: float, time_s: float, p2p_power: float) -> float:
    return energy_j - p2p_power * time_s


def record_of(cfg: Config, time_s: float, energy_j: float, **extra) -> dict:
    r = {"freq": cfg.freq, "overlap_start": cfg.overlap[0], "overlap_end": cfg.overlap[1], "sm": cfg.sm,
         "block": cfg.block, "time_s": time_s, "energy_j": energy_j}
    if cfg.nano != 2:
        r["nano"] = cfg.nano
    r.update(extra)
    return r


def config_of(rec: dict) -> Config:
    return Config(int(rec["freq"]), int(rec["sm"]), (rec["overlap_start"], rec["overlap_end"]), int(rec["block"]),
                  int(rec.get("nano", 2)))


def load_eval_log(path) -> List[dict]:
    p = Path(path)
    if not p.exists():
        return []
    out, seen = [], set()
    for line in p.read_text().splitlines():
        try:
            r = json.loads(line)
            k = config_of(r).key()
        except (ValueError, KeyError, TypeError):
            continue
        if k not in seen:
            seen.add(k)
            out.append(r)
    return out


def append_eval_log(path, records: Iterable[dict]) -> None:
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    with p.open("a") as f:
        for r in records:
            f.write(json.dumps(r) + "\n")


@dataclass
class BOResult:
    records: List[dict]
    pareto_effective: List[dict]
    pareto_real: List[dict]
    timing: List[dict]


def _pick(scores: np.ndarray, k: int, taken: set) -> List[int]:
    out = []
    for i in np.argsort(-scores):
        if len(out) >= k:
            break
        if int(i) not in taken:
            out.append(int(i))
            taken.add(int(i))
    return out


def select_batch(space: SearchSpace, sur: Surrogates, Xc: np.ndarray, measured_Y_eff: np.ndarray,
                 measured_Y_real: np.ndarray, k: int) -> Tuple[List[int], List[str]]:
    """Indices into the candidate matrix ``Xc`` and the reason each was picked."""
    e_eff, e_real, t = sur.predict(Xc)
    ref_eff = measured_Y_eff.max(0) * 1.1 + 1e-9
    ref_real = measured_Y_real.max(0) * 1.1 + 1e-9
    s_real = hv_improvement(measured_Y_real[pareto_mask(measured_Y_real)], np.stack([t, e_real], 1), ref_real)
    s_dyn = hv_improvement(measured_Y_eff[pareto_mask(measured_Y_eff)], np.stack([t, e_eff], 1), ref_eff)
    n_real = int(round(k * space.real_fraction))
    n_dyn = int(round(k * space.dynamic_fraction))
    n_time = int(round(k * space.time_fraction))
    n_unc = max(0, k - n_real - n_dyn - n_time)
    taken: set = set()
    idx, why = [], []
    for scores, n, tag in ((s_real, n_real, "real_ehvi"), (s_dyn, n_dyn, "dynamic_ehvi"), (-t, n_time, "time"),
                           (sur.uncertainty(Xc), n_unc, "uncertainty")):
        got = _pick(np.asarray(scores, dtype=float), n, taken)
        idx += got
        why += [tag] * len(got)
    return idx, why


def run_bo_search(space: SearchSpace, freqs: Sequence[int], evaluate: Evaluator, logs_dir, p2p_power: float,
                  seed: int = 0, n_init: Optional[int] = None, batches: Optional[int] = None,
                  acq_batch: Optional[int] = None, log: Callable[[str], None] = lambda s: None) -> BOResult:
    logs = Path(logs_dir)
    logs.mkdir(parents=True, exist_ok=True)
    eval_path = logs / "eval_results.jsonl"
    n_init = space.n_init if n_init is None else n_init
    batches = space.batches if batches is None else batches
    acq_batch = space.acq_batch if acq_batch is None else acq_batch
    grid = space.grid(freqs)
    by_key = {c.key(): c for c in grid}
    rng = random.Random(seed)
    records = [r for r in load_eval_log(eval_path) if config_of(r).key() in by_key]
    done = {config_of(r).key() for r in records}
    timing: List[dict] = []

    def measure(cfgs: List[Config], tag: str, reasons: Optional[List[str]] = None) -> float:
        if not cfgs:
            return 0.0
        t0 = time.time()
        res = evaluate(cfgs)
        new = [record_of(c, t, e, selection=(reasons[i] if reasons else tag)) for i, (c, (t, e)) in
               enumerate(zip(cfgs, res))]
        append_eval_log(eval_path, new)
        records.extend(new)
        done.update(c.key() for c in cfgs)
        return time.time() - t0

    # initial design (resume: only what is missing)
    todo = [c for c in grid if c.key() not in done]
    need = max(0, min(n_init, len(grid)) - len(records))
    if need:
        log(f"initial design: measuring {need} of {len(grid)} configurations ({len(records)} cached)")
        timing.append({"batch": "init", "train_s": 0.0, "select_s": 0.0, "eval_s": measure(rng.sample(todo, min(need, len(todo))), "init")})
    # batches already covered by the cache are skipped
    covered = max(0, (len(records) - n_init) // max(acq_batch, 1)) if len(records) > n_init else 0
    for b in range(covered, batches):
        cand = [c for c in grid if c.key() not in done]
        if not cand:
            break
        t0 = time.time()
        X = space.encode([config_of(r) for r in records], freqs)
        tt = np.array([r["time_s"] for r in records])
        ee = np.array([r["energy_j"] for r in records])
        eff = ee - p2p_power * tt
        sur = Surrogates(p2p_power, seed=seed + b).fit(X, eff, tt)
        t1 = time.time()
        idx, why = select_batch(space, sur, space.encode(cand, freqs), np.stack([tt, eff], 1), np.stack([tt, ee], 1),
                                min(acq_batch, len(cand)))
        t2 = time.time()
        ev = measure([cand[i] for i in idx], f"batch{b}", why)
        timing.append({"batch": b, "train_s": t1 - t0, "select_s": t2 - t1, "eval_s": ev})
        log(f"batch {b}: measured {len(idx)} configurations, {len(records)} total")
    res = summarize(records, p2p_power)
    write_outputs(logs, records, res, timing, p2p_power)
    return BOResult(records, res[0], res[1], timing)


def summarize(records: Sequence[dict], p2p_power: float):
    tt = np.array([r["time_s"] for r in records])
    ee = np.array([r["energy_j"] for r in records])
    eff = ee - p2p_power * tt
    pe = [records[i] for i in np.nonzero(pareto_mask(np.stack([tt, eff], 1)))[0]]
    pr = [records[i] for i in np.nonzero(pareto_mask(np.stack([tt, ee], 1)))[0]]
    key = lambda r: r["time_s"]
    return sorted(pe, key=key), sorted(pr, key=key)


def _row(r: dict, p2p_power: float) -> list:
    return [r["freq"], r["overlap_start"], r["overlap_end"], r["sm"], r["block"], r["time_s"], r["energy_j"],
            effective_energy(r["energy_j"], r["time_s"], p2p_power)]


def write_outputs(logs: Path, records, res, timing, p2p_power: float) -> None:
    for name, rows in (("results_all.csv", records), ("results_pareto_frontier_effective.csv", res[0]),
                       ("results_pareto_frontier_real.csv", res[1])):
        with (logs / name).open("w", newline="") as f:
            w = csv.writer(f)
            w.writerow(RESULTS_HEADER)
            for r in rows:
                w.writerow(_row(r, p2p_power))
    with (logs / "bo_timing.csv").open("w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["batch", "train_s", "select_s", "eval_s"])
        for t in timing:
            w.writerow([t["batch"], t["train_s"], t["select_s"], t["eval_s"]])
