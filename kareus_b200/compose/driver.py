"""Plan driver: profile CSV → one ``freqs_pipeline_NNNNN.py`` / ``scheds_pipeline_NNNNN.py`` pair per
solver iteration (reference ``tests/kareus/run_optimization.py:340-491``; frequency-only variant for
the Perseus baselines: ``tests/perseus/run_optimization.py``).

Costs handed to the solver are effective energies ``E − P_p2p·t`` (per GPU column); the trailer
written under each plan gives the iteration's cost change, total effective cost and
``total + num_stages·T·P_p2p`` ("with P2P").
"""
from __future__ import annotations

import csv
from pathlib import Path
from typing import Dict, List, Optional, Sequence

from ..config import get_p2p_power
from ..plan.freqs import emit_freqs_text
from ..plan.schedule import (BWD_KEYS_CP, BWD_KEYS_TP, FWD_KEYS_CP, FWD_KEYS_TP, ScheduleItem, emit_schedule_text,
                             parse_config_string)
from .solver import ExecutionOption, plan_pipeline


def read_profile_csv(path):
    with open(path, newline="") as f:
        rows = list(csv.DictReader(f))
    if not rows:
        raise RuntimeError(f"{path} has no candidates")
    cols = rows[0].keys()
    mode = "cp" if "fwd_qkv_ar" in cols else ("tp_ac" if "recompute_attention_configs" in cols else
                                             ("tp" if "attention_configs" in cols else "freq"))
    return rows, mode


def _knob(row, mode: str, kind: str):
    f = int(float(row["frequency"]))
    if mode == "freq":
        return (f,)
    if mode == "cp":
        keys = FWD_KEYS_CP if kind == "forward" else (FWD_KEYS_CP + BWD_KEYS_CP)
        vals = [row[k] for k in keys]
        if kind == "backward" and all(v == "" for v in vals[: len(FWD_KEYS_CP)]):
            vals = vals[len(FWD_KEYS_CP):]
        return (f,) + tuple(vals)
    if mode == "tp_ac" and kind == "backward":
        return (f, row["recompute_attention_configs"], row["recompute_mlp_configs"], row["attention_configs"],
                row["mlp_configs"])
    return (f, row["attention_configs"], row["mlp_configs"])


def build_options(rows, mode: str, num_stages: int, unit_time: float, p2p_power: float):
    opts: Dict[int, Dict[str, List[ExecutionOption]]] = {s: {"forward": [], "backward": []} for s in range(num_stages)}
    for r in rows:
        s, kind = int(r["stage"]), r["instruction"]
        if s >= num_stages:
            continue
        o = ExecutionOption(float(r["time"]), unit_time, float(r["energy"]), _knob(r, mode, kind))
        o.cost -= p2p_power * o.quant_time * unit_time
        opts[s][kind].append(o)
    for s in range(num_stages):
        for k in ("forward", "backward"):
            if not opts[s][k]:
                raise RuntimeError(f"profile has no {k} candidate for stage {s}")
    return opts


def _sched_item(kind: str, knob: tuple, mode: str) -> ScheduleItem:
    cp = mode == "cp"
    fk = FWD_KEYS_CP if cp else FWD_KEYS_TP
    bk = BWD_KEYS_CP if cp else BWD_KEYS_TP
    allk = fk + bk
    cfgs = list(knob[1:])
    if kind == "forward":
        keys = fk
    elif len(cfgs) == len(allk):
        keys = allk
    else:
        keys = bk
    d = {k: None for k in allk}
    for k, c in zip(keys, cfgs):
        d[k] = parse_config_string(c)
    return ScheduleItem(kind, tuple(d.items()), cp)


def _pair_items(stage_instructions, num_mbs: int, mode: str) -> List[ScheduleItem]:
    """One item per microbatch holding the forward keys of its forward instruction and the backward keys of its
    backward instruction."""
    cp = mode == "cp"
    fk = FWD_KEYS_CP if cp else FWD_KEYS_TP
    bk = BWD_KEYS_CP if cp else BWD_KEYS_TP
    by_mb: Dict[int, Dict[str, object]] = {mb: {k: None for k in fk + bk} for mb in range(num_mbs)}
    for inst in stage_instructions:
        d = _sched_item(inst.kind, inst.assigned_knob, mode).as_dict()
        for k in (fk if inst.kind == "forward" else bk):
            by_mb[inst.micro_batch][k] = d[k]
    return [ScheduleItem("both", tuple(by_mb[mb].items()), cp) for mb in range(num_mbs)]


def run_optimization(inst_profile, output_dir, num_stages: int, num_mbs: int, gpu_type: str = "B200",
                     unit_time: float = 1e-3, noise_factor: float = 0.9, use_activation_checkpointing: bool = True,
                     p2p_power: Optional[float] = None, max_iterations: Optional[int] = None,
                     use_native: Optional[bool] = None, write_every: int = 1) -> List[dict]:
    """Returns the per-iteration summary; plan files are written under ``output_dir``."""
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    rows, mode = read_profile_csv(inst_profile)
    p2p = get_p2p_power(gpu_type) if p2p_power is None else p2p_power
    opts = build_options(rows, mode, num_stages, unit_time, p2p)
    summary = []
    log = (out / "job.log").open("a")
    for res, stages in plan_pipeline(num_stages, num_mbs, opts, unit_time, noise_factor, use_native, max_iterations):
        real_cost = res.cost + num_stages * res.real_time * p2p
        summary.append({"iteration": res.iteration, "time_s": res.real_time, "cost": res.cost,
                        "cost_change": res.cost_change, "cost_with_p2p": real_cost})
        log.write(f"iteration {res.iteration} time {res.real_time:.6f} cost {res.cost:.6f} with_p2p {real_cost:.6f}\n")
        if res.iteration % write_every:
            continue
        freqs = [[(i.kind, int(i.assigned_knob[0])) for i in st] for st in stages]
        trailer = dict(iteration=res.iteration, cost_change=res.cost_change, total_cost=res.cost,
                       total_cost_p2p=real_cost)
        (out / f"freqs_pipeline_{res.iteration:05d}.py").write_text(emit_freqs_text(freqs, **trailer))
        if mode != "freq":
            if use_activation_checkpointing:
                items = [[_sched_item(i.kind, i.assigned_knob, mode) for i in st] for st in stages]
            else:
                # without recompute a plan lists, per stage, one (forward, backward) pair per microbatch
                # (writer in the reference: tests/kareus/run_optimization.py:205-252, 297-333)
                items = [_pair_items(st, num_mbs, mode) for st in stages]
            (out / f"scheds_pipeline_{res.iteration:05d}.py").write_text(
                emit_schedule_text(items, use_activation_checkpointing, **trailer))
    log.close()
    return summary
