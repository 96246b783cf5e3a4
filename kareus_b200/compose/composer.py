"""Frontier composer: per-partition profile points → per-stage forward/backward candidates.

Arithmetic of the reference (``tests/kareus/generate_profile_csv.py:180-252,259-445,452-705``):
for every clock that all partitions were profiled at, take the cartesian product of the
partitions' configs **at that clock**, sum time and energy, apply the ×1.15 fudge, multiply by
``layers_per_stage × nanobatches`` (each key is executed once per nanobatch per layer), add the
embedding on the first stage and the head + loss on the last, and keep the Pareto front in
(time, effective energy) with ``E_eff = E − P_p2p·t``.  With activation recompute the backward
candidate is the product of the recompute-forward configs and the backward configs.

Inputs/outputs keep the reference's formats: ``logs/<model>/cp<C>-tp<T>-bs<B>-seq<S>/<partition>/
eval_results.jsonl`` and ``nonpartition/<freq>/*_energy.csv`` in, ``profile_<model>_cp.._tp.._bs.._seq..csv``
out (headers as in ``generate_profile_csv.py:314-317,516-521``).
"""
from __future__ import annotations

import csv
import itertools
import json
import os
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

from ..config import get_model_config, get_p2p_power
from ..plan.schedule import BWD_KEYS_CP, BWD_KEYS_TP, FWD_KEYS_CP, FWD_KEYS_TP

Point = Tuple[tuple, Tuple[float, float]]   # (config, (time, energy))
SCALE = 1.15

CSV_COLUMNS_TP = {"fwd_attn": "attention_configs", "fwd_mlp": "mlp_configs",
                  "bwd_attn": "attention_configs", "bwd_mlp": "mlp_configs"}
REC_COLUMNS_TP = {"fwd_attn": "recompute_attention_configs", "fwd_mlp": "recompute_mlp_configs"}


def run_dir(base, model: str, cp: int, tp: int, bs: int, seq: int) -> Path:
    return Path(base) / "logs" / model / f"cp{cp}-tp{tp}-bs{bs}-seq{seq}"


def read_bo_jsonl(path, nano: Optional[int] = None) -> Dict[int, List[Point]]:
    """``{frequency: [((overlap_start, overlap_end, sm, block), (time_s, energy_j)), ...]}``.  ``nano``: keep the
    measurements taken with that many nanobatches (a search over the split count writes them into one file; a
    row without the field was measured with two)."""
    out: Dict[int, List[Point]] = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            try:
                row = json.loads(line)
                if nano is not None and int(row.get("nano", 2)) != nano:
                    continue
                key = (row["overlap_start"], row["overlap_end"], int(row["sm"]), int(row["block"]))
                out.setdefault(int(row["freq"]), []).append((key, (float(row["time_s"]), float(row["energy_j"]))))
            except (ValueError, KeyError, TypeError):
                continue          # malformed lines are skipped, like the reference does
    return out


def read_time_energy_csv(path) -> Tuple[float, float]:
    """First row of a non-partition CSV ``time (s),total_energy (J),per_rank_energy (J)``."""
    with open(path) as f:
        rows = list(csv.reader(f))
    if len(rows) < 2 or len(rows[1]) < 3:
        raise RuntimeError(f"malformed CSV {path}")
    hdr, row = rows[0], rows[1]
    idx = hdr.index("per_rank_energy (J)") if "per_rank_energy (J)" in hdr else 2
    return float(row[0]), float(row[idx])


NONPARTITION_FILES = {"forward-embedding": "preprocess_energy.csv", "forward-output": "postprocess_energy.csv",
                      "loss-func": "loss_energy.csv", "backward-embedding": "preprocess_backward_energy.csv",
                      "backward-output": "postprocess_backward_energy.csv"}


def read_prepost(base_dir, freqs: Sequence[int]) -> Dict[int, Dict[str, Tuple[float, float]]]:
    out = {}
    for f in freqs:
        d = Path(base_dir) / "nonpartition" / str(f)
        out[int(f)] = {k: read_time_energy_csv(d / v) for k, v in NONPARTITION_FILES.items()}
    return out


# Fused sequence-parallel path: every reference key has a second partition (the all-gather→GEMM segment
# in front of it) that a plan does not name; at run time it inherits the key's sm with the launch slot
# "first" (plan/schedule.py).  Its measured cost therefore belongs to the key's point with the same sm.
FUSED_CHILD = {"fwd_attn": "fwd_attn_ag", "fwd_mlp": "fwd_mlp_ag", "bwd_attn": "bwd_attn_ag", "bwd_mlp": "bwd_mlp_ag"}


def merge_fused_partitions(maps: Dict[str, Dict[int, List[Point]]]) -> Dict[str, Dict[int, List[Point]]]:
    """Fold the ``*_ag`` partitions of the fused path into their reference keys: for every clock and every
    point of the key, add the child's point measured with the same sm (its fastest one if several launch
    slots were tried); points whose sm the child was never measured at are dropped."""
    out = {k: v for k, v in maps.items() if k not in FUSED_CHILD.values()}
    for parent, child in FUSED_CHILD.items():
        if child not in maps or parent not in maps:
            continue
        merged: Dict[int, List[Point]] = {}
        for f, pts in maps[parent].items():
            by_sm: Dict[int, Tuple[float, float]] = {}
            for cfg, (t, e) in maps[child].get(f, []):
                if cfg[2] not in by_sm or t < by_sm[cfg[2]][0]:
                    by_sm[cfg[2]] = (t, e)
            rows = [(cfg, (t + by_sm[cfg[2]][0], e + by_sm[cfg[2]][1])) for cfg, (t, e) in pts if cfg[2] in by_sm]
            if rows:
                merged[f] = rows
        out[parent] = merged
    return out


def pareto_optimal(points: Sequence[Point], p2p_power: float, tol: float = 1e-4) -> List[Point]:
    best = float("inf")
    keep: List[Point] = []
    for cfg, (t, e) in sorted(points, key=lambda x: (x[1][0], x[1][1])):
        eff = e - p2p_power * t
        if eff + tol < best:
            keep.append((cfg, (t, e)))
            best = eff
    return keep


def layers_per_stage(num_layers: int, pp: int, first: Optional[int] = None, last: Optional[int] = None) -> List[int]:
    if pp <= 0:
        raise ValueError("pipeline size must be positive")
    if pp == 1:
        return [num_layers]
    if pp == 2:
        f = min(num_layers, first if first is not None else (num_layers + 1) // 2)
        return [f, num_layers - f]
    f = first if first is not None else None
    l = last if last is not None else None
    if f is None or l is None:
        base, rem = divmod(num_layers, pp)
        return [base + (1 if i < rem else 0) for i in range(pp)]
    mid = num_layers - f - l
    base, rem = divmod(max(mid, 0), pp - 2)
    return [f] + [base + (1 if i < rem else 0) for i in range(pp - 2)] + [max(0, num_layers - f - max(mid, 0))]


def cfg_string(cfg: tuple) -> str:
    return "-".join(str(x) for x in cfg)


def _combine(maps: Sequence[Dict[int, List[Point]]], freq: int, p2p_power: float, prefilter_tol: Optional[float],
             limit: int = 200000):
    lists = [m.get(freq, []) for m in maps]
    size = 1
    for l in lists:
        size *= max(len(l), 1)
    if prefilter_tol is not None and size > limit:
        lists = [pareto_optimal(l, p2p_power, prefilter_tol) for l in lists]
    for combo in itertools.product(*lists):
        t = sum(c[1][0] for c in combo)
        e = sum(c[1][1] for c in combo)
        yield tuple(c[0] for c in combo), t, e


def compose(partition_maps: Dict[str, Dict[int, List[Point]]], prepost: Dict[int, Dict[str, Tuple[float, float]]],
            layers: Sequence[int], p2p_power: float, context_parallel: bool = False,
            use_activation_checkpointing: bool = True, scale_time_energy: bool = True, nanobatches: int = 2):
    """Returns ``{stage: {"forward": [Point], "backward": [Point]}}`` of Pareto candidates whose
    config is ``(frequency, cfg_key0, cfg_key1, ...)`` in plan-file key order."""
    fk = FWD_KEYS_CP if context_parallel else FWD_KEYS_TP
    bk = BWD_KEYS_CP if context_parallel else BWD_KEYS_TP
    missing = [k for k in fk + bk if k not in partition_maps]
    if missing:
        raise KeyError(f"missing partition profiles: {missing}")
    freqs = None
    for k in fk + bk:
        s = set(partition_maps[k])
        freqs = s if freqs is None else freqs & s
    if not freqs:
        raise RuntimeError("no clock was profiled for every partition")
    scale = SCALE if scale_time_energy else 1.0
    pp = len(layers)
    tol_bwd = 0.01 if context_parallel else 1e-4
    out = {s: {"forward": [], "backward": []} for s in range(pp)}
    for f in sorted(freqs):
        pre = prepost[f]
        for cfgs, t, e in _combine([partition_maps[k] for k in fk], f, p2p_power, 1e-4):
            for s in range(pp):
                st, se = t * scale * layers[s] * nanobatches, e * scale * layers[s] * nanobatches
                if s == 0:
                    st += pre["forward-embedding"][0]
                    se += pre["forward-embedding"][1]
                if s == pp - 1:
                    st += pre["forward-output"][0] + pre["loss-func"][0]
                    se += pre["forward-output"][1] + pre["loss-func"][1]
                out[s]["forward"].append(((f,) + cfgs, (st, se)))
        keys = (fk + bk) if use_activation_checkpointing else bk
        for cfgs, t, e in _combine([partition_maps[k] for k in keys], f, p2p_power, tol_bwd):
            for s in range(pp):
                st, se = t * scale * layers[s] * nanobatches, e * scale * layers[s] * nanobatches
                if s == 0:
                    st += pre["backward-embedding"][0] * 2
                    se += pre["backward-embedding"][1] * 2
                if s == pp - 1:
                    st += pre["backward-output"][0]
                    se += pre["backward-output"][1]
                out[s]["backward"].append(((f,) + cfgs, (st, se)))
    for s in range(pp):
        out[s]["forward"] = pareto_optimal(out[s]["forward"], p2p_power)
        out[s]["backward"] = pareto_optimal(out[s]["backward"], p2p_power, tol_bwd)
    return out


def profile_csv_header(context_parallel: bool, use_activation_checkpointing: bool) -> List[str]:
    if context_parallel:
        return ["stage", "instruction", "frequency"] + list(FWD_KEYS_CP) + list(BWD_KEYS_CP) + ["time", "energy"]
    if use_activation_checkpointing:
        return ["stage", "instruction", "frequency", "recompute_attention_configs", "recompute_mlp_configs",
                "attention_configs", "mlp_configs", "time", "energy"]
    return ["stage", "instruction", "frequency", "attention_configs", "mlp_configs", "time", "energy"]


def write_profile_csv(path, candidates, context_parallel: bool, use_activation_checkpointing: bool) -> None:
    hdr = profile_csv_header(context_parallel, use_activation_checkpointing)
    fk = FWD_KEYS_CP if context_parallel else FWD_KEYS_TP
    bk = BWD_KEYS_CP if context_parallel else BWD_KEYS_TP
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(hdr)
        for s in sorted(candidates):
            for kind in ("forward", "backward"):
                for cfg, (t, e) in candidates[s][kind]:
                    freq, cfgs = cfg[0], [cfg_string(c) for c in cfg[1:]]
                    nf, nb = len(fk), len(bk)
                    if context_parallel:
                        if kind == "forward":
                            cols = cfgs + [""] * nb
                        elif use_activation_checkpointing:
                            cols = cfgs
                        else:
                            cols = [""] * nf + cfgs
                    elif use_activation_checkpointing:
                        cols = (["", ""] + cfgs) if kind == "forward" else cfgs
                    else:
                        cols = cfgs
                    w.writerow([s, kind, freq] + cols + [t, e])


def generate_profile_csv(model_name: str, tp: int, cp: int, pp: int, batch_size: int, seq_len: int,
                         bayesian_profile_dir: str = ".", prepost_profile_dir: Optional[str] = None,
                         output_dir: str = ".", gpu_type: str = "B200", use_activation_checkpointing: bool = True,
                         scale_time_energy: bool = True, nanobatches: int = 2) -> Path:
    """File-to-file driver with the reference's CLI arguments (``generate_profile_csv.py:32-57``)."""
    cfg = get_model_config(model_name)
    base = run_dir(bayesian_profile_dir, model_name, cp, tp, batch_size, seq_len)
    pre_base = run_dir(prepost_profile_dir or bayesian_profile_dir, model_name, cp, tp, batch_size, seq_len)
    context_parallel = cp > 1
    keys = (FWD_KEYS_CP + BWD_KEYS_CP) if context_parallel else (FWD_KEYS_TP + BWD_KEYS_TP)
    maps = {k: read_bo_jsonl(base / k / "eval_results.jsonl", nanobatches) for k in keys}
    if not context_parallel:
        for child in FUSED_CHILD.values():          # logs of the fused sequence-parallel path, if profiled
            if (base / child / "eval_results.jsonl").exists():
                maps[child] = read_bo_jsonl(base / child / "eval_results.jsonl", nanobatches)
        maps = merge_fused_partitions(maps)
    freqs = set.intersection(*(set(m) for m in maps.values()))
    prepost = read_prepost(pre_base, sorted(freqs))
    first = cfg.num_layers_in_first_pipeline_stage
    layers = layers_per_stage(cfg.num_layers, pp, first, cfg.num_layers - first if first else None)
    cands = compose(maps, prepost, layers, get_p2p_power(gpu_type), context_parallel, use_activation_checkpointing,
                    scale_time_energy, nanobatches)
    os.makedirs(output_dir, exist_ok=True)
    out = Path(output_dir) / f"profile_{model_name}_cp{cp}_tp{tp}_bs{batch_size}_seq{seq_len}.csv"
    write_profile_csv(out, cands, context_parallel, use_activation_checkpointing)
    return out
