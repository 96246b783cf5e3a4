"""Bayesian partition search on a synthetic time/energy surface."""
import json

import numpy as np
import pytest

from kareus_b200.profile.bo import load_eval_log, run_bo_search
from kareus_b200.profile.space import PARTITION_SPACES, SearchSpace, TP_PARTITIONS
from kareus_b200.profile.surrogates import hv_improvement, hypervolume_2d, pareto_mask

FREQS = [1500, 1350, 1200, 1050, 900]


def surface(c):
    slot_penalty = {"norm_0": 0.0, "linear_0": 0.08, "rope_0": 0.15, "attn_0": 0.2}[c.overlap[0]]
    comm = 6.0 / c.sm                       # more CTAs → faster collective, slower compute
    t = (2.0 * 1500 / c.freq) * (1 + 0.01 * c.sm + slot_penalty) + 0.2 * comm
    e = 300.0 * (c.freq / 1500) ** 2 * 2.0 + 190.0 * t
    return t * 1e-3, e * 1e-3


def test_hypervolume_and_pareto():
    Y = np.array([[1.0, 3.0], [2.0, 2.0], [3.0, 1.0], [2.5, 2.5]])
    assert pareto_mask(Y).tolist() == [True, True, True, False]
    assert hypervolume_2d(Y, (4.0, 4.0)) == pytest.approx(3 + 2 + 1)
    gain = hv_improvement(Y[:3], np.array([[1.5, 2.2], [3.5, 3.5]]), (4.0, 4.0))
    assert gain[0] > 0 and gain[1] == 0


def test_partition_registry_matches_reference_spaces():
    assert set(TP_PARTITIONS) <= set(PARTITION_SPACES) and len(PARTITION_SPACES) == 14
    kind, sp = PARTITION_SPACES["fwd_attn"]
    assert kind == "all_reduce" and sp.sm_values == list(range(3, 31, 3)) and len(sp.grid(range(18))) == 720
    assert PARTITION_SPACES["bwd_a_rs"][1].sm_values == list(range(1, 21))


def test_bo_finds_frontier_and_resumes(tmp_path):
    space = PARTITION_SPACES["fwd_attn"][1]
    calls = []

    def evaluate(cfgs):
        calls.append(len(cfgs))
        return [surface(c) for c in cfgs]

    res = run_bo_search(space, FREQS, evaluate, tmp_path, p2p_power=190.0, seed=3, n_init=24, batches=3, acq_batch=12)
    assert len(res.records) == 24 + 3 * 12 and calls == [24, 12, 12, 12]
    # the true fastest point is (max clock, norm_0, some mid SM); BO must have measured a near-fastest one
    grid = space.grid(FREQS)
    best_t = min(surface(c)[0] for c in grid)
    assert min(r["time_s"] for r in res.records) <= best_t * 1.03
    # frontier is sorted and strictly improving in effective energy
    eff = [r["energy_j"] - 190.0 * r["time_s"] for r in res.pareto_effective]
    assert all(a > b for a, b in zip(eff, eff[1:]))
    hdr = (tmp_path / "results_all.csv").read_text().splitlines()[0]
    assert hdr == "frequency,overlap_start,overlap_end,comm_sm_number,comm_block_size,time_s,avg_energy_J,effect_energy_J"
    rec = json.loads((tmp_path / "eval_results.jsonl").read_text().splitlines()[0])
    assert {"freq", "overlap_start", "overlap_end", "sm", "block", "time_s", "energy_j"} <= set(rec)
    # resume: nothing left to measure for the same budget
    calls.clear()
    res2 = run_bo_search(space, FREQS, evaluate, tmp_path, p2p_power=190.0, seed=3, n_init=24, batches=3, acq_batch=12)
    assert calls == [] and len(res2.records) == len(res.records)
    # a larger budget only measures the missing batch
    res3 = run_bo_search(space, FREQS, evaluate, tmp_path, p2p_power=190.0, seed=3, n_init=24, batches=4, acq_batch=12)
    assert calls == [12] and len(load_eval_log(tmp_path / "eval_results.jsonl")) == 72


def test_nanobatch_axis():
    sp = SearchSpace([("norm_0", "none")], [4, 8], nano_values=[1, 2, 4])
    g = sp.grid([1500, 1200])
    assert len(g) == 12 and sp.encode(g, [1500, 1200]).shape == (12, 4)
