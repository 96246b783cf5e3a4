"""Composer arithmetic, Pareto filter, the time–cost solver and plan emission on synthetic profiles."""
import csv
import json
import math
import random

import pytest

from kareus_b200.compose import (ExecutionOption, compare_frontiers, compose, dominates, frontier_from_plans,
                                 generate_profile_csv, pareto_optimal, plan_pipeline, run_optimization, summarize_run)
from kareus_b200.compose.composer import layers_per_stage
from kareus_b200.compose.mincut import bounded_min_cut
from kareus_b200.plan import (PipelineCommScheduler, parse_freqs_file, parse_schedule_file, sample_frontier,
                              select_max_throughput)

FREQS = [1500, 1350, 1200, 1050, 900]     # five clock levels


def _points(base_t, base_e, rng):
    """Synthetic partition profile: slower clock → longer, cheaper (dynamic) but static power adds up."""
    out = {}
    for f in FREQS:
        pts = []
        for sm in (6, 12, 18):
            for slot in ("norm_0", "linear_0"):
                t = base_t * (1500 / f) * (1 + 0.05 * (sm == 6) + 0.02 * rng.random())
                e = base_e * (f / 1500) ** 2 * (1 + 0.03 * (sm == 18)) + 190.0 * t
                pts.append(((slot, "none", sm, 1024), (t, e)))
        out[f] = pts
    return out


def _prepost():
    return {f: {k: (1e-3 * 1500 / f, 0.5) for k in ("forward-embedding", "forward-output", "loss-func",
                                                   "backward-embedding", "backward-output")} for f in FREQS}


def test_pareto_and_layers():
    pts = [(("a",), (1.0, 300.0)), (("b",), (1.1, 295.0)), (("c",), (1.2, 400.0)), (("d",), (0.9, 500.0))]
    keep = pareto_optimal(pts, p2p_power=100.0)
    assert [c[0][0] for c in keep] == ["d", "a", "b"]
    assert layers_per_stage(28, 2, 15, 13) == [15, 13]
    assert layers_per_stage(28, 1) == [28]
    assert sum(layers_per_stage(32, 4)) == 32


def test_compose_arithmetic():
    rng = random.Random(0)
    maps = {"fwd_attn": _points(2e-3, 1.0, rng), "fwd_mlp": _points(3e-3, 1.5, rng),
            "bwd_attn": _points(4e-3, 2.0, rng), "bwd_mlp": _points(6e-3, 3.0, rng)}
    cands = compose(maps, _prepost(), [15, 13], p2p_power=190.0)
    assert set(cands) == {0, 1}
    # one hand-computed candidate at 1500 MHz: fastest attn + fastest mlp config
    fa = min(maps["fwd_attn"][1500], key=lambda p: p[1][0])
    fm = min(maps["fwd_mlp"][1500], key=lambda p: p[1][0])
    want_t = (fa[1][0] + fm[1][0]) * 1.15 * 15 * 2 + 1e-3
    fastest = min(cands[0]["forward"], key=lambda p: p[1][0])
    assert fastest[0][0] == 1500
    assert fastest[1][0] == pytest.approx(want_t, rel=1e-9)
    # Pareto: sorted by time, effective energy strictly decreasing
    for kind in ("forward", "backward"):
        eff = [e - 190.0 * t for _, (t, e) in cands[1][kind]]
        assert all(a > b for a, b in zip(eff, eff[1:]))
    assert len(cands[0]["backward"][0][0]) == 5      # (freq, rec_attn, rec_mlp, attn, mlp)


def test_bounded_min_cut_native_matches_python():
    edges = [(0, 1, 1.0, 4.0), (0, 2, 0.0, 2.0), (1, 3, 0.5, 3.0), (2, 3, 0.0, 5.0), (1, 2, 0.0, 1e18)]
    py = bounded_min_cut(4, edges, 0, 3, use_native=False)
    assert py is not None and py[0] == 1 and py[3] == 0
    try:
        nat = bounded_min_cut(4, edges, 0, 3, use_native=True)
    except RuntimeError:
        pytest.skip("library not built")
    def cut(side):
        return sum(ub for u, v, lb, ub in edges if side[u] and not side[v]) - \
            sum(lb for u, v, lb, ub in edges if side[v] and not side[u])
    assert cut(nat) == pytest.approx(cut(py))
    # infeasible lower bounds
    assert bounded_min_cut(3, [(0, 1, 5.0, 6.0), (1, 2, 0.0, 1.0)], 0, 2, use_native=False) is None


def _options(unit):
    opts = {}
    for s in range(2):
        opts[s] = {}
        for kind, base in (("forward", 0.020), ("backward", 0.045)):
            lst = []
            for f in FREQS:
                t = base * (1500 / f) * (1.0 + 0.1 * s)
                e = 40.0 * base * (f / 1500) ** 2
                lst.append(ExecutionOption(t, unit, e, (f,)))
            opts[s][kind] = lst
    return opts


def test_solver_walks_a_monotone_frontier():
    unit = 1e-3
    results = []
    for res, stages in plan_pipeline(2, 4, _options(unit), unit, use_native=False):
        results.append((res.quant_time, res.cost, res.cost_change,
                        [[(i.kind, i.assigned_knob[0], i.duration) for i in st] for st in stages]))
    assert len(results) > 20
    times = [r[0] for r in results]
    costs = [r[1] for r in results]
    assert all(a - b == 1 for a, b in zip(times, times[1:])), "each iteration removes exactly one time unit"
    assert all(b >= a - 1e-9 for a, b in zip(costs, costs[1:])), "energy grows as time shrinks"
    assert all(c >= -1e-9 for c in (r[2] for r in results))
    # ends at the all-fastest critical path: stage-0 warm-up F + 4x(F,B) chain at max clock
    last = results[-1][3]
    assert last[1][0][1] == 1500 and all(k in ("forward", "backward") for k, _, _ in last[0])
    # marginal cost is non-decreasing (convex frontier)
    ch = [r[2] for r in results]
    assert ch[-1] >= ch[0] - 1e-9


def test_driver_writes_compatible_plan_files(tmp_path):
    rng = random.Random(1)
    base = tmp_path / "bo" / "logs" / "llama3.2_3b" / "cp1-tp8-bs8-seq4096"
    for part, (t, e) in {"fwd_attn": (2e-3, 1.0), "fwd_mlp": (3e-3, 1.5), "bwd_attn": (4e-3, 2.0),
                         "bwd_mlp": (6e-3, 3.0)}.items():
        d = base / part
        d.mkdir(parents=True)
        with (d / "eval_results.jsonl").open("w") as f:
            for freq, pts in _points(t, e, rng).items():
                for (s0, s1, sm, blk), (tt, ee) in pts:
                    f.write(json.dumps({"freq": freq, "overlap_start": s0, "overlap_end": s1, "sm": sm, "block": blk,
                                        "time_s": tt, "energy_j": ee}) + "\n")
            f.write("not json\n")
    for freq, d in _prepost().items():
        nd = base / "nonpartition" / str(freq)
        nd.mkdir(parents=True)
        for key, fname in {"forward-embedding": "preprocess_energy.csv", "forward-output": "postprocess_energy.csv",
                           "loss-func": "loss_energy.csv", "backward-embedding": "preprocess_backward_energy.csv",
                           "backward-output": "postprocess_backward_energy.csv"}.items():
            (nd / fname).write_text(f"time (s),total_energy (J),per_rank_energy (J)\n{d[key][0]},{d[key][1] * 8},{d[key][1]}\n")
    csv_path = generate_profile_csv("llama3.2_3b", 8, 1, 2, 8, 4096, bayesian_profile_dir=str(tmp_path / "bo"),
                                    output_dir=str(tmp_path), gpu_type="B200")
    assert csv_path.read_text().splitlines()[0] == ("stage,instruction,frequency,recompute_attention_configs,"
                                                    "recompute_mlp_configs,attention_configs,mlp_configs,time,energy")
    out = tmp_path / "lowtime"
    summary = run_optimization(csv_path, out, num_stages=2, num_mbs=8, gpu_type="B200", use_native=False,
                               max_iterations=60)
    assert len(summary) == 60
    names = sorted(p.name for p in out.glob("freqs_pipeline_*.py"))
    assert names[0] == "freqs_pipeline_00000.py" and len(names) == 60
    best = select_max_throughput(names)
    freqs = parse_freqs_file(out / best)
    assert len(freqs) == 2 and len(freqs[0]) == 16 and freqs[0][0][0] == "forward"
    sched = parse_schedule_file(out / best.replace("freqs", "scheds"), True, False)
    s = PipelineCommScheduler.from_parsed(sched, 1, 8, use_activation_checkpointing=True)
    s.on_instruction_begin("forward")
    assert s.current_schedule.get("fwd_attn").block_size == 1024
    trailer = (out / best).read_text().splitlines()[-1]
    assert trailer.startswith(f"# Iteration {int(best[-8:-3])} total cost with P2P:")
    kept = sample_frontier(names)
    assert len(kept) == 10 and kept[-1] == names[-1]
    fr = frontier_from_plans(out, 2, 190.0)
    assert len(fr) == 60 and fr[0][0] > fr[-1][0]
    # the same logs planned for a run WITHOUT activation recompute: the profile drops the recompute columns and
    # the plan lists one (forward, backward) pair per microbatch and stage
    csv2 = generate_profile_csv("llama3.2_3b", 8, 1, 2, 8, 4096, bayesian_profile_dir=str(tmp_path / "bo"),
                                output_dir=str(tmp_path / "noac"), gpu_type="B200", use_activation_checkpointing=False)
    assert csv2.read_text().splitlines()[0] == "stage,instruction,frequency,attention_configs,mlp_configs,time,energy"
    out2 = tmp_path / "lowtime_noac"
    run_optimization(csv2, out2, num_stages=2, num_mbs=8, gpu_type="B200", use_native=False, max_iterations=5,
                     use_activation_checkpointing=False)
    text = (out2 / "scheds_pipeline_00004.py").read_text()
    pairs = parse_schedule_file(out2 / "scheds_pipeline_00004.py", False, False)
    assert len(pairs) == 2 and len(pairs[0]) == 8 and pairs[0][0].kind == "both" and "(('forward'," in text
    s2 = PipelineCommScheduler.from_parsed(pairs, 0, 8, use_activation_checkpointing=False)
    s2.on_instruction_begin("forward")
    assert s2.current_schedule.get("fwd_mlp").block_size == 1024
    s2.on_instruction_end("forward")
    s2.on_instruction_begin("backward")
    assert s2.current_schedule.get("bwd_attn") is not None


def test_compare_methods(tmp_path):
    def write_run(d, t, e):
        d.mkdir(parents=True)
        for r in range(2):
            rows = ["start_time,window_name,elapsed_time,gpu0_energy"]
            for i in range(30):
                rows.append(f"{i},training_step,{t + 1},{e + 5}")
                rows.append(f"{i},training_step_fwd_bwd_step_call,{t + 0.01 * r},{e}")
            (d / f"zeus_monitor_global_rank-{r}_local_rank-{r}.txt").write_text("\n".join(rows) + "\n")
    write_run(tmp_path / "megatron", 5.0, 1000.0)
    write_run(tmp_path / "kareus", 4.0, 900.0)
    a, b = summarize_run(tmp_path / "megatron"), summarize_run(tmp_path / "kareus")
    assert a["time_s"] == pytest.approx(5.01) and a["energy_j"] == pytest.approx(2000.0) and a["iterations"] == 20
    assert b["time_s"] < a["time_s"]
    ours = [(4.0, 2700.0), (5.0, 2300.0), (6.0, 2250.0)]
    base = [(4.5, 2800.0), (5.5, 2400.0)]
    assert dominates(ours, base)
    cmp = compare_frontiers(ours, base)
    assert cmp["iso_time_energy_reduction_pct"] > 0


def test_frequency_profile_from_timer_and_poller_files(tmp_path):
    """The reference's baseline route: a piecewise-linear curve through the energy poller's samples,
    evaluated at the instruction timers' start/end stamps; stage time = max over its ranks, stage
    energy = mean per rank; warm-up iterations skipped."""
    from kareus_b200.compose.perseus import PiecewiseLinearEnergy, profile_from_timer_files
    m = PiecewiseLinearEnergy([0.0, 1.0, 3.0], [0.0, 100.0, 500.0])
    assert m(0.5) == 50.0 and m(2.0) == 300.0 and abs(m.between(0.5, 2.0) - 250.0) < 1e-12
    with pytest.raises(ValueError):
        m(3.5)
    with pytest.raises(ValueError):
        PiecewiseLinearEnergy([0.0, 1.0], [5.0, 4.0])
    mb, warm, prof = 2, 1, 2
    for node, ranks in (("node0", (0, 1)), ("node1", (2, 3))):           # 2 stages x 2 ranks
        for freq, watts in ((1200, 400.0), (1500, 600.0)):
            d = tmp_path / node / str(freq) / "timers"
            d.mkdir(parents=True)
            for r in ranks:
                p_r = watts + 10.0 * r                                     # constant power per rank
                (d / f"time-energy-{r}-{r % 2}.csv").write_text(
                    "time,energy\n" + "\n".join(f"{t / 10.0},{p_r * t / 10.0}" for t in range(0, 400)))
                rows, t = ["instruction,start,end"], 1.0
                for it in range(warm + prof):
                    for _ in range(mb):
                        f_len = (0.9 if it < warm else 0.2 + 0.01 * r) * 1500.0 / freq
                        rows.append(f"forward-compute,{t},{t + f_len}")
                        t += f_len + 0.05
                        rows.append(f"backward-compute,{t},{t + 2 * f_len}")
                        t += 2 * f_len + 0.05
                (d / f"instructions-{r}-{r % 2}.csv").write_text("\n".join(rows))
    out = profile_from_timer_files(tmp_path, num_microbatches=mb, prof_iters=prof, warmup_iters=warm, ranks_per_stage=2)
    got = {(int(r["stage"]), r["instruction"], int(r["frequency"])): (float(r["time"]), float(r["energy"]))
           for r in csv.DictReader(out.open())}
    assert len(got) == 2 * 2 * 2
    t, e = got[(0, "forward", 1500)]
    assert abs(t - 0.21) < 1e-9                                           # slower rank of stage 0 (rank 1)
    assert abs(e - (600.0 * 0.20 + 610.0 * 0.21) / 2) < 1e-6             # mean per rank of P x dt
    t, e = got[(1, "backward", 1200)]
    assert abs(t - 2 * 0.23 * 1500 / 1200) < 1e-9
    assert abs(e - (420.0 * 2 * 0.22 + 430.0 * 2 * 0.23) * 1500 / 1200 / 2) < 1e-6


def test_fused_path_partitions_fold_into_the_reference_keys():
    """The all-gather→GEMM partition in front of a key is not named by a plan: it inherits the key's sm,
    so its measured point with that sm is added to the key's point; other sm values drop out."""
    from kareus_b200.compose.composer import merge_fused_partitions
    maps = {
        "fwd_attn": {1500: [(("rope_0", "none", 8, 1024), (1.0, 10.0)), (("attn_0", "none", 16, 1024), (0.9, 11.0)),
                            (("attn_0", "none", 32, 1024), (0.8, 12.0))]},
        "fwd_attn_ag": {1500: [(("norm_0", "none", 8, 1024), (0.5, 5.0)), (("norm_0", "none", 16, 1024), (0.4, 6.0)),
                               (("first", "none", 16, 1024), (0.45, 5.5))]},
        "fwd_mlp": {1500: [(("activation_0", "none", 8, 1024), (2.0, 20.0))]},
    }
    out = merge_fused_partitions(maps)
    assert set(out) == {"fwd_attn", "fwd_mlp"}
    got = dict(out["fwd_attn"][1500])
    assert got[("rope_0", "none", 8, 1024)] == (1.5, 15.0)
    assert got[("attn_0", "none", 16, 1024)] == (0.9 + 0.4, 11.0 + 6.0)          # child's faster point at sm 16
    assert ("attn_0", "none", 32, 1024) not in got                                # child never measured at 32
    assert out["fwd_mlp"] == maps["fwd_mlp"]                                      # no child logs: unchanged


def _fake_run(d, times, energies, ranks=2):
    d.mkdir(parents=True, exist_ok=True)
    for r in range(ranks):
        with (d / f"zeus_monitor_global_rank-{r}_local_rank-{r}.txt").open("w") as f:
            f.write("start_time,window_name,elapsed_time,gpu0_energy\n")
            for t, e in zip(times, energies):
                f.write(f"0.0,training_step_fwd_bwd_step_call,{t},{e / ranks}\n")


def test_results_tree_tables_and_measured_frontiers(tmp_path):
    """The comparison over a whole results tree: per configuration every method against the one-nanobatch run,
    and the measured frontier runs of each method against the frequency-only method's frontier."""
    from kareus_b200.compose.compare import format_table, iso_reductions, load_frontier_runs, results_table
    cfg = tmp_path / "llama3.2_3b" / "cp1_tp8_mbs8_seq4096"
    _fake_run(cfg / "megatron", [1.0] * 4, [1000.0] * 4)
    _fake_run(cfg / "perseus", [1.0] * 4, [900.0] * 4)
    _fake_run(cfg / "kareus", [0.8] * 4, [700.0] * 4)
    (tmp_path / "llama3.2_3b" / "notes").mkdir()                      # not a layout directory: ignored
    rows = results_table(tmp_path, skip=1, take=3)
    assert rows[0][:2] == ["model", "layout"] and len(rows) == 2
    line = dict(zip(rows[0], rows[1]))
    assert line["kareus time"] == "+20.0%" and line["kareus energy"] == "+30.0%" and line["perseus energy"] == "+10.0%"
    assert line["nanobatch_perseus time"] == "n/a"
    assert format_table(rows).splitlines()[1].startswith("|---|")
    # measured frontiers: perseus spans (1.0 s, 900 J) .. (1.3 s, 700 J)
    for i, (t, e) in enumerate([(1.0, 900.0), (1.15, 780.0), (1.3, 700.0)]):
        _fake_run(cfg / "perseus" / "frontier" / f"pipeline_{i:05d}", [t] * 4, [e] * 4)
    for i, (t, e) in enumerate([(0.8, 800.0), (0.95, 650.0), (1.2, 600.0)]):
        _fake_run(cfg / "kareus" / "frontier" / f"pipeline_{i:05d}", [t] * 4, [e] * 4)
    ref = load_frontier_runs(cfg / "perseus", 1, 3)
    ours = load_frontier_runs(cfg / "kareus", 1, 3, expected=3)
    r = iso_reductions(ours, ref)
    # as fast as perseus' fastest run (1.0 s): kareus' cheapest such run uses 650 J instead of 900 J
    assert abs(r["iso_time_energy_reduction_pct"] - 100 * (900 - 650) / 900) < 1e-9
    # no more energy than perseus' most frugal run (700 J): kareus' fastest such run takes 0.95 s instead of 1.3 s
    assert abs(r["iso_energy_time_reduction_pct"] - 100 * (1.3 - 0.95) / 1.3) < 1e-9
    rows = results_table(tmp_path, 1, 3, frontier=True)
    line = dict(zip(rows[0], rows[1]))
    assert line["kareus iso-time energy"] == "+27.8%" and line["nanobatch_perseus iso-energy time"] == "n/a"
    import pytest
    with pytest.raises(ValueError):
        load_frontier_runs(cfg / "kareus", 1, 3, expected=10)


def test_frontier_runner_trains_under_every_sampled_plan(tmp_path):
    from kareus_b200.cli import compare, run_frontier
    from kareus_b200.plan.freqs import emit_freqs_text
    plans = tmp_path / "plans"
    plans.mkdir()
    for i, f in enumerate([900, 1200, 1500]):
        (plans / f"freqs_pipeline_{i:05d}.py").write_text(
            emit_freqs_text([[("forward", f), ("backward", f), ("forward", f), ("backward", f)]], iteration=i,
                            cost_change=0.0, total_cost=1.0, total_cost_p2p=2.0))
    rc = run_frontier.main(["--method", "perseus", "--plans-dir", str(plans), "--model", "tiny", "--mbs", "2", "--gbs",
                            "4", "--seq", "32", "--steps", "3", "--out", str(tmp_path / "exp"), "--comm-backend", "nccl"])
    assert rc == 0
    runs = sorted((tmp_path / "exp" / "tiny" / "cp1_tp1_mbs2_seq32" / "perseus" / "frontier").iterdir())
    assert [r.name for r in runs] == ["pipeline_00001", "pipeline_00002"]          # positions 0 dropped, last kept
    assert compare.main(["--root", str(tmp_path / "exp"), "--frontier", "--skip", "1", "--take", "2"]) == 0


def test_composer_reads_one_nanobatch_count_at_a_time(tmp_path):
    """A search over the nanobatch split writes all counts into one log; composition takes one of them."""
    from kareus_b200.compose.composer import read_bo_jsonl
    f = tmp_path / "eval_results.jsonl"
    rows = [{"freq": 1500, "overlap_start": "norm_0", "overlap_end": "none", "sm": 6, "block": 1024, "time_s": 1e-3,
             "energy_j": 1.0},
            {"freq": 1500, "overlap_start": "norm_0", "overlap_end": "none", "sm": 6, "block": 1024, "time_s": 2e-3,
             "energy_j": 2.0, "nano": 1},
            {"freq": 1500, "overlap_start": "norm_0", "overlap_end": "none", "sm": 9, "block": 1024, "time_s": 5e-4,
             "energy_j": 0.5, "nano": 4}]
    f.write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    assert len(read_bo_jsonl(f)[1500]) == 3
    assert [p[1][0] for p in read_bo_jsonl(f, 2)[1500]] == [1e-3]
    assert [p[0][2] for p in read_bo_jsonl(f, 4)[1500]] == [9]
    assert read_bo_jsonl(f, 8) == {}
