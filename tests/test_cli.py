"""Drivers end to end on CPU: training run with plans → monitor files → comparison."""
import json

import pytest

from kareus_b200.cli import compare as cli_compare, run_train
from kareus_b200.plan import emit_freqs_text, emit_schedule_text, uniform_freqs, uniform_schedule


def test_run_train_cpu_with_plans(tmp_path, capsys):
    order = ["forward", "backward"] * 2
    (tmp_path / "freqs_pipeline_00001.py").write_text(emit_freqs_text(uniform_freqs(1, order, 1500), 1, 0.0, 1.0, 2.0))
    (tmp_path / "scheds_pipeline_00001.py").write_text(
        emit_schedule_text(uniform_schedule(1, order), True, 1, 0.0, 1.0, 2.0))
    rc = run_train.main(["--method", "kareus", "--model", "tiny", "--mbs", "2", "--gbs", "4", "--seq", "32",
                         "--steps", "2", "--freqs", str(tmp_path / "freqs_pipeline_00001.py"),
                         "--scheds", str(tmp_path / "scheds_pipeline_00001.py"), "--out", str(tmp_path / "exp"),
                         "--enable-timers"])
    assert rc == 0
    out = capsys.readouterr().out
    assert "step 1 loss" in out
    assert (tmp_path / "exp" / "tiny" / "cp1_tp1_mbs2_seq32" / "kareus" / "timers" / "instructions-0-0.csv").exists()


def test_compare_cli(tmp_path, capsys):
    for name, t in (("megatron", 5.0), ("kareus", 4.0)):
        d = tmp_path / name
        d.mkdir()
        rows = ["start_time,window_name,elapsed_time,gpu0_energy"] + \
               [f"{i},training_step_fwd_bwd_step_call,{t},{t * 200}" for i in range(30)]
        (d / "zeus_monitor_global_rank-0_local_rank-0.txt").write_text("\n".join(rows) + "\n")
    assert cli_compare.main(["--base", str(tmp_path / "megatron"), "--runs", str(tmp_path / "kareus")]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert lines[1]["time_reduction_pct"] == pytest.approx(20.0)


def test_perseus_profile_and_frequency_only_plan(tmp_path, capsys):
    from kareus_b200.cli import run_perseus_profile
    from kareus_b200.compose import run_optimization
    out = tmp_path / "perseus.csv"
    rc = run_perseus_profile.main(["--model", "tiny", "--mbs", "2", "--gbs", "4", "--seq", "32", "--steps", "2",
                                   "--skip", "0", "--freqs", "1500", "1200", "900", "--out", str(out)])
    assert rc == 0
    rows = out.read_text().strip().splitlines()
    assert rows[0] == "stage,instruction,frequency,time,energy" and len(rows) == 1 + 2 * 3
    summary = run_optimization(out, tmp_path / "plans", num_stages=1, num_mbs=2, gpu_type="B200", unit_time=1e-4,
                               use_native=False, max_iterations=5)
    assert (tmp_path / "plans" / "freqs_pipeline_00000.py").exists() or summary == []
    assert not list((tmp_path / "plans").glob("scheds_pipeline_*.py"))


def test_perseus_profile_through_timer_and_poller_files(tmp_path):
    """Same table through the reference's route: instruction timers + energy poller files per frequency."""
    from kareus_b200.cli import run_perseus_profile
    out = tmp_path / "perseus.csv"
    rc = run_perseus_profile.main(["--model", "tiny", "--mbs", "2", "--gbs", "4", "--seq", "32", "--steps", "3",
                                   "--skip", "1", "--freqs", "1500", "900", "--route", "timers",
                                   "--timer-dir", str(tmp_path / "sweep"), "--out", str(out)])
    assert rc == 0
    assert (tmp_path / "sweep" / "900" / "timers" / "instructions-0-0.csv").read_text().startswith("instruction,start,end")
    assert (tmp_path / "sweep" / "900" / "timers" / "time-energy-0-0.csv").read_text().startswith("time,energy")
    rows = out.read_text().strip().splitlines()
    assert rows[0] == "stage,instruction,frequency,time,energy" and len(rows) == 1 + 2 * 2
    for r in rows[1:]:
        st, inst, f, t, e = r.split(",")
        assert float(t) > 0 and float(e) >= 0


def test_run_kareus_end_to_end_cpu(tmp_path, capsys):
    """Synthetic partition profiles → compose → plan → train under the max-throughput plan."""
    import json
    import random
    from kareus_b200.cli import run_kareus
    rng = random.Random(0)
    freqs = [1500, 1200, 900]
    base = tmp_path / "bo" / "logs" / "tiny" / "cp1-tp1-bs2-seq32"
    for part, (t, e) in {"fwd_attn": (2e-3, 1.0), "fwd_mlp": (3e-3, 1.5), "bwd_attn": (4e-3, 2.0), "bwd_mlp": (6e-3, 3.0)}.items():
        (base / part).mkdir(parents=True)
        with (base / part / "eval_results.jsonl").open("w") as f:
            for fr in freqs:
                for sm in (6, 12):
                    tt = t * 1500 / fr * (1 + 0.05 * (sm == 6) + 0.01 * rng.random())
                    f.write(json.dumps({"freq": fr, "overlap_start": "norm_0", "overlap_end": "none", "sm": sm,
                                        "block": 1024, "time_s": tt, "energy_j": e * (fr / 1500) ** 2 + 190 * tt}) + "\n")
    for fr in freqs:
        d = base / "nonpartition" / str(fr)
        d.mkdir(parents=True)
        for fname in ("preprocess_energy.csv", "postprocess_energy.csv", "loss_energy.csv",
                      "preprocess_backward_energy.csv", "postprocess_backward_energy.csv"):
            (d / fname).write_text(f"time (s),total_energy (J),per_rank_energy (J)\n{1e-3 * 1500 / fr},0.5,0.5\n")
    rc = run_kareus.main(["--model", "tiny", "--mbs", "2", "--gbs", "4", "--seq", "32", "--steps", "2",
                          "--bayesian-dir", str(tmp_path / "bo"), "--workdir", str(tmp_path / "exp"),
                          "--max-iterations", "12", "--comm-backend", "nccl"])
    assert rc == 0
    out = capsys.readouterr().out
    assert "planned 12 frontier points" in out and "step 1 loss" in out
    plans = tmp_path / "exp" / "tiny" / "cp1_tp1_mbs2_seq32" / "kareus" / "lowtime"
    assert (plans / "freqs_pipeline_00011.py").exists() and (plans / "scheds_pipeline_00011.py").exists()
    # frontier mode: one run per sampled plan, each in <method>/frontier/pipeline_NNNNN/
    rc = run_kareus.main(["--model", "tiny", "--mbs", "2", "--gbs", "4", "--seq", "32", "--steps", "2",
                          "--bayesian-dir", str(tmp_path / "bo"), "--workdir", str(tmp_path / "exp"),
                          "--skip-planning", "--frontier", "--comm-backend", "nccl"])
    assert rc == 0
    runs = sorted((tmp_path / "exp" / "tiny" / "cp1_tp1_mbs2_seq32" / "kareus" / "frontier").iterdir())
    assert runs and all(r.name.startswith("pipeline_") for r in runs)
    assert all((r / "zeus_monitor_global_rank-0_local_rank-0.txt").exists() for r in runs)


def test_pretrain_from_yaml(tmp_path, capsys):
    from kareus_b200.cli import pretrain
    (tmp_path / "c.yaml").write_text("""
name: tiny_yaml
trainer: {devices: 1, num_nodes: 1, precision: 32, max_steps: 2}
model:
  micro_batch_size: 2
  global_batch_size: 4
  tensor_model_parallel_size: 1
  pipeline_model_parallel_size: 1
  encoder_seq_length: 32
  num_layers: 2
  hidden_size: 64
  ffn_hidden_size: 128
  num_attention_heads: 4
  num_query_groups: 2
  vocab_size: 256
  activations_checkpoint_granularity: full
  enable_megatron_timers: true
""")
    rc = pretrain.main(["--config", str(tmp_path / "c.yaml"), "--out", str(tmp_path / "exp"), "model.hidden_dropout=0.0"])
    assert rc == 0 and "step 1 loss" in capsys.readouterr().out
    assert (tmp_path / "exp" / "tiny_yaml" / "cp1_tp1_mbs2_seq32" / "nanobatch" / "timers" / "instructions-0-0.csv").exists()


def test_bench_reference_arm_says_why_it_is_unavailable():
    """`bench.py --impl reference` prints one JSON line with the reason and exits 0 (the reference's training
    stack cannot be installed offline); it must not start the package's own engine."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    r = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                        "--warmup", "3"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]
    assert "value" not in line


def test_profiler_clock_grid_from_driver_environment(monkeypatch):
    """FREQ_START / FREQ_END / FREQ_STEP of the reference's driver scripts give the profiler's clock grid."""
    from kareus_b200.cli.run_bayesian import env_freq_grid
    for k in ("FREQ_START", "FREQ_END", "FREQ_STEP"):
        monkeypatch.delenv(k, raising=False)
    assert env_freq_grid() is None
    monkeypatch.setenv("FREQ_START", "900")
    monkeypatch.setenv("FREQ_END", "1410")
    monkeypatch.setenv("FREQ_STEP", "30")
    grid = env_freq_grid()
    assert grid[0] == 1410 and grid[-1] == 900 and len(grid) == 18


def test_small_frontiers_keep_the_max_throughput_plan():
    from kareus_b200.plan.frontier import sample_frontier
    names = [f"freqs_pipeline_{i:05d}.py" for i in range(2496)]
    picked = sample_frontier(names)
    assert len(picked) == 10 and picked[-1] == names[-1]            # the reference's counts: unchanged
    for n in (1, 2, 3, 5, 7, 9):
        got = sample_frontier(names[:n])
        assert got and got[-1] == names[n - 1], (n, got)


def _noac_worker(rank, world, out):
    """Two nanobatches, no activation recompute: train under a plan in the per-microbatch pair layout."""
    import torch.distributed as dist
    from kareus_b200.cli import run_train
    from kareus_b200.plan.schedule import DEFAULT_CONFIG, ScheduleItem, emit_schedule_text, FWD_KEYS_TP, BWD_KEYS_TP
    plan = out + "/scheds_pipeline_00001.py"
    if rank == 0:
        item = ScheduleItem("both", tuple((k, DEFAULT_CONFIG) for k in FWD_KEYS_TP + BWD_KEYS_TP), False)
        with open(plan, "w") as f:
            f.write(emit_schedule_text([[item, item]], False, 1, 0.0, 1.0, 2.0))
    dist.barrier()
    rc = run_train.main(["--method", "kareus", "--model", "tiny", "--tp", "2", "--mbs", "4", "--gbs", "8", "--seq", "32",
                         "--steps", "2", "--tp-comm", "allreduce", "--scheds", plan, "--no-recompute", "--out",
                         out + "/runs", "--keep-process-group"])
    assert rc == 0


def test_training_without_recompute_under_a_pair_layout_plan(tmp_path):
    from dist_utils import run_distributed
    run_distributed(_noac_worker, 2, str(tmp_path), timeout=300.0)


def test_plan_server_process_serves_a_training_run(tmp_path, capsys):
    """The stand-alone plan server (environment of the reference's drivers) hands the clocks of a plan file to a
    training run that only knows its URL."""
    import json
    import os
    import socket
    import subprocess
    import sys
    import time
    import urllib.request
    from kareus_b200.cli import run_train
    from kareus_b200.plan.freqs import emit_freqs_text
    plan = tmp_path / "freqs_pipeline_00007.py"
    plan.write_text(emit_freqs_text([[("forward", 1500), ("backward", 1200), ("forward", 1500), ("backward", 1200)]],
                                    iteration=7, cost_change=0.0, total_cost=1.0, total_cost_p2p=2.0))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, PFO_PORT=str(port), ZEUS_PFO_SCHEDULER_ARGS=json.dumps({"solution_path": str(plan)}))
    proc = subprocess.Popen([sys.executable, "-m", "kareus_b200.cli.pfo_server", "--once-after", "60"], env=env,
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        url = f"http://127.0.0.1:{port}"
        for _ in range(100):
            try:
                with urllib.request.urlopen(url + "/health", timeout=1) as r:
                    assert json.loads(r.read())["stages"] == 1
                break
            except OSError:
                time.sleep(0.1)
        else:
            raise AssertionError("the plan server did not come up")
        rc = run_train.main(["--method", "perseus", "--model", "tiny", "--mbs", "2", "--gbs", "4", "--seq", "32", "--steps",
                             "2", "--pfo-url", url, "--out", str(tmp_path / "runs"), "--keep-process-group"])
        assert rc == 0 and "step 1 loss" in capsys.readouterr().out
    finally:
        proc.terminate()
        proc.wait(timeout=10)


def test_nanobatch_count_of_a_run(tmp_path, capsys):
    """`--nano 4`: four nanobatches along the batch, or along the sequence when the micro batch is 1; same first
    loss as the two-nanobatch run of the same batch (the split changes the schedule, not the math)."""
    from kareus_b200.cli import run_train
    losses = {}
    for tag, extra in {"n2": ["--mbs", "4", "--gbs", "8"], "n4": ["--mbs", "4", "--gbs", "8", "--nano", "4"],
                       "seq4": ["--mbs", "1", "--gbs", "2", "--nano", "4"]}.items():
        rc = run_train.main(["--method", "nanobatch", "--model", "tiny", "--seq", "32", "--steps", "1", "--out",
                             str(tmp_path / tag), "--keep-process-group"] + extra)
        assert rc == 0
        losses[tag] = float(capsys.readouterr().out.split("step 0 loss")[1].split()[0])
    assert abs(losses["n2"] - losses["n4"]) < 1e-3
    assert 6.5 < losses["seq4"] < 7.5
    import pytest
    with pytest.raises(SystemExit):
        run_train.main(["--method", "nanobatch", "--model", "tiny", "--mbs", "3", "--gbs", "3", "--seq", "33", "--nano", "2",
                        "--steps", "1", "--out", str(tmp_path / "bad"), "--keep-process-group"])
