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
