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
