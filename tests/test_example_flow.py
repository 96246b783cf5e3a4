"""The example script that chains every phase driver (profile → compose/plan → train per method → compare)
runs to the end on two CPU ranks with the tiny model."""
import json
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _free_port() -> str:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return str(s.getsockname()[1])

# the two-rank tensor-parallel flow always runs; the other layouts take another minute each
long_tests = pytest.mark.skipif(os.environ.get("KAREUS_LONG_TESTS", "0") != "1",
                                reason="set KAREUS_LONG_TESTS=1 for the pipeline-only and TP x CP flows")


def test_artifact_flow_on_two_cpu_ranks(tmp_path):
    env = dict(os.environ, NPROC="2", TP="2", MODEL="tiny", SEQ="32", MBS="4", GBS="8", STEPS="4", QUICK="1",
               WORK=str(tmp_path / "w"), MASTER_PORT=_free_port(), CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(["bash", str(ROOT / "examples" / "artifact_flow.sh")], cwd=ROOT, env=env, capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + "\n" + r.stderr[-3000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{") and '"run"' in l]
    assert [Path(l["run"]).name for l in lines] == ["megatron", "nanobatch", "perseus", "nanobatch_perseus", "kareus"]
    assert all(l["iterations"] == 3 and l["ranks"] == 2 for l in lines)
    assert "energy_reduction_pct" in lines[1]
    runs = tmp_path / "w" / "runs" / "tiny" / "cp1_tp2_mbs4_seq32"
    assert list((runs / "kareus" / "lowtime").glob("freqs_pipeline_*.py"))
    assert (tmp_path / "w" / "perseus_profile.csv").exists() and (tmp_path / "w" / "nanobatch_perseus_profile.csv").exists()
    assert (tmp_path / "w" / "bayesian" / "logs" / "tiny" / "cp1-tp2-bs4-seq32" / "fwd_attn_ag" / "eval_results.jsonl").exists()


@long_tests
def test_artifact_flow_with_pipeline_stages_only(tmp_path):
    """Two pipeline stages, no tensor parallelism: nothing to profile per partition, the frequency-only plan is
    the whole story."""
    env = dict(os.environ, NPROC="2", TP="1", PP="2", MODEL="tiny", SEQ="32", MBS="2", GBS="8", STEPS="4", QUICK="1",
               WORK=str(tmp_path / "w"), MASTER_PORT=_free_port(), CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(["bash", str(ROOT / "examples" / "artifact_flow.sh")], cwd=ROOT, env=env, capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + "\n" + r.stderr[-3000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{") and '"run"' in l]
    assert [Path(l["run"]).name for l in lines] == ["megatron", "nanobatch", "perseus", "nanobatch_perseus"]
    assert list((tmp_path / "w" / "perseus_plans").glob("freqs_pipeline_*.py"))


@long_tests
def test_artifact_flow_with_tensor_and_context_parallelism(tmp_path):
    """TP2 x CP2 on four ranks: the twelve context-parallel partitions are profiled, composed into the
    context-parallel profile CSV, planned, and the run executes the 5 + 12 entry plan."""
    env = dict(os.environ, NPROC="4", TP="2", CP="2", MODEL="tiny", SEQ="64", MBS="2", GBS="4", STEPS="4", QUICK="1",
               WORK=str(tmp_path / "w"), MASTER_PORT=_free_port(), CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(["bash", str(ROOT / "examples" / "artifact_flow.sh")], cwd=ROOT, env=env, capture_output=True,
                       text=True, timeout=1200)
    assert r.returncode == 0, r.stdout[-3000:] + "\n" + r.stderr[-3000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{") and '"run"' in l]
    assert [Path(l["run"]).name for l in lines] == ["megatron", "nanobatch", "perseus", "nanobatch_perseus", "kareus"]
    logs = tmp_path / "w" / "bayesian" / "logs" / "tiny" / "cp2-tp2-bs2-seq64"
    for key in ("fwd_qkv_ar", "fwd_qkv_ag", "fwd_ao_ag", "fwd_ao_ar", "fwd_mlp", "bwd_qkv_ar", "bwd_qkv_rs", "bwd_a_rs",
                "bwd_a_ag", "bwd_o_ag", "bwd_o_ar", "bwd_mlp"):
        assert (logs / key / "eval_results.jsonl").exists(), key
