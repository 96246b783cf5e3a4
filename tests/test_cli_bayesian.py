"""run_bayesian driver end to end on two gloo ranks with a simulated NVML."""
import os

from dist_utils import run_distributed


def _worker(rank, world, out):
    from kareus_b200.cli import run_bayesian
    import torch.distributed as dist
    # the driver initialises (and tears down) the process group itself when launched by torchrun;
    # here the group already exists, so keep it alive for the harness barrier
    real_destroy = dist.destroy_process_group
    dist.destroy_process_group = lambda *a, **k: None
    try:
        rc = run_bayesian.main(["--partition", "fwd_attn", "-m", "tiny", "-w", "2", "-tp", "2", "-b", "4", "-s", "32",
                                "--out", out, "--freqs", "1500", "1200", "--n-init", "4", "--batches", "1",
                                "--acq-batch", "2", "--measure-s", "0.05", "--cooldown-s", "0.0",
                                "--comm-backend", "nccl"])
    finally:
        dist.destroy_process_group = real_destroy
    assert rc == 0


def test_run_bayesian_two_ranks(tmp_path):
    run_distributed(_worker, 2, str(tmp_path))
    d = tmp_path / "logs" / "tiny" / "cp1-tp2-bs4-seq32" / "fwd_attn"
    rows = (d / "eval_results.jsonl").read_text().strip().splitlines()
    assert len(rows) == 6
    assert (d / "results_pareto_frontier_effective.csv").exists() and (d / "bo_timing.csv").exists()


def _worker_all(rank, world, out):
    from kareus_b200.cli import run_bayesian
    import torch.distributed as dist
    real_destroy = dist.destroy_process_group
    dist.destroy_process_group = lambda *a, **k: None
    try:
        rc = run_bayesian.main(["--partition", "all", "--tp-comm", "sp", "-m", "tiny", "-w", "2", "-tp", "2", "-b", "4",
                                "-s", "32", "--out", out, "--freqs", "1500", "--n-init", "3", "--batches", "1",
                                "--acq-batch", "1", "--measure-s", "0.02", "--cooldown-s", "0.0",
                                "--comm-backend", "nccl"])
    finally:
        dist.destroy_process_group = real_destroy
    assert rc == 0


def test_all_partitions_of_the_sequence_parallel_path_and_their_composition(tmp_path):
    """`--partition all` profiles the eight partitions of the sequence-parallel path in one process; the
    composer folds the all-gather partitions into the four reference keys and yields stage candidates."""
    from kareus_b200.compose.composer import FUSED_CHILD, merge_fused_partitions, read_bo_jsonl
    from kareus_b200.profile.space import SP_FUSED_PARTITIONS
    run_distributed(_worker_all, 2, str(tmp_path), timeout=400.0)
    base = tmp_path / "logs" / "tiny" / "cp1-tp2-bs4-seq32"
    maps = {}
    for part in SP_FUSED_PARTITIONS:
        f = base / part / "eval_results.jsonl"
        assert f.exists(), part
        maps[part] = read_bo_jsonl(f)
        assert maps[part][1500]
    merged = merge_fused_partitions(maps)
    assert set(merged) == set(FUSED_CHILD)
    for k in FUSED_CHILD:
        assert merged[k].get(1500), f"{k}: no point shares an sm value with its all-gather partition"
