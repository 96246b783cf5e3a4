"""End-to-end driver: compose → plan → pick plan(s) → train under the plan → collect results.

The reference's ``tests/artifact/run_kareus.sh`` flow (its lines 302-339 compose and plan, 338-339
pick the last plan as the max-throughput one, 214-282 the frontier mode, 373-447 start the plan
server and launch training) as one command that runs inside the ranks started by torchrun:

    torchrun --nproc-per-node 8 -m kareus_b200.cli.run_kareus --model llama3.2_3b --tp 8 --pp 1 \
        --mbs 8 --seq 4096 --gbs 64 --bayesian-dir . --workdir nemo_experiments [--frontier] [--skip-planning]

Environment variables of the reference drivers are honoured as defaults: ``FRONTIER``,
``SKIP_PROFILING`` (profiling is a separate step here: ``run_bayesian``), ``GPU_TYPE``, ``PFO_PORT``.
Rank 0 composes and plans (CPU work), every rank then trains with the chosen
``freqs_pipeline_*.py`` / ``scheds_pipeline_*.py`` pair; in frontier mode the training run is repeated
for each of the 10 sampled plans under ``<method>/frontier/pipeline_NNNNN/``.
"""
from __future__ import annotations

import argparse
import os
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3.2_3b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--cp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--mbs", type=int, default=8)
    ap.add_argument("--gbs", type=int, default=64)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--bayesian-dir", default=".")
    ap.add_argument("--workdir", default="nemo_experiments")
    ap.add_argument("--gpu_type", default=os.environ.get("GPU_TYPE", "B200"))
    ap.add_argument("--frontier", action="store_true", default=os.environ.get("FRONTIER", "false").lower() == "true")
    ap.add_argument("--skip-planning", action="store_true")
    ap.add_argument("--no-recompute", action="store_true", help="plan and train without activation recompute")
    ap.add_argument("--nano", type=int, default=2,
                    help="nanobatches per microbatch: composes the measurements taken with this split and trains with it")
    ap.add_argument("--max-iterations", type=int, default=None)
    ap.add_argument("--clock-mode", default="advisory", choices=["off", "advisory", "locked"])
    ap.add_argument("--tp-comm", default="allreduce")
    ap.add_argument("--comm-backend", default="kernel")
    a = ap.parse_args(argv)

    import torch.distributed as dist
    from ..compose.composer import generate_profile_csv
    from ..compose.driver import run_optimization
    from ..parallel.mesh import init_distributed
    from ..plan.frontier import create_frontier, select_max_throughput
    from . import run_train

    rank, world, _ = init_distributed()
    tag = f"cp{a.cp}_tp{a.tp}_mbs{a.mbs}_seq{a.seq}"
    base = Path(a.workdir) / a.model / tag / "kareus"
    plans = base / "lowtime"
    num_mbs = a.gbs // (a.mbs * max(1, world // (a.tp * a.cp * a.pp)))
    if rank == 0 and not a.skip_planning:
        csv_path = generate_profile_csv(a.model, a.tp, a.cp, a.pp, a.mbs, a.seq, a.bayesian_dir, None, str(base),
                                        a.gpu_type, not a.no_recompute, True, a.nano)
        summary = run_optimization(csv_path, plans, a.pp, num_mbs, a.gpu_type, max_iterations=a.max_iterations,
                                   use_activation_checkpointing=not a.no_recompute)
        print(f"planned {len(summary)} frontier points: T {summary[0]['time_s']:.3f}s → {summary[-1]['time_s']:.3f}s")
    if rank == 0 and a.frontier:
        have = list((plans / "frontier").glob("*_pipeline_*.py"))
        if not a.skip_planning:
            for p in have:                                # samples of an earlier planning run
                p.unlink()
            have = []
        if not have:
            create_frontier(plans, plans / "frontier")   # also after --skip-planning, from the plans already there
    if world > 1:
        dist.barrier()
    chosen = []
    if a.frontier:
        chosen = sorted(p.name for p in (plans / "frontier").glob("freqs_pipeline_*.py"))
    else:
        chosen = [select_max_throughput([p.name for p in plans.glob("freqs_pipeline_*.py")])]
    for name in chosen:
        src = (plans / "frontier" / name) if a.frontier else (plans / name)
        # one run directory per sampled plan: <method>/frontier/pipeline_NNNNN/zeus_monitor_*.txt
        run_dir = str(base / "frontier" / name[len("freqs_"):-3]) if a.frontier else None
        argv2 = ["--method", "kareus", "--model", a.model, "--tp", str(a.tp), "--cp", str(a.cp), "--pp", str(a.pp),
                 "--mbs", str(a.mbs), "--gbs", str(a.gbs), "--seq", str(a.seq), "--steps", str(a.steps),
                 "--freqs", str(src), "--scheds", str(src.parent / name.replace("freqs", "scheds")),
                 "--clock-mode", a.clock_mode, "--tp-comm", a.tp_comm, "--comm-backend", a.comm_backend,
                 "--out", str(Path(a.workdir)), "--keep-process-group", "--nano", str(a.nano)] + (["--run-dir", run_dir] if run_dir else []) + (["--no-recompute"] if a.no_recompute else [])
        run_train.main(argv2)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
