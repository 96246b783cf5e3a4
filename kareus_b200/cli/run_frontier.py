"""Train once under every sampled plan of a frontier: ``<out>/<model>/<layout>/<method>/frontier/pipeline_NNNNN/``.

    torchrun --nproc-per-node 8 -m kareus_b200.cli.run_frontier --method perseus --plans-dir perseus_plans \\
        --model llama3.2_3b --tp 8 --mbs 8 --gbs 64 --seq 4096 --steps 30 --out nemo_experiments

The ``FRONTIER=true`` mode of the reference's per-method scripts (``tests/artifact/run_perseus.sh``,
``run_nanobatch_perseus.sh``, ``run_kareus.sh:214-282``): the plan directory is sampled with the frontier rule
(``create_frontier``) unless ``<plans-dir>/frontier`` already holds plans, then the method is run under each one.
``cli.compare --root <out> --frontier`` reads the result.  For ``kareus`` the overlap plans
(``scheds_pipeline_*.py``) travel with the frequency plans.
"""
from __future__ import annotations

import argparse
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--method", required=True, choices=["perseus", "nanobatch_perseus", "kareus"])
    ap.add_argument("--plans-dir", required=True)
    ap.add_argument("--model", default="llama3.2_3b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--cp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--mbs", type=int, default=8)
    ap.add_argument("--gbs", type=int, default=64)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--tp-comm", default="sp_fused")
    ap.add_argument("--comm-backend", default="kernel")
    ap.add_argument("--clock-mode", default="advisory", choices=["off", "advisory", "locked"])
    ap.add_argument("--out", default="nemo_experiments")
    ap.add_argument("--no-recompute", action="store_true")
    a = ap.parse_args(argv)

    import torch.distributed as dist
    from ..parallel.mesh import init_distributed
    from ..plan.frontier import create_frontier
    from . import run_train

    rank, world, _ = init_distributed()
    plans = Path(a.plans_dir)
    with_scheds = a.method == "kareus"
    if rank == 0 and not list((plans / "frontier").glob("freqs_pipeline_*.py")):
        create_frontier(plans, plans / "frontier", with_scheds=with_scheds)
    if world > 1:
        dist.barrier()
    names = sorted(p.name for p in (plans / "frontier").glob("freqs_pipeline_*.py"))
    if not names:
        raise SystemExit(f"no freqs_pipeline_*.py under {plans}")
    tag = f"cp{a.cp}_tp{a.tp}_mbs{a.mbs}_seq{a.seq}"
    base = Path(a.out) / a.model / tag / a.method / "frontier"
    for name in names:
        src = plans / "frontier" / name
        argv2 = ["--method", a.method, "--model", a.model, "--tp", str(a.tp), "--cp", str(a.cp), "--pp", str(a.pp),
                 "--mbs", str(a.mbs), "--gbs", str(a.gbs), "--seq", str(a.seq), "--steps", str(a.steps),
                 "--freqs", str(src), "--clock-mode", a.clock_mode, "--tp-comm", a.tp_comm, "--comm-backend",
                 a.comm_backend, "--out", a.out, "--run-dir", str(base / name[len("freqs_"):-3]),
                 "--keep-process-group"]
        if with_scheds:
            argv2 += ["--scheds", str(src.parent / name.replace("freqs", "scheds"))]
        if a.no_recompute:
            argv2.append("--no-recompute")
        if rank == 0:
            print(f"== {a.method} under {name}", flush=True)
        run_train.main(argv2)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
