"""Compare measured runs (``zeus_monitor_*.txt``) of several methods, or two plan frontiers.

    python -m kareus_b200.cli.compare --base nemo_experiments/m/tag/megatron --runs .../kareus .../perseus
    python -m kareus_b200.cli.compare --frontier-ours plans/kareus/frontier --frontier-base plans/perseus/frontier \
        --num_stages 2 --gpu_type B200
    python -m kareus_b200.cli.compare --root nemo_experiments [--frontier]      # table over every configuration

``--root``: the reference's ``compare_method.py`` over a results tree — per ``<model>/<layout>`` the time and
energy reduction of perseus / nanobatch_perseus / kareus against the megatron run, or with ``--frontier`` the
iso-time energy and iso-energy time reduction of each method's measured ``frontier/pipeline_*`` runs against the
perseus frontier.
"""
from __future__ import annotations

import argparse
import json


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base")
    ap.add_argument("--runs", nargs="*", default=[])
    ap.add_argument("--skip", type=int, default=10)
    ap.add_argument("--take", type=int, default=20)
    ap.add_argument("--root", help="results tree: <root>/<model>/<cp.._tp.._mbs.._seq..>/<method>/")
    ap.add_argument("--frontier", action="store_true", help="with --root: compare measured frontier runs")
    ap.add_argument("--frontier-count", type=int, default=0, help="expected pipeline_* runs per method; 0: any")
    ap.add_argument("--frontier-ours")
    ap.add_argument("--frontier-base")
    ap.add_argument("--num_stages", type=int, default=2)
    ap.add_argument("--gpu_type", default="B200")
    a = ap.parse_args(argv)
    from ..compose.compare import compare_frontiers, dominates, frontier_from_plans, reduction, summarize_run
    from ..config import get_p2p_power
    if a.root:
        from ..compose.compare import format_table, results_table
        rows = results_table(a.root, a.skip, a.take, a.frontier, a.frontier_count or None)
        print(format_table(rows))
        if len(rows) == 1:
            print(f"no configuration with a {'perseus frontier' if a.frontier else 'megatron run'} under {a.root}")
    if a.base:
        base = summarize_run(a.base, a.skip, a.take)
        print(json.dumps({"run": a.base, **base}))
        for r in a.runs:
            s = summarize_run(r, a.skip, a.take)
            print(json.dumps({"run": r, **s, **reduction(base, s)}))
    if a.frontier_ours and a.frontier_base:
        p = get_p2p_power(a.gpu_type)
        ours = frontier_from_plans(a.frontier_ours, a.num_stages, p)
        base = frontier_from_plans(a.frontier_base, a.num_stages, p)
        res = {k: (None if isinstance(v, float) and v != v else v) for k, v in compare_frontiers(ours, base).items()}
        print(json.dumps({**res, "dominates": dominates(ours, base)}))      # frontiers that do not overlap: null
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
