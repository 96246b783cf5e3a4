"""Compare measured runs (``zeus_monitor_*.txt``) of several methods, or two plan frontiers.

    python -m kareus_b200.cli.compare --base nemo_experiments/m/tag/megatron --runs .../kareus .../perseus
    python -m kareus_b200.cli.compare --frontier-ours plans/kareus/frontier --frontier-base plans/perseus/frontier \
        --num_stages 2 --gpu_type B200
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
    ap.add_argument("--frontier-ours")
    ap.add_argument("--frontier-base")
    ap.add_argument("--num_stages", type=int, default=2)
    ap.add_argument("--gpu_type", default="B200")
    a = ap.parse_args(argv)
    from ..compose.compare import compare_frontiers, dominates, frontier_from_plans, reduction, summarize_run
    from ..config import get_p2p_power
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
        print(json.dumps({**compare_frontiers(ours, base), "dominates": dominates(ours, base)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
