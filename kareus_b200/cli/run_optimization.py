"""Phase 2b: time–energy plan search; writes ``freqs_pipeline_%05d.py`` / ``scheds_pipeline_%05d.py``.

    python -m kareus_b200.cli.run_optimization --inst_profile profile_....csv --output_dir lowtime \
        --num_stages 2 --num_mbs 8 --gpu_type B200
"""
from __future__ import annotations

import argparse
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--inst_profile", required=True)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--num_stages", type=int, required=True)
    ap.add_argument("--num_mbs", type=int, required=True)
    ap.add_argument("--gpu_type", default="B200")
    ap.add_argument("--unit_time", type=float, default=1e-3)
    ap.add_argument("--noise_factor", type=float, default=0.9)
    ap.add_argument("--p2p_power", type=float, default=None)
    ap.add_argument("--max_iterations", type=int, default=None)
    ap.add_argument("--create_frontier", action="store_true", help="also sample the 10-plan frontier")
    a = ap.parse_args(argv)
    from ..compose.driver import run_optimization
    from ..plan.frontier import create_frontier
    t0 = time.time()
    summary = run_optimization(a.inst_profile, a.output_dir, a.num_stages, a.num_mbs, a.gpu_type, a.unit_time,
                               a.noise_factor, True, a.p2p_power, a.max_iterations)
    print(f"{len(summary)} plans written to {a.output_dir} in {time.time() - t0:.1f}s; "
          f"T {summary[0]['time_s']:.3f}s → {summary[-1]['time_s']:.3f}s")
    if a.create_frontier:
        kept = create_frontier(a.output_dir, f"{a.output_dir}/frontier")
        print(f"frontier: {len(kept)} files")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
