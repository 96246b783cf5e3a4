"""Plan server: serves the clocks of a ``freqs_pipeline_*.py`` plan to the training ranks over HTTP.

    python -m kareus_b200.cli.pfo_server --freqs plans/freqs_pipeline_02495.py [--host 0.0.0.0] [--port 7787]
    torchrun ... -m kareus_b200.cli.run_train --method perseus --pfo-url http://$MASTER_ADDR:7787 ...

The reference starts zeus' pipeline-frequency server for this on the master node
(``uvicorn zeus.optimizer.pipeline_frequency.server.router:app --port $PFO_PORT`` with the plan named in
``ZEUS_PFO_SCHEDULER_ARGS``; ``tests/artifact/run_kareus.sh:373-385``).  The same environment is honoured here:
``PFO_PORT`` is the default port and ``ZEUS_PFO_SCHEDULER_ARGS`` (a JSON object with ``solution_path``) the
default plan.  The process serves until it is interrupted; ``--once-after S`` stops it after S seconds (tests).
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import sys
import threading


def main(argv=None) -> int:
    env_args = {}
    try:
        env_args = json.loads(os.environ.get("ZEUS_PFO_SCHEDULER_ARGS", "") or "{}")
    except json.JSONDecodeError:
        print("ZEUS_PFO_SCHEDULER_ARGS is not a JSON object; ignored", file=sys.stderr)
    ap = argparse.ArgumentParser()
    ap.add_argument("--freqs", default=env_args.get("solution_path"), help="freqs_pipeline_*.py to serve")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=int(os.environ.get("PFO_PORT", "7787")))
    ap.add_argument("--once-after", type=float, default=None, help="stop by itself after this many seconds")
    a = ap.parse_args(argv)
    if not a.freqs:
        ap.error("--freqs (or ZEUS_PFO_SCHEDULER_ARGS with solution_path) is required")
    from ..energy.pfo import PFOServer, PointSolution
    solution = PointSolution.from_file(a.freqs)
    server = PFOServer(solution, host=a.host, port=a.port).start()
    print(f"serving {a.freqs} ({len(solution.plan)} pipeline stages) on {server.url}", flush=True)
    done = threading.Event()
    for sig in (signal.SIGINT, signal.SIGTERM):
        try:
            signal.signal(sig, lambda *_: done.set())
        except ValueError:          # not the main thread (tests)
            pass
    done.wait(a.once_after)
    server.stop()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
