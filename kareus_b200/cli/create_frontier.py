"""Sample the 10-plan frontier out of a solver output directory (``create_frontier.sh``).

    python -m kareus_b200.cli.create_frontier kareus <lowtime dir> <target dir>
"""
from __future__ import annotations

import sys


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) != 3 or argv[0] not in ("kareus", "nanobatch", "perseus"):
        print("usage: create_frontier <kareus|nanobatch|perseus> <source dir> <target dir>", file=sys.stderr)
        return 1
    from ..plan.frontier import create_frontier
    kept = create_frontier(argv[1], argv[2], with_scheds=(argv[0] == "kareus"))
    print(f"Done. Frontier written to: {argv[2]} ({len(kept)} files)")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
