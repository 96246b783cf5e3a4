"""Frontier sampling: pick 10 plans out of the solver's per-iteration output.

Rule (reference ``tests/artifact/create_frontier.sh:20-26,96-143``): sort plan files by name,
take a stride of ``ceil(total/15)`` walking down from the last file, re-sort ascending, then drop
positions 0, 2, 4, 6 and 8.  With the solver's usual output (hundreds of plans, 15 picked) the highest-numbered
file (max throughput) is position 14 and survives; with fewer than ten picked files it could sit on a dropped
position, so it is kept explicitly: a frontier is never empty.
"""
from __future__ import annotations

import shutil
from pathlib import Path
from typing import List, Sequence, Union

DROP_POSITIONS = (0, 2, 4, 6, 8)


def sample_frontier(names: Sequence[str], num_samples: int = 15,
                    drop: Sequence[int] = DROP_POSITIONS) -> List[str]:
    files = sorted(names)
    total = len(files)
    if total == 0:
        raise ValueError("no plan files to sample")
    if 0 < num_samples < total:
        stride = max(1, (total + num_samples - 1) // num_samples)
        picked = sorted(files[i] for i in range(total - 1, -1, -stride))
    else:
        picked = files
    dropset = set(drop)
    last = len(picked) - 1
    return [f for i, f in enumerate(picked) if i not in dropset or i == last]


def select_max_throughput(names: Sequence[str]) -> str:
    """Highest-numbered plan = last solver iteration (``tests/artifact/run_kareus.sh:338-339``)."""
    def key(n: str):
        digits = "".join(c for c in Path(n).stem if c.isdigit())
        return int(digits) if digits else -1
    return max(names, key=key)


def create_frontier(source_dir: Union[str, Path], target_dir: Union[str, Path],
                    with_scheds: bool = True, num_samples: int = 15) -> List[Path]:
    src, dst = Path(source_dir), Path(target_dir)
    dst.mkdir(parents=True, exist_ok=True)
    out: List[Path] = []
    for pattern in ("freqs_pipeline_*.py",) + (("scheds_pipeline_*.py",) if with_scheds else ()):
        names = [p.name for p in src.glob(pattern)]
        if not names:
            raise FileNotFoundError(f"no {pattern} under {src}")
        for n in sample_frontier(names, num_samples):
            shutil.copy2(src / n, dst / n)
            out.append(dst / n)
    return out
