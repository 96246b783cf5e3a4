"""``freqs_pipeline_NNNNN.py`` plan files: per-stage, per-instruction SM clock in 1F1B order.

Contract (reference writer ``tests/kareus/run_optimization.py:189-252,476-484``; shipped example
``tests/kareus/schedules/megatron_llama3.2_3b/cp1_tp8_mbs8_seq4096/frontier/freqs_pipeline_00324.py``):
a list literal with one list per pipeline stage of ``('forward'|'backward', MHz)`` tuples in
that stage's execution order, followed by three ``# Iteration N ...`` comment lines.
"""
from __future__ import annotations

from pathlib import Path
from typing import List, Optional, Sequence, Tuple, Union

from .schedule import _load_literal, _trailer, read_trailer  # noqa: F401  (re-exported)

FreqPlan = List[List[Tuple[str, int]]]


def parse_freqs_text(text: str) -> FreqPlan:
    parsed = _load_literal(text)
    if not isinstance(parsed, list):
        raise TypeError("top level of a frequency plan must be a list")
    out: FreqPlan = []
    for si, stage in enumerate(parsed):
        if not isinstance(stage, list):
            raise TypeError(f"stage {si}: expected a list")
        row = []
        for tup in stage:
            if not (isinstance(tup, tuple) and len(tup) == 2 and tup[0] in ("forward", "backward")):
                raise TypeError(f"stage {si}: expected ('forward'|'backward', MHz), got {tup!r}")
            row.append((tup[0], int(tup[1])))
        out.append(row)
    return out


def parse_freqs_file(path: Union[str, Path]) -> FreqPlan:
    return parse_freqs_text(Path(path).read_text(encoding="utf-8"))


def emit_freqs_text(plan: Sequence[Sequence[Tuple[str, int]]], iteration: Optional[int] = None,
                    cost_change: Optional[float] = None, total_cost: Optional[float] = None,
                    total_cost_p2p: Optional[float] = None) -> str:
    lines = ["["]
    for stage in plan:
        lines.append("[" + ", ".join(repr((k, int(f))) for k, f in stage) + "],")
    lines.append("]")
    return "\n".join(lines) + "\n" + _trailer(iteration, cost_change, total_cost, total_cost_p2p)


def uniform_freqs(num_stages: int, instructions: Sequence[str], mhz: int) -> FreqPlan:
    return [[(k, int(mhz)) for k in instructions] for _ in range(num_stages)]
