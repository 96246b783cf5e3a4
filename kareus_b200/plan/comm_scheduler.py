"""Per-microbatch communication scheduler.

Walks this pipeline stage's list of :class:`ScheduleItem` as the training loop reports
instructions, exposing the active one as ``current_schedule`` (reference
``kareus/scheduler/pipeline_comm_scheduler.py:13-144``).  In the checkpointing layout every
instruction consumes one item and its kind is verified; in the pair layout only forwards advance.
``on_step_end`` checks that the plan was consumed exactly.
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import List, Optional, Sequence, Union

from .schedule import ScheduleItem, parse_schedule_file


class PipelineCommScheduler:
    def __init__(self, configs_pipeline: Union[str, os.PathLike], pp_rank: int, num_microbatches: int,
                 use_activation_checkpointing: bool = False, context_parallel: bool = False):
        p = Path(str(configs_pipeline))
        if p.suffix != ".py" or not p.is_file():
            raise FileNotFoundError(f"configs_pipeline must be an existing .py file, got: {p}")
        parsed = parse_schedule_file(p, use_activation_checkpointing, context_parallel)
        self._setup(parsed, pp_rank, num_microbatches, use_activation_checkpointing, context_parallel)
        self.path: Optional[Path] = p.resolve()

    @classmethod
    def from_parsed(cls, parsed: Sequence[Sequence[ScheduleItem]], pp_rank: int, num_microbatches: int,
                    use_activation_checkpointing: bool = False,
                    context_parallel: bool = False) -> "PipelineCommScheduler":
        """Build from a plan parsed elsewhere (rank 0 parses, everyone receives a broadcast)."""
        self = cls.__new__(cls)
        self.path = None
        self._setup(parsed, pp_rank, num_microbatches, use_activation_checkpointing, context_parallel)
        return self

    def _setup(self, parsed, pp_rank, num_microbatches, ac, cp):
        if not 0 <= pp_rank < len(parsed):
            raise IndexError(f"pp_rank {pp_rank} out of range for a plan with {len(parsed)} stages")
        self.ac_mode = bool(ac)
        self.context_parallel = bool(cp)
        self.pp_rank = pp_rank
        self.items: List[ScheduleItem] = list(parsed[pp_rank])
        want = 2 * num_microbatches if self.ac_mode else num_microbatches
        if len(self.items) != want:
            raise ValueError(
                f"plan has {len(self.items)} items for stage {pp_rank}, expected {want} "
                f"({num_microbatches} microbatches, {'instruction' if self.ac_mode else 'pair'} layout)")
        self._pos = 0
        self.current_schedule: Optional[ScheduleItem] = None

    # hooks -----------------------------------------------------------------
    def on_step_begin(self) -> None:
        pass

    def on_instruction_begin(self, name: str) -> None:
        if name not in ("forward", "backward"):
            raise ValueError(f"unknown instruction {name!r}")
        if self.ac_mode:
            if self._pos >= len(self.items):
                raise RuntimeError("no scheduled instruction left for this step")
            item = self.items[self._pos]
            if item.kind != name:
                raise RuntimeError(f"plan/loop mismatch at instruction {self._pos}: plan says "
                                   f"{item.kind!r}, loop runs {name!r}")
            self._pos += 1
            self.current_schedule = item
        elif name == "forward":
            if self._pos >= len(self.items):
                raise RuntimeError("no forward microbatch left for this step")
            self.current_schedule = self.items[self._pos]
            self._pos += 1

    def on_instruction_end(self, name: Optional[str] = None) -> None:
        pass

    def on_step_end(self) -> None:
        if self._pos != len(self.items):
            raise RuntimeError(f"step ended after {self._pos} of {len(self.items)} scheduled items")
        self._pos = 0
        self.current_schedule = None
