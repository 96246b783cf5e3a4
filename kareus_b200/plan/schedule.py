"""``scheds_pipeline_NNNNN.py`` plan files: parse, emit and the per-instruction schedule item.

File contract (reference ``kareus/scheduler/parser.py:24-60,66-101,104-318``): the file is one
Python list literal, one inner list per pipeline stage.

* activation-checkpointing layout: a flat list of the stage's 1F1B instructions,
  ``('forward', cfg...)`` carrying the forward keys and ``('backward', cfg...)`` carrying the
  recompute-forward keys followed by the backward keys;
* non-checkpointing layout: one ``((forward...), (backward...))`` pair per microbatch.

A cfg string is ``<start_slot>-<end_slot|none>-<sm>-<block>`` with slot names such as ``norm_0``
or, in old files, integers (``-1--1-16-1024``).  This module is table driven: the key order of
the tensor-parallel and context-parallel flavours is data, so new key sets (for example the
sequence-parallel ``*_ag`` keys) only extend the tables.
"""
from __future__ import annotations

import ast
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

OverlapWindow = Tuple[Union[int, str], Union[int, str]]
ResourceShape = Tuple[int, int]

FWD_KEYS_TP: Tuple[str, ...] = ("fwd_attn", "fwd_mlp")
BWD_KEYS_TP: Tuple[str, ...] = ("bwd_attn", "bwd_mlp")
FWD_KEYS_CP: Tuple[str, ...] = ("fwd_qkv_ar", "fwd_qkv_ag", "fwd_ao_ag", "fwd_ao_ar", "fwd_mlp")
BWD_KEYS_CP: Tuple[str, ...] = (
    "bwd_qkv_ar", "bwd_qkv_rs", "bwd_a_rs", "bwd_a_ag", "bwd_o_ag", "bwd_o_ar", "bwd_mlp",
)
TRAIL_KEYS: Tuple[str, ...] = ("fwd_trail", "bwd_trail")

# Keys that only exist under sequence parallelism inherit the value of the reference key that
# governs the same half of the layer when a plan file does not name them.
_INHERIT: Dict[str, str] = {
    "fwd_attn_ag": "fwd_attn", "fwd_mlp_ag": "fwd_mlp",
    "bwd_attn_ag": "bwd_attn", "bwd_mlp_ag": "bwd_mlp",
}


@dataclass(frozen=True)
class CommConfig:
    """Where a collective is launched inside a partition and with how many CTAs."""

    overlap_window: OverlapWindow
    resource_shape: ResourceShape

    @property
    def start(self):
        return self.overlap_window[0]

    @property
    def sm_num(self) -> int:
        return self.resource_shape[0]

    @property
    def block_size(self) -> int:
        return self.resource_shape[1]

    def to_string(self) -> str:
        s, e = self.overlap_window
        return f"{s}-{e}-{self.resource_shape[0]}-{self.resource_shape[1]}"


TRAIL_CONFIG = CommConfig(("norm_0", "none"), (20, 1024))
DEFAULT_CONFIG = CommConfig(("norm_0", "none"), (16, 1024))

_INT_CFG = re.compile(r"^(-?\d+)-(-?\d+)-(-?\d+)-(-?\d+)$")
_SLOT_CFG = re.compile(r"^([A-Za-z_]+\w*)-([A-Za-z_]+\w*)-(\d+)-(\d+)$")


def parse_config_string(cfg: str) -> CommConfig:
    if not isinstance(cfg, str):
        raise TypeError(f"config must be a string, got {type(cfg).__name__}")
    m = _INT_CFG.match(cfg)
    if m:
        a, b, sm, blk = (int(g) for g in m.groups())
        return CommConfig((a, b), (sm, blk))
    m = _SLOT_CFG.match(cfg)
    if m:
        return CommConfig((m.group(1), m.group(2)), (int(m.group(3)), int(m.group(4))))
    raise ValueError(
        f"bad comm config {cfg!r}: expected '<start>-<end>-<sm>-<block>' with slot names or integers"
    )


@dataclass(frozen=True)
class ScheduleItem:
    """Configs of one pipeline instruction (or one microbatch in the pair layout).

    Keys are looked up by name with :meth:`get`; attribute access works for every key so code
    written against the reference's ``ScheduleItem``/``ScheduleItemCP`` field names keeps working.
    """

    kind: str  # "forward", "backward" or "both"
    configs: Tuple[Tuple[str, Optional[CommConfig]], ...]
    context_parallel: bool = False

    def as_dict(self) -> Dict[str, Optional[CommConfig]]:
        return dict(self.configs)

    def get(self, key: str, default: Optional[CommConfig] = None) -> Optional[CommConfig]:
        d = dict(self.configs)
        if key in d and d[key] is not None:
            return d[key]
        if key in TRAIL_KEYS:
            return TRAIL_CONFIG
        parent = _INHERIT.get(key)
        if parent is not None and d.get(parent) is not None:
            # the parent's slot names belong to another segment: keep its launch shape and start
            # the collective with the first operator of this one
            return CommConfig(("first", "none"), d[parent].resource_shape)
        return default

    def __getattr__(self, name: str):
        if name.startswith("fwd_") or name.startswith("bwd_"):
            return self.get(name)
        raise AttributeError(name)


def _item(kind: str, keys: Sequence[str], cfgs: Sequence[str], cp: bool,
          all_keys: Sequence[str]) -> ScheduleItem:
    parsed = {k: None for k in all_keys}
    for k, c in zip(keys, cfgs):
        parsed[k] = parse_config_string(c)
    return ScheduleItem(kind, tuple(parsed.items()), cp)


def _load_literal(text: str):
    try:
        return ast.literal_eval(text.strip())
    except (SyntaxError, ValueError) as e:
        raise ValueError(f"plan file is not a Python literal: {e}") from e


def parse_schedule_text(text: str, use_activation_checkpointing: bool,
                        context_parallel: bool) -> List[List[ScheduleItem]]:
    parsed = _load_literal(text)
    if not isinstance(parsed, list):
        raise TypeError("top level of a schedule file must be a list (one entry per pipeline stage)")
    fk = FWD_KEYS_CP if context_parallel else FWD_KEYS_TP
    bk = BWD_KEYS_CP if context_parallel else BWD_KEYS_TP
    allk = fk + bk
    out: List[List[ScheduleItem]] = []
    for si, stage in enumerate(parsed):
        if not isinstance(stage, list):
            raise TypeError(f"stage {si}: expected a list")
        items: List[ScheduleItem] = []
        if use_activation_checkpointing:
            for tup in stage:
                if not isinstance(tup, tuple) or not tup or not isinstance(tup[0], str):
                    raise TypeError(f"stage {si}: instruction must be a tuple starting with its name")
                name, cfgs = tup[0], tup[1:]
                if name == "forward":
                    if len(cfgs) != len(fk):
                        raise TypeError(f"stage {si}: forward needs {len(fk)} configs, got {len(cfgs)}")
                    items.append(_item("forward", fk, cfgs, context_parallel, allk))
                elif name == "backward":
                    if len(cfgs) != len(fk) + len(bk):
                        raise TypeError(
                            f"stage {si}: backward needs {len(fk)} recompute + {len(bk)} backward configs, "
                            f"got {len(cfgs)}")
                    items.append(_item("backward", allk, cfgs, context_parallel, allk))
                else:
                    raise ValueError(f"stage {si}: unknown instruction {name!r}")
        else:
            for pair in stage:
                if not (isinstance(pair, tuple) and len(pair) == 2):
                    raise TypeError(f"stage {si}: expected ((forward...), (backward...)) pairs")
                f, b = pair
                if not (isinstance(f, tuple) and isinstance(b, tuple) and f and b):
                    raise TypeError(f"stage {si}: malformed microbatch pair")
                if f[0] != "forward" or b[0] != "backward":
                    raise ValueError(f"stage {si}: expected ('forward',..),('backward',..), got {f[0]!r},{b[0]!r}")
                if len(f) - 1 != len(fk) or len(b) - 1 != len(bk):
                    raise TypeError(f"stage {si}: pair needs {len(fk)} forward and {len(bk)} backward configs")
                items.append(_item("both", allk, tuple(f[1:]) + tuple(b[1:]), context_parallel, allk))
        out.append(items)
    return out


def parse_schedule_file(path: Union[str, Path], use_activation_checkpointing: bool,
                        context_parallel: bool) -> List[List[ScheduleItem]]:
    return parse_schedule_text(Path(path).read_text(encoding="utf-8"),
                               use_activation_checkpointing, context_parallel)


def _trailer(iteration: Optional[int], cost_change: Optional[float], total_cost: Optional[float],
             total_cost_p2p: Optional[float]) -> str:
    if iteration is None:
        return ""
    return (f"# Iteration {iteration} cost change: {cost_change}\n"
            f"# Iteration {iteration} total cost: {total_cost}\n"
            f"# Iteration {iteration} total cost with P2P: {total_cost_p2p}\n")


def emit_schedule_text(stages: Sequence[Sequence[ScheduleItem]], use_activation_checkpointing: bool,
                       iteration: Optional[int] = None, cost_change: Optional[float] = None,
                       total_cost: Optional[float] = None, total_cost_p2p: Optional[float] = None) -> str:
    """Inverse of :func:`parse_schedule_text` (writer in the reference:
    ``tests/kareus/run_optimization.py:189-337``)."""
    lines = ["["]
    for stage in stages:
        parts = []
        for it in stage:
            cp = it.context_parallel
            fk = FWD_KEYS_CP if cp else FWD_KEYS_TP
            bk = BWD_KEYS_CP if cp else BWD_KEYS_TP
            d = it.as_dict()

            def s(keys):
                return tuple(d[k].to_string() for k in keys)

            if use_activation_checkpointing:
                if it.kind == "forward":
                    parts.append(repr(("forward",) + s(fk)))
                elif it.kind == "backward":
                    parts.append(repr(("backward",) + s(fk) + s(bk)))
                else:
                    raise ValueError("pair items cannot be written in the checkpointing layout")
            else:
                parts.append(repr((("forward",) + s(fk), ("backward",) + s(bk))))
        lines.append("[" + ", ".join(parts) + "],")
    lines.append("]")
    return "\n".join(lines) + "\n" + _trailer(iteration, cost_change, total_cost, total_cost_p2p)


def read_trailer(text: str) -> Dict[str, float]:
    """Return ``{'iteration', 'cost_change', 'total_cost', 'total_cost_p2p'}`` from a plan file."""
    out: Dict[str, float] = {}
    for line in text.splitlines():
        m = re.match(r"#\s*Iteration\s+(\d+)\s+(cost change|total cost with P2P|total cost):\s*(\S+)", line)
        if m:
            out["iteration"] = int(m.group(1))
            key = {"cost change": "cost_change", "total cost": "total_cost",
                   "total cost with P2P": "total_cost_p2p"}[m.group(2)]
            out[key] = float(m.group(3))
    return out


def uniform_schedule(num_stages: int, instructions: Sequence[str], cfg: CommConfig = DEFAULT_CONFIG,
                     context_parallel: bool = False) -> List[List[ScheduleItem]]:
    """A plan that uses the same config everywhere (the fixed ``norm_0-none-16-1024`` schedule)."""
    fk = FWD_KEYS_CP if context_parallel else FWD_KEYS_TP
    bk = BWD_KEYS_CP if context_parallel else BWD_KEYS_TP
    allk = fk + bk
    s = cfg.to_string()
    stages = []
    for _ in range(num_stages):
        items = []
        for name in instructions:
            if name == "forward":
                items.append(_item("forward", fk, [s] * len(fk), context_parallel, allk))
            else:
                items.append(_item("backward", allk, [s] * len(allk), context_parallel, allk))
        stages.append(items)
    return stages
