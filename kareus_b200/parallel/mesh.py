"""Process mesh: rank ↔ (tp, cp, dp, pp) coordinates and the process groups of each axis.

Rank order is tp-cp-dp-pp with tp fastest, the order the reference initialises Megatron with
(``3rdparty/Megatron-LM/megatron/core/parallel_state.py:431-445``), so a TP (and CP) group is a
contiguous block of ranks that lives on one NVSwitch domain.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class Coord:
    tp: int
    cp: int
    dp: int
    pp: int


class Mesh:
    AXES = ("tp", "cp", "dp", "pp")

    def __init__(self, tp: int = 1, cp: int = 1, dp: int = 1, pp: int = 1,
                 rank: Optional[int] = None, world_size: Optional[int] = None,
                 create_groups: bool = True):
        self.shape = {"tp": tp, "cp": cp, "dp": dp, "pp": pp}
        n = tp * cp * dp * pp
        if world_size is None:
            world_size = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        if rank is None:
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        if n != world_size:
            raise ValueError(f"tp*cp*dp*pp = {n} does not match world size {world_size}")
        self.world_size = world_size
        self.rank = rank
        self.coord = self.coord_of(rank)
        self.groups: Dict[str, object] = {}
        self.group_ranks: Dict[str, List[int]] = {}
        for axes in (("tp",), ("cp",), ("dp",), ("pp",), ("dp", "cp"), ("tp", "cp"), ("tp", "pp")):
            name = "_".join(axes)
            mine = None
            for ranks in self._enumerate_groups(axes):
                g = None
                if create_groups and world_size > 1 and len(ranks) > 1 and dist.is_initialized():
                    g = dist.new_group(ranks)
                if rank in ranks:
                    mine = (ranks, g)
            self.group_ranks[name] = mine[0]
            self.groups[name] = mine[1]
        # first and last pipeline stage of every (tp, cp, dp) column: the two holders of a tied
        # embedding / output weight (Megatron's embedding group, parallel_state.py)
        self.group_ranks["embd"], self.groups["embd"] = [rank], None
        if pp > 1:
            for t in range(tp):
                for c in range(cp):
                    for d in range(dp):
                        ranks = [self.rank_of(t, c, d, 0), self.rank_of(t, c, d, pp - 1)]
                        g = dist.new_group(ranks) if create_groups and dist.is_initialized() else None
                        if rank in ranks:
                            self.group_ranks["embd"], self.groups["embd"] = ranks, g

    # coordinates ------------------------------------------------------------
    def coord_of(self, rank: int) -> Coord:
        s = self.shape
        tp = rank % s["tp"]
        r = rank // s["tp"]
        cp = r % s["cp"]
        r //= s["cp"]
        dp = r % s["dp"]
        r //= s["dp"]
        return Coord(tp, cp, dp, r)

    def rank_of(self, tp: int, cp: int, dp: int, pp: int) -> int:
        s = self.shape
        return ((pp * s["dp"] + dp) * s["cp"] + cp) * s["tp"] + tp

    def _enumerate_groups(self, axes: Tuple[str, ...]) -> List[List[int]]:
        s = self.shape
        others = [a for a in self.AXES if a not in axes]
        groups: Dict[Tuple[int, ...], List[int]] = {}
        for r in range(self.world_size):
            c = self.coord_of(r)
            key = tuple(getattr(c, a) for a in others)
            groups.setdefault(key, []).append(r)
        return [sorted(v) for _, v in sorted(groups.items())]

    # accessors ----------------------------------------------------------------
    def size(self, axis: str) -> int:
        n = 1
        for a in axis.split("_"):
            n *= self.shape[a]
        return n

    def group(self, axis: str):
        return self.groups[axis]

    def ranks(self, axis: str) -> List[int]:
        return self.group_ranks[axis]

    def axis_rank(self, axis: str) -> int:
        return self.group_ranks[axis].index(self.rank)

    @property
    def tp(self) -> int: return self.shape["tp"]
    @property
    def cp(self) -> int: return self.shape["cp"]
    @property
    def dp(self) -> int: return self.shape["dp"]
    @property
    def pp(self) -> int: return self.shape["pp"]
    @property
    def tp_rank(self) -> int: return self.coord.tp
    @property
    def cp_rank(self) -> int: return self.coord.cp
    @property
    def dp_rank(self) -> int: return self.coord.dp
    @property
    def pp_rank(self) -> int: return self.coord.pp
    @property
    def is_first_stage(self) -> bool: return self.coord.pp == 0
    @property
    def is_last_stage(self) -> bool: return self.coord.pp == self.shape["pp"] - 1

    def pp_neighbor(self, delta: int) -> int:
        c = self.coord
        return self.rank_of(c.tp, c.cp, c.dp, (c.pp + delta) % self.shape["pp"])

    def folded_tp_rank(self) -> Tuple[int, int]:
        """(rank, degree) with CP folded into TP, the coordinate the frequency planner uses
        (reference ``3rdparty/NeMo/.../megatron_base_model.py:705-711``)."""
        return self.coord.cp * self.shape["tp"] + self.coord.tp, self.shape["tp"] * self.shape["cp"]


def init_distributed(backend: Optional[str] = None, device: Optional[torch.device] = None,
                     timeout_s: Optional[float] = None) -> Tuple[int, int, int]:
    """Initialise ``torch.distributed`` from the torchrun environment.  Returns (rank, world, local)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if timeout_s is not None:
            import datetime
            kw["timeout"] = datetime.timedelta(seconds=timeout_s)
        if backend == "nccl":
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kw)
    return rank, world, local
