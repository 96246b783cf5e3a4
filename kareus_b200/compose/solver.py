"""Iteration-level time–energy planner: Phillips–Dessouky time–cost trade-off on the 1F1B DAG.

The reference delegates this to the ``lowtime`` package (``tests/kareus/run_optimization.py:24-40,
369-429,464-487``); this is an independent implementation of the same algorithm:

1. every (stage, forward|backward) instruction type has candidate execution options
   ``(time, effective energy, knob)``; options are quantised to ``unit_time`` and reduced to their
   Pareto front, and an exponential ``cost(t) = a·exp(b·t) + c`` is fitted through them so that
   cost is defined for every integer duration between the fastest and the slowest option;
2. all instructions start at their slowest (cheapest) duration; the dependency DAG is the in-stage
   1F1B order plus ``F(s,m) → F(s+1,m)`` and ``B(s+1,m) → B(s,m)``;
3. each iteration finds the critical sub-DAG, gives every critical instruction the flow bounds
   ``[cost(d) − cost(d+1), cost(d−1) − cost(d)]`` (what slowing it by one unit saves, what speeding it
   up costs), solves a minimum cut with lower bounds, speeds up the instructions cut forward and
   slows down those cut backward.  The iteration time drops by exactly one ``unit_time`` at the least
   possible energy increase.  It stops when the cut is unbounded.

``plan_pipeline`` yields one result per iteration with each instruction's planned duration and the
knob of the option to run it with (largest option time ≤ planned duration).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Generator, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from ..parallel.pipeline import one_f_one_b_order
from .mincut import INF, bounded_min_cut


# ----------------------------------------------------------------------------- options / cost model
@dataclass
class ExecutionOption:
    real_time: float          # seconds
    unit_time: float          # seconds per quantum
    cost: float               # (effective) energy, joules
    knob: tuple

    @property
    def quant_time(self) -> int:
        return max(1, int(round(self.real_time / self.unit_time)))


def pareto_options(options: Sequence[ExecutionOption], noise_factor: float = 1.0) -> List[ExecutionOption]:
    """Keep options that are not dominated in (quant_time, cost): walking from fast to slow, a
    slower option stays only if it is cheaper than everything faster (by ``noise_factor``)."""
    best: Dict[int, ExecutionOption] = {}
    for o in options:
        q = o.quant_time
        if q not in best or o.cost < best[q].cost:
            best[q] = o
    out: List[ExecutionOption] = []
    cheapest = math.inf
    for q in sorted(best):
        o = best[q]
        if o.cost < cheapest * noise_factor or not out:
            if o.cost < cheapest:
                cheapest = o.cost
            out.append(o)
    # remove leftovers that noise tolerance let through but are strictly dominated
    if noise_factor == 1.0:
        return out
    return out


class ExponentialModel:
    """``cost(t) = a·exp(b·t) + c`` through the Pareto options (falls back to piecewise-linear
    interpolation when the fit is not decreasing/convex or fails)."""

    def __init__(self, options: Sequence[ExecutionOption]):
        pts = sorted({(o.quant_time, o.cost) for o in options})
        self.ts = np.array([p[0] for p in pts], dtype=float)
        self.cs = np.array([p[1] for p in pts], dtype=float)
        self.params: Optional[Tuple[float, float, float]] = None
        if len(pts) >= 3:
            self.params = self._fit()

    def _fit(self) -> Optional[Tuple[float, float, float]]:
        try:
            from scipy.optimize import curve_fit
        except Exception:  # pragma: no cover
            return None
        t0, scale = self.ts.min(), max(self.ts.max() - self.ts.min(), 1.0)
        x = (self.ts - t0) / scale
        cspan = max(self.cs.max() - self.cs.min(), 1e-9)

        def f(x, a, b, c):
            return a * np.exp(b * x) + c

        try:
            (a, b, c), _ = curve_fit(f, x, self.cs, p0=(cspan, -2.0, self.cs.min()), maxfev=20000)
        except Exception:
            return None
        if not (a > 0 and b < 0) or not np.all(np.isfinite([a, b, c])):
            return None
        resid = np.abs(f(x, a, b, c) - self.cs).max()
        if resid > 0.25 * cspan:
            return None
        # back to absolute quanta: a·exp(b·(t − t0)/scale) + c
        return (a * math.exp(-b * t0 / scale), b / scale, c)

    def __call__(self, t: float) -> float:
        if self.params is not None:
            a, b, c = self.params
            return a * math.exp(b * t) + c
        return float(np.interp(t, self.ts, self.cs))


@dataclass
class OperationSpec:
    options: List[ExecutionOption]
    model: ExponentialModel

    @classmethod
    def build(cls, options: Sequence[ExecutionOption], noise_factor: float = 1.0) -> "OperationSpec":
        po = pareto_options(options)
        if len(po) <= 3 and noise_factor != 1.0:
            po = pareto_options(options, noise_factor)
        if not po:
            raise ValueError("an instruction type needs at least one execution option")
        return cls(po, ExponentialModel(po))

    @property
    def min_duration(self) -> int:
        return min(o.quant_time for o in self.options)

    @property
    def max_duration(self) -> int:
        return max(o.quant_time for o in self.options)

    def knob_for(self, duration: int) -> tuple:
        """Option with the largest quantised time not exceeding ``duration``."""
        fit = [o for o in self.options if o.quant_time <= duration]
        o = max(fit, key=lambda o: o.quant_time) if fit else min(self.options, key=lambda o: o.quant_time)
        return o.knob


# ----------------------------------------------------------------------------- DAG
@dataclass
class Instruction:
    kind: str               # "forward" | "backward"
    stage: int
    micro_batch: int
    spec: OperationSpec
    duration: int = 0
    assigned_knob: tuple = ()

    def __post_init__(self):
        self.duration = self.spec.max_duration
        self.assigned_knob = self.spec.knob_for(self.duration)

    @property
    def cost(self) -> float:
        return self.spec.model(self.duration)


def build_1f1b_dag(num_stages: int, num_micro_batches: int,
                   specs: Dict[int, Dict[str, OperationSpec]]):
    """Returns ``(per-stage instruction lists, edges)`` with edges as index pairs into the flat list."""
    stages: List[List[Instruction]] = []
    flat: List[Instruction] = []
    index: Dict[Tuple[str, int, int], int] = {}
    edges: List[Tuple[int, int]] = []
    for s in range(num_stages):
        row = []
        prev = None
        for kind, mb in one_f_one_b_order(num_stages, s, num_micro_batches):
            inst = Instruction(kind, s, mb, specs[s][kind])
            idx = len(flat)
            flat.append(inst)
            row.append(inst)
            index[(kind, s, mb)] = idx
            if prev is not None:
                edges.append((prev, idx))
            prev = idx
        stages.append(row)
    for s in range(num_stages - 1):
        for mb in range(num_micro_batches):
            edges.append((index[("forward", s, mb)], index[("forward", s + 1, mb)]))
            edges.append((index[("backward", s + 1, mb)], index[("backward", s, mb)]))
    return stages, flat, edges


@dataclass
class IterationResult:
    iteration: int
    cost: float             # Σ effective energy of all instructions
    cost_change: float
    quant_time: int
    real_time: float        # seconds


def _schedule(flat: Sequence[Instruction], edges: Sequence[Tuple[int, int]]):
    n = len(flat)
    succ = [[] for _ in range(n)]
    pred = [[] for _ in range(n)]
    indeg = [0] * n
    for u, v in edges:
        succ[u].append(v)
        pred[v].append(u)
        indeg[v] += 1
    order, stack = [], [i for i in range(n) if indeg[i] == 0]
    deg = indeg[:]
    while stack:
        u = stack.pop()
        order.append(u)
        for v in succ[u]:
            deg[v] -= 1
            if deg[v] == 0:
                stack.append(v)
    if len(order) != n:
        raise RuntimeError("instruction graph has a cycle")
    es = [0] * n
    for u in order:
        for p in pred[u]:
            es[u] = max(es[u], es[p] + flat[p].duration)
    total = max(es[u] + flat[u].duration for u in range(n))
    lf = [total] * n
    for u in reversed(order):
        for v in succ[u]:
            lf[u] = min(lf[u], lf[v] - flat[v].duration)
    return es, lf, total, succ, pred


class PhillipsDessouky:
    def __init__(self, flat: Sequence[Instruction], edges: Sequence[Tuple[int, int]], unit_time: float,
                 use_native: Optional[bool] = None):
        self.flat, self.edges, self.unit_time, self.use_native = list(flat), list(edges), unit_time, use_native

    def total_cost(self) -> float:
        return sum(i.cost for i in self.flat)

    def iteration_time(self) -> int:
        return _schedule(self.flat, self.edges)[2]

    def run(self, max_iterations: Optional[int] = None) -> Generator[IterationResult, None, None]:
        it = 0
        while max_iterations is None or it < max_iterations:
            step = self._reduce_once()
            if step is None:
                return
            cost_change, total = step
            for inst in self.flat:
                inst.assigned_knob = inst.spec.knob_for(inst.duration)
            yield IterationResult(it, self.total_cost(), cost_change, total, total * self.unit_time)
            it += 1

    def _reduce_once(self):
        flat = self.flat
        es, lf, total, succ, pred = _schedule(flat, self.edges)
        crit = [u for u in range(len(flat)) if es[u] + flat[u].duration == lf[u]]
        cset = set(crit)
        # activity-on-edge network: node u becomes edge (2k, 2k+1); s = 2C, t = 2C+1
        pos = {u: k for k, u in enumerate(crit)}
        C = len(crit)
        S, T = 2 * C, 2 * C + 1
        net: List[Tuple[int, int, float, float]] = []
        op_edge: List[int] = []
        for u in crit:
            inst = flat[u]
            d = inst.duration
            lb = inst.spec.model(d) - inst.spec.model(d + 1) if d < inst.spec.max_duration else 0.0
            ub = inst.spec.model(d - 1) - inst.spec.model(d) if d > inst.spec.min_duration else INF
            lb = max(lb, 0.0)
            ub = max(ub, lb) if ub < INF else INF
            op_edge.append(len(net))
            net.append((2 * pos[u], 2 * pos[u] + 1, lb, ub))
            if es[u] == 0:
                net.append((S, 2 * pos[u], 0.0, INF))
            if lf[u] == total:
                net.append((2 * pos[u] + 1, T, 0.0, INF))
        for u, v in self.edges:
            if u in cset and v in cset and es[u] + flat[u].duration == es[v]:
                net.append((2 * pos[u] + 1, 2 * pos[v], 0.0, INF))
        side = bounded_min_cut(2 * C + 2, net, S, T, use_native=self.use_native)
        if side is None:
            return None
        change = 0.0
        speed, slow = [], []
        for k, u in enumerate(crit):
            a, b, lb, ub = net[op_edge[k]]
            if side[a] and not side[b]:
                if ub >= INF:
                    return None           # the cheapest way to shorten the schedule is impossible
                speed.append(u)
                change += ub
            elif side[b] and not side[a]:
                slow.append(u)
                change -= lb
        # dummy edges crossing forward make the cut unbounded
        for a, b, lb, ub in net:
            if ub >= INF and side[a] and not side[b]:
                return None
        if not speed:
            return None
        for u in speed:
            flat[u].duration -= 1
        for u in slow:
            if flat[u].duration < flat[u].spec.max_duration:
                flat[u].duration += 1
        new_total = _schedule(flat, self.edges)[2]
        return change, new_total


def plan_pipeline(num_stages: int, num_micro_batches: int, options: Dict[int, Dict[str, Sequence[ExecutionOption]]],
                  unit_time: float = 1e-3, noise_factor: float = 1.0, use_native: Optional[bool] = None,
                  max_iterations: Optional[int] = None):
    """Generator of ``(IterationResult, per-stage instruction lists)``; instruction objects are
    updated in place between yields, so consume (or snapshot) each result before advancing."""
    specs = {s: {k: OperationSpec.build(v, noise_factor) for k, v in kinds.items()} for s, kinds in options.items()}
    stages, flat, edges = build_1f1b_dag(num_stages, num_micro_batches, specs)
    solver = PhillipsDessouky(flat, edges, unit_time, use_native)
    produced = False
    for res in solver.run(max_iterations):
        produced = True
        yield res, stages
    if not produced:
        # nothing can be shortened (e.g. one measured option per instruction): the minimum-energy schedule
        # is the whole frontier, and still a plan that a run can execute
        for inst in flat:
            inst.assigned_knob = inst.spec.knob_for(inst.duration)
        total = _schedule(flat, edges)[2]
        yield IterationResult(0, solver.total_cost(), 0.0, total, total * unit_time), stages
