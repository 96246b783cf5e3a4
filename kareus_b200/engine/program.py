"""Partition programs: N-way nanobatch interleaving of a tensor graph and its executor.

A graph's node list is cut at every collective into *segments* ``(compute nodes, trailing
collective)``.  The program visits ``(segment, nanobatch)`` pairs round-robin; each visit is a
*step* (the reference's "partition") that runs the segment's compute for one nanobatch on the
compute stream while the collective produced by the previous visit (another nanobatch) runs on
the side stream.  With two nanobatches this reproduces the reference's interleaving
(``kareus/megatron/core/partitions/partition_builder.py:81-183``: NB0 carries the previous
segment's collective of NB1, NB1 carries this segment's collective of NB0); the same rule gives
valid programs for 1 (no overlap) and 4 nanobatches.

Launch and wait protocol (reference ``partition_base.py:186-299``, ``forward_partition.py:30-127``,
``backward_partition.py:36-145``): the plan entry of the step's key gives
``(overlap_start slot, sm_num, block_size)``.  The collective is enqueued on the side stream just
before the compute node that the slot names, after the side stream has waited for the event that
marks its input ready; at the end of the step (``sync="partition_end"``) or at the first consumer
(``sync="lazy"``) the compute stream waits for the collective's event.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .context import NanoBatchContext, OpContext
from .graph import Node, TensorGraph

MEMORY_BOUND_GROUPS = frozenset({"norm", "rope", "activation"})
KNOWN_GROUPS = frozenset({"norm", "rope", "activation", "linear", "attn"})


def build_overlap_slots(nodes: Sequence[Node]) -> Dict[str, int]:
    """Slot name → index of the compute node before which a collective may be launched.

    Neighbouring memory-bound operators of the same group share one slot; every GEMM and
    attention gets its own (vocabulary ``norm_k, rope_k, activation_k, linear_k, attn_k``;
    reference ``partition_base.py:22-110``).
    """
    slots: Dict[str, int] = {}
    counter: Dict[str, int] = {}
    prev: Optional[str] = None
    for i, n in enumerate(nodes):
        g = n.group
        if g not in KNOWN_GROUPS:
            raise ValueError(f"operator {n.name!r} has unknown slot group {g!r}")
        if g in MEMORY_BOUND_GROUPS:
            if g == prev:
                continue
            prev = g
        else:
            prev = None
        k = counter.get(g, 0)
        counter[g] = k + 1
        slots[f"{g}_{k}"] = i
    return slots


def resolve_slot(slots: Dict[str, int], name) -> int:
    """Index for a slot name; ``none`` and negative legacy integers mean "not inside the step"."""
    if isinstance(name, int):
        return name
    if name == "none":
        return -1
    if name == "first":
        return 0
    if name not in slots:
        raise KeyError(f"unknown overlap slot {name!r}; this step offers {sorted(slots)}")
    return slots[name]


@dataclass
class Segment:
    index: int
    compute: List[Node]
    comm: Optional[Node]
    key: str


@dataclass
class Step:
    index: int
    key: str
    nb: int
    segment: int
    compute: List[Node]
    comm: Optional[Node] = None      # collective launched during this step ...
    comm_nb: int = -1                # ... on behalf of this nanobatch
    comm_segment: int = -1
    slots: Dict[str, int] = field(default_factory=dict)

    def describe(self) -> str:
        c = f" || comm[{self.comm.kind.value}](nb{self.comm_nb})" if self.comm is not None else ""
        return f"step {self.index} key={self.key!r} nb{self.nb}: {[n.name for n in self.compute]}{c}"


def split_segments(nodes: Sequence[Node], trail_key: str) -> List[Segment]:
    segs: List[Segment] = []
    cur: List[Node] = []
    for n in nodes:
        if not n.is_comm:
            cur.append(n)
            continue
        if cur or not segs or segs[-1].comm is not None:
            # a collective with no compute before it still forms a (compute-less) segment so that
            # back-to-back collectives keep their order
            segs.append(Segment(len(segs), cur, n, n.key))
            cur = []
        else:
            segs[-1].comm = n
            segs[-1].key = n.key
    if cur:
        segs.append(Segment(len(segs), cur, None, trail_key))
    return segs


def _rec():
    from ..kernels import replay
    return replay


def record_event(stream):
    """New event recorded on ``stream`` (mirrored into an open launch-list recording)."""
    ev = torch.cuda.Event()
    ev.record(stream)
    _rec().note_event_record(ev, stream)
    return ev


def wait_event(stream, ev) -> None:
    stream.wait_event(ev)
    _rec().note_stream_wait(stream, ev)


def wait_stream(stream, other) -> None:
    """``stream`` waits for everything enqueued on ``other`` so far."""
    wait_event(stream, record_event(other))


def record_stream(t, stream) -> None:
    """``t`` is used on ``stream`` although it was allocated on another one."""
    if isinstance(t, torch.Tensor) and t.is_cuda:
        t.record_stream(stream)
        _rec().note_cross_stream_use(t)


class StreamSet:
    """Compute/side stream pair.  On CPU everything is ``None`` and waits are no-ops."""

    def __init__(self, device: Optional[torch.device] = None):
        self.cuda = device is not None and torch.device(device).type == "cuda"
        self.device = device
        self._comm = None

    @property
    def comm(self):
        if self.cuda and self._comm is None:
            self._comm = _shared_comm_stream(self.device)
        return self._comm

    def comm_for(self, nb: int):
        """Side stream of a nanobatch.  By default all nanobatches share one ordered side stream (the
        reference's single comm stream); with ``KAREUS_COMM_STREAMS=per_nanobatch`` each nanobatch
        gets its own, so two fused GEMM+collective kernels (one link bound, one compute bound) can
        run side by side."""
        if not self.cuda:
            return None
        if _per_nb_streams():
            return _shared_comm_stream(self.device, slot=1 + nb)
        return self.comm

    def compute(self):
        return torch.cuda.current_stream(self.device) if self.cuda else None

    def record(self, stream):
        if not self.cuda:
            return None
        return record_event(stream)


_COMM_STREAMS: Dict[tuple, "torch.cuda.Stream"] = {}


def _per_nb_streams() -> bool:
    import os
    return os.environ.get("KAREUS_COMM_STREAMS", "shared") == "per_nanobatch"


def _shared_comm_stream(device, slot: int = 0) -> "torch.cuda.Stream":
    """One side stream per device shared by all collectives, which keeps them ordered among
    themselves (reference ``kareus/msccl/msccl_comm.py:577``)."""
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if (idx, slot) not in _COMM_STREAMS:
        _COMM_STREAMS[(idx, slot)] = torch.cuda.Stream(device=idx, priority=-1)
    return _COMM_STREAMS[(idx, slot)]


class PartitionProgram:
    def __init__(self, graph: TensorGraph, num_nanobatches: int, backward: bool,
                 sync: str = "partition_end", reverse_nb: bool = False, cp_keys: bool = False):
        if sync not in ("partition_end", "lazy"):
            raise ValueError(sync)
        self.graph = graph
        self.n = int(num_nanobatches)
        self.backward = backward
        self.sync = sync
        # sequence-split nanobatches: a later nanobatch's attention backward produces dK/dV for the
        # earlier ones, so the backward program visits nanobatches last-to-first
        self.nb_order = list(reversed(range(self.n))) if reverse_nb else list(range(self.n))
        self.trail_key = "bwd_trail" if backward else "fwd_trail"
        # context-parallel plan files name a step after its compute segment AND the collective it
        # carries (fwd_qkv_ar, fwd_qkv_ag, fwd_ao_ag, ...: reference transformer_block.py:193-203)
        self.cp_keys = cp_keys
        self.segments = split_segments(graph.nodes, self.trail_key)
        self.steps = self._form_steps()
        self._last_use = self._compute_last_use()
        self.keep_ids: set = set(graph.final.values())
        self.free_dead = True      # profilers re-run single steps and switch this off

    # ------------------------------------------------------------------ formation
    def _form_steps(self) -> List[Step]:
        steps: List[Step] = []
        prev: Optional[Tuple[int, int]] = None
        for seg in self.segments:
            for nb in self.nb_order:
                st = Step(index=len(steps), key=seg.key, nb=nb, segment=seg.index,
                          compute=seg.compute, slots=build_overlap_slots(seg.compute))
                if prev is not None:
                    ps, pnb = prev
                    pc = self.segments[ps].comm
                    if pc is not None:
                        st.comm, st.comm_nb, st.comm_segment = pc, pnb, ps
                if self.cp_keys:
                    st.key = self._cp_key(seg, st.comm)
                steps.append(st)
                prev = (seg.index, nb)
        if prev is not None and self.segments[prev[0]].comm is not None:
            ps, pnb = prev
            steps.append(Step(index=len(steps), key=self.trail_key, nb=pnb, segment=ps + 1,
                              compute=[], comm=self.segments[ps].comm, comm_nb=pnb, comm_segment=ps))
        return steps

    def _cp_key(self, seg: Segment, carried: Optional[Node]) -> str:
        if seg.comm is None or not seg.comm.segment:
            return seg.key
        d = "bwd" if self.backward else "fwd"
        name = seg.comm.segment
        if name == "mlp":
            return f"{d}_mlp"
        short = carried.short if carried is not None and carried.short else seg.comm.short
        return f"{d}_{name}_{short}"

    def expected_keys(self) -> List[str]:
        return [s.key for s in self.steps]

    def _compute_last_use(self) -> Dict[str, int]:
        last: Dict[str, int] = {}
        for n in self.graph.nodes:
            for p in n.inputs:
                last[p.tensor_id] = n.index
        return last

    # ------------------------------------------------------------------ execution
    def run(self, ctxs: Sequence[NanoBatchContext], schedule=None, streams: Optional[StreamSet] = None,
            grad_enabled: bool = True, release_saved: bool = True,
            default_shape: Tuple[Optional[int], Optional[int]] = (None, None)) -> None:
        """Execute all steps.  ``ctxs[i].store`` must already hold the graph's external tensors."""
        self.run_steps(ctxs, self.steps, schedule, streams, grad_enabled, release_saved, default_shape)

    def run_steps(self, ctxs: Sequence[NanoBatchContext], steps: Sequence[Step], schedule=None,
                  streams: Optional[StreamSet] = None, grad_enabled: bool = True, release_saved: bool = True,
                  default_shape: Tuple[Optional[int], Optional[int]] = (None, None)) -> None:
        """Execute a contiguous run of steps (the whole program, or one step for a profiler)."""
        if len(ctxs) != self.n:
            raise ValueError(f"program was formed for {self.n} nanobatches, got {len(ctxs)} contexts")
        streams = streams or StreamSet(None)
        pending: List[Tuple[Node, int, object]] = []  # (comm node, nb, done event) not yet waited

        for st in steps:
            cfg = schedule.get(st.key) if schedule is not None else None
            planned = cfg is not None
            if planned:
                start = resolve_slot(st.slots, cfg.start) if st.compute else -1
                shape = cfg.resource_shape
            else:
                start, shape = 0, default_shape
            launched = st.comm is None
            if self.n == 1 and st.comm is not None:
                # a single nanobatch has nothing to hide the collective behind
                self._launch_comm(st, ctxs, streams, shape, pending, planned, release_saved)
                self._wait_all(pending, ctxs, streams)
                launched = True
            for i, node in enumerate(st.compute):
                if not launched and i == start:
                    self._launch_comm(st, ctxs, streams, shape, pending, planned, release_saved)
                    launched = True
                self._run_compute(node, ctxs[st.nb], streams, grad_enabled, release_saved)
            if st.compute:
                ctxs[st.nb].ready_event[st.segment] = streams.record(streams.compute())
            if not launched:
                self._launch_comm(st, ctxs, streams, shape, pending, planned, release_saved)
            if self.sync == "partition_end":
                self._wait_all(pending, ctxs, streams)
        self._wait_all(pending, ctxs, streams)

    # -- compute
    def _run_compute(self, node: Node, nbctx: NanoBatchContext, streams: StreamSet,
                     grad_enabled: bool, release_saved: bool) -> None:
        store = nbctx.store
        ins = []
        for p in node.inputs:
            ev = store.event(p.tensor_id)
            if ev is not None:
                if streams.cuda:
                    wait_event(streams.compute(), ev)
                store.clear_event(p.tensor_id)
            ins.append(store.get(p.tensor_id))
        op = node.operator
        if not self.backward:
            ctx = nbctx.ctx_for(node.op_id)
            ctx.requires_grad = grad_enabled
            outs = op.forward(ctx, *ins)
        else:
            ctx = nbctx.ctx_for(node.op_id, create=False)
            outs = op.backward(ctx, *ins)
            if release_saved:
                nbctx.release_op(node.op_id)
        if not isinstance(outs, (tuple, list)):
            outs = (outs,)
        if len(outs) != len(node.outputs):
            raise RuntimeError(f"{node.name} returned {len(outs)} tensors for {len(node.outputs)} ports")
        for p, t in zip(node.outputs, outs):
            store.put(p.tensor_id, t)
        self._free_dead(node, store)

    def _free_dead(self, node: Node, store) -> None:
        if not self.free_dead:
            return
        for p in node.inputs:
            tid = p.tensor_id
            if self._last_use.get(tid) == node.index and tid not in self.keep_ids \
                    and not tid.startswith("ext_"):
                store.pop(tid)

    # -- collectives
    def _launch_comm(self, st: Step, ctxs, streams: StreamSet, shape, pending, planned: bool = False,
                     release_saved: bool = True) -> None:
        node, nb = st.comm, st.comm_nb
        nbctx = ctxs[nb]
        store = nbctx.store
        ins = [store.get(p.tensor_id) for p in node.inputs]
        side = streams.comm_for(nb)
        if streams.cuda:
            ready = nbctx.ready_event.get(st.comm_segment)
            if ready is not None:
                wait_event(side, ready)
            else:
                wait_stream(side, streams.compute())
            for p in node.inputs:           # input produced by an earlier collective
                ev = store.event(p.tensor_id)
                if ev is not None:
                    wait_event(side, ev)
        sm_num, block = shape if shape is not None else (None, None)
        ctx = nbctx.ctx_for(node.op_id) if getattr(node.operator, "needs_ctx", False) else None
        # operators whose sm_num has a second meaning when it comes from a plan entry are told so
        kw = {"planned": planned} if getattr(node.operator, "takes_planned", False) else {}
        if streams.cuda:
            with torch.cuda.stream(side):
                outs = node.operator.run(ins, sm_num=sm_num, block_size=block, backward=self.backward,
                                         nb=nb, ctx=ctx, **kw)
            done = streams.record(side)
            for t in ins:
                record_stream(t, side)
        else:
            outs = node.operator.run(ins, sm_num=sm_num, block_size=block, backward=self.backward,
                                     nb=nb, ctx=ctx, **kw)
            done = None
        if self.backward and release_saved and getattr(node.operator, "releases_ctx", False):
            # a fused backward node is the last user of its layer's saved tensors (a profiler that re-runs
            # one step keeps them: release_saved=False)
            nbctx.release_op(node.op_id)
        if not isinstance(outs, (tuple, list)):
            outs = (outs,)
        for p, t in zip(node.outputs, outs):
            store.put(p.tensor_id, t, event=done)
            if streams.cuda:
                record_stream(t, streams.compute())
        self._free_dead(node, store)
        pending.append((node, nb, done))

    def _wait_all(self, pending, ctxs, streams: StreamSet) -> None:
        for node, nb, done in pending:
            if done is not None and streams.cuda:
                wait_event(streams.compute(), done)
            for p in node.outputs:
                ctxs[nb].store.clear_event(p.tensor_id)
        pending.clear()

    def describe(self) -> str:
        return "\n".join(s.describe() for s in self.steps)
