"""Named-channel dataflow graph of one transformer block.

Operators declare which *channels* they read and write (``main``, ``residual``, ``key``,
``value``, ``rotary_pos_emb`` and the ``grad_*`` mirrors).  The builder turns a flat operator
list into nodes whose ports carry tensor ids, so producers and consumers that are not adjacent
(residual branches, K/V) connect without the operators knowing about each other.  The backward
graph is derived from the same operators in reverse with input/output channels swapped and
shares ``op_id`` with the forward node so saved state can be found.

Same role as the reference's ``kareus/megatron/core/partitions/tensor_graph.py:22-334``; the
differences are that a collective node may carry compute (a fused all-gather→GEMM is still one
node that the engine places on the side stream) and that every collective names the plan key of
the compute segment it terminates.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple


class CommKind(enum.Enum):
    ALL_REDUCE = "all_reduce"
    ALL_GATHER = "all_gather"            # sequence-parallel gather of activations (TP group)
    REDUCE_SCATTER = "reduce_scatter"    # sequence-parallel scatter of partial sums (TP group)
    ALL_GATHER_KV = "all_gather_kv"      # context-parallel gather of K and V
    REDUCE_SCATTER_KV = "reduce_scatter_kv"
    FUSED = "fused"                      # collective fused with a GEMM (runs on the side stream)


def grad_channel(name: str) -> str:
    return "grad_" + name


_UID = [0]


def operator_uid(op) -> int:
    """Process-wide unique id of an operator object, assigned on first use."""
    uid = getattr(op, "_graph_uid", None)
    if uid is None:
        _UID[0] += 1
        uid = _UID[0]
        try:
            object.__setattr__(op, "_graph_uid", uid)
        except Exception:  # pragma: no cover - objects without a __dict__
            raise TypeError(f"cannot tag {type(op).__name__} with a graph uid")
    return uid


@dataclass(frozen=True)
class Port:
    channel: str
    tensor_id: str


@dataclass
class Node:
    """One executable step of the graph."""

    index: int
    op_id: int
    operator: object
    inputs: Tuple[Port, ...]
    outputs: Tuple[Port, ...]
    is_comm: bool = False
    kind: Optional[CommKind] = None
    key: str = ""          # plan key of the compute segment this collective terminates
    backward: bool = False
    segment: str = ""      # context-parallel plan vocabulary: segment name (qkv, ao, a, o, mlp) ...
    short: str = ""        # ... and collective type (ar, ag, rs)

    @property
    def name(self) -> str:
        return getattr(self.operator, "name", type(self.operator).__name__)

    @property
    def group(self) -> str:
        return getattr(self.operator, "group", "other")


@dataclass
class ComputeSpec:
    operator: object
    in_channels: Tuple[str, ...]
    out_channels: Tuple[str, ...]
    backward: bool = False


@dataclass
class CommSpec:
    operator: object               # object with .run(tensors, sm_num, block_size, backward) semantics
    kind: CommKind
    in_channels: Tuple[str, ...]
    out_channels: Tuple[str, ...]
    key: str
    backward: bool = False
    segment: str = ""
    short: str = ""


class GraphOperator:
    """Base class of operators that can be placed in the graph.

    ``in_channels``/``out_channels`` describe the forward compute.  ``no_grad_inputs`` lists input
    channels that never receive a gradient (for example the RoPE table).  Subclasses may wrap the
    compute with collectives by overriding :meth:`forward_specs` / :meth:`backward_specs`.
    """

    name: str = "op"
    group: str = "other"   # slot vocabulary: norm | linear | rope | attn | activation
    in_channels: Tuple[str, ...] = ("main",)
    out_channels: Tuple[str, ...] = ("main",)
    no_grad_inputs: Tuple[str, ...] = ()

    def forward(self, ctx, *inputs):
        raise NotImplementedError

    def backward(self, ctx, *grad_outputs):
        raise NotImplementedError

    # graph declaration ------------------------------------------------------
    def forward_specs(self) -> List[object]:
        return [ComputeSpec(self, tuple(self.in_channels), tuple(self.out_channels))]

    def backward_specs(self) -> List[object]:
        gin = tuple(grad_channel(c) for c in self.out_channels)
        gout = tuple(grad_channel(c) for c in self.in_channels if c not in self.no_grad_inputs)
        return [ComputeSpec(self, gin, gout, backward=True)]

    def parameters(self) -> List[object]:
        return []


class TensorGraph:
    def __init__(self, nodes: List[Node], initial: Dict[str, str], final: Dict[str, str]):
        self.nodes = nodes
        self.initial = dict(initial)   # channel -> external tensor id
        self.final = dict(final)       # channel -> tensor id holding the graph's result

    def compute_nodes(self) -> List[Node]:
        return [n for n in self.nodes if not n.is_comm]

    def comm_nodes(self) -> List[Node]:
        return [n for n in self.nodes if n.is_comm]

    def validate(self) -> None:
        """Every input port must have been produced earlier or be external."""
        known = set(self.initial.values())
        for n in self.nodes:
            for p in n.inputs:
                if p.tensor_id not in known:
                    raise RuntimeError(f"node {n.index} ({n.name}) reads {p.tensor_id} on channel "
                                       f"{p.channel!r} before it is produced")
            for p in n.outputs:
                known.add(p.tensor_id)


class TensorGraphBuilder:
    def __init__(self):
        self._nodes: List[Node] = []
        self._current: Dict[str, str] = {}
        self._initial: Dict[str, str] = {}
        self._next_tensor = 0

    def add_initial_channels(self, mapping: Dict[str, str]) -> None:
        for ch, tid in mapping.items():
            self._current[ch] = tid
            self._initial[ch] = tid

    def _new_tensor(self) -> str:
        tid = f"t_{self._next_tensor}"
        self._next_tensor += 1
        return tid

    def _read(self, ch: str, who: str) -> Port:
        if ch not in self._current:
            raise KeyError(f"{who}: channel {ch!r} has no producer; live channels: {sorted(self._current)}")
        return Port(ch, self._current[ch])

    def add(self, spec) -> Node:
        who = getattr(spec.operator, "name", type(spec.operator).__name__)
        ins = tuple(self._read(c, who) for c in spec.in_channels)
        outs = []
        for c in spec.out_channels:
            tid = self._new_tensor()
            self._current[c] = tid
            outs.append(Port(c, tid))
        is_comm = isinstance(spec, CommSpec)
        node = Node(index=len(self._nodes), op_id=operator_uid(spec.operator), operator=spec.operator, inputs=ins,
                    outputs=tuple(outs), is_comm=is_comm, kind=getattr(spec, "kind", None),
                    key=getattr(spec, "key", ""), backward=spec.backward,
                    segment=getattr(spec, "segment", ""), short=getattr(spec, "short", ""))
        self._nodes.append(node)
        return node

    def build(self) -> TensorGraph:
        g = TensorGraph(self._nodes, self._initial, dict(self._current))
        g.validate()
        return g


def build_graphs(operators: Sequence[GraphOperator],
                 forward_inputs: Dict[str, str], backward_inputs: Dict[str, str]
                 ) -> Tuple[TensorGraph, TensorGraph]:
    """Forward graph over ``operators`` and the mirrored backward graph.

    A compute node's ``op_id`` is the operator's process-wide uid, so the forward and backward
    nodes of one operator (in this graph or in a graph over a sub-range of the same operators)
    find the same saved context.
    """
    fb = TensorGraphBuilder()
    fb.add_initial_channels(forward_inputs)
    for op in operators:
        for spec in op.forward_specs():
            fb.add(spec)
    bb = TensorGraphBuilder()
    bb.add_initial_channels(backward_inputs)
    for op in reversed(list(operators)):
        for spec in op.backward_specs():
            bb.add(spec)
    return fb.build(), bb.build()
