"""Graph wiring, segment/step formation for N nanobatches, slot names, tensor lifetime."""
import pytest
import torch

from kareus_b200.engine.graph import CommKind, CommSpec, ComputeSpec, GraphOperator, build_graphs
from kareus_b200.engine.program import PartitionProgram, build_overlap_slots, resolve_slot, split_segments


class Op(GraphOperator):
    def __init__(self, name, group, ins=("main",), outs=("main",), comm_after=None, comm_bwd=None):
        self.name, self.group, self.in_channels, self.out_channels = name, group, ins, outs
        self.comm_after, self.comm_bwd = comm_after, comm_bwd

    def forward(self, ctx, *xs):
        return tuple(xs[0] + 1 for _ in self.out_channels)

    def backward(self, ctx, *gs):
        return tuple(sum(gs) for _ in self.in_channels)

    def forward_specs(self):
        out = [ComputeSpec(self, tuple(self.in_channels), tuple(self.out_channels))]
        if self.comm_after:
            out.append(CommSpec(_AR(), CommKind.ALL_REDUCE, ("main",), ("main",), self.comm_after))
        return out

    def backward_specs(self):
        out = super().backward_specs()
        if self.comm_bwd:
            out.append(CommSpec(_AR(), CommKind.ALL_REDUCE, ("grad_main",), ("grad_main",), self.comm_bwd, backward=True))
        return out


class _AR:
    name = "ar"

    def run(self, tensors, **kw):
        return tensors


def layer(i):
    return [Op(f"fork{i}", "norm", outs=("main", "residual")), Op(f"norm{i}", "norm"),
            Op(f"qkv{i}", "linear", comm_bwd="bwd_attn"), Op(f"rope{i}", "rope"), Op(f"attn{i}", "attn"),
            Op(f"proj{i}", "linear", comm_after="fwd_attn"), Op(f"bda{i}", "norm", ins=("main", "residual")),
            Op(f"norm2{i}", "norm"), Op(f"fc1{i}", "linear", comm_bwd="bwd_mlp"), Op(f"act{i}", "activation"),
            Op(f"fc2{i}", "linear", comm_after="fwd_mlp"), Op(f"bda2{i}", "norm")]


def test_graph_wiring_and_backward_mirror():
    ops = layer(0)
    fwd, bwd = build_graphs(ops, {"main": "ext_main"}, {"grad_main": "ext_grad_main"})
    assert [n.name for n in fwd.nodes if n.is_comm] == ["ar", "ar"]
    bda = next(n for n in fwd.nodes if n.name == "bda0")
    fork = next(n for n in fwd.nodes if n.name == "fork0")
    assert bda.inputs[1].tensor_id == fork.outputs[1].tensor_id          # residual skips five operators
    # backward shares op ids with forward and reverses the order
    f_ids = [n.op_id for n in fwd.nodes if not n.is_comm]
    b_ids = [n.op_id for n in bwd.nodes if not n.is_comm]
    assert b_ids == f_ids[::-1]
    assert [n.key for n in bwd.nodes if n.is_comm] == ["bwd_mlp", "bwd_attn"]


@pytest.mark.parametrize("n", [1, 2, 4])
def test_step_formation(n):
    ops = layer(0) + layer(1)
    fwd, _ = build_graphs(ops, {"main": "ext_main"}, {"grad_main": "ext_grad_main"})
    prog = PartitionProgram(fwd, n, backward=False)
    segs = prog.segments
    assert [s.key for s in segs] == ["fwd_attn", "fwd_mlp", "fwd_attn", "fwd_mlp", "fwd_trail"]
    assert len(prog.steps) == len(segs) * n          # last segment has no collective → no extra step
    # the collective of (segment s, nanobatch i) is carried by the very next step
    for k, st in enumerate(prog.steps):
        if k == 0:
            assert st.comm is None
            continue
        prev = prog.steps[k - 1]
        if segs[prev.segment].comm is not None:
            assert st.comm is segs[prev.segment].comm and st.comm_nb == prev.nb and st.comm_segment == prev.segment
        else:
            assert st.comm is None
    if n == 2:   # the reference's interleaving: NB0 carries the previous segment's collective of NB1
        s = prog.steps[2]
        assert (s.segment, s.nb, s.comm_segment, s.comm_nb) == (1, 0, 0, 1)
    # reversed nanobatch order (sequence split) keeps the pairing rule
    rev = PartitionProgram(fwd, n, backward=False, reverse_nb=True)
    assert [s.nb for s in rev.steps[:n]] == list(reversed(range(n)))


def test_slots_and_resolution():
    ops = layer(0)
    fwd, _ = build_graphs(ops, {"main": "ext_main"}, {"grad_main": "ext_grad_main"})
    seg = split_segments(fwd.nodes, "fwd_trail")[0]
    slots = build_overlap_slots(seg.compute)
    assert slots == {"norm_0": 0, "linear_0": 2, "rope_0": 3, "attn_0": 4, "linear_1": 5}
    assert resolve_slot(slots, "none") == -1 and resolve_slot(slots, "first") == 0 and resolve_slot(slots, 3) == 3
    with pytest.raises(KeyError):
        resolve_slot(slots, "activation_0")
    bad = Op("weird", "mystery")
    with pytest.raises(ValueError):
        build_overlap_slots(build_graphs([bad], {"main": "ext_main"}, {"grad_main": "g"})[0].nodes)


def test_execution_frees_dead_tensors_and_matches_sequential():
    from kareus_b200.engine.context import NanoBatchContext
    ops = layer(0) + layer(1)
    fwd, _ = build_graphs(ops, {"main": "ext_main"}, {"grad_main": "ext_grad_main"})
    prog = PartitionProgram(fwd, 2, backward=False)
    ctxs = [NanoBatchContext(i) for i in range(2)]
    for i, c in enumerate(ctxs):
        c.store.put("ext_main", torch.full((2,), float(i)))
    prog.run(ctxs)
    final = fwd.final["main"]
    # every operator adds 1 on the main channel: 11 main-channel hops per layer (fork passes x+1 twice)
    assert ctxs[0].store.get(final)[0].item() == ctxs[1].store.get(final)[0].item() - 1
    assert len(ctxs[0].store) <= 3                       # external input, final output (+ maybe one live residual)
