"""Block engine: one autograd boundary around all layers × partitions × nanobatches.

``BlockEngine`` owns the forward/backward tensor graphs and partition programs of a stack of
transformer layers and runs them behind a single ``torch.autograd.Function`` (the reference's
``TransformerBlockAutogradFunction``, ``kareus/megatron/core/partitions/autograd_function.py:
98-372``).  Differences:

* any number of nanobatches (1, 2 or 4) instead of exactly two;
* parameter gradients accumulate into ``param.main_grad`` inside the backward operators, so
  parameters are not passed through autograd (the reference passes every parameter twice);
* activation recompute works on *chunks* of layers: the first pass runs the whole block without
  saving and keeps only each chunk's input; backward re-runs one chunk's forward program and
  then its backward program, so live activations are one chunk instead of the whole block
  (``recompute_layers = num_layers`` reproduces the reference's whole-block recompute).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .context import NanoBatchContext
from .graph import GraphOperator, TensorGraph, build_graphs
from .program import PartitionProgram, StreamSet

FWD_INPUTS = {"main": "ext_main", "rotary_pos_emb": "ext_rotary_pos_emb"}
BWD_INPUTS = {"grad_main": "ext_grad_main"}


class _Chunk:
    def __init__(self, operators: Sequence[GraphOperator], n: int, sync: str, seq_split: bool = False,
                 cp_keys: bool = False):
        self.operators = list(operators)
        self.fwd_graph, self.bwd_graph = build_graphs(self.operators, FWD_INPUTS, BWD_INPUTS)
        self.fwd = PartitionProgram(self.fwd_graph, n, backward=False, sync=sync, cp_keys=cp_keys)
        self.bwd = PartitionProgram(self.bwd_graph, n, backward=True, sync=sync, reverse_nb=seq_split,
                                    cp_keys=cp_keys)


class BlockEngine:
    def __init__(self, layer_operators: Sequence[Sequence[GraphOperator]], num_nanobatches: int = 2,
                 recompute: bool = True, recompute_layers: Optional[int] = None,
                 sync: str = "partition_end", scheduler=None, seq_split: bool = False, cp_keys: bool = False):
        self.layers = [list(ops) for ops in layer_operators]
        self.n = int(num_nanobatches)
        self.recompute = bool(recompute)
        self.sync = sync
        self.scheduler = scheduler
        self.default_shape: Tuple[Optional[int], Optional[int]] = (None, None)
        L = len(self.layers)
        self.recompute_layers = L if recompute_layers is None else max(1, min(int(recompute_layers), L))
        all_ops = [op for ops in self.layers for op in ops]
        self.seq_split = seq_split
        self.full = _Chunk(all_ops, self.n, sync, seq_split, cp_keys)
        self.chunks: List[_Chunk] = []
        self._boundary_ids: List[str] = []
        if self.recompute and self.recompute_layers < L:
            bounds = list(range(0, L, self.recompute_layers))
            for s in bounds:
                ops = [op for l in self.layers[s:s + self.recompute_layers] for op in l]
                self.chunks.append(_Chunk(ops, self.n, sync, seq_split, cp_keys))
            # tensor ids of the full forward graph that enter each chunk
            first_nodes = {id(c.operators[0]): i for i, c in enumerate(self.chunks)}
            ids: Dict[int, str] = {}
            for node in self.full.fwd_graph.nodes:
                ci = first_nodes.get(id(node.operator))
                if ci is not None and not node.is_comm and ci not in ids:
                    ids[ci] = next(p.tensor_id for p in node.inputs if p.channel == "main")
            self._boundary_ids = [ids[i] for i in range(len(self.chunks))]
            self.full.fwd.keep_ids |= set(self._boundary_ids)
        else:
            self.chunks = [self.full]
            self._boundary_ids = ["ext_main"]

    # ------------------------------------------------------------------ helpers
    def current_schedule(self):
        return self.scheduler.current_schedule if self.scheduler is not None else None

    def _streams(self, t: torch.Tensor) -> StreamSet:
        return StreamSet(t.device if t.is_cuda else None)

    def _seed(self, ctxs, inputs, rotary, graph: TensorGraph, channel_map) -> None:
        for i, (c, x) in enumerate(zip(ctxs, inputs)):
            c.store.put(graph.initial[channel_map], x)
            if rotary is not None and "rotary_pos_emb" in graph.initial:
                # one table for all nanobatches, or one per nanobatch (sequence-split nanobatches)
                c.store.put(graph.initial["rotary_pos_emb"], rotary[i] if isinstance(rotary, (list, tuple)) else rotary)

    def run_forward(self, chunk: _Chunk, inputs, rotary, grad_enabled: bool, ctxs=None):
        ctxs = ctxs or [NanoBatchContext(i) for i in range(self.n)]
        self._seed(ctxs, inputs, rotary, chunk.fwd_graph, "main")
        chunk.fwd.run(ctxs, schedule=self.current_schedule(), streams=self._streams(inputs[0]),
                      grad_enabled=grad_enabled, default_shape=self.default_shape)
        return ctxs

    def run_backward(self, chunk: _Chunk, ctxs, grads):
        for c, g in zip(ctxs, grads):
            c.store.clear()
            c.ready_event.clear()
            c.store.put(chunk.bwd_graph.initial["grad_main"], g)
        chunk.bwd.run(ctxs, schedule=self.current_schedule(), streams=self._streams(grads[0]),
                      default_shape=self.default_shape)
        if grads[0].is_cuda:
            from .program import _per_nb_streams, _shared_comm_stream
            if _per_nb_streams():       # weight-gradient GEMMs funnelled through the ordered side stream
                torch.cuda.current_stream(grads[0].device).wait_stream(_shared_comm_stream(grads[0].device, 0))
        out_id = chunk.bwd_graph.final["grad_main"]
        return [c.store.get(out_id) for c in ctxs]

    # ------------------------------------------------------------------ public
    def __call__(self, inputs: Sequence[torch.Tensor], rotary: Optional[torch.Tensor]) -> List[torch.Tensor]:
        if len(inputs) != self.n:
            raise ValueError(f"expected {self.n} nanobatch tensors, got {len(inputs)}")
        outs = _BlockFunction.apply(self, rotary, torch.is_grad_enabled(), *inputs)
        return list(outs)


class _BlockFunction(torch.autograd.Function):
    @staticmethod
    def forward(fctx, engine: BlockEngine, rotary, grad_enabled: bool, *inputs):
        fctx.engine = engine
        fctx.rotary = rotary
        n = engine.n
        final_id = engine.full.fwd_graph.final["main"]
        if engine.recompute or not grad_enabled:
            ctxs = engine.run_forward(engine.full, inputs, rotary, grad_enabled=False)
            outs = tuple(c.store.get(final_id) for c in ctxs)
            if grad_enabled:
                saved = []
                for bid in engine._boundary_ids:
                    for i, c in enumerate(ctxs):
                        saved.append(inputs[i] if bid == "ext_main" else c.store.get(bid))
                fctx.save_for_backward(*saved)
            for c in ctxs:
                c.reset()
            fctx.ctxs = None
        else:
            ctxs = engine.run_forward(engine.full, inputs, rotary, grad_enabled=True)
            outs = tuple(c.store.get(final_id) for c in ctxs)
            for c in ctxs:
                c.store.clear()
            fctx.ctxs = ctxs
        return outs

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(fctx, *grads):
        engine: BlockEngine = fctx.engine
        n = engine.n
        grads = [g.contiguous() for g in grads]
        if fctx.ctxs is not None:
            dins = engine.run_backward(engine.full, fctx.ctxs, grads)
            for c in fctx.ctxs:
                c.reset()
            fctx.ctxs = None
            return (None, None, None) + tuple(dins)
        saved = fctx.saved_tensors
        cur = grads
        for ci in range(len(engine.chunks) - 1, -1, -1):
            chunk = engine.chunks[ci]
            xs = saved[ci * n:(ci + 1) * n]
            ctxs = engine.run_forward(chunk, xs, fctx.rotary, grad_enabled=True)
            cur = engine.run_backward(chunk, ctxs, cur)
            for c in ctxs:
                c.reset()
        return (None, None, None) + tuple(cur)
