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
  (``recompute_layers = num_layers`` reproduces the reference's whole-block recompute);
* launch lists: with recompute on, the no-grad forward pass and every chunk's recompute+backward
  pass are self-contained regions whose launches repeat from microbatch to microbatch.  The first
  time a region is seen it runs as usual (lazy buffers get created), the second time its launches
  are recorded (:mod:`kareus_b200.kernels.replay`), afterwards the recorded list is replayed from
  C++ with the new inputs copied into the recorded input buffers.  ``KAREUS_REPLAY=0`` switches it
  off.  Regions with operators that launch work outside this library (NCCL collectives, context
  parallel attention, dropout with per-call seeds, qk-norm) always run through the interpreter.
"""
from __future__ import annotations

import os
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


def replay_safe(op) -> bool:
    """True for operators whose every GPU launch goes through this library's recordable entry points
    with arguments that do not change between calls (apart from channel epochs)."""
    from ..ops.attention import AttentionOp, QKVPostOp, RotaryOp
    from ..ops.basic import DropoutAddOp, RMSNormOp, ResidualFork, SwiGLUOp
    from ..ops.fused import _FusedBase
    from ..ops.linear import _LinearBase
    if isinstance(op, (ResidualFork, RMSNormOp, SwiGLUOp, RotaryOp, _LinearBase, _FusedBase)):
        return True
    if isinstance(op, DropoutAddOp):
        return op.p == 0.0 or not op.training
    if isinstance(op, QKVPostOp):
        return not op.qk_norm
    if isinstance(op, AttentionOp):
        return op.cp == 1 and op.seq_nano <= 1
    return False


class _Recorded:
    """A recorded region: its launch list, the input buffers baked into it and its output tensors."""

    __slots__ = ("lst", "static_in", "outs")

    def __init__(self, lst, static_in, outs):
        self.lst, self.static_in, self.outs = lst, static_in, outs


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
        self.replay = os.environ.get("KAREUS_REPLAY", "1") != "0"
        self._recorded: Dict[tuple, _Recorded] = {}
        self._seen: Dict[tuple, int] = {}
        self._pool = None
        self._static_ok: Optional[bool] = None
        self.replayed_regions = 0
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

    # ------------------------------------------------------------------ launch lists
    def can_replay(self, inputs, rotary) -> bool:
        if not (self.replay and self.recompute) or self.seq_split or isinstance(rotary, (list, tuple)):
            return False
        x = inputs[0]
        if not (x.is_cuda and x.dtype == torch.bfloat16):
            return False
        from .. import kernels as K
        if K.library_baseline():         # cuBLAS / flash-attention launches are invisible to a recording
            return False
        from ..ops.basic import DropoutAddOp
        if self._static_ok is None:
            self._static_ok = all(isinstance(n.operator, DropoutAddOp) or replay_safe(n.operator)
                                  for g in (self.full.fwd_graph, self.full.bwd_graph) for n in g.nodes)
        return self._static_ok and all(replay_safe(op) for ops in self.layers for op in ops
                                       if isinstance(op, DropoutAddOp))

    def _region_key(self, tag, programs, inputs, rotary) -> tuple:
        sch = self.current_schedule()
        sk = None
        if sch is not None:
            keys = sorted({k for p in programs for k in p.expected_keys()})
            sk = tuple((k, None if sch.get(k) is None else (sch.get(k).start, tuple(sch.get(k).resource_shape)))
                       for k in keys)
        return (tag, tuple(tuple(x.shape) for x in inputs), rotary.data_ptr() if rotary is not None else 0, sk,
                tuple(self.default_shape))

    def run_region(self, key: tuple, inputs: Sequence[torch.Tensor], fn) -> List[torch.Tensor]:
        """Run ``fn(inputs) -> outputs`` as a replayable region (see the module docstring).  The returned
        tensors are the caller's own (copies of the list's output buffers when replaying)."""
        rec = self._recorded.get(key)
        if rec is not None:
            for s, x in zip(rec.static_in, inputs):
                if s.data_ptr() != x.data_ptr():
                    s.copy_(x)
            rec.lst.replay()
            self.replayed_regions += 1
            return [o.clone() for o in rec.outs]
        seen = self._seen.get(key, 0)
        self._seen[key] = seen + 1
        if seen == 0:
            return list(fn(list(inputs)))
        from ..kernels import replay as R
        if self._pool is None:
            self._pool = torch.cuda.MemPool()
        with torch.cuda.use_mem_pool(self._pool):
            static_in = [torch.empty(x.shape, dtype=x.dtype, device=x.device) for x in inputs]
            for s, x in zip(static_in, inputs):
                s.copy_(x)
            with R.Recording() as r:
                outs = list(fn(static_in))
            self._recorded[key] = _Recorded(r.result, static_in, outs)
        return [o.clone() for o in outs]

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
            from .program import _per_nb_streams, _shared_comm_stream, wait_stream
            if _per_nb_streams():       # weight-gradient GEMMs funnelled through the ordered side stream
                wait_stream(torch.cuda.current_stream(grads[0].device), _shared_comm_stream(grads[0].device, 0))
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
            inner = [b for b in engine._boundary_ids if b != "ext_main"]

            def region(xs):
                ctxs = engine.run_forward(engine.full, xs, rotary, grad_enabled=False)
                res = [c.store.get(final_id) for c in ctxs]
                res += [c.store.get(bid) for bid in inner for c in ctxs]
                for c in ctxs:
                    c.reset()
                return res

            fctx.replay = engine.can_replay(inputs, rotary)
            if fctx.replay:
                res = engine.run_region(engine._region_key("fwd", [engine.full.fwd], inputs, rotary), inputs, region)
            else:
                res = region(list(inputs))
            outs = tuple(res[:n])
            if grad_enabled:
                saved, k = [], n
                for bid in engine._boundary_ids:
                    if bid == "ext_main":
                        saved += list(inputs)
                    else:
                        saved += res[k:k + n]
                        k += n
                fctx.save_for_backward(*saved)
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

            def region(ts, chunk=chunk):
                ctxs = engine.run_forward(chunk, ts[:n], fctx.rotary, grad_enabled=True)
                dins = engine.run_backward(chunk, ctxs, ts[n:])
                for c in ctxs:
                    c.reset()
                return dins

            both = list(xs) + list(cur)
            if getattr(fctx, "replay", False):
                key = engine._region_key(("bwd", ci), [chunk.fwd, chunk.bwd], both, fctx.rotary)
                cur = engine.run_region(key, both, region)
            else:
                cur = region(both)
        return (None, None, None) + tuple(cur)
