"""Run ONE partition (compute of a segment for one nanobatch ‖ the collective of another) in
isolation, repeatedly, for the profiler.

The reference builds a one-partition graph from an operator list plus a physical collective and,
for backward partitions, runs a compute-only forward first to populate the saved contexts
(``tests/bayesian/common/partition_executor.py:74-318``; used by every
``tests/bayesian/partitions/*/overlap_test.py``).  Here the partition is taken out of the real
one-layer program of the engine: all steps before it run once to produce valid inputs and saved
state, then ``execute(overlap_window, (sm, block))`` re-runs just that step.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..config import ModelConfig, ParallelConfig
from ..engine.block import BWD_INPUTS, FWD_INPUTS, _Chunk
from ..engine.context import NanoBatchContext
from ..engine.program import StreamSet
from ..kernels import ref
from ..models.llama import TransformerLayer, _torch_dtype
from ..parallel.collectives import CommFactory
from ..plan.schedule import CommConfig


class _OneKeySchedule:
    def __init__(self, key: str, cfg: CommConfig):
        self.key, self.cfg = key, cfg

    def get(self, key, default=None):
        return self.cfg if key == self.key else default


class PartitionExecutor:
    def __init__(self, model_cfg: ModelConfig, par: ParallelConfig, key: str, micro_batch_size: int, seq_len: int,
                 mesh=None, comm: Optional[CommFactory] = None, device="cpu", dtype="bf16", seed: int = 0):
        self.key, self.par = key, par
        self.device = torch.device(device)
        dt = _torch_dtype(dtype)
        self.comm = comm or CommFactory(mesh, par.comm_backend)
        self.layer = TransformerLayer(model_cfg, par, self.comm, 0, dt, self.device, seed=seed)
        n = par.num_nanobatches
        # same step naming as the model's block: with tensor x context parallelism (all-reduce flavour) steps
        # carry the reference's context-parallel keys (fwd_qkv_ar, fwd_qkv_ag, fwd_ao_ag, ...)
        cp_keys = par.cp > 1 and par.tp > 1 and par.tp_comm == "allreduce"
        self.backward = key.startswith("bwd_")
        self.layers = [self.layer]
        for depth in (1, 2):
            # some steps exist only between two layers: a layer's first segment beside the collective that
            # the previous layer's last segment started (fwd_qkv_ar, bwd_o_ar of the context-parallel plan)
            if depth == 2:
                self.layers.append(TransformerLayer(model_cfg, par, self.comm, 1, dt, self.device, seed=seed + 1))
            ops = [op for l in self.layers for op in l.operators()]
            self.chunk = _Chunk(ops, n, "partition_end", cp_keys=cp_keys)
            prog = self.chunk.bwd if self.backward else self.chunk.fwd
            cands = [s for s in prog.steps if s.key == key and s.compute]
            if cands:
                break
        if not cands:
            raise KeyError(f"partition key {key!r} does not occur with tp_comm={par.tp_comm!r}, cp={par.cp}; "
                           f"program keys: {sorted(set(prog.expected_keys()))}")
        with_comm = [s for s in cands if s.comm is not None]
        self.step = (with_comm or cands)[-1]
        self.program = prog
        for pr in (self.chunk.fwd, self.chunk.bwd):
            pr.free_dead = False
        s_local = seq_len // par.cp
        s_rows = s_local // par.tp if par.sequence_parallel else s_local
        b = max(1, micro_batch_size // n)
        g = torch.Generator(device="cpu").manual_seed(seed)
        self.inputs = [torch.randn(s_rows, b, model_cfg.hidden_size, generator=g).to(dtype=dt, device=self.device)
                       for _ in range(n)]
        self.rotary = ref.rope_table(s_local, model_cfg.hd, model_cfg.rope_theta, device=self.device)
        self.streams = StreamSet(self.device if self.device.type == "cuda" else None)
        self.ctxs = [NanoBatchContext(i) for i in range(n)]
        self._prepare()

    def _seed(self, graph, tensors, channel):
        for c, x in zip(self.ctxs, tensors):
            c.store.put(graph.initial[channel], x)
            if "rotary_pos_emb" in graph.initial:
                c.store.put(graph.initial["rotary_pos_emb"], self.rotary)

    @torch.no_grad()
    def _prepare(self) -> None:
        fwd, bwd = self.chunk.fwd, self.chunk.bwd
        self._seed(self.chunk.fwd_graph, self.inputs, "main")
        if not self.backward:
            fwd.run_steps(self.ctxs, fwd.steps[: self.step.index], streams=self.streams, grad_enabled=False)
            return
        fwd.run(self.ctxs, streams=self.streams, grad_enabled=True)
        final = self.chunk.fwd_graph.final["main"]
        grads = [torch.randn_like(c.store.get(final)) for c in self.ctxs]
        for c, g in zip(self.ctxs, grads):
            c.store.clear()
            c.ready_event.clear()
            c.store.put(self.chunk.bwd_graph.initial["grad_main"], g)
        bwd.run_steps(self.ctxs, bwd.steps[: self.step.index], streams=self.streams, release_saved=False)

    @torch.no_grad()
    def execute(self, overlap_window: Tuple[str, str] = ("norm_0", "none"),
                resource_shape: Tuple[Optional[int], Optional[int]] = (16, 1024)) -> None:
        sched = _OneKeySchedule(self.key, CommConfig(tuple(overlap_window), tuple(resource_shape)))
        self.program.run_steps(self.ctxs, [self.step], schedule=sched, streams=self.streams,
                               grad_enabled=False, release_saved=False)

    def slots(self):
        return dict(self.step.slots)
