"""Training step driver: the framework's public entry point for running iterations.

``Trainer.train_step(batch)`` takes one global-batch share for this data-parallel rank as pinned
host tensors ``tokens, labels, loss_mask [n_micro * mbs, s]``, copies it to the device, runs all
microbatches through the (pipeline) schedule with the per-instruction hooks, reduces gradients,
applies AdamW and returns the loss as a host float.  It is the counterpart of the reference's
``MegatronGPTModel.training_step`` (``kareus/nemo/collections/nlp/models/language_modeling/
megatron_gpt_model.py:599-846``) without NeMo/Lightning: the hook order is the same —
``on_step_begin``; per instruction ``on_instruction_begin/end("forward"|"backward")`` for the
frequency client first and the comm scheduler second; the ``training_step_fwd_bwd_step_call``
energy window around forward/backward; ``on_step_end``.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..config import ModelConfig, ParallelConfig, TrainConfig
from ..models.llama import GPTModel
from ..parallel.collectives import CommFactory
from ..parallel.mesh import Mesh
from ..parallel.pipeline import P2P, PipelineSchedule, one_f_one_b_order
from .optimizer import DistributedAdamW

FWD_BWD_WINDOW = "training_step_fwd_bwd_step_call"
STEP_WINDOW = "training_step"


def stage_layer_range(cfg: ModelConfig, pp: int, pp_rank: int) -> range:
    """Layers of a pipeline stage; ``num_layers_in_first_pipeline_stage`` gives the uneven split the
    reference ships (15/13 of 28: the last stage also carries the head and the loss)."""
    L = cfg.num_layers
    if pp == 1:
        return range(L)
    first = cfg.num_layers_in_first_pipeline_stage
    if first is None or pp != 2:
        per = (L + pp - 1) // pp
        return range(min(L, pp_rank * per), min(L, (pp_rank + 1) * per))
    return range(0, first) if pp_rank == 0 else range(first, L)


class Trainer:
    def __init__(self, model_cfg: ModelConfig, par: ParallelConfig, train_cfg: TrainConfig,
                 mesh: Optional[Mesh] = None, device=None, dtype: Optional[str] = None,
                 monitor=None, freq_client=None, comm_scheduler=None, heap=None, heap_cp=None,
                 recompute_layers: Optional[int] = None, sync: str = "partition_end"):
        self.model_cfg, self.par, self.cfg = model_cfg, par, train_cfg
        self.mesh = mesh or Mesh(par.tp, par.cp, par.dp, par.pp)
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.dtype = dtype or train_cfg.dtype
        self.monitor, self.freq_client, self.comm_scheduler = monitor, freq_client, comm_scheduler
        mesh = self.mesh
        comm = CommFactory(mesh, par.comm_backend, heap=heap, heap_cp=heap_cp)
        self.model = GPTModel(model_cfg, par, mesh=mesh, comm=comm, dtype=self.dtype, device=self.device,
                              seed=train_cfg.seed, pre_process=mesh.is_first_stage,
                              post_process=mesh.is_last_stage,
                              layer_range=stage_layer_range(model_cfg, mesh.pp, mesh.pp_rank),
                              recompute_layers=recompute_layers, sync=sync,
                              micro_batch_size=train_cfg.micro_batch_size)
        if comm_scheduler is not None:
            self.model.decoder.set_scheduler(comm_scheduler)
        mp_group = mesh.group("tp_pp") if mesh.size("tp_pp") > 1 else None
        self.optimizer = DistributedAdamW(self.model.parameters(), train_cfg, dp_group=mesh.group("dp_cp"),
                                          dp_size=mesh.size("dp_cp"), dp_rank=mesh.axis_rank("dp_cp"),
                                          mp_group=mp_group, tp_rank=mesh.tp_rank)
        self.num_microbatches = train_cfg.num_microbatches(par.dp)
        self.p2p: Optional[P2P] = None
        self.step_index = 0
        self._hooks = [h for h in (freq_client, comm_scheduler) if h is not None]

    # ------------------------------------------------------------------ helpers
    def _msg_shapes(self, mbs: int, s_local: int):
        n = self.par.num_nanobatches
        s = s_local // self.par.tp if self.par.sequence_parallel else s_local
        if self.model.seq_split:
            return [(s // n, mbs, self.model_cfg.hidden_size)] * n
        return [(s, mbs // n, self.model_cfg.hidden_size)] * n

    def instruction_order(self) -> List[str]:
        return [k for k, _ in one_f_one_b_order(self.mesh.pp, self.mesh.pp_rank, self.num_microbatches)]

    def to_device(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        if self.device.type != "cuda":
            return batch
        return {k: v.to(self.device, non_blocking=True) for k, v in batch.items()}

    # ------------------------------------------------------------------ step
    def forward_backward(self, batch: Dict[str, torch.Tensor], loss_denominator: float,
                         forward_only: bool = False) -> torch.Tensor:
        """All microbatches of one step; returns the summed loss (device scalar; 0 off the last stage).
        ``forward_only``: no backward pass (evaluation; the caller disables autograd)."""
        mesh, M = self.mesh, self.num_microbatches
        mbs = self.cfg.micro_batch_size
        tokens, labels, mask = batch["tokens"], batch["labels"], batch["loss_mask"]

        def mb_slice(t, i):
            return t[i * mbs:(i + 1) * mbs]

        def forward_fn(mb, inputs):
            if mesh.is_last_stage:
                return self.model(tokens=mb_slice(tokens, mb) if mesh.is_first_stage else None,
                                  labels=mb_slice(labels, mb), loss_mask=mb_slice(mask, mb), hidden=inputs,
                                  loss_denominator=loss_denominator)
            return self.model(tokens=mb_slice(tokens, mb) if mesh.is_first_stage else None, hidden=inputs)

        if mesh.pp > 1 and self.p2p is None:
            dt = next(self.model.parameters()).dtype
            self.p2p = P2P(mesh, self._msg_shapes(mbs, tokens.shape[1]), dt, self.device)
        sched = PipelineSchedule(mesh, self.p2p, forward_fn, hooks=() if forward_only else self._hooks)
        losses = sched.run_forward_only(M) if forward_only else sched.run(M)
        if losses:
            return torch.stack(losses).sum()
        return torch.zeros((), device=self.device)

    def train_step(self, batch: Dict[str, torch.Tensor], loss_denominator: Optional[float] = None,
                   return_loss: bool = True):
        for h in self._hooks:
            h.on_step_begin()
        if self.monitor is not None:
            self.monitor.begin_window(STEP_WINDOW)
        if loss_denominator is None:
            # tokens that count, over the whole global batch (host-side: the mask is a host tensor)
            loss_denominator = float(batch["loss_mask"].sum()) * self.par.dp * self.par.cp
        dev_batch = self.to_device(batch)
        self.optimizer.zero_grad()
        if self.monitor is not None:
            self.monitor.begin_window(FWD_BWD_WINDOW)
        loss = self.forward_backward(dev_batch, loss_denominator)
        if self.monitor is not None:
            self.monitor.end_window(FWD_BWD_WINDOW)
        self.model.finalize_grads()
        self.optimizer.step()
        for h in self._hooks:
            h.on_step_end()
        out = None
        if return_loss:
            out = self.reduce_loss(loss)
        if self.monitor is not None:
            self.monitor.end_window(STEP_WINDOW)
        self.step_index += 1
        return out

    @torch.no_grad()
    def evaluate(self, batch: Dict[str, torch.Tensor], loss_denominator: Optional[float] = None) -> float:
        """Mean loss of one global batch without touching gradients, optimizer state or the step count (the
        reference's validation pass: ``trainer.val_check_interval`` / ``limit_val_batches`` of its run
        configs).  Same batch layout and the same value on every rank as ``train_step``."""
        if loss_denominator is None:
            loss_denominator = float(batch["loss_mask"].sum()) * self.par.dp * self.par.cp
        was_training = self.model.training
        self.model.eval()
        try:
            loss = self.forward_backward(self.to_device(batch), loss_denominator, forward_only=True)
        finally:
            self.model.train(was_training)
        return self.reduce_loss(loss)

    # ------------------------------------------------------------------ checkpoint
    def save_checkpoint(self, ckpt_dir, common: Optional[dict] = None) -> None:
        """Collective over all ranks: model and optimizer state in the Megatron distributed-checkpoint
        layout (reshardable), plus the step index."""
        from ..models import checkpoint as ck
        mesh = self.mesh
        c = dict(common or {})
        c["iteration"] = self.step_index
        ck.save(self.model, ckpt_dir, rank=mesh.rank, tp_rank=mesh.tp_rank, tp=mesh.tp,
                dp_rank=mesh.axis_rank("dp_cp"), common=c, optimizer=self.optimizer)

    def load_checkpoint(self, ckpt_dir, strict: bool = True) -> dict:
        """Resume from a checkpoint written under any TP x PP x DP layout."""
        from ..models import checkpoint as ck
        mesh = self.mesh
        common = ck.load(self.model, ckpt_dir, tp_rank=mesh.tp_rank, tp=mesh.tp, strict=strict,
                         optimizer=self.optimizer, dp_rank=mesh.axis_rank("dp_cp"))
        self.step_index = int(common.get("iteration", 0))
        return common

    def reduce_loss(self, loss: torch.Tensor) -> float:
        """Global mean token loss on every rank (sum over dp×cp shares; broadcast from the last stage)."""
        mesh = self.mesh
        t = loss.detach().to(torch.float32).reshape(1).clone()
        if mesh.size("dp_cp") > 1:
            dist.all_reduce(t, group=mesh.group("dp_cp"))
        if mesh.pp > 1:
            src = mesh.rank_of(mesh.tp_rank, mesh.cp_rank, mesh.dp_rank, mesh.pp - 1)
            dist.broadcast(t, src=src, group=mesh.group("pp"))
        return float(t.item())


def synthetic_batch(model_cfg: ModelConfig, train_cfg: TrainConfig, num_microbatches: int, seed: int = 0,
                    pin: bool = True, cp: int = 1, cp_rank: int = 0) -> Dict[str, torch.Tensor]:
    """Uniform-random tokens and labels for one step of one data-parallel rank (host tensors)."""
    g = torch.Generator().manual_seed(seed)
    n = num_microbatches * train_cfg.micro_batch_size
    s = train_cfg.seq_len
    tokens = torch.randint(0, model_cfg.vocab_size, (n, s), generator=g, dtype=torch.int64)
    labels = torch.randint(0, model_cfg.vocab_size, (n, s), generator=g, dtype=torch.int64)
    mask = torch.ones(n, s, dtype=torch.float32)
    if cp > 1:
        from ..parallel.collectives import dual_chunk_ids
        c = s // (2 * cp)
        a, b = dual_chunk_ids(cp, cp_rank)
        idx = torch.cat([torch.arange(a * c, (a + 1) * c), torch.arange(b * c, (b + 1) * c)])
        tokens, labels, mask = tokens[:, idx].contiguous(), labels[:, idx].contiguous(), mask[:, idx].contiguous()
    out = {"tokens": tokens, "labels": labels, "loss_mask": mask}
    if pin and torch.cuda.is_available():
        out = {k: v.pin_memory() for k, v in out.items()}
    return out
