"""Distributed AdamW over flat buffers (ZeRO-1 style) with fp32 master weights.

All parameters of a model stage are re-homed into one contiguous bf16 buffer and their
``main_grad`` into one contiguous fp32 buffer, so that zeroing gradients is one memset, the
gradient norm one reduction kernel and the AdamW update ONE launch over the shard this data-
parallel rank owns.  With ``dp > 1`` gradients are reduce-scattered and updated parameters
all-gathered over the data-parallel group in the flat space (the reference relies on Megatron's
``DistributedDataParallel`` + ``DistributedOptimizer`` for the same dataflow:
``3rdparty/Megatron-LM/megatron/core/distributed/param_and_grad_buffer.py:356-388``,
``megatron/core/optimizer/distrib_optimizer.py``; AdamW hyper-parameters from
``tests/artifact/conf/megatron_llama3.2_3b_config.yaml:180-191``).
"""
from __future__ import annotations

import math
from typing import Iterable, List, Optional

import torch
import torch.distributed as dist

from .. import kernels as K
from ..config import TrainConfig

_ALIGN = 128  # elements; keeps every parameter 256-byte aligned in the bf16 buffer


def cosine_lr(step: int, cfg: TrainConfig) -> float:
    if step < cfg.warmup_steps:
        return cfg.lr * (step + 1) / max(1, cfg.warmup_steps)
    t = min(1.0, (step - cfg.warmup_steps) / max(1, cfg.max_steps - cfg.warmup_steps))
    return cfg.min_lr + 0.5 * (cfg.lr - cfg.min_lr) * (1.0 + math.cos(math.pi * t))


class DistributedAdamW:
    def __init__(self, params: Iterable[torch.nn.Parameter], cfg: TrainConfig, dp_group=None, dp_size: int = 1,
                 dp_rank: int = 0, mp_group=None, tp_rank: int = 0):
        self.cfg = cfg
        self.dp_group, self.dp, self.dp_rank = dp_group, int(dp_size), int(dp_rank)
        self.mp_group, self.tp_rank = mp_group, tp_rank
        seen, plist = set(), []
        for p in params:
            if id(p) not in seen and p.requires_grad:
                seen.add(id(p))
                plist.append(p)
        # TP-replicated parameters (norm weights) go last so their norm can be counted once
        def replicated(p):
            return p.dim() == 1
        self.params: List[torch.nn.Parameter] = [p for p in plist if not replicated(p)] + \
                                                [p for p in plist if replicated(p)]
        if not self.params:
            raise ValueError("no parameters")
        dev, dt = self.params[0].device, self.params[0].dtype
        self.offsets, o = [], 0
        self.replicated_start = None
        # flat ranges left out of the gradient norm (second copy of a weight tied across stages)
        self.norm_exclude = []
        for p in self.params:
            if getattr(p, "norm_exclude", False):
                self.norm_exclude.append((o, o + p.numel()))
            if replicated(p) and self.replicated_start is None:
                self.replicated_start = o
            self.offsets.append(o)
            o += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        if self.replicated_start is None:
            self.replicated_start = o
        chunk = _ALIGN * self.dp
        self.total = (o + chunk - 1) // chunk * chunk
        acc = torch.float64 if dt == torch.float64 else torch.float32
        self.param_flat = torch.zeros(self.total, dtype=dt, device=dev)
        self.grad_flat = torch.zeros(self.total, dtype=acc, device=dev)
        for p, off in zip(self.params, self.offsets):
            n = p.numel()
            self.param_flat[off:off + n].copy_(p.data.reshape(-1))
            p.data = self.param_flat[off:off + n].view(p.shape)
            old = getattr(p, "main_grad", None)
            p.main_grad = self.grad_flat[off:off + n].view(p.shape)
            if old is not None:
                p.main_grad.copy_(old)
        self.shard = self.total // self.dp
        lo = self.dp_rank * self.shard
        self.lo, self.hi = lo, lo + self.shard
        self.master = self.param_flat[lo:lo + self.shard].to(acc).clone()
        self.m = torch.zeros(self.shard, dtype=acc, device=dev)
        self.v = torch.zeros(self.shard, dtype=acc, device=dev)
        self.grad_shard = self.grad_flat[lo:lo + self.shard] if self.dp == 1 else \
            torch.empty(self.shard, dtype=acc, device=dev)
        self.step_count = 0
        self.last_grad_norm: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------
    def zero_grad(self) -> None:
        self.grad_flat.zero_()
        for p in self.params:
            p.grad = None

    def _reduce_grads(self) -> torch.Tensor:
        """Sum over the data(+context)-parallel group: the loss is already divided by the global
        token count, so shares add up."""
        if self.dp == 1:
            return self.grad_flat
        if self.grad_flat.is_cuda:
            dist.reduce_scatter_tensor(self.grad_shard, self.grad_flat, op=dist.ReduceOp.SUM, group=self.dp_group)
        else:
            dist.all_reduce(self.grad_flat, group=self.dp_group)
            self.grad_shard.copy_(self.grad_flat[self.lo:self.hi])
        return self.grad_shard

    def _grad_norm(self, g: torch.Tensor) -> torch.Tensor:
        """Global L2 norm: every element counted once across tp × pp × dp-shards."""
        total = K.sumsq(g)
        if self.tp_rank != 0:
            a, b = max(self.replicated_start, self.lo), self.hi
            if b > a:
                total = total - K.sumsq(g[a - self.lo:b - self.lo] if self.dp > 1 else self.grad_flat[a:b])
        for a0, b0 in self.norm_exclude:
            a, b = max(a0, self.lo), min(b0, self.hi)
            if b > a:
                total = total - K.sumsq(g[a - self.lo:b - self.lo] if self.dp > 1 else self.grad_flat[a:b])
        total = total.reshape(1).clone()
        if self.dp > 1:
            dist.all_reduce(total, group=self.dp_group)
        if self.mp_group is not None:
            dist.all_reduce(total, group=self.mp_group)
        return total.sqrt()[0]

    def step(self, lr: Optional[float] = None) -> torch.Tensor:
        """Reduce, clip, update.  Returns the gradient norm as a device scalar (no host sync)."""
        cfg = self.cfg
        g = self._reduce_grads()
        norm = self._grad_norm(g)
        self.last_grad_norm = norm
        scale_t = None
        if cfg.grad_clip and cfg.grad_clip > 0:
            scale_t = torch.clamp(cfg.grad_clip / (norm + 1e-6), max=1.0).to(torch.float32).reshape(1)
        self.step_count += 1
        lr = cosine_lr(self.step_count - 1, cfg) if lr is None else lr
        p_shard = self.param_flat[self.lo:self.hi]
        if g.is_cuda and g.dtype == torch.float32:
            from ..kernels import cuda as KC
            KC.adamw_step(p_shard, g, self.m, self.v, self.master, lr, cfg.betas[0], cfg.betas[1], cfg.eps,
                          cfg.weight_decay, self.step_count, 1.0, grad_scale_tensor=scale_t)
        else:
            gs = float(scale_t.item()) if scale_t is not None else 1.0
            K.ref.adamw_step(p_shard, g, self.m, self.v, self.master, lr, cfg.betas[0], cfg.betas[1], cfg.eps,
                             cfg.weight_decay, self.step_count, gs)
        if self.dp > 1:
            dist.all_gather_into_tensor(self.param_flat, p_shard.clone(), group=self.dp_group)
        return norm

    # ------------------------------------------------------------------ checkpoint
    def gather_state(self) -> dict:
        """Full-length flat AdamW state ``{exp_avg, exp_avg_sq, fp32_param}`` (length ``total``) on every
        rank: the data-parallel shards all-gathered.  Collective over the data-parallel group."""
        out = {}
        for name, t in (("exp_avg", self.m), ("exp_avg_sq", self.v), ("fp32_param", self.master)):
            if self.dp == 1:
                out[name] = t
            else:
                full = torch.empty(self.total, dtype=t.dtype, device=t.device)
                dist.all_gather_into_tensor(full, t.contiguous(), group=self.dp_group)
                out[name] = full
        return out

    def empty_full_state(self) -> dict:
        """Destination buffers for :meth:`scatter_state` (a checkpoint loader fills them in model space)."""
        return {name: torch.zeros(self.total, dtype=self.master.dtype, device=self.master.device)
                for name in ("exp_avg", "exp_avg_sq", "fp32_param")}

    def scatter_state(self, full: dict, step: int) -> None:
        """Take this data-parallel rank's shard of full-length state and refresh the parameters from the
        fp32 master values."""
        self.m.copy_(full["exp_avg"][self.lo:self.hi])
        self.v.copy_(full["exp_avg_sq"][self.lo:self.hi])
        self.master.copy_(full["fp32_param"][self.lo:self.hi])
        self.step_count = int(step)
        self.param_flat[self.lo:self.hi].copy_(self.master.to(self.param_flat.dtype))
        if self.dp > 1:
            dist.all_gather_into_tensor(self.param_flat, self.param_flat[self.lo:self.hi].clone(), group=self.dp_group)

    def state_dict(self) -> dict:
        return {"step": self.step_count, "master": self.master, "exp_avg": self.m, "exp_avg_sq": self.v,
                "shard": (self.lo, self.hi), "total": self.total}

    def load_state_dict(self, sd: dict) -> None:
        if tuple(sd["shard"]) != (self.lo, self.hi) or sd["total"] != self.total:
            raise ValueError("optimizer shard layout differs from the checkpoint")
        self.step_count = int(sd["step"])
        self.master.copy_(sd["master"])
        self.m.copy_(sd["exp_avg"])
        self.v.copy_(sd["exp_avg_sq"])
        self.param_flat[self.lo:self.hi].copy_(self.master.to(self.param_flat.dtype))
