"""Memory-bound graph operators: residual fork, RMSNorm, SwiGLU, dropout-add.

Counterparts of the reference's ``kareus/megatron/core/extensions/ops/`` wrappers
(``residual_fork.py:13-107``, ``te_norm.py:15-61``, ``bias_swiglu.py:14-239``,
``bias_dropout_add.py:15-186``).  The math runs in :mod:`kareus_b200.kernels`: hand-written
sm_100a kernels for CUDA tensors, PyTorch statements on CPU.  Parameter gradients are accumulated
into ``param.main_grad`` (fp32) instead of being returned, so the two nanobatches add into one
buffer without passing every parameter through autograd twice.
"""
from __future__ import annotations

import collections
import itertools
from typing import Optional

import torch
import torch.nn as nn

from .. import kernels as K
from ..engine.graph import GraphOperator


def accumulate_grad(param: torch.nn.Parameter, grad: torch.Tensor) -> None:
    """``main_grad += grad`` (creating the fp32 buffer on first use)."""
    mg = getattr(param, "main_grad", None)
    if mg is None:
        acc = torch.float64 if param.dtype == torch.float64 else torch.float32
        mg = torch.zeros(param.shape, dtype=acc, device=param.device)
        param.main_grad = mg
    mg.add_(grad.reshape(param.shape).to(mg.dtype))


def ensure_main_grad(param: torch.nn.Parameter) -> torch.Tensor:
    mg = getattr(param, "main_grad", None)
    if mg is None:
        acc = torch.float64 if param.dtype == torch.float64 else torch.float32
        mg = torch.zeros(param.shape, dtype=acc, device=param.device)
        param.main_grad = mg
    return mg


class ResidualFork(GraphOperator):
    """``x → (x, x)``; backward adds the two incoming gradients."""

    group = "norm"
    in_channels = ("main",)
    out_channels = ("main", "residual")

    def __init__(self, name: str = "fork"):
        self.name = name

    def forward(self, ctx, x):
        return x, x

    def backward(self, ctx, g_main, g_res):
        return (K.add(g_main, g_res),)


class RMSNormOp(nn.Module, GraphOperator):
    group = "norm"
    in_channels = ("main",)
    out_channels = ("main",)

    def __init__(self, hidden: int, eps: float = 1e-5, name: str = "norm", dtype=torch.float32,
                 device=None, sequence_parallel: bool = False):
        super().__init__()
        self.name = name
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden, dtype=dtype, device=device))
        # under sequence parallelism each TP rank sees different rows, so the weight gradient
        # must be summed over the TP group after backward
        self.weight.sequence_parallel = sequence_parallel

    def forward(self, ctx, x):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        y, rstd = K.rmsnorm_fwd(x2, self.weight, self.eps)
        if ctx.requires_grad:
            ctx.save_for_backward(x2, rstd)
        return (y.reshape(shp),)

    def backward(self, ctx, dy):
        x2, rstd = ctx.saved_tensors
        shp = dy.shape
        dx, _ = K.rmsnorm_bwd(dy.reshape(-1, shp[-1]), x2, rstd, self.weight, dw_accum=ensure_main_grad(self.weight))
        return (dx.reshape(shp),)

    def parameters_list(self):
        return [self.weight]


class SwiGLUOp(GraphOperator):
    """``silu(gate) * up`` on a ``[gate | up]`` packed last dim (reference ``bias_swiglu.py:18-19``)."""

    group = "activation"

    def __init__(self, name: str = "swiglu"):
        self.name = name

    def forward(self, ctx, x):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        y = K.swiglu_fwd(x2)
        if ctx.requires_grad:
            ctx.save_for_backward(x2)
        return (y.reshape(shp[:-1] + (shp[-1] // 2,)),)

    def backward(self, ctx, dy):
        (x2,) = ctx.saved_tensors
        dx = K.swiglu_bwd(dy.reshape(-1, dy.shape[-1]), x2)
        return (dx.reshape(dy.shape[:-1] + (x2.shape[-1],)),)


_SEED_COUNTER = itertools.count(1)


class DropoutAddOp(GraphOperator):
    """``residual + dropout(x)``.

    The mask is a function of a per-call seed kept in the context, so nothing mask-sized is saved
    and a recompute pass reproduces the forward by reusing the seed (the reference stores the
    mask and restores global RNG state: ``bias_dropout_add.py:24-30,108-110``,
    ``autograd_function.py:143-146,263-266``).
    """

    group = "norm"
    in_channels = ("main", "residual")
    out_channels = ("main",)

    def __init__(self, p: float = 0.0, name: str = "bda", base_seed: int = 1234):
        self.name = name
        self.p = float(p)
        self.base_seed = base_seed
        self.training = True
        self._replay = {}  # nanobatch -> FIFO of seeds to reuse during recompute

    def forward(self, ctx, x, residual):
        p = self.p if self.training else 0.0
        seed = 0
        if p > 0.0:
            key = ctx.nb_index
            queue = self._replay.setdefault(key, collections.deque())
            if queue and ctx.requires_grad:
                seed = queue.popleft()   # recompute pass: microbatches come back in forward order
            else:
                seed = (self.base_seed * 1000003 + next(_SEED_COUNTER)) & 0x7FFFFFFF
                if not ctx.requires_grad:
                    queue.append(seed)
        ctx.extra["seed"] = seed
        ctx.extra["p"] = p
        return (K.dropout_add_fwd(x, residual, p, seed),)

    def backward(self, ctx, dy):
        dx, dres = K.dropout_add_bwd(dy, ctx.extra["p"], ctx.extra["seed"])
        return dx, dres
