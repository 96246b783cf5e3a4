"""Tensor-parallel linear operators and how they place collectives in the graph.

* ``tp_comm="allreduce"`` — the reference's layout (``kareus/megatron/core/extensions/ops/
  te_linear.py:303-445``): a column-parallel layer declares a backward ``ALL_REDUCE(grad_main)``
  after its dgrad, a row-parallel layer a forward ``ALL_REDUCE(main)`` after its GEMM.
* ``tp_comm="sp"`` — sequence parallelism: column-parallel = ``ALL_GATHER(main)`` then GEMM
  (backward: dgrad then ``REDUCE_SCATTER(grad_main)``); row-parallel = GEMM then
  ``REDUCE_SCATTER(main)`` (backward: ``ALL_GATHER(grad_main)`` then dgrad/wgrad).
* ``tp_comm="sp_fused"`` — same dataflow, but forward gather+GEMM and GEMM+scatter are single
  fused kernels (``FUSED`` nodes that the engine runs on the side stream).

Weights are ``[out_features_local, in_features_local]`` (K-major for the forward GEMM).  The wgrad
GEMM accumulates straight into the fp32 ``main_grad`` of the weight.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn as nn

from .. import kernels as K
from ..engine.graph import CommKind, CommSpec, ComputeSpec, GraphOperator, grad_channel
from ..parallel.collectives import AllGather, AllReduce, CommFactory, ReduceScatter
from .basic import ensure_main_grad


class _LinearBase(nn.Module, GraphOperator):
    group = "linear"
    in_channels = ("main",)
    out_channels = ("main",)

    def __init__(self, in_features: int, out_features: int, name: str, key: str, tp_comm: str,
                 comm: Optional[CommFactory], dtype=torch.float32, device=None, init_std: float = 0.02,
                 seed: Optional[int] = None):
        super().__init__()
        self.name = name
        self.key = key                      # "attn" or "mlp": which plan key family governs us
        self.tp_comm = tp_comm
        self.in_features = in_features
        self.out_features = out_features
        comm = comm or CommFactory()
        self.tp, tp_rank = comm._args("tp")[1], comm._args("tp")[2]
        w = torch.empty(out_features, in_features, dtype=torch.float32)
        g = torch.Generator().manual_seed(seed * 64 + tp_rank) if seed is not None else None
        w.normal_(0.0, init_std, generator=g)
        self.weight = nn.Parameter(w.to(dtype=dtype, device=device))
        self._comm_factory = comm

    # compute -------------------------------------------------------------------
    def _fwd_staging(self, shape, dtype, nb, device):
        """Where the forward result should be written so the following collective needs no copy."""
        return None

    def _bwd_staging(self, shape, dtype, nb, device):
        return None

    def forward(self, ctx, x):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        out = self._fwd_staging((x2.shape[0], self.out_features), x2.dtype, ctx.nb_index, x2.device)
        y = K.gemm(x2, self.weight, trans_b=True, out=out)
        if ctx.requires_grad:
            ctx.save_for_backward(x2)
        return (y.reshape(shp[:-1] + (self.out_features,)),)

    def backward(self, ctx, dy):
        (x2,) = ctx.saved_tensors
        shp = dy.shape
        dy2 = dy.reshape(-1, shp[-1])
        out = self._bwd_staging((dy2.shape[0], self.in_features), dy2.dtype, ctx.nb_index, dy2.device)
        dx = K.gemm(dy2, self.weight, trans_b=False, out=out)              # [M,N]·[N,K]
        K.gemm(dy2, x2, trans_a=True, trans_b=False, accumulate=ensure_main_grad(self.weight))
        return (dx.reshape(shp[:-1] + (self.in_features,)),)


class ColumnParallelLinear(_LinearBase):
    """Output features sharded over TP (QKV, FC1)."""

    tp_shard_axis = 0

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        f = self._comm_factory
        self.bwd_allreduce = f.make(AllReduce, "tp", f"{self.name}.bwd_ar")
        self.fwd_allgather = f.make(AllGather, "tp", f"{self.name}.fwd_ag")
        self.bwd_reducescatter = f.make(ReduceScatter, "tp", f"{self.name}.bwd_rs")
        self.fused_ag_gemm = None   # set by kareus_b200.ops.fused when tp_comm == "sp_fused"
        self.fused_dgrad_rs = None

    def _bwd_staging(self, shape, dtype, nb, device):
        if self.tp == 1:
            return None
        op = self.bwd_allreduce if self.tp_comm == "allreduce" else self.bwd_reducescatter
        return op.staging(shape, dtype, nb, device)

    def forward_specs(self) -> List[object]:
        compute = ComputeSpec(self, ("main",), ("main",))
        if self.tp == 1 or self.tp_comm == "allreduce":
            return [compute]
        if self.tp_comm == "sp_fused" and self.fused_ag_gemm is not None:
            return [CommSpec(self.fused_ag_gemm, CommKind.FUSED, ("main",), ("main",), f"fwd_{self.key}_ag")]
        return [CommSpec(self.fwd_allgather, CommKind.ALL_GATHER, ("main",), ("main",), f"fwd_{self.key}_ag"),
                compute]

    def backward_specs(self) -> List[object]:
        compute = ComputeSpec(self, ("grad_main",), ("grad_main",), backward=True)
        if self.tp == 1:
            return [compute]
        if self.tp_comm == "allreduce":
            return [compute, CommSpec(self.bwd_allreduce, CommKind.ALL_REDUCE, ("grad_main",), ("grad_main",),
                                      f"bwd_{self.key}", backward=True,
                                      segment="qkv" if self.key == "attn" else "mlp", short="ar")]
        if self.tp_comm == "sp_fused" and self.fused_dgrad_rs is not None:
            return [CommSpec(self.fused_dgrad_rs, CommKind.FUSED, ("grad_main",), ("grad_main",),
                             f"bwd_{self.key}", backward=True)]
        return [compute, CommSpec(self.bwd_reducescatter, CommKind.REDUCE_SCATTER, ("grad_main",),
                                  ("grad_main",), f"bwd_{self.key}", backward=True)]


class RowParallelLinear(_LinearBase):
    """Input features sharded over TP (attention out-proj, FC2); output is a partial sum."""

    tp_shard_axis = 1

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        f = self._comm_factory
        self.fwd_allreduce = f.make(AllReduce, "tp", f"{self.name}.fwd_ar")
        self.fwd_reducescatter = f.make(ReduceScatter, "tp", f"{self.name}.fwd_rs")
        self.bwd_allgather = f.make(AllGather, "tp", f"{self.name}.bwd_ag")
        self.fused_gemm_rs = None
        self.fused_ag_dgrad = None

    def _fwd_staging(self, shape, dtype, nb, device):
        if self.tp == 1:
            return None
        op = self.fwd_allreduce if self.tp_comm == "allreduce" else self.fwd_reducescatter
        return op.staging(shape, dtype, nb, device)

    def forward_specs(self) -> List[object]:
        compute = ComputeSpec(self, ("main",), ("main",))
        if self.tp == 1:
            return [compute]
        if self.tp_comm == "allreduce":
            return [compute, CommSpec(self.fwd_allreduce, CommKind.ALL_REDUCE, ("main",), ("main",),
                                      f"fwd_{self.key}", segment="ao" if self.key == "attn" else "mlp", short="ar")]
        if self.tp_comm == "sp_fused" and self.fused_gemm_rs is not None:
            return [CommSpec(self.fused_gemm_rs, CommKind.FUSED, ("main",), ("main",), f"fwd_{self.key}")]
        return [compute, CommSpec(self.fwd_reducescatter, CommKind.REDUCE_SCATTER, ("main",), ("main",),
                                  f"fwd_{self.key}")]

    def backward_specs(self) -> List[object]:
        compute = ComputeSpec(self, ("grad_main",), ("grad_main",), backward=True)
        if self.tp == 1 or self.tp_comm == "allreduce":
            return [compute]
        if self.tp_comm == "sp_fused" and self.fused_ag_dgrad is not None:
            return [CommSpec(self.fused_ag_dgrad, CommKind.FUSED, ("grad_main",), ("grad_main",),
                             f"bwd_{self.key}_ag", backward=True)]
        return [CommSpec(self.bwd_allgather, CommKind.ALL_GATHER, ("grad_main",), ("grad_main",),
                         f"bwd_{self.key}_ag", backward=True), compute]
