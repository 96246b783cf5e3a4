"""Operators the benchmark models do not use but the reference's operator set has: LayerNorm (the
other branch of its norm factory, ``kareus/megatron/core/extensions/ops/te_norm.py:15-61``) and a
bias operator that follows a linear layer (``kareus/transformer_engine/pytorch/ops/basic/bias.py``;
``add_bias_linear`` is false for Llama and Qwen)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_void_p

import torch
import torch.nn as nn

from ..engine.graph import GraphOperator
from ..kernels import cuda as KC
from .basic import RMSNormOp, accumulate_grad


def _cuda_bf16(t) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16


def _call(name, *args):
    fn = getattr(KC.lib(), name)
    fn.restype = c_int
    KC._check(fn(*args), name)
    KC._count()


class LayerNormOp(nn.Module, GraphOperator):
    group = "norm"

    def __init__(self, hidden: int, eps: float = 1e-5, name: str = "layernorm", dtype=torch.float32, device=None,
                 sequence_parallel: bool = False):
        super().__init__()
        self.name, self.eps = name, eps
        self.weight = nn.Parameter(torch.ones(hidden, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(hidden, dtype=dtype, device=device))
        self.weight.sequence_parallel = sequence_parallel
        self.bias.sequence_parallel = sequence_parallel

    def forward(self, ctx, x):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        rows, H = x2.shape
        if _cuda_bf16(x2):
            y = torch.empty_like(x2)
            mean = torch.empty(rows, dtype=torch.float32, device=x2.device)
            rstd = torch.empty_like(mean)
            _call("kb_layernorm_fwd", c_void_p(x2.data_ptr()), c_void_p(self.weight.data_ptr()),
                  c_void_p(self.bias.data_ptr()), c_void_p(y.data_ptr()), c_void_p(mean.data_ptr()),
                  c_void_p(rstd.data_ptr()), c_int(rows), c_int(H), c_float(self.eps), c_void_p(KC._stream()))
        else:
            acc = torch.float64 if x2.dtype == torch.float64 else torch.float32
            xf = x2.to(acc)
            mean = xf.mean(-1)
            rstd = torch.rsqrt(xf.var(-1, unbiased=False) + self.eps)
            y = ((xf - mean[:, None]) * rstd[:, None] * self.weight.to(acc) + self.bias.to(acc)).to(x2.dtype)
        if ctx.requires_grad:
            ctx.save_for_backward(x2, mean, rstd)
        return (y.reshape(shp),)

    def backward(self, ctx, dy):
        x2, mean, rstd = ctx.saved_tensors
        shp = dy.shape
        d2 = dy.reshape(-1, shp[-1]).contiguous()
        rows, H = x2.shape
        if _cuda_bf16(x2):
            L = KC.lib()
            L.kb_layernorm_bwd_scratch_elems.restype = c_long
            n = L.kb_layernorm_bwd_scratch_elems(c_int(rows), c_int(H))
            scratch = torch.empty(n, dtype=torch.float32, device=x2.device)
            dx = torch.empty_like(x2)
            dw = torch.empty(H, dtype=torch.float32, device=x2.device)
            db = torch.empty_like(dw)
            _call("kb_layernorm_bwd", c_void_p(d2.data_ptr()), c_void_p(x2.data_ptr()), c_void_p(mean.data_ptr()),
                  c_void_p(rstd.data_ptr()), c_void_p(self.weight.data_ptr()), c_void_p(dx.data_ptr()),
                  c_void_p(dw.data_ptr()), c_void_p(db.data_ptr()), c_void_p(scratch.data_ptr()), c_int(rows), c_int(H),
                  c_void_p(KC._stream()))
        else:
            acc = torch.float64 if x2.dtype == torch.float64 else torch.float32
            xh = (x2.to(acc) - mean[:, None]) * rstd[:, None]
            gy = d2.to(acc)
            g = gy * self.weight.to(acc)
            dx = ((g - g.mean(-1, keepdim=True) - xh * (g * xh).mean(-1, keepdim=True)) * rstd[:, None]).to(x2.dtype)
            dw, db = (gy * xh).sum(0), gy.sum(0)
        accumulate_grad(self.weight, dw)
        accumulate_grad(self.bias, db)
        return (dx.reshape(shp),)


class BiasOp(nn.Module, GraphOperator):
    """``y = x + b`` after a linear layer; with ``tp_shard=True`` the bias is sharded like a
    column-parallel output."""

    group = "norm"

    def __init__(self, features: int, name: str = "bias", dtype=torch.float32, device=None):
        super().__init__()
        self.name = name
        self.bias = nn.Parameter(torch.zeros(features, dtype=dtype, device=device))

    def forward(self, ctx, x):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        if _cuda_bf16(x2):
            x2 = x2.contiguous()
            y = torch.empty_like(x2)
            _call("kb_bias_add", c_void_p(x2.data_ptr()), c_void_p(self.bias.data_ptr()), c_void_p(y.data_ptr()),
                  c_long(x2.shape[0]), c_int(x2.shape[1]), c_void_p(KC._stream()))
        else:
            y = x2 + self.bias.to(x2.dtype)
        return (y.reshape(shp),)

    def backward(self, ctx, dy):
        d2 = dy.reshape(-1, dy.shape[-1])
        if _cuda_bf16(d2):
            from .basic import ensure_main_grad
            d2 = d2.contiguous()
            _call("kb_colsum_accumulate", c_void_p(d2.data_ptr()), c_void_p(ensure_main_grad(self.bias).data_ptr()),
                  c_long(d2.shape[0]), c_int(d2.shape[1]), c_void_p(KC._stream()))
        else:
            accumulate_grad(self.bias, d2.sum(0))
        return (dy,)


def make_norm(kind: str, hidden: int, eps: float, name: str, **kw):
    """Norm factory: ``"RMSNorm"`` or ``"LayerNorm"`` (the reference's ``TENormOp``)."""
    if kind.lower() == "rmsnorm":
        return RMSNormOp(hidden, eps, name, **kw)
    if kind.lower() == "layernorm":
        return LayerNormOp(hidden, eps, name, **kw)
    raise ValueError(f"unknown normalization {kind!r}")
