"""Operators the benchmark models do not use but the reference's operator set has: LayerNorm (the
other branch of its norm factory, ``kareus/megatron/core/extensions/ops/te_norm.py:15-61``), a
bias operator that follows a linear layer (``kareus/transformer_engine/pytorch/ops/basic/bias.py``;
``add_bias_linear`` is false for Llama and Qwen), and linear layers with a bias and an optional
activation whose forward runs in the GEMM's epilogue (``ops/basic/basic_linear_bias.py:34-315``,
``ops/fused/forward_linear_bias_activation.py:37-213``)."""
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


class LinearBiasOp(nn.Module, GraphOperator):
    """``y = act(x Wᵀ + b)`` as ONE forward kernel: bias and activation are applied to the GEMM's fp32
    accumulator in its epilogue.

    ``skip_bias_add=True`` is Megatron's ``return_bias``: the layer leaves the bias out of ``y`` and exposes
    it as ``self.bias`` for a later fused bias-dropout-add.  With an activation and gradients required the
    pre-activation is kept (the GEMM then writes ``x Wᵀ + b`` and the activation runs as its own kernel);
    without gradients everything stays in the one launch."""

    group = "linear"

    def __init__(self, in_features: int, out_features: int, name: str = "linear_bias", activation=None,
                 skip_bias_add: bool = False, dtype=torch.float32, device=None, init_std: float = 0.02, seed=None):
        super().__init__()
        if activation not in (None, "gelu"):
            raise ValueError(f"unsupported activation {activation!r}")
        self.name, self.activation, self.skip_bias_add = name, activation, skip_bias_add
        self.in_features, self.out_features = in_features, out_features
        w = torch.empty(out_features, in_features, dtype=torch.float32)
        w.normal_(0.0, init_std, generator=torch.Generator().manual_seed(seed) if seed is not None else None)
        self.weight = nn.Parameter(w.to(dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device))

    def forward(self, ctx, x):
        from .. import kernels as K
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        bias = None if self.skip_bias_add else self.bias
        if self.activation is None or not ctx.requires_grad:
            y = K.gemm(x2, self.weight, trans_b=True, bias=bias, activation=self.activation)
            if ctx.requires_grad:
                ctx.save_for_backward(x2, None)
        else:
            z = K.gemm(x2, self.weight, trans_b=True, bias=bias)
            y = _gelu_fwd(z)
            ctx.save_for_backward(x2, z)
        return (y.reshape(shp[:-1] + (self.out_features,)),)

    def backward(self, ctx, dy):
        from .. import kernels as K
        from .basic import ensure_main_grad
        x2, z = ctx.saved_tensors
        shp = dy.shape
        d2 = dy.reshape(-1, shp[-1])
        if z is not None:
            d2 = _gelu_bwd(d2, z)
        if not self.skip_bias_add:
            if _cuda_bf16(d2):
                d2 = d2.contiguous()
                _call("kb_colsum_accumulate", c_void_p(d2.data_ptr()), c_void_p(ensure_main_grad(self.bias).data_ptr()),
                      c_long(d2.shape[0]), c_int(d2.shape[1]), c_void_p(KC._stream()))
            else:
                accumulate_grad(self.bias, d2.sum(0))
        dx = K.gemm(d2, self.weight, trans_b=False)
        K.gemm(d2, x2, trans_a=True, trans_b=False, accumulate=ensure_main_grad(self.weight))
        return (dx.reshape(shp[:-1] + (self.in_features,)),)


def _gelu_fwd(z):
    from .activations import gelu_forward
    return gelu_forward(z)


def _gelu_bwd(dy, z):
    from .activations import gelu_backward
    return gelu_backward(dy, z)
