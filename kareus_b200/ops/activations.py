"""GELU and GeGLU graph operators (reference ``kareus/megatron/core/extensions/ops/bias_gelu.py``,
``bias_geglu.py``); the benchmark models use :class:`kareus_b200.ops.basic.SwiGLUOp`."""
from __future__ import annotations

import math
from ctypes import c_int, c_long, c_void_p

import torch

from ..engine.graph import GraphOperator
from ..kernels import cuda as KC

_C = math.sqrt(2.0 / math.pi)


def gelu_ref(x):
    return 0.5 * x * (1.0 + torch.tanh(_C * x * (1.0 + 0.044715 * x * x)))


def gelu_grad_ref(x):
    t = torch.tanh(_C * x * (1.0 + 0.044715 * x * x))
    return 0.5 * x * ((1 - t * t) * (_C + 3 * 0.044715 * _C * x * x)) + 0.5 * (1 + t)


def _launch(fn_name, args):
    L = KC.lib()
    fn = getattr(L, fn_name)
    fn.restype = c_int
    KC._check(fn(*args), fn_name)
    KC._count()


class _GeluBase(GraphOperator):
    group = "activation"
    gated = False

    def __init__(self, name: str = "gelu"):
        self.name = name

    def forward(self, ctx, x):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        F = shp[-1] // 2 if self.gated else shp[-1]
        if x2.is_cuda and x2.dtype == torch.bfloat16:
            x2 = x2.contiguous()
            y = torch.empty(x2.shape[0], F, dtype=x2.dtype, device=x2.device)
            _launch("kb_gelu_fwd", [c_void_p(x2.data_ptr()), c_void_p(y.data_ptr()), c_long(x2.shape[0]), c_int(F),
                                    c_int(1 if self.gated else 0), c_void_p(KC._stream())])
        else:
            acc = torch.float64 if x2.dtype == torch.float64 else torch.float32
            xf = x2.to(acc)
            y = (gelu_ref(xf[:, :F]) * xf[:, F:] if self.gated else gelu_ref(xf)).to(x2.dtype)
        if ctx.requires_grad:
            ctx.save_for_backward(x2)
        return (y.reshape(shp[:-1] + (F,)),)

    def backward(self, ctx, dy):
        (x2,) = ctx.saved_tensors
        F = x2.shape[1] // 2 if self.gated else x2.shape[1]
        d2 = dy.reshape(-1, F)
        if x2.is_cuda and x2.dtype == torch.bfloat16:
            d2 = d2.contiguous()
            dx = torch.empty_like(x2)
            _launch("kb_gelu_bwd", [c_void_p(d2.data_ptr()), c_void_p(x2.data_ptr()), c_void_p(dx.data_ptr()),
                                    c_long(x2.shape[0]), c_int(F), c_int(1 if self.gated else 0),
                                    c_void_p(KC._stream())])
        else:
            acc = torch.float64 if x2.dtype == torch.float64 else torch.float32
            xf, g = x2.to(acc), d2.to(acc)
            if self.gated:
                a, b = xf[:, :F], xf[:, F:]
                dx = torch.cat([g * b * gelu_grad_ref(a), g * gelu_ref(a)], dim=1).to(x2.dtype)
            else:
                dx = (g * gelu_grad_ref(xf)).to(x2.dtype)
        return (dx.reshape(dy.shape[:-1] + (x2.shape[1],)),)


class GeluOp(_GeluBase):
    gated = False


class GegluOp(_GeluBase):
    gated = True


def gelu_forward(x2: torch.Tensor) -> torch.Tensor:
    """GELU of a 2-D tensor (kernel on bf16 CUDA tensors, PyTorch statement otherwise)."""
    if x2.is_cuda and x2.dtype == torch.bfloat16:
        x2 = x2.contiguous()
        y = torch.empty_like(x2)
        _launch("kb_gelu_fwd", [c_void_p(x2.data_ptr()), c_void_p(y.data_ptr()), c_long(x2.shape[0]), c_int(x2.shape[1]),
                                c_int(0), c_void_p(KC._stream())])
        return y
    acc = torch.float64 if x2.dtype == torch.float64 else torch.float32
    return gelu_ref(x2.to(acc)).to(x2.dtype)


def gelu_backward(dy2: torch.Tensor, x2: torch.Tensor) -> torch.Tensor:
    """``dy * gelu'(x)`` for 2-D tensors."""
    if x2.is_cuda and x2.dtype == torch.bfloat16:
        dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        _launch("kb_gelu_bwd", [c_void_p(dy2.data_ptr()), c_void_p(x2.data_ptr()), c_void_p(dx.data_ptr()),
                                c_long(x2.shape[0]), c_int(x2.shape[1]), c_int(0), c_void_p(KC._stream())])
        return dx
    acc = torch.float64 if x2.dtype == torch.float64 else torch.float32
    return (dy2.to(acc) * gelu_grad_ref(x2.to(acc))).to(x2.dtype)
