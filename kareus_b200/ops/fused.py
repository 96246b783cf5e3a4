"""Graph nodes that run a GEMM fused with its sequence-parallel collective.

``FusedAGGemm`` (all-gather → column-parallel GEMM) and ``FusedGemmRS`` (row-parallel GEMM →
reduce-scatter) wrap the kernels of ``csrc/fused_gemm_comm.cu``.  To the partition engine they are
collective nodes: they run on the side stream, take the plan entry's ``sm_num`` (copy-driver /
reducer CTAs) and overlap with the other nanobatch's compute, but they also produce the GEMM
result, so the graph has no separate compute node for that linear layer in forward.  Backward
uses the linear operator's ordinary dgrad/wgrad with the (unfused) mirrored collective.

State the forward leaves for backward (the gathered input, or the row-parallel input) goes into
the linear operator's own context: these nodes share its graph uid.
"""
from __future__ import annotations

import ctypes
import re
from ctypes import c_int, c_uint32, c_uint64, c_void_p

import torch

from ..engine.graph import operator_uid
from ..kernels import cuda as KC

_DECLARED = False


def _lib():
    global _DECLARED
    L = KC.lib()
    if not _DECLARED:
        P, I, U32, U64 = c_void_p, c_int, c_uint32, c_uint64
        L.kb_ag_gemm_bf16.argtypes = [P, I, I, U64, U64, P, P, I, I, I, I, P, U32, I, I, P, P]
        L.kb_gemm_rs_bf16.argtypes = [P, I, I, U64, U64, U64, P, I, P, I, P, I, I, I, P, U32, I, I, P, P]
        L.kb_fused_tiles_n.argtypes = [I]
        for n in ("kb_ag_gemm_bf16", "kb_gemm_rs_bf16", "kb_fused_tiles_n"):
            getattr(L, n).restype = c_int
        _DECLARED = True
    return L


class _FusedBase:
    needs_ctx = True
    group = "linear"

    def __init__(self, linear, heap, default_sm: int):
        self.linear, self.heap, self.default_sm = linear, heap, default_sm
        self.name = linear.name + "." + type(self).__name__
        # one set of heap buffers per call site, shared by all layers (see CollectiveBase.tag)
        self.tag = re.sub(r"layers\.\d+\.", "", linear.name)
        self._graph_uid = operator_uid(linear)
        self._local = {}

    def _local_flags(self, key, n):
        t = self._local.get(key)
        if t is None or t.numel() < n:
            t = torch.zeros(n, dtype=torch.int32, device=self.heap.device)
            self._local[key] = t
        return t


class FusedAGGemm(_FusedBase):
    def run(self, tensors, sm_num=None, block_size=None, backward=False, nb=0, ctx=None):
        (x,) = tensors
        heap, lin = self.heap, self.linear
        world, rank = heap.world, heap.rank
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        ms, k = x2.shape
        m, n = ms * world, lin.out_features
        if ms % 128 or x2.dtype != torch.bfloat16:
            raise KC.KernelError(f"fused all-gather GEMM needs bf16 and a multiple of 128 rows per rank, got {ms}")
        ch = heap.channel(f"{self.tag}/ag_gemm/{nb}")
        off, _ = heap.buffer(ch, "xg", m * k * 2)
        xg = heap.view(off, (m, k), torch.bfloat16)
        xg[rank * ms:(rank + 1) * ms].copy_(x2)
        ready = self._local_flags(("ready", nb), m // 128)
        ch.epoch += 1
        y = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
        st = KC.status_word(x.device)
        w = lin.weight
        rc = _lib().kb_ag_gemm_bf16(heap._bases_arr, rank, world, ch.flag_off, off, w.data_ptr(), y.data_ptr(), m, n, k,
                                    w.stride(0), ready.data_ptr(), ch.epoch, int(sm_num or self.default_sm), 0,
                                    st.data_ptr(), KC._stream())
        KC._check(rc, f"ag_gemm {lin.name}")
        KC._count()
        if ctx is not None and ctx.requires_grad:
            ctx.save_for_backward(xg.clone())         # gathered input for the wgrad GEMM
        return (y.reshape((lead[0] * world,) + tuple(lead[1:]) + (n,)),)


class FusedGemmRS(_FusedBase):
    def run(self, tensors, sm_num=None, block_size=None, backward=False, nb=0, ctx=None):
        (a,) = tensors
        heap, lin = self.heap, self.linear
        world, rank = heap.world, heap.rank
        lead = a.shape[:-1]
        a2 = a.reshape(-1, a.shape[-1])
        if not KC._rowmajor_ok(a2):
            a2 = a2.contiguous()
        m, k = a2.shape
        n = lin.out_features
        ms = m // world
        if m % (world * 128) or a2.dtype != torch.bfloat16:
            raise KC.KernelError(f"fused GEMM reduce-scatter needs bf16 and rows divisible by {world * 128}, got {m}")
        L = _lib()
        tiles_n = L.kb_fused_tiles_n(n)
        ch = heap.channel(f"{self.tag}/gemm_rs/{nb}")
        stage_off, _ = heap.buffer(ch, "stage", m * n * 2)
        cnt_off, _ = heap.buffer(ch, "cnt", world * (ms // 128) * tiles_n * 4)
        go = self._local_flags(("go", nb), 1)
        ch.epoch += 1
        out = torch.empty(ms, n, dtype=torch.bfloat16, device=a.device)
        st = KC.status_word(a.device)
        w = lin.weight
        rc = L.kb_gemm_rs_bf16(heap._bases_arr, rank, world, ch.flag_off, stage_off, cnt_off, a2.data_ptr(),
                               a2.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), m, n, k, go.data_ptr(), ch.epoch,
                               int(sm_num or self.default_sm), 0, st.data_ptr(), KC._stream())
        KC._check(rc, f"gemm_rs {lin.name}")
        KC._count()
        if ctx is not None and ctx.requires_grad:
            ctx.save_for_backward(a2)
        return (out.reshape((lead[0] // world,) + tuple(lead[1:]) + (n,)),)


def attach_fused(layer, heap, default_sm: int = 16) -> None:
    """Give the four linear layers of a transformer layer their fused forward nodes."""
    layer.qkv.fused_ag_gemm = FusedAGGemm(layer.qkv, heap, default_sm)
    layer.fc1.fused_ag_gemm = FusedAGGemm(layer.fc1, heap, default_sm)
    layer.proj.fused_gemm_rs = FusedGemmRS(layer.proj, heap, default_sm)
    layer.fc2.fused_gemm_rs = FusedGemmRS(layer.fc2, heap, default_sm)
