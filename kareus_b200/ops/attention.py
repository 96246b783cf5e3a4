"""QKV unpacking, rotary embedding and causal GQA attention as graph operators.

Reference counterparts: ``kareus/megatron/core/extensions/ops/qkv_postprocess.py:14-244``,
``rotary_embedding.py:19-256``, ``te_attention.py:71-432`` and the all-gather context-parallel
attention in ``kareus/transformer_engine/pytorch/attention/dot_product_attention/
context_parallel.py:247-506,596-797``.

Layout choices that differ from the reference: Q, K and V are strided *views* of the packed QKV
GEMM output ``[s, b, groups, (q_per_group + 2) * d]`` (same packing order, so checkpoints stay
compatible), RoPE rotates them in place, and the attention kernels take strides, so no transposes
or ``contiguous()`` copies sit between the QKV GEMM and attention.  In backward, attention writes
dQ/dK/dV straight into one packed buffer that becomes the QKV GEMM's ``dy``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import kernels as K
from ..engine.graph import CommKind, CommSpec, ComputeSpec, GraphOperator
from ..parallel.collectives import AllGatherKV, CommFactory, ReduceScatterKV, dual_chunk_ids
from .basic import accumulate_grad


class QKVPostOp(nn.Module, GraphOperator):
    """Split the packed QKV projection into q ``[s,b,hq,d]``, k and v ``[s,b,g,d]`` views.

    Optional per-head RMSNorm of q and k (Qwen3 ``qk_layernorm``).
    """

    group = "rope"
    in_channels = ("main",)
    out_channels = ("main", "key", "value")

    def __init__(self, num_heads_local: int, num_groups_local: int, head_dim: int, qk_norm: bool = False,
                 eps: float = 1e-6, name: str = "qkv_post", dtype=torch.float32, device=None):
        super().__init__()
        self.name = name
        self.hq, self.g, self.d = num_heads_local, num_groups_local, head_dim
        self.rep = num_heads_local // num_groups_local
        self.eps = eps
        self.qk_norm = qk_norm
        if qk_norm:
            self.q_norm_weight = nn.Parameter(torch.ones(head_dim, dtype=dtype, device=device))
            self.k_norm_weight = nn.Parameter(torch.ones(head_dim, dtype=dtype, device=device))
            # every TP rank normalises different heads with the same weight: gradients are partial
            self.q_norm_weight.tp_partial_grad = True
            self.k_norm_weight.tp_partial_grad = True

    def split(self, x):
        s, b, _ = x.shape
        p = x.view(s, b, self.g, (self.rep + 2) * self.d)
        q = p[..., : self.rep * self.d].unflatten(-1, (self.rep, self.d))   # [s,b,g,rep,d] view
        k = p[..., self.rep * self.d:(self.rep + 1) * self.d]               # [s,b,g,d] view
        v = p[..., (self.rep + 1) * self.d:]
        return q, k, v

    def forward(self, ctx, x):
        s, b, _ = x.shape
        q, k, v = self.split(x)
        if self.qk_norm:
            qc = q.reshape(-1, self.d)
            kc = k.reshape(-1, self.d)
            qn, q_rstd = K.rmsnorm_fwd(qc, self.q_norm_weight, self.eps)
            kn, k_rstd = K.rmsnorm_fwd(kc, self.k_norm_weight, self.eps)
            if ctx.requires_grad:
                ctx.save_for_backward(qc, q_rstd, kc, k_rstd)
            return qn.view(s, b, self.g, self.rep, self.d), kn.view(s, b, self.g, self.d), v
        return q, k, v

    def backward(self, ctx, dq, dk, dv):
        packed = getattr(dq, "_packed_base", None)
        if self.qk_norm:
            qc, q_rstd, kc, k_rstd = ctx.saved_tensors
            dqc, dwq = K.rmsnorm_bwd(dq.reshape(-1, self.d), qc, q_rstd, self.q_norm_weight)
            dkc, dwk = K.rmsnorm_bwd(dk.reshape(-1, self.d), kc, k_rstd, self.k_norm_weight)
            accumulate_grad(self.q_norm_weight, dwq)
            accumulate_grad(self.k_norm_weight, dwk)
            dq = dqc.view(dq.shape)
            dk = dkc.view(dk.shape)
            packed = None
        if packed is not None:
            return (packed,)
        s, b = dv.shape[0], dv.shape[1]
        out = torch.empty(s, b, self.g, (self.rep + 2) * self.d, dtype=dv.dtype, device=dv.device)
        out[..., : self.rep * self.d] = dq.reshape(s, b, self.g, self.rep * self.d)
        out[..., self.rep * self.d:(self.rep + 1) * self.d] = dk
        out[..., (self.rep + 1) * self.d:] = dv
        return (out.view(s, b, -1),)


def q_heads(q):
    """Number of query heads of a 4-D ``[s,b,h,d]`` or 5-D ``[s,b,g,rep,d]`` query view."""
    return q.shape[2] if q.dim() == 4 else q.shape[2] * q.shape[3]


def alloc_packed_grads(q, k):
    """One ``[s,b,g,(rep+2)*d]`` buffer and its dq ``[s,b,g,rep,d]``, dk, dv ``[s,b,g,d]`` views."""
    s, b = q.shape[0], q.shape[1]
    g, d = k.shape[2], k.shape[3]
    rep = q_heads(q) // g
    base = torch.empty(s, b, g, (rep + 2) * d, dtype=q.dtype, device=q.device)
    dq = base[..., : rep * d].unflatten(-1, (rep, d))
    dk = base[..., rep * d:(rep + 1) * d]
    dv = base[..., (rep + 1) * d:]
    return base, dq, dk, dv


class RotaryOp(GraphOperator):
    """Rotate-half RoPE on q and k, in place (they are views of the QKV buffer nobody else keeps)."""

    group = "rope"
    in_channels = ("main", "key", "rotary_pos_emb")
    out_channels = ("main", "key")
    no_grad_inputs = ("rotary_pos_emb",)

    def __init__(self, name: str = "rope"):
        self.name = name

    def forward(self, ctx, q, k, freqs):
        if freqs is None or isinstance(freqs, tuple):
            raise ValueError("rotary_pos_emb must be a single [s, d] angle table")
        if ctx.requires_grad:
            ctx.save_for_backward(freqs)
        K.rope_inplace(q, k, freqs, inverse=False)
        return q, k

    def backward(self, ctx, dq, dk):
        (freqs,) = ctx.saved_tensors
        K.rope_inplace(dq, dk, freqs, inverse=True)
        return dq, dk


class AttentionOp(GraphOperator):
    """Causal GQA attention; with ``cp > 1`` the all-gather context-parallel variant.

    Context parallelism (dual-chunk ownership): this rank's local sequence is chunks ``r`` and
    ``2cp-1-r`` of the global one.  K and V arrive gathered in sequence order (the ``ALL_GATHER_KV``
    node placed before this operator); each local query chunk ``c`` attends to keys
    ``[0, (c+1)·chunk)`` with the causal diagonal at offset ``c·chunk``.  Backward accumulates dK/dV
    for the full sequence and the ``REDUCE_SCATTER_KV`` node returns this rank's shard.
    """

    group = "attn"
    in_channels = ("main", "key", "value")
    out_channels = ("main",)

    def __init__(self, head_dim: int, name: str = "core_attn", comm: Optional[CommFactory] = None,
                 key: str = "attn", cp_comm: str = "all_gather"):
        self.name = name
        self.d = head_dim
        self.scale = 1.0 / math.sqrt(head_dim)
        comm = comm or CommFactory()
        self.cp = comm._args("cp")[1]
        self.cp_rank = comm._args("cp")[2]
        self.cp_comm = cp_comm
        self.key = key
        if self.cp > 1:
            self.ag_kv = comm.make(AllGatherKV, "cp", f"{name}.ag_kv")
            self.ag_kv_bwd = comm.make(AllGatherKV, "cp", f"{name}.ag_kv_bwd")
            self.rs_kv = comm.make(ReduceScatterKV, "cp", f"{name}.rs_kv")
        # sequence-split nanobatches: nanobatch i holds rows [i·s/N, (i+1)·s/N) of every sequence and
        # attends to the keys of nanobatches 0..i, which they leave in this per-layer bank
        self._seq_nano = 0
        self._kv_bank = {}
        self._dkv_bank = {}
        self.ring = None
        if self.cp > 1 and cp_comm == "ring":
            from ..parallel.ring_attention import RingAttention
            self.ring = RingAttention(comm._args("cp")[0], self.cp, self.cp_rank, heap=getattr(comm, "heap_cp", None),
                                      name=f"{name}.ring")

    @property
    def seq_nano(self) -> int:
        return self._seq_nano

    @seq_nano.setter
    def seq_nano(self, n: int) -> None:
        self._seq_nano = int(n)
        if self.cp > 1 and self.cp_comm != "ring":
            # each nanobatch then gathers / reduces one half of the sequence (one chunk per rank)
            for op in (self.ag_kv, self.rs_kv):
                op.half_mode = self._seq_nano > 1

    # graph --------------------------------------------------------------------
    def forward_specs(self):
        compute = ComputeSpec(self, self.in_channels, self.out_channels)
        if self.cp == 1 or self.cp_comm == "ring":
            return [compute]
        return [CommSpec(self.ag_kv, CommKind.ALL_GATHER_KV, ("key", "value"), ("key", "value"), "fwd_qkv_ag",
                         segment="qkv", short="ag"),
                compute]

    def backward_specs(self):
        compute = ComputeSpec(self, ("grad_main",), ("grad_main", "grad_key", "grad_value"), backward=True)
        if self.cp == 1 or self.cp_comm == "ring":
            return [compute]
        if self.seq_nano > 1:
            # sequence-split nanobatches keep the gathered K/V of their half: nothing to gather again
            return [compute,
                    CommSpec(self.rs_kv, CommKind.REDUCE_SCATTER_KV, ("grad_key", "grad_value"),
                             ("grad_key", "grad_value"), "bwd_a_rs", backward=True, segment="a", short="rs")]
        # K/V are gathered again for backward by a schedulable collective of its own; it has no
        # graph input (it re-reads the local shards kept by the forward), so it is modelled as a
        # pass-through on grad_main that stashes the gathered tensors for the compute node.
        return [CommSpec(_RegatherKV(self), CommKind.ALL_GATHER_KV, ("grad_main",), ("grad_main",),
                         "bwd_a_ag", backward=True, segment="o", short="ag"),
                compute,
                CommSpec(self.rs_kv, CommKind.REDUCE_SCATTER_KV, ("grad_key", "grad_value"),
                         ("grad_key", "grad_value"), "bwd_a_rs", backward=True, segment="a", short="rs")]

    # compute --------------------------------------------------------------------
    def forward(self, ctx, q, k, v):
        s, b = q.shape[0], q.shape[1]
        if self.seq_nano > 1:
            return self._forward_seq_split(ctx, q, k, v)
        if self.cp > 1 and self.cp_comm == "ring":
            out, lse = self.ring.forward(q, k, v, self.scale, nb=ctx.nb_index)
            if ctx.requires_grad:
                ctx.save_for_backward(q, k, v, out, lse)
            return (out.reshape(s, b, -1),)
        if self.cp == 1:
            out, lse = K.attention_fwd(q, k, v, self.scale, causal=True)
            if ctx.requires_grad:
                ctx.save_for_backward(q, k, v, out, lse)
            return (out.reshape(s, b, -1),)
        # all-gather CP: k, v are full length in sequence order
        c = s // 2
        outs, lses = [], []
        for half, cid in enumerate(dual_chunk_ids(self.cp, self.cp_rank)):
            o, l = K.attention_fwd(q[half * c:(half + 1) * c], k, v, self.scale, causal=True,
                                   q_offset=cid * c, kv_len=(cid + 1) * c)
            outs.append(o)
            lses.append(l)
        out = torch.cat(outs, dim=0)
        if ctx.requires_grad:
            # keep only the local K/V shards; backward gathers again (reference keeps K_TO_SAVE /
            # V_TO_SAVE: all_gather_kv.py:30-33)
            a, bb = dual_chunk_ids(self.cp, self.cp_rank)
            k_loc = torch.cat([k[a * c:(a + 1) * c], k[bb * c:(bb + 1) * c]], dim=0)
            v_loc = torch.cat([v[a * c:(a + 1) * c], v[bb * c:(bb + 1) * c]], dim=0)
            ctx.save_for_backward(q, k_loc, v_loc, out, lses[0], lses[1])
        return (out.reshape(s, b, -1),)

    def _seq_split_window(self, i: int, chunk_rows: int):
        """(absolute position of the nanobatch's first query, number of visible keys)."""
        if self.cp == 1:
            return i * chunk_rows, None
        # dual-chunk ownership: nanobatch 0 is this rank's early chunk r, nanobatch 1 its late chunk 2cp-1-r;
        # the keys at hand are the gathered halves 0..i of the sequence
        cid = dual_chunk_ids(self.cp, self.cp_rank)[i]
        return cid * chunk_rows, (cid + 1) * chunk_rows

    def _forward_seq_split(self, ctx, q, k, v):
        if self.cp > 1 and (self.seq_nano != 2 or self.cp_comm != "all_gather"):
            raise NotImplementedError("sequence-split nanobatches with context parallelism: two nanobatches and "
                                      "cp_comm='all_gather' only")
        i, s, b = ctx.nb_index, q.shape[0], q.shape[1]
        self._kv_bank[i] = (k, v)
        if i > 0:
            k_all = torch.cat([self._kv_bank[j][0] for j in range(i + 1)], dim=0)
            v_all = torch.cat([self._kv_bank[j][1] for j in range(i + 1)], dim=0)
        else:
            k_all, v_all = k, v
        if i == self.seq_nano - 1:
            self._kv_bank.clear()
        q_off, kv_len = self._seq_split_window(i, s)
        if kv_len is None:
            out, lse = K.attention_fwd(q, k_all, v_all, self.scale, causal=True, q_offset=q_off)
        else:
            out, lse = K.attention_fwd(q, k_all, v_all, self.scale, causal=True, q_offset=q_off, kv_len=kv_len)
        if ctx.requires_grad:
            ctx.save_for_backward(q, k_all, v_all, out, lse)
        return (out.reshape(s, b, -1),)

    def _backward_seq_split(self, ctx, dout):
        q, k_all, v_all, out, lse = ctx.saved_tensors
        i, s, b = ctx.nb_index, q.shape[0], q.shape[1]
        do = dout.reshape(s, b, q_heads(q), self.d)
        q_off, kv_len = self._seq_split_window(i, s)
        if kv_len is None:
            dq, dk_all, dv_all = K.attention_bwd(do, q, k_all, v_all, out, lse, self.scale, causal=True, q_offset=q_off)
        else:
            dq, dk_all, dv_all = K.attention_bwd(do, q, k_all, v_all, out, lse, self.scale, causal=True,
                                                 q_offset=q_off, kv_len=kv_len)
        w = s * self.cp                               # keys per nanobatch: its (gathered) part of the sequence
        dk, dv = dk_all[i * w:(i + 1) * w], dv_all[i * w:(i + 1) * w]
        late = self._dkv_bank.pop(i, None)            # contributions of the nanobatches after this one
        if late is not None:
            dk, dv = dk + late[0], dv + late[1]
        for j in range(i):
            part = (dk_all[j * w:(j + 1) * w], dv_all[j * w:(j + 1) * w])
            old = self._dkv_bank.get(j)
            self._dkv_bank[j] = part if old is None else (old[0] + part[0], old[1] + part[1])
        return dq, dk, dv

    def backward(self, ctx, dout):
        if self.seq_nano > 1:
            return self._backward_seq_split(ctx, dout)
        if self.cp > 1 and self.cp_comm != "ring":
            return self._backward_cp(ctx, dout)
        q, k, v, out, lse = ctx.saved_tensors
        s, b = q.shape[0], q.shape[1]
        do = dout.reshape(s, b, q_heads(q), self.d)
        base, dq, dk, dv = alloc_packed_grads(q, k)
        if self.cp > 1:
            self.ring.backward(do, q, k, v, out, lse, self.scale, out_grads=(dq, dk, dv), nb=ctx.nb_index)
        else:
            K.attention_bwd(do, q, k, v, out, lse, self.scale, causal=True, out=(dq, dk, dv))
        base3 = base.view(s, b, -1)
        for t in (dq, dk, dv):
            t._packed_base = base3
        return dq, dk, dv

    def _backward_cp(self, ctx, dout):
        q, k_loc, v_loc, out, lse0, lse1 = ctx.saved_tensors
        # left in place: the engine drops the operator's context after backward, and a profiler that runs this
        # step again (release_saved=False) finds it still there
        k, v = ctx.extra["regathered"]
        s, b = q.shape[0], q.shape[1]
        c = s // 2
        do = dout.reshape(s, b, q_heads(q), self.d)
        dk = torch.zeros_like(k)
        dv = torch.zeros_like(v)
        dqs = []
        for half, (cid, lse) in enumerate(zip(dual_chunk_ids(self.cp, self.cp_rank), (lse0, lse1))):
            sl = slice(half * c, (half + 1) * c)
            dq_h, dk_h, dv_h = K.attention_bwd(do[sl], q[sl], k, v, out[sl], lse, self.scale, causal=True,
                                               q_offset=cid * c, kv_len=(cid + 1) * c)
            dqs.append(dq_h)
            dk += dk_h
            dv += dv_h
        return torch.cat(dqs, dim=0), dk, dv


class _RegatherKV:
    """Backward-time K/V all-gather (plan keys ``bwd_a_ag`` / ``bwd_o_ag`` in the reference)."""

    needs_ctx = True
    group = "attn"

    def __init__(self, attn: AttentionOp):
        self.attn = attn
        self.name = attn.name + ".regather_kv"
        from ..engine.graph import operator_uid
        self._graph_uid = operator_uid(attn)   # share the attention operator's saved context

    def run(self, tensors, sm_num=None, block_size=None, backward=True, nb=0, ctx=None):
        (g,) = tensors
        _, k_loc, v_loc, *_ = ctx.saved_tensors
        k, v = self.attn.ag_kv_bwd.run((k_loc, v_loc), sm_num=sm_num, block_size=block_size,
                                       backward=True, nb=nb)
        ctx.extra["regathered"] = (k, v)
        return (g,)
