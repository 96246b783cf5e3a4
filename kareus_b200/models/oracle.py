"""Unpartitioned single-process Llama written with ordinary autograd.

The numerical oracle for the engine: no nanobatches, no tensor/context/pipeline parallelism, no
custom backward.  ``load_from_shards`` assembles its full weights from the per-rank shards of
``GPTModel`` instances so that partitioned and oracle runs start from identical parameters.
"""
from __future__ import annotations

import math
from typing import Dict, List, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig
from ..kernels import ref


class OracleLlama(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype=torch.float64):
        super().__init__()
        self.cfg = cfg
        h, d = cfg.hidden_size, cfg.hd
        hq, g, f = cfg.num_attention_heads, cfg.num_query_groups, cfg.ffn_hidden_size
        self.emb = nn.Parameter(torch.zeros(cfg.vocab_size, h, dtype=dtype))
        self.out = None if cfg.tie_embeddings else nn.Parameter(torch.zeros(cfg.vocab_size, h, dtype=dtype))
        self.final_norm = nn.Parameter(torch.ones(h, dtype=dtype))
        self.layers = nn.ModuleList()
        for _ in range(cfg.num_layers):
            l = nn.Module()
            l.input_norm = nn.Parameter(torch.ones(h, dtype=dtype))
            l.qkv = nn.Parameter(torch.zeros((hq + 2 * g) * d, h, dtype=dtype))
            l.proj = nn.Parameter(torch.zeros(h, hq * d, dtype=dtype))
            l.pre_mlp_norm = nn.Parameter(torch.ones(h, dtype=dtype))
            l.fc1 = nn.Parameter(torch.zeros(2 * f, h, dtype=dtype))
            l.fc2 = nn.Parameter(torch.zeros(h, f, dtype=dtype))
            if cfg.qk_layernorm:
                l.q_norm = nn.Parameter(torch.ones(d, dtype=dtype))
                l.k_norm = nn.Parameter(torch.ones(d, dtype=dtype))
            self.layers.append(l)

    @staticmethod
    def _norm(x, w, eps):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w

    def forward(self, tokens, labels, loss_mask):
        """``[b, s]`` inputs → masked mean token loss."""
        cfg = self.cfg
        b, s = tokens.shape
        hq, g, d = cfg.num_attention_heads, cfg.num_query_groups, cfg.hd
        rep = hq // g
        x = self.emb[tokens]                                   # b s h
        fr = ref.rope_table(s, d, cfg.rope_theta).to(x.dtype)
        cos, sin = fr.cos()[None, :, None, :], fr.sin()[None, :, None, :]

        def rope(t):
            t1, t2 = t[..., : d // 2], t[..., d // 2:]
            return t * cos + torch.cat([-t2, t1], -1) * sin

        for l in self.layers:
            y = self._norm(x, l.input_norm, cfg.norm_eps)
            qkv = (y @ l.qkv.t()).view(b, s, g, (rep + 2) * d)
            q = qkv[..., : rep * d].reshape(b, s, hq, d)
            k = qkv[..., rep * d:(rep + 1) * d]
            v = qkv[..., (rep + 1) * d:]
            if cfg.qk_layernorm:
                q = self._norm(q, l.q_norm, cfg.norm_eps)
                k = self._norm(k, l.k_norm, cfg.norm_eps)
            q, k = rope(q), rope(k)
            kk = k.repeat_interleave(rep, dim=2)
            vv = v.repeat_interleave(rep, dim=2)
            sc = torch.einsum("bqhd,bkhd->bhqk", q, kk) / math.sqrt(d)
            mask = torch.triu(torch.ones(s, s, dtype=torch.bool), 1)
            sc = sc.masked_fill(mask, float("-inf"))
            a = torch.einsum("bhqk,bkhd->bqhd", sc.softmax(-1), vv).reshape(b, s, hq * d)
            x = x + a @ l.proj.t()
            y = self._norm(x, l.pre_mlp_norm, cfg.norm_eps)
            u = y @ l.fc1.t()
            gate, up = u.chunk(2, dim=-1)
            x = x + (F.silu(gate) * up) @ l.fc2.t()
        x = self._norm(x, self.final_norm, cfg.norm_eps)
        w_out = self.emb if self.out is None else self.out
        logits = x @ w_out.t()
        lp = F.log_softmax(logits, dim=-1)
        nll = -lp.gather(-1, labels.unsqueeze(-1)).squeeze(-1)
        m = loss_mask.to(nll.dtype)
        return (nll * m).sum() / m.sum()


def _cat_qkv(shards: Sequence[torch.Tensor]) -> torch.Tensor:
    return torch.cat(list(shards), dim=0)          # groups are contiguous per rank


def _cat_fc1(shards: Sequence[torch.Tensor]) -> torch.Tensor:
    gates = [s.chunk(2, dim=0)[0] for s in shards]
    ups = [s.chunk(2, dim=0)[1] for s in shards]
    return torch.cat(gates + ups, dim=0)


def load_from_shards(oracle: OracleLlama, tp_models: Sequence[nn.Module]) -> None:
    """Fill ``oracle`` from the TP shards (one ``GPTModel`` per TP rank, all layers)."""
    dt = oracle.emb.dtype

    def f(t):
        return t.detach().to(dt).cpu()

    with torch.no_grad():
        oracle.emb.copy_(torch.cat([f(m.embedding.weight) for m in tp_models], 0))
        if oracle.out is not None:
            oracle.out.copy_(torch.cat([f(m.output_layer.weight) for m in tp_models], 0))
        oracle.final_norm.copy_(f(tp_models[0].final_norm.weight))
        for i, l in enumerate(oracle.layers):
            ls = [m.decoder.layers[i] for m in tp_models]
            l.input_norm.copy_(f(ls[0].input_norm.weight))
            l.pre_mlp_norm.copy_(f(ls[0].pre_mlp_norm.weight))
            l.qkv.copy_(_cat_qkv([f(x.qkv.weight) for x in ls]))
            l.proj.copy_(torch.cat([f(x.proj.weight) for x in ls], 1))
            l.fc1.copy_(_cat_fc1([f(x.fc1.weight) for x in ls]))
            l.fc2.copy_(torch.cat([f(x.fc2.weight) for x in ls], 1))
            if oracle.cfg.qk_layernorm:
                l.q_norm.copy_(f(ls[0].qkv_post.q_norm_weight))
                l.k_norm.copy_(f(ls[0].qkv_post.k_norm_weight))


def shard_of_oracle_grad(oracle: OracleLlama, name: str, layer: int, tp: int, rank: int) -> torch.Tensor:
    """The slice of an oracle gradient that corresponds to a TP rank's shard of parameter ``name``."""
    l = oracle.layers[layer] if layer >= 0 else None
    if name == "qkv":
        return l.qkv.grad.chunk(tp, 0)[rank]
    if name == "proj":
        return l.proj.grad.chunk(tp, 1)[rank]
    if name == "fc1":
        gate, up = l.fc1.grad.chunk(2, 0)
        return torch.cat([gate.chunk(tp, 0)[rank], up.chunk(tp, 0)[rank]], 0)
    if name == "fc2":
        return l.fc2.grad.chunk(tp, 1)[rank]
    if name == "input_norm":
        return l.input_norm.grad
    if name == "pre_mlp_norm":
        return l.pre_mlp_norm.grad
    if name == "emb":
        return oracle.emb.grad.chunk(tp, 0)[rank]
    if name == "out":
        return oracle.out.grad.chunk(tp, 0)[rank]
    if name == "final_norm":
        return oracle.final_norm.grad
    raise KeyError(name)
