"""Llama-architecture GPT model on the partition engine.

Structure mirrors the reference's L3 (``kareus/megatron/core/models/gpt/gpt_model.py:81-423``,
``transformer/transformer_block.py:74-590``, ``transformer_layer.py:148-174``,
``attention.py``, ``mlp.py``): embedding → block of layers run as nanobatch partitions → final
norm → vocab-parallel output projection → vocab-parallel cross entropy.  Operator order inside
a layer: ``attn_fork, input_norm, qkv, qkv_post, rope, core_attn, proj, attn_bda, mlp_fork,
pre_mlp_norm, fc1, swiglu, fc2, mlp_bda``.

The microbatch is split into nanobatches *before* the embedding so each nanobatch is a contiguous
``[s, b/N, h]`` tensor from the start (the reference slices ``[s, b, h]`` along ``b`` inside the
block and re-materialises contiguous copies at every GEMM), and the head + loss also run per
nanobatch, which halves the live logits.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.distributed as dist

from .. import kernels as K
from ..config import ModelConfig, ParallelConfig
from ..engine.block import BlockEngine
from ..kernels import ref
from ..ops.attention import AttentionOp, QKVPostOp, RotaryOp
from ..ops.basic import DropoutAddOp, RMSNormOp, ResidualFork, SwiGLUOp, accumulate_grad, ensure_main_grad
from ..ops.linear import ColumnParallelLinear, RowParallelLinear
from ..parallel.collectives import CommFactory, dual_chunk_ids


def _torch_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    return {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32, "fp64": torch.float64}[name]


class TransformerLayer(nn.Module):
    """Holds the operators of one layer; it is never called directly (the block runs the graph)."""

    def __init__(self, cfg: ModelConfig, par: ParallelConfig, comm: CommFactory, layer_number: int,
                 dtype, device, seed: int):
        super().__init__()
        tp = par.tp
        h, d = cfg.hidden_size, cfg.hd
        if cfg.num_attention_heads % tp or cfg.num_query_groups % tp or cfg.ffn_hidden_size % tp:
            raise ValueError("heads, query groups and ffn size must be divisible by tp")
        hq, g, f = cfg.num_attention_heads // tp, cfg.num_query_groups // tp, cfg.ffn_hidden_size // tp
        sp = par.sequence_parallel
        n = f"layers.{layer_number}"
        out_std = cfg.init_std / math.sqrt(2.0 * cfg.num_layers)
        kw = dict(dtype=dtype, device=device)
        self.layer_number = layer_number
        self.attn_fork = ResidualFork(f"{n}.attn_fork")
        self.input_norm = RMSNormOp(h, cfg.norm_eps, f"{n}.input_layernorm", sequence_parallel=sp, **kw)
        self.qkv = ColumnParallelLinear(h, (hq + 2 * g) * d, f"{n}.self_attention.linear_qkv", "attn",
                                        par.tp_comm, comm, init_std=cfg.init_std, seed=seed * 16 + 1, **kw)
        self.qkv_post = QKVPostOp(hq, g, d, cfg.qk_layernorm, cfg.norm_eps, f"{n}.qkv_post", **kw)
        self.rope = RotaryOp(f"{n}.rope")
        self.core_attn = AttentionOp(d, f"{n}.core_attention", comm, cp_comm=par.cp_comm)
        self.proj = RowParallelLinear(hq * d, h, f"{n}.self_attention.linear_proj", "attn",
                                      par.tp_comm, comm, init_std=out_std, seed=seed * 16 + 2, **kw)
        self.attn_bda = DropoutAddOp(cfg.hidden_dropout, f"{n}.attn_bda", base_seed=seed * 16 + 3)
        self.mlp_fork = ResidualFork(f"{n}.mlp_fork")
        self.pre_mlp_norm = RMSNormOp(h, cfg.norm_eps, f"{n}.pre_mlp_layernorm", sequence_parallel=sp, **kw)
        self.fc1 = ColumnParallelLinear(h, 2 * f, f"{n}.mlp.linear_fc1", "mlp", par.tp_comm, comm,
                                        init_std=cfg.init_std, seed=seed * 16 + 4, **kw)
        self.act = SwiGLUOp(f"{n}.mlp.swiglu")
        self.fc2 = RowParallelLinear(f, h, f"{n}.mlp.linear_fc2", "mlp", par.tp_comm, comm,
                                     init_std=out_std, seed=seed * 16 + 5, **kw)
        self.mlp_bda = DropoutAddOp(cfg.hidden_dropout, f"{n}.mlp_bda", base_seed=seed * 16 + 6)
        if par.tp_comm == "sp_fused" and tp > 1 and getattr(comm, "heap", None) is not None \
                and dtype == torch.bfloat16 and torch.device(device or "cpu").type == "cuda":
            from ..ops.fused import attach_fused
            attach_fused(self, comm.heap)

    def operators(self):
        return [self.attn_fork, self.input_norm, self.qkv, self.qkv_post, self.rope, self.core_attn,
                self.proj, self.attn_bda, self.mlp_fork, self.pre_mlp_norm, self.fc1, self.act,
                self.fc2, self.mlp_bda]

    def forward(self, *a, **k):
        raise RuntimeError("TransformerLayer is executed by TransformerBlock's partition engine")

    def train(self, mode: bool = True):
        super().train(mode)
        self.attn_bda.training = mode
        self.mlp_bda.training = mode
        return self


class TransformerBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, par: ParallelConfig, comm: CommFactory, layer_range: range,
                 dtype, device, seed: int = 0, recompute_layers: Optional[int] = None,
                 sync: str = "partition_end", seq_split: bool = False):
        super().__init__()
        self.cfg, self.par = cfg, par
        self.layers = nn.ModuleList(
            TransformerLayer(cfg, par, comm, i, dtype, device, seed=seed * 1000 + i) for i in layer_range)
        if seq_split:
            for l in self.layers:
                l.core_attn.seq_nano = par.num_nanobatches
        self.engine = BlockEngine([l.operators() for l in self.layers], par.num_nanobatches,
                                  recompute=par.recompute, recompute_layers=recompute_layers, sync=sync,
                                  seq_split=seq_split,
                                  cp_keys=(par.cp > 1 and par.tp > 1 and par.tp_comm == "allreduce"
                                           and par.cp_comm == "all_gather"))

    def set_scheduler(self, scheduler) -> None:
        self.engine.scheduler = scheduler

    def forward(self, hidden: Sequence[torch.Tensor], rotary: torch.Tensor) -> List[torch.Tensor]:
        if len(self.layers) == 0:
            return list(hidden)
        return self.engine(hidden, rotary)


# ----------------------------------------------------------------------------- embedding / head
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, weight, vocab_start, tp_op, sp_op, module):
        out = K.embedding_fwd(tokens, weight, vocab_start)          # [s, b, h]
        ctx.save_for_backward(tokens)
        ctx.module, ctx.vocab_start, ctx.tp_op, ctx.sp_op = module, vocab_start, tp_op, sp_op
        if sp_op is not None:
            (out,) = sp_op.run((out,))
        elif tp_op is not None:
            (out,) = tp_op.run((out,))
        return out

    @staticmethod
    def backward(ctx, dout):
        (tokens,) = ctx.saved_tensors
        w = ctx.module.weight
        if ctx.sp_op is not None:
            (dout,) = ctx.module.bwd_gather.run((dout.contiguous(),))
        K.embedding_bwd(dout, tokens, ensure_main_grad(w), ctx.vocab_start)
        return None, None, None, None, None, None


class VocabParallelEmbedding(nn.Module):
    """Embedding sharded over the vocabulary; the partial lookups are summed over TP (all-reduce, or
    reduce-scatter to sequence shards under SP) (reference path: Megatron ``VocabParallelEmbedding``
    via ``LanguageModelEmbedding``)."""

    def __init__(self, cfg: ModelConfig, par: ParallelConfig, comm: CommFactory, dtype, device, seed: int):
        super().__init__()
        from ..parallel.collectives import AllGather, AllReduce, ReduceScatter
        g, tp, rank = comm._args("tp")
        if cfg.vocab_size % tp:
            raise ValueError("vocab size must be divisible by tp")
        self.v_local = cfg.vocab_size // tp
        self.vocab_start = rank * self.v_local
        w = torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=torch.float32)
        w.normal_(0.0, cfg.init_std, generator=torch.Generator().manual_seed(seed))
        self.weight = nn.Parameter(w[self.vocab_start:self.vocab_start + self.v_local].to(dtype=dtype, device=device))
        self.sp = par.sequence_parallel
        self.reduce = comm.make(AllReduce, "tp", "embedding.ar") if tp > 1 and not self.sp else None
        self.scatter = comm.make(ReduceScatter, "tp", "embedding.rs") if tp > 1 and self.sp else None
        self.bwd_gather = comm.make(AllGather, "tp", "embedding.bwd_ag") if tp > 1 and self.sp else None

    def forward(self, tokens_sb: torch.Tensor) -> torch.Tensor:
        """``tokens_sb`` is ``[s, b]`` int64; returns ``[s(/tp), b, h]``."""
        return _EmbeddingFn.apply(tokens_sb, self.weight, self.vocab_start, self.reduce, self.scatter, self)


class _HeadLossFn(torch.autograd.Function):
    """Final norm output → vocab-parallel logits → cross entropy, fused so logits never reach
    autograd: the logits buffer is overwritten with its own gradient and consumed by the dgrad and
    wgrad GEMMs inside ``forward`` (the loss scale is known up front: it is ``loss_mask / n``).
    Reference: output ``ColumnParallelLinear`` + TE parallel cross entropy
    (``gpt_model.py:401-421``; ``3rdparty/TransformerEngine/.../triton/cross_entropy.py``)."""

    @staticmethod
    def forward(ctx, x, module, labels, loss_weight, want_grad):
        # x: [s, b, h] (full sequence); labels, loss_weight: [s, b]
        w = module.weight
        in_shape = x.shape
        if module.fwd_gather is not None:                                 # sequence shard → full sequence
            (x,) = module.fwd_gather.run((x.contiguous(),))
        s, b, h = x.shape
        x2 = x.reshape(-1, h)
        logits = K.gemm(x2, w, trans_b=True)                            # [T, V_local]
        tgt = labels.reshape(-1)
        m, se, tl = K.cross_entropy_local_stats(logits, tgt, module.vocab_start)
        if module.tp > 1:
            stats = torch.stack([m, se, tl], dim=0)                        # [3, T]
            flat = torch.empty((module.tp * 3, stats.shape[1]), dtype=stats.dtype, device=stats.device)
            dist.all_gather_into_tensor(flat, stats.contiguous(), group=module.group)
            gathered = flat.view(module.tp, 3, -1)
            gm = gathered[:, 0].max(dim=0).values
            gs = (gathered[:, 1] * torch.exp(gathered[:, 0] - gm)).sum(0)
            gt = gathered[:, 2].sum(0)
        else:
            gm, gs, gt = m, se, tl
        per_token = (gm + torch.log(gs) - gt)                              # [T] fp32
        lw = loss_weight.reshape(-1).to(per_token.dtype)
        loss = (per_token * lw).sum()
        if want_grad:
            K.cross_entropy_finish(logits, tgt, module.vocab_start, gm, gs, lw)   # logits := dlogits
            dx = K.gemm(logits, w, trans_b=False)                          # [T, h] partial over TP
            K.gemm(logits, x2, trans_a=True, trans_b=False, accumulate=ensure_main_grad(w))
            ctx.save_for_backward(dx)
            ctx.shape = x.shape
            ctx.in_shape = in_shape
            ctx.module = module
        return loss

    @staticmethod
    def backward(ctx, dloss):
        (dx,) = ctx.saved_tensors
        module = ctx.module
        # dloss is a scalar (1/num_microbatches scaling etc.); weights got the unscaled gradient,
        # so the caller must keep dloss == 1 or rescale main_grad — enforced by GPTModel.
        dx = dx * dloss.to(dx.dtype)
        dx = dx.reshape(ctx.shape)
        if module.tp > 1 and not module.sp:
            dist.all_reduce(dx, group=module.group)
        elif module.tp > 1:
            (dx,) = module.bwd_scatter.run((dx,))
        return dx, None, None, None, None


class OutputHead(nn.Module):
    def __init__(self, cfg: ModelConfig, par: ParallelConfig, comm: CommFactory, dtype, device, seed: int,
                 tied_weight: Optional[nn.Parameter] = None):
        super().__init__()
        from ..parallel.collectives import AllGather, ReduceScatter
        self.group, self.tp, rank = comm._args("tp")
        self.v_local = cfg.vocab_size // self.tp
        self.vocab_start = rank * self.v_local
        self.sp = par.sequence_parallel
        if tied_weight is not None:
            self.weight = tied_weight
        else:
            w = torch.empty(cfg.vocab_size, cfg.hidden_size, dtype=torch.float32)
            w.normal_(0.0, cfg.init_std, generator=torch.Generator().manual_seed(seed))
            self.weight = nn.Parameter(w[self.vocab_start:self.vocab_start + self.v_local].to(dtype=dtype, device=device))
        self.fwd_gather = comm.make(AllGather, "tp", "head.fwd_ag") if self.tp > 1 and self.sp else None
        self.bwd_scatter = comm.make(ReduceScatter, "tp", "head.bwd_rs") if self.tp > 1 and self.sp else None

    def forward(self, x, labels, loss_weight):
        return _HeadLossFn.apply(x, self, labels, loss_weight, torch.is_grad_enabled())


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, module):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        y, rstd = K.rmsnorm_fwd(x2, module.weight, module.eps)
        ctx.save_for_backward(x2, rstd)
        ctx.module, ctx.shp = module, shp
        return y.reshape(shp)

    @staticmethod
    def backward(ctx, dy):
        x2, rstd = ctx.saved_tensors
        dx, dw = K.rmsnorm_bwd(dy.reshape(-1, ctx.shp[-1]).contiguous(), x2, rstd, ctx.module.weight)
        accumulate_grad(ctx.module.weight, dw)
        return dx.reshape(ctx.shp), None


class GPTModel(nn.Module):
    """One pipeline stage of a Llama-style decoder.

    ``forward(tokens, labels, loss_mask)`` with ``[b, s]`` tensors returns the summed masked
    token loss divided by ``loss_denominator`` (first/last stage duties depend on ``pre_process``
    / ``post_process``; middle stages take and return hidden-state lists).
    """

    def __init__(self, cfg: ModelConfig, par: Optional[ParallelConfig] = None, mesh=None,
                 comm: Optional[CommFactory] = None, dtype="bf16", device=None, seed: int = 42,
                 pre_process: bool = True, post_process: bool = True,
                 layer_range: Optional[range] = None, recompute_layers: Optional[int] = None,
                 sync: str = "partition_end", micro_batch_size: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        self.par = par or ParallelConfig()
        self.mesh = mesh
        self.comm = comm or CommFactory(mesh, self.par.comm_backend)
        dt = _torch_dtype(dtype)
        self.dtype, self.device = dt, device
        self.pre_process, self.post_process = pre_process, post_process
        layer_range = layer_range if layer_range is not None else range(cfg.num_layers)
        self.embedding = VocabParallelEmbedding(cfg, self.par, self.comm, dt, device, seed + 1) if pre_process else None
        # nanobatches split the batch when it is large enough, otherwise the sequence (MBS = 1)
        d = self.par.nano_split_dim
        if d == "auto":
            d = "seq" if (micro_batch_size is not None and micro_batch_size % self.par.num_nanobatches) else "batch"
        self.seq_split = d == "seq" and self.par.num_nanobatches > 1
        self.decoder = TransformerBlock(cfg, self.par, self.comm, layer_range, dt, device, seed=seed,
                                        recompute_layers=recompute_layers, sync=sync, seq_split=self.seq_split)
        if post_process:
            self.final_norm = RMSNormOp(cfg.hidden_size, cfg.norm_eps, "final_layernorm", dtype=dt,
                                        device=device, sequence_parallel=self.par.sequence_parallel)
            tied = self.embedding.weight if (cfg.tie_embeddings and pre_process) else None
            # tied weights on different pipeline stages: the last stage holds a copy with the same
            # initial values (same seed as the embedding); finalize_grads sums the two gradients so
            # both copies take identical updates (Megatron: copy of the init + all-reduce of the shared
            # embedding gradients over the embedding group)
            head_seed = seed + 1 if (cfg.tie_embeddings and not pre_process) else seed + 2
            self.output_layer = OutputHead(cfg, self.par, self.comm, dt, device, head_seed, tied_weight=tied)
        self.tied_across_stages = bool(cfg.tie_embeddings and (pre_process != post_process)
                                       and mesh is not None and mesh.pp > 1)
        if self.tied_across_stages:
            w = self.embedding.weight if pre_process else self.output_layer.weight
            w.shared_embedding = True
            # the copy on the last stage is left out of the global gradient norm (counted once)
            w.norm_exclude = not pre_process
        self._rope_cache: Dict[Tuple, torch.Tensor] = {}

    # ------------------------------------------------------------------ helpers
    @property
    def n(self) -> int:
        return self.par.num_nanobatches

    def rotary(self, s_local: int, device) -> torch.Tensor:
        """Angle table for this rank's sequence positions (dual-chunk slice under CP)."""
        cp = self.par.cp
        cp_rank = self.comm._args("cp")[2]
        key = (s_local, cp, cp_rank, str(device))
        t = self._rope_cache.get(key)
        if t is None:
            if cp == 1:
                t = ref.rope_table(s_local, self.cfg.hd, self.cfg.rope_theta, device=device)
            else:
                c = s_local // 2
                a, b = dual_chunk_ids(cp, cp_rank)
                pos = torch.cat([torch.arange(a * c, (a + 1) * c), torch.arange(b * c, (b + 1) * c)]).to(device)
                t = ref.rope_table(s_local, self.cfg.hd, self.cfg.rope_theta, device=device, positions=pos)
            self._rope_cache[key] = t
        return t

    def split_nanobatches(self, t_bs: torch.Tensor) -> List[torch.Tensor]:
        """``[b, s]`` → N tensors ``[s, b/N]`` (batch split) or ``[s/N, b]`` (sequence split), each in
        sequence-major token order."""
        if self.seq_split:
            if t_bs.shape[1] % self.n:
                raise ValueError("sequence length must be divisible by the number of nanobatches")
            return [c.t().contiguous() for c in t_bs.chunk(self.n, dim=1)]
        if t_bs.shape[0] % self.n:
            raise ValueError(f"micro batch {t_bs.shape[0]} is not divisible by {self.n} nanobatches; "
                             "build the model with nano_split_dim='seq'")
        return [c.t().contiguous() for c in t_bs.chunk(self.n, dim=0)]

    # ------------------------------------------------------------------ forward
    def embed(self, tokens: torch.Tensor) -> List[torch.Tensor]:
        return [self.embedding(t) for t in self.split_nanobatches(tokens)]

    def run_block(self, hidden: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        s_local = hidden[0].shape[0] * (self.par.tp if self.par.sequence_parallel else 1)
        if self.seq_split:
            full = self.rotary(s_local * self.n, hidden[0].device)
            return self.decoder(hidden, [full[i * s_local:(i + 1) * s_local] for i in range(self.n)])
        return self.decoder(hidden, self.rotary(s_local, hidden[0].device))

    def head_loss(self, hidden: Sequence[torch.Tensor], labels: torch.Tensor, loss_mask: torch.Tensor,
                  loss_denominator: Optional[float] = None) -> torch.Tensor:
        lab = self.split_nanobatches(labels)
        msk = self.split_nanobatches(loss_mask)
        if loss_denominator is None:
            loss_denominator = float(loss_mask.sum().item()) or 1.0
        total = None
        for h, l, m in zip(hidden, lab, msk):
            y = _NormFn.apply(h, self.final_norm)
            acc = torch.float64 if self.dtype == torch.float64 else torch.float32
            part = self.output_layer(y, l, m.to(acc) / loss_denominator)
            total = part if total is None else total + part
        return total

    def forward(self, tokens=None, labels=None, loss_mask=None, hidden=None, loss_denominator=None):
        if self.pre_process:
            hidden = self.embed(tokens)
        hidden = self.run_block(hidden)
        if not self.post_process:
            return hidden
        return self.head_loss(hidden, labels, loss_mask, loss_denominator)

    # ------------------------------------------------------------------ grads
    def finalize_grads(self) -> None:
        """Move autograd ``.grad`` into ``main_grad`` and all-reduce sequence-parallel parameter
        gradients over TP (Megatron ``finalize_model_grads``)."""
        sp_params = []
        for p in self.parameters():
            if p.grad is not None:
                accumulate_grad(p, p.grad)
                p.grad = None
            partial = (getattr(p, "sequence_parallel", False) and self.par.sequence_parallel) \
                or getattr(p, "tp_partial_grad", False)
            if partial and getattr(p, "main_grad", None) is not None:
                sp_params.append(p)
        if self.tied_across_stages:
            w = self.embedding.weight if self.pre_process else self.output_layer.weight
            dist.all_reduce(ensure_main_grad(w), group=self.mesh.group("embd"))
        tp_group, tp, _ = self.comm._args("tp")
        if tp > 1 and sp_params:
            flat = torch.cat([p.main_grad.reshape(-1) for p in sp_params])
            dist.all_reduce(flat, group=tp_group)
            o = 0
            for p in sp_params:
                n = p.main_grad.numel()
                p.main_grad.copy_(flat[o:o + n].view_as(p.main_grad))
                o += n

    def zero_grad_buffers(self) -> None:
        for p in self.parameters():
            mg = getattr(p, "main_grad", None)
            if mg is not None:
                mg.zero_()
            p.grad = None
