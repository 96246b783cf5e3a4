"""Plain PyTorch statements of every kernel's math.

These are the numerical oracle for the sm_100a kernels (tests compare a kernel against the same
function evaluated in fp32) and the implementation used for CPU tensors, which is how the engine
runs under ``gloo`` without a GPU.  Shapes follow the engine's layout: activations are
``[tokens, features]`` with tokens ordered ``(s, b)``; attention tensors are ``[s, b, heads, d]``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def _acc(x: torch.Tensor) -> torch.dtype:
    return torch.float64 if x.dtype == torch.float64 else torch.float32


# ----------------------------------------------------------------------------- RMSNorm
def rmsnorm_fwd(x, w, eps: float):
    xf = x.to(_acc(x))
    rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
    y = (xf * rstd.unsqueeze(-1) * w.to(xf.dtype)).to(x.dtype)
    return y, rstd


def rmsnorm_bwd(dy, x, rstd, w):
    acc = _acc(x)
    xf, dyf, wf = x.to(acc), dy.to(acc), w.to(acc)
    xhat = xf * rstd.unsqueeze(-1)
    g = dyf * wf
    c = (g * xhat).mean(-1, keepdim=True)
    dx = ((g - xhat * c) * rstd.unsqueeze(-1)).to(x.dtype)
    dw = (dyf * xhat).reshape(-1, x.shape[-1]).sum(0)
    return dx, dw


# ----------------------------------------------------------------------------- RoPE
def rope_table(seq_len: int, dim: int, theta: float, device=None, offset: int = 0,
               positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``[s, dim]`` fp32 angles, halves duplicated (rotate-half convention; reference
    ``3rdparty/Megatron-LM/megatron/core/models/common/embeddings/rotary_pos_embedding.py:161-171``)."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    pos = positions.to(torch.float32) if positions is not None else \
        torch.arange(offset, offset + seq_len, dtype=torch.float32, device=device)
    fr = torch.outer(pos, inv)
    return torch.cat([fr, fr], dim=-1)


def rope_apply(t, freqs, inverse: bool = False):
    """Rotate ``t [s, b, h, d]`` by ``freqs [s, d]``; ``inverse`` applies the transpose (backward)."""
    acc = _acc(t)
    tf = t.to(acc)
    bshape = (freqs.shape[0],) + (1,) * (t.dim() - 2) + (freqs.shape[-1],)
    cos = freqs.cos().to(acc).reshape(bshape)
    sin = freqs.sin().to(acc).reshape(bshape)
    if inverse:
        sin = -sin
    d = t.shape[-1]
    t1, t2 = tf[..., : d // 2], tf[..., d // 2:]
    rot = torch.cat([-t2, t1], dim=-1)
    return (tf * cos + rot * sin).to(t.dtype)


# ----------------------------------------------------------------------------- SwiGLU
def swiglu_fwd(x):
    a, b = x.chunk(2, dim=-1)
    acc = _acc(x)
    return (F.silu(a.to(acc)) * b.to(acc)).to(x.dtype)


def swiglu_bwd(dy, x):
    acc = _acc(x)
    a, b = x.chunk(2, dim=-1)
    a, b, g = a.to(acc), b.to(acc), dy.to(acc)
    s = torch.sigmoid(a)
    da = g * b * (s * (1 + a * (1 - s)))
    db = g * (a * s)
    return torch.cat([da, db], dim=-1).to(x.dtype)


# ----------------------------------------------------------------------------- dropout + residual
def dropout_mask(shape, p: float, seed: int, device) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed) & 0x7FFFFFFFFFFFFFFF)
    return (torch.rand(shape, generator=g, device="cpu") >= p).to(device)


def dropout_add_fwd(x, residual, p: float, seed: int, bias=None):
    acc = _acc(x)
    v = x.to(acc)
    if bias is not None:
        v = v + bias.to(acc)
    if p > 0.0:
        m = dropout_mask(x.shape, p, seed, x.device)
        v = v * m.to(acc) / (1.0 - p)
    return (residual.to(acc) + v).to(x.dtype)


def dropout_add_bwd(dy, p: float, seed: int):
    """Returns ``(dx, dresidual)``."""
    if p > 0.0:
        m = dropout_mask(dy.shape, p, seed, dy.device)
        dx = (dy.to(_acc(dy)) * m / (1.0 - p)).to(dy.dtype)
    else:
        dx = dy
    return dx, dy


# ----------------------------------------------------------------------------- GEMM
def gemm(a, b, trans_a: bool = False, trans_b: bool = True, out_dtype=None, accumulate=None):
    """``op(a) @ op(b)`` with fp32 accumulation; ``accumulate`` (fp32) is added to in place."""
    A = a.t() if trans_a else a
    B = b.t() if trans_b else b
    if accumulate is not None:
        accumulate.add_((A.to(_acc(a)) @ B.to(_acc(a))).to(accumulate.dtype))
        return accumulate
    out = A.to(_acc(a)) @ B.to(_acc(a)) if a.dtype in (torch.bfloat16, torch.float16) else A @ B
    return out.to(out_dtype or a.dtype)


# ----------------------------------------------------------------------------- attention
def gelu(x):
    """tanh approximation (the one Megatron's fused bias-GELU uses)."""
    xf = x.to(_acc(x))
    return (0.5 * xf * (1.0 + torch.tanh(0.7978845608028654 * xf * (1.0 + 0.044715 * xf * xf)))).to(x.dtype)


def bias_act(y, bias=None, activation=None):
    """Epilogue of a linear layer: ``act(y + bias)``."""
    if bias is not None:
        y = (y.to(_acc(y)) + bias.to(_acc(y))).to(y.dtype)
    if activation in (None, "none"):
        return y
    if activation == "gelu":
        return gelu(y)
    raise ValueError(f"unknown activation {activation!r}")


def _heads4(t):
    """``[s,b,g,rep,d]`` → ``[s,b,g*rep,d]`` (copy if the strides need it)."""
    if t.dim() == 5:
        return t.reshape(t.shape[0], t.shape[1], t.shape[2] * t.shape[3], t.shape[4])
    return t


def attention_fwd(q, k, v, scale: float, causal: bool = True, q_offset: int = 0,
                  kv_len: Optional[int] = None):
    """GQA attention on ``[s, b, h, d]`` tensors.  Returns ``(out [sq,b,hq,d], lse [b,hq,sq] fp32)``.

    ``q_offset`` is the absolute position of the first query row relative to the first key row
    (used when queries are a slice of the sequence); ``kv_len`` limits the visible keys.
    """
    q = _heads4(q)
    sq, b, hq, d = q.shape
    sk = k.shape[0] if kv_len is None else kv_len
    hk = k.shape[2]
    rep = hq // hk
    acc = _acc(q)
    qf = q.to(acc).permute(1, 2, 0, 3)                       # b hq sq d
    kf = k[:sk].to(acc).permute(1, 2, 0, 3).repeat_interleave(rep, dim=1)
    vf = v[:sk].to(acc).permute(1, 2, 0, 3).repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        qi = torch.arange(sq, device=q.device)[:, None] + q_offset
        ki = torch.arange(sk, device=q.device)[None, :]
        s = s.masked_fill(ki > qi, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.matmul(p, vf).permute(2, 0, 1, 3).contiguous().to(q.dtype)
    return o, lse.to(_acc(q))


def attention_bwd(do, q, k, v, o, lse, scale: float, causal: bool = True, q_offset: int = 0,
                  kv_len: Optional[int] = None):
    q_shape = q.shape
    q, do, o = _heads4(q), _heads4(do), _heads4(o)
    sq, b, hq, d = q.shape
    sk_full = k.shape[0]
    sk = sk_full if kv_len is None else kv_len
    hk = k.shape[2]
    rep = hq // hk
    acc = _acc(q)
    qf = q.to(acc).permute(1, 2, 0, 3)
    kf = k[:sk].to(acc).permute(1, 2, 0, 3).repeat_interleave(rep, dim=1)
    vf = v[:sk].to(acc).permute(1, 2, 0, 3).repeat_interleave(rep, dim=1)
    dof = do.to(acc).permute(1, 2, 0, 3)
    of = o.to(acc).permute(1, 2, 0, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        qi = torch.arange(sq, device=q.device)[:, None] + q_offset
        ki = torch.arange(sk, device=q.device)[None, :]
        s = s.masked_fill(ki > qi, float("-inf"))
    p = torch.nan_to_num(torch.exp(s - lse.to(acc).unsqueeze(-1)), nan=0.0)
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    dq = dq.permute(2, 0, 1, 3).contiguous().to(q.dtype).reshape(q_shape)
    dk = dk.reshape(b, hk, rep, sk, d).sum(2).permute(2, 0, 1, 3)
    dv = dv.reshape(b, hk, rep, sk, d).sum(2).permute(2, 0, 1, 3)
    dk_full = torch.zeros_like(k)
    dv_full = torch.zeros_like(v)
    dk_full[:sk] = dk.to(k.dtype)
    dv_full[:sk] = dv.to(v.dtype)
    return dq, dk_full, dv_full


def merge_attention(o1, lse1, o2, lse2):
    """Combine two partial attention results over disjoint key sets (log-sum-exp algebra;
    reference ``3rdparty/TransformerEngine/.../context_parallel.py:94-162``).
    ``o`` is ``[s,b,h,d]``, ``lse`` is ``[b,h,s]``."""
    lse = torch.logaddexp(lse1, lse2)
    w1 = torch.exp(lse1 - lse).permute(2, 0, 1).unsqueeze(-1)
    w2 = torch.exp(lse2 - lse).permute(2, 0, 1).unsqueeze(-1)
    w1 = torch.nan_to_num(w1, nan=0.0)
    w2 = torch.nan_to_num(w2, nan=0.0)
    o = (o1.to(torch.float32) * w1 + o2.to(torch.float32) * w2).to(o1.dtype)
    return o, lse


def _logical_kv(sources, table, chunk_rows):
    k = torch.cat([sources[src][0][base:base + chunk_rows] for src, base in table], dim=0)
    v = torch.cat([sources[src][1][base:base + chunk_rows] for src, base in table], dim=0)
    return k, v


def attention_fwd_chunked(q, sources, table, chunk_rows: int, q_positions, scale: float, causal: bool = True):
    """Attention over a logical key sequence that is stored as chunks of ``chunk_rows`` keys in several
    buffers (``sources[i] = (k_i, v_i)``; logical chunk ``c`` is rows ``base .. base+chunk_rows`` of source
    ``src`` with ``table[c] = (src, base)``).  The local queries are ``len(q_positions)`` equal chunks whose
    first rows sit at those absolute positions.  Returns ``(out [sq,b,h,d], lse [b,h,sq])``."""
    k, v = _logical_kv(sources, table, chunk_rows)
    qc = q.shape[0] // len(q_positions)
    outs, lses = [], []
    for i, pos in enumerate(q_positions):
        o, l = attention_fwd(q[i * qc:(i + 1) * qc], k, v, scale, causal, q_offset=pos,
                             kv_len=min(k.shape[0], pos + qc) if causal else None)
        outs.append(o)
        lses.append(l)
    return torch.cat(outs, dim=0), torch.cat(lses, dim=-1)


def attention_bwd_chunked(do, q, sources, table, chunk_rows: int, q_positions, o, lse, scale: float,
                          causal: bool = True):
    """Gradients of :func:`attention_fwd_chunked`: ``(dq, dk, dv)`` with dk/dv over the LOGICAL key
    sequence (``len(table) * chunk_rows`` rows)."""
    k, v = _logical_kv(sources, table, chunk_rows)
    qc = q.shape[0] // len(q_positions)
    h = o.shape[-2]
    do4 = do.reshape(q.shape[0], q.shape[1], h, -1)
    acc = _acc(q)
    dk = torch.zeros(k.shape, dtype=acc, device=k.device)
    dv = torch.zeros(v.shape, dtype=acc, device=v.device)
    dqs = []
    for i, pos in enumerate(q_positions):
        sl = slice(i * qc, (i + 1) * qc)
        dq_i, dk_i, dv_i = attention_bwd(do4[sl], q[sl], k, v, o[sl], lse[..., sl], scale, causal, q_offset=pos,
                                         kv_len=min(k.shape[0], pos + qc) if causal else None)
        dqs.append(dq_i)
        dk += dk_i.to(acc)
        dv += dv_i.to(acc)
    return torch.cat(dqs, dim=0), dk.to(k.dtype), dv.to(v.dtype)


# ----------------------------------------------------------------------------- cross entropy
def cross_entropy_local_stats(logits, targets, vocab_start: int):
    """Per-row ``(max, sum exp(x - max), target logit or 0)`` over this rank's vocab shard."""
    lf = logits.to(_acc(logits))
    m = lf.max(dim=-1).values
    se = torch.exp(lf - m.unsqueeze(-1)).sum(-1)
    v = logits.shape[-1]
    local = targets - vocab_start
    inside = (local >= 0) & (local < v)
    idx = local.clamp(0, v - 1)
    tl = torch.where(inside, lf.gather(-1, idx.unsqueeze(-1)).squeeze(-1), torch.zeros_like(m))
    return m, se, tl


def cross_entropy_finish(logits, targets, vocab_start: int, gmax, gsum, grad_scale):
    """In-place gradient ``(softmax - onehot) * grad_scale[row]`` given the global max and sum."""
    lf = logits.to(_acc(logits))
    p = torch.exp(lf - gmax.unsqueeze(-1)) / gsum.unsqueeze(-1)
    v = logits.shape[-1]
    local = targets - vocab_start
    inside = (local >= 0) & (local < v)
    idx = local.clamp(0, v - 1)
    onehot = torch.zeros_like(p)
    onehot.scatter_(-1, idx.unsqueeze(-1), inside.to(p.dtype).unsqueeze(-1))
    g = (p - onehot) * grad_scale.unsqueeze(-1)
    logits.copy_(g.to(logits.dtype))
    return logits


# ----------------------------------------------------------------------------- optimizer
def adamw_step(p, g, m, v, master, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    """One AdamW update on fp32 ``master`` with moments ``m, v``; ``p`` gets the rounded copy."""
    gf = g.to(torch.float32) * grad_scale
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (v / bc2).sqrt_().add_(eps)
    master.mul_(1 - lr * wd).addcdiv_(m / bc1, denom, value=-lr)
    if p is not master:
        p.copy_(master.to(p.dtype))


def sumsq(t) -> torch.Tensor:
    return t.to(torch.float32).pow(2).sum()


# ----------------------------------------------------------------------------- embedding
def embedding_fwd(tokens, weight, vocab_start: int):
    """Rows of ``weight`` for tokens in ``[vocab_start, vocab_start+V_local)``, zeros elsewhere."""
    v = weight.shape[0]
    local = tokens - vocab_start
    inside = (local >= 0) & (local < v)
    out = weight[local.clamp(0, v - 1)]
    return out * inside.unsqueeze(-1).to(out.dtype)


def embedding_bwd(dout, tokens, grad_weight, vocab_start: int):
    v = grad_weight.shape[0]
    local = (tokens - vocab_start).reshape(-1)
    inside = (local >= 0) & (local < v)
    d = dout.reshape(-1, dout.shape[-1]).to(grad_weight.dtype) * inside.unsqueeze(-1).to(grad_weight.dtype)
    grad_weight.index_add_(0, local.clamp(0, v - 1), d)
    return grad_weight
