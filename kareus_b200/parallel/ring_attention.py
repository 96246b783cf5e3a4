"""Context-parallel attention without a materialised K/V all-gather.

Every CP rank publishes its post-RoPE K and V shards in the symmetric heap; the flash-attention
kernels then read the K/V tiles of *other* ranks' chunks straight out of peer memory with their own
TMA loads (no multicast), chunk by chunk, and the partial results are merged with log-sum-exp
algebra.  With dual-chunk causal load balance (rank r owns sequence chunks r and 2cp−1−r) a query
chunk ``c`` attends to key chunks ``0..c``: all of them unmasked except the diagonal one.  This is the
arithmetic of ring attention (``3rdparty/TransformerEngine/.../context_parallel.py:94-162,676-712``,
unreachable in the reference, which all-gathers K/V instead: ``context_parallel.py:247-506``) with
pulls over NVSwitch in place of a rotating ring.

Backward re-reads the peers' K/V the same way, accumulates dK/dV for every key chunk it touched and
reduce-scatters them to their owners.

Without a heap (CPU / gloo) the K/V shards are exchanged with ``all_gather`` and the same chunk
schedule and merge run on the PyTorch statements, which is how the math is tested without GPUs.
"""
from __future__ import annotations

import re
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import kernels as K
from ..kernels import ref
from ..kernels.cuda import KernelError
from .collectives import ReduceScatterKV, dual_chunk_ids


def chunk_owner(j: int, cp: int) -> Tuple[int, int]:
    """(rank, half) holding sequence chunk ``j``."""
    return (j, 0) if j < cp else (2 * cp - 1 - j, 1)


class RingAttention:
    def __init__(self, group, cp: int, cp_rank: int, heap=None, name: str = "ring"):
        self.group, self.cp, self.rank, self.heap = group, cp, cp_rank, heap
        self.name = re.sub(r"layers\.\d+\.", "", name)      # heap buffers shared by all layers
        self.rs = ReduceScatterKV(group, cp, cp_rank, backend="kernel" if heap is not None else "nccl", heap=heap,
                                  name=self.name + ".rs_dkv")

    # ------------------------------------------------------------------ K/V publication
    def _publish(self, k, v, nb: int, tag: str) -> List[Tuple[torch.Tensor, torch.Tensor]]:
        """Returns ``[(K_r, V_r) for r in ranks]`` — peer-memory views on GPUs, gathered copies on CPU."""
        if self.heap is not None and k.is_cuda:
            if K.library_baseline():
                raise KernelError("ring attention over the symmetric heap is refused with "
                                  "KAREUS_B200_LIBRARY_BASELINE=1: the library attention kernels would receive "
                                  "peer memory; use cp_comm='all_gather' for the library baseline")
            if k.dtype != torch.bfloat16:
                raise KernelError(f"ring attention over the symmetric heap needs bf16 K/V, got {k.dtype}")
            heap = self.heap
            ch = heap.channel(f"{self.name}/{tag}/{nb}")
            n = k.numel() * k.element_size()
            off, _ = heap.buffer(ch, "kv", 2 * n)
            heap.barrier(ch)                                   # peers finished reading the previous contents
            heap.view(off, k.shape, k.dtype).copy_(k)
            heap.view(off + n, v.shape, v.dtype).copy_(v)
            heap.barrier(ch)                                   # everyone's shards are in place
            return [(heap.peer_view(r, off, k.shape, k.dtype), heap.peer_view(r, off + n, v.shape, v.dtype))
                    for r in range(self.cp)]
        ks = [torch.empty_like(k) for _ in range(self.cp)]
        vs = [torch.empty_like(v) for _ in range(self.cp)]
        dist.all_gather(ks, k.contiguous(), group=self.group)
        dist.all_gather(vs, v.contiguous(), group=self.group)
        return list(zip(ks, vs))

    def _peer(self, k) -> bool:
        """True when ``_publish`` hands out views of other GPUs' memory: every attention call must then
        be announced as such (``peer=True``), which pins it to this package's own kernels."""
        return self.heap is not None and k.is_cuda

    def _kv_chunk(self, kv, j: int, c: int):
        r, half = chunk_owner(j, self.cp)
        return kv[r][0][half * c:(half + 1) * c], kv[r][1][half * c:(half + 1) * c]

    # ------------------------------------------------------------------ forward / backward
    def forward(self, q, k, v, scale: float, nb: int = 0):
        s = q.shape[0]
        c = s // 2
        kv = self._publish(k, v, nb, "fwd")
        peer = self._peer(k)
        outs, lses = [], []
        for half, cid in enumerate(dual_chunk_ids(self.cp, self.rank)):
            qc = q[half * c:(half + 1) * c]
            o = lse = None
            for j in range(cid + 1):
                kj, vj = self._kv_chunk(kv, j, c)
                oj, lj = K.attention_fwd(qc, kj, vj, scale, causal=(j == cid), peer=peer)
                if o is None:
                    o, lse = oj, lj
                else:
                    o, lse = ref.merge_attention(o, lse, oj, lj)
            outs.append(o)
            lses.append(lse)
        return torch.cat(outs, dim=0), torch.stack(lses, dim=0)       # lse: [2, b, h, c]

    def backward(self, do, q, k, v, out, lse, scale: float, out_grads=None, nb: int = 0):
        s = q.shape[0]
        c = s // 2
        kv = self._publish(k, v, nb, "bwd")
        peer = self._peer(k)
        acc = torch.float64 if q.dtype == torch.float64 else torch.float32
        dk_full = torch.zeros((2 * self.cp * c,) + tuple(k.shape[1:]), dtype=acc, device=k.device)
        dv_full = torch.zeros_like(dk_full)
        dqs = []
        for half, cid in enumerate(dual_chunk_ids(self.cp, self.rank)):
            sl = slice(half * c, (half + 1) * c)
            dq = None
            for j in range(cid + 1):
                kj, vj = self._kv_chunk(kv, j, c)
                dqj, dkj, dvj = K.attention_bwd(do[sl], q[sl], kj, vj, out[sl], lse[half], scale, causal=(j == cid),
                                                peer=peer)
                dq = dqj.to(acc) if dq is None else dq + dqj.to(acc)
                dk_full[j * c:(j + 1) * c] += dkj.to(acc)
                dv_full[j * c:(j + 1) * c] += dvj.to(acc)
            dqs.append(dq.to(q.dtype))
        dk, dv = self.rs.run((dk_full.to(k.dtype), dv_full.to(v.dtype)), sm_num=16, nb=nb)
        dq = torch.cat(dqs, dim=0)
        if out_grads is not None:
            out_grads[0].copy_(dq.reshape(out_grads[0].shape))
            out_grads[1].copy_(dk)
            out_grads[2].copy_(dv)
            return out_grads
        return dq, dk, dv
