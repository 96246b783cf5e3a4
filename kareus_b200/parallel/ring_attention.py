"""Context-parallel attention without a materialised K/V all-gather.

Every CP rank publishes its post-RoPE K and V shards in the symmetric heap; ONE flash-attention
launch per direction then walks the whole visible key range and fetches the tiles of *other* ranks'
chunks straight out of peer memory with its own TMA loads (no multicast), picking the buffer per
chunk from a table (``csrc/attention_chunks.h``).  With dual-chunk causal load balance (rank r owns
sequence chunks r and 2cp−1−r) the local queries are two chunks with their own absolute positions;
the kernel carries the running maximum and sum across chunks, so nothing is merged afterwards.  This
is the arithmetic of ring attention (``3rdparty/TransformerEngine/.../context_parallel.py:94-162,
676-712``, unreachable in the reference, which all-gathers K/V instead:
``context_parallel.py:247-506``) with pulls over NVSwitch in place of a rotating ring.

Backward is again one launch: it re-reads the peers' K/V the same way, keeps dK/dV of every key chunk
it touched in fp32 and converts them straight into the rank-ordered input buffer of a reduce-scatter
(one all-pairs kernel over the heap) that returns each rank the sums for its own two chunks.

Per layer and direction: two peer barriers and two copies to publish K/V, one attention launch, and in
backward one reduce-scatter — instead of one launch per (query chunk, key chunk) pair with eager
merges in between.

Without a heap (CPU / gloo) the K/V shards are exchanged with ``all_gather`` and the same chunk tables
drive the PyTorch statement of the math, which is how the logic is tested without GPUs.
"""
from __future__ import annotations

import re
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import kernels as K
from ..kernels.cuda import KernelError
from .collectives import ReduceScatterKV, dual_chunk_ids


def chunk_owner(j: int, cp: int) -> Tuple[int, int]:
    """(rank, half) holding sequence chunk ``j``."""
    return (j, 0) if j < cp else (2 * cp - 1 - j, 1)


def chunk_table(cp: int, c: int) -> List[Tuple[int, int]]:
    """Logical chunk → (source rank, first row in that rank's ``[2c, ...]`` shard)."""
    return [(r, half * c) for r, half in (chunk_owner(j, cp) for j in range(2 * cp))]


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

    def _q_positions(self, c: int) -> List[int]:
        return [cid * c for cid in dual_chunk_ids(self.cp, self.rank)]

    # ------------------------------------------------------------------ forward / backward
    def forward(self, q, k, v, scale: float, nb: int = 0):
        """``q`` ``[2c, b, ...]`` (this rank's two chunks), ``k``/``v`` ``[2c, b, g, d]``.  Returns
        ``(out [2c,b,h,d], lse [b,h,2c])``."""
        c = q.shape[0] // 2
        kv = self._publish(k, v, nb, "fwd")
        return K.attention_fwd_chunked(q, kv, chunk_table(self.cp, c), c, self._q_positions(c), scale, causal=True,
                                       peer=self._peer(k))

    def backward(self, do, q, k, v, out, lse, scale: float, out_grads=None, nb: int = 0):
        c = q.shape[0] // 2
        cp = self.cp
        kv = self._publish(k, v, nb, "bwd")
        table = chunk_table(cp, c)
        # dK and dV of all 2cp chunks in the layout the reduce-scatter shards by rank: rank r's block is
        # [dK chunk r | dK chunk 2cp-1-r | dV chunk r | dV chunk 2cp-1-r]
        rows = cp * 4 * c
        shape = (rows,) + tuple(k.shape[1:])
        dkv = None
        if self._peer(k):
            dkv = self.rs.staging(shape, k.dtype, nb, k.device)     # the collective's own input buffer
        if dkv is None:
            dkv = torch.empty(shape, dtype=k.dtype, device=k.device)
        dk_base = [r * 4 * c + half * c for r, half in (chunk_owner(j, cp) for j in range(2 * cp))]
        dv_base = [b + 2 * c for b in dk_base]
        dq = out_grads[0] if out_grads is not None else torch.empty_like(q)
        K.attention_bwd_chunked(do, q, kv, table, c, self._q_positions(c), out, lse, scale, dq, dkv, dk_base, dv_base,
                                causal=True, peer=self._peer(k))
        mine = self.rs.reduce_rows(dkv, nb=nb)                      # [4c, b, g, d]: this rank's dK | dV
        dk, dv = mine[:2 * c], mine[2 * c:]
        if out_grads is not None:
            out_grads[1].copy_(dk)
            out_grads[2].copy_(dv)
            return out_grads
        return dq, dk, dv
