"""Collective operators that the partition engine schedules on the side stream.

Each operator exposes ``run(tensors, sm_num, block_size, backward, nb, ctx) -> tensors``.  Two
backends: ``"nccl"`` goes through ``torch.distributed`` (NCCL on GPUs, gloo on CPU), ``"kernel"``
uses this package's all-pairs kernels over the symmetric heap, launched with ``sm_num`` CTAs of
``block_size`` threads — the two knobs a plan entry carries.  If a plan gives no launch shape the
kernel backend falls back to the library call, like the reference's operators
(``kareus/transformer_engine/pytorch/ops/basic/all_reduce.py:135-178``,
``all_gather_kv.py:116-204``, ``reduce_scatter_kv.py:117-207``).

Buffers are owned per nanobatch: every operator instance is created for one group and indexes
its symmetric buffers by ``nb``, so two nanobatches never alias each other's staging memory.
"""
from __future__ import annotations

import re
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


class CollectiveBase:
    needs_ctx = False
    group_name = "tp"

    def __init__(self, group, world: int, rank: int, backend: str = "nccl", heap=None, name: str = ""):
        self.group = group
        self.world = int(world)
        self.rank = int(rank)
        self.backend = backend
        if heap is not None and (int(heap.world) != int(world) or int(heap.rank) != int(rank)):
            # a heap maps the memory of ONE process group; running this collective over it would sum
            # or gather across the wrong set of ranks
            raise ValueError(f"{name or type(self).__name__}: symmetric heap spans {heap.world} ranks (rank "
                             f"{heap.rank}) but the collective's group has {world} (rank {rank})")
        self.heap = heap
        self.name = name or type(self).__name__
        # heap buffers are shared by the same call site of every layer (layers run one after another
        # on the ordered side stream), so the tag drops the layer index
        self.tag = re.sub(r"layers\.\d+\.", "", self.name)
        self.calls = 0

    def staging(self, shape, dtype, nb: int, device) -> Optional[torch.Tensor]:
        """Heap buffer this collective reads its input from (kernel backend only), so the producing
        GEMM can write there directly; ``None`` when the library path is used."""
        if self.backend == "kernel" and self.heap is not None and self.world > 1 and device.type == "cuda" \
                and dtype == torch.bfloat16 and self.staging_kind is not None:
            return self.heap.staging(self.staging_kind, self.tag, nb, shape, dtype)
        return None

    staging_kind: Optional[str] = None

    def _use_kernel(self, t, sm_num) -> bool:
        # the heap kernels sum and move bf16 only; every other dtype (fp32/fp64 numerics runs) takes
        # the torch.distributed path
        return (self.backend == "kernel" and self.heap is not None and sm_num is not None
                and isinstance(t, torch.Tensor) and t.is_cuda and self.world > 1
                and t.dtype == torch.bfloat16)


class AllReduce(CollectiveBase):
    """In-place sum over the group."""

    staging_kind = "ar"

    def run(self, tensors, sm_num=None, block_size=None, backward=False, nb=0, ctx=None):
        (x,) = tensors
        self.calls += 1
        if self.world == 1:
            return (x,)
        if self._use_kernel(x, sm_num):
            return (self.heap.all_reduce(x, nb=nb, sm_num=sm_num, block_size=block_size, tag=self.tag),)
        if not x.is_contiguous():
            x = x.contiguous()
        dist.all_reduce(x, group=self.group)
        return (x,)


class AllGather(CollectiveBase):
    """Gather along dim 0 (sequence shards → full sequence)."""

    def run(self, tensors, sm_num=None, block_size=None, backward=False, nb=0, ctx=None):
        (x,) = tensors
        self.calls += 1
        if self.world == 1:
            return (x,)
        if self._use_kernel(x, sm_num):
            # the forward gather feeds a linear layer that keeps its input for wgrad
            return (self.heap.all_gather(x, nb=nb, sm_num=sm_num, block_size=block_size, tag=self.tag,
                                         keep=not backward),)
        x = x.contiguous()
        out = torch.empty((x.shape[0] * self.world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=self.group)
        return (out,)


class ReduceScatter(CollectiveBase):
    """Sum over the group, each rank keeps its dim-0 shard."""

    staging_kind = "rs"

    def run(self, tensors, sm_num=None, block_size=None, backward=False, nb=0, ctx=None):
        (x,) = tensors
        self.calls += 1
        if self.world == 1:
            return (x,)
        if x.shape[0] % self.world:
            raise ValueError(f"{self.name}: dim 0 ({x.shape[0]}) not divisible by group size {self.world}")
        if self._use_kernel(x, sm_num):
            return (self.heap.reduce_scatter(x, nb=nb, sm_num=sm_num, block_size=block_size, tag=self.tag),)
        x = x.contiguous()
        out = torch.empty((x.shape[0] // self.world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        if x.is_cuda:
            dist.reduce_scatter_tensor(out, x, group=self.group)
        else:  # gloo has no reduce_scatter_tensor
            dist.all_reduce(x, group=self.group)
            n = out.shape[0]
            out.copy_(x[self.rank * n:(self.rank + 1) * n])
        return (out,)


# ----------------------------------------------------------------------------- context parallel
def dual_chunk_ids(cp: int, rank: int) -> Tuple[int, int]:
    """Sequence chunks owned by a CP rank: ``r`` and ``2cp-1-r`` (causal load balance; reference
    ``kareus/nemo/.../megatron_gpt_model.py:1036-1056``)."""
    return rank, 2 * cp - 1 - rank


def to_sequence_order(gathered: torch.Tensor, cp: int) -> torch.Tensor:
    """``[cp*2c, ...]`` in rank order (rank j holds chunks j and 2cp-1-j) → sequence order."""
    c = gathered.shape[0] // (2 * cp)
    chunks = gathered.reshape((cp, 2, c) + tuple(gathered.shape[1:]))
    order = [None] * (2 * cp)
    for j in range(cp):
        a, b = dual_chunk_ids(cp, j)
        order[a] = chunks[j, 0]
        order[b] = chunks[j, 1]
    return torch.cat(order, dim=0)


def to_rank_order(seq: torch.Tensor, cp: int) -> torch.Tensor:
    c = seq.shape[0] // (2 * cp)
    chunks = seq.reshape((2 * cp, c) + tuple(seq.shape[1:]))
    out = []
    for j in range(cp):
        a, b = dual_chunk_ids(cp, j)
        out += [chunks[a], chunks[b]]
    return torch.cat(out, dim=0)


def half_to_sequence_order(gathered: torch.Tensor, cp: int, half: int) -> torch.Tensor:
    """One chunk per rank (sequence-split nanobatch ``half`` of a dual-chunk layout): rank j contributed global
    chunk j (half 0: already in sequence order) or 2cp-1-j (half 1: reverse the ranks).  Its own inverse."""
    if half == 0:
        return gathered
    c = gathered.shape[0] // cp
    chunks = gathered.reshape((cp, c) + tuple(gathered.shape[1:]))
    return chunks.flip(0).reshape(gathered.shape)


class AllGatherKV(CollectiveBase):
    """CP all-gather of K and V into full-length, sequence-ordered tensors.

    ``half_mode`` (sequence-split nanobatches, two per microbatch): nanobatch ``nb`` carries one of this
    rank's two chunks, so the gathered tensor is one half of the sequence: chunks 0..cp-1 for nanobatch 0,
    cp..2cp-1 for nanobatch 1."""

    group_name = "cp"
    half_mode = False

    def run(self, tensors, sm_num=None, block_size=None, backward=False, nb=0, ctx=None):
        k, v = tensors
        self.calls += 1
        if self.world == 1:
            return (k, v)
        outs = []
        for t in (k, v):
            t = t.contiguous()
            if self._use_kernel(t, sm_num):
                g = self.heap.all_gather(t, nb=nb, sm_num=sm_num, block_size=block_size,
                                         tag=self.tag + ("_k" if t is k else "_v"))
            else:
                g = torch.empty((t.shape[0] * self.world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
                dist.all_gather_into_tensor(g, t, group=self.group)
            outs.append(half_to_sequence_order(g, self.world, nb) if self.half_mode
                        else to_sequence_order(g, self.world))
        return tuple(outs)


class ReduceScatterKV(CollectiveBase):
    """CP reduce-scatter of full-length, sequence-ordered dK and dV (``half_mode``: of one half of the
    sequence, see :class:`AllGatherKV`)."""

    group_name = "cp"
    staging_kind = "rs"
    half_mode = False

    def reduce_rows(self, x, nb=0, sm_num=16, block_size=1024):
        """Plain dim-0 reduce-scatter of a tensor that is already in rank order (the chunked attention
        backward writes dK|dV per rank straight into :meth:`staging`)."""
        self.calls += 1
        if self.world == 1:
            return x
        if self._use_kernel(x, sm_num):
            return self.heap.reduce_scatter(x, nb=nb, sm_num=sm_num, block_size=block_size, tag=self.tag)
        x = x.contiguous()
        out = torch.empty((x.shape[0] // self.world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        if x.is_cuda:
            dist.reduce_scatter_tensor(out, x, group=self.group)
        else:
            dist.all_reduce(x, group=self.group)
            n = out.shape[0]
            out.copy_(x[self.rank * n:(self.rank + 1) * n])
        return out

    def run(self, tensors, sm_num=None, block_size=None, backward=False, nb=0, ctx=None):
        dk, dv = tensors
        self.calls += 1
        if self.world == 1:
            return (dk, dv)
        outs = []
        for t in (dk, dv):
            t = (half_to_sequence_order(t, self.world, nb) if self.half_mode
                 else to_rank_order(t, self.world)).contiguous()
            if self._use_kernel(t, sm_num):
                o = self.heap.reduce_scatter(t, nb=nb, sm_num=sm_num, block_size=block_size,
                                             tag=self.tag + ("_k" if t is dk else "_v"))
            else:
                o = torch.empty((t.shape[0] // self.world,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
                if t.is_cuda:
                    dist.reduce_scatter_tensor(o, t, group=self.group)
                else:
                    dist.all_reduce(t, group=self.group)
                    n = o.shape[0]
                    o.copy_(t[self.rank * n:(self.rank + 1) * n])
            outs.append(o)
        return tuple(outs)


class CommFactory:
    """Creates the collective operators of one model for a mesh/backend pair."""

    def __init__(self, mesh=None, backend: str = "nccl", heap=None, heap_cp=None):
        self.mesh = mesh
        self.backend = backend
        self.heap = heap              # symmetric heap of the tensor-parallel group
        self.heap_cp = heap_cp        # symmetric heap of the context-parallel group

    def heap_for(self, axis: str):
        """The heap that maps the memory of ``axis``'s group, or ``None`` (library collectives)."""
        return {"tp": self.heap, "cp": self.heap_cp}.get(axis)

    def _args(self, axis: str):
        if self.mesh is None:
            return None, 1, 0
        return self.mesh.group(axis), self.mesh.size(axis), self.mesh.axis_rank(axis)

    def make(self, cls, axis: str, name: str):
        g, w, r = self._args(axis)
        return cls(g, w, r, backend=self.backend, heap=self.heap_for(axis), name=name)
