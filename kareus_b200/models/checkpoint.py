"""Distributed checkpoint in the Megatron layout, written as PyTorch distributed-checkpoint files.

``sharded_state_dict(model)`` describes every local tensor as a :class:`ShardedTensor` with the
reference's contract (``3rdparty/Megatron-LM/megatron/core/dist_checkpointing/mapping.py:48-87``;
module side: ``kareus/megatron/core/transformer/transformer_block.py:529-590``, ``mlp.py:141-271``,
``extensions/ops/te_linear.py:361-366,434-439``, ``models/gpt/gpt_model.py:446-495``):

* keys ``embedding.word_embeddings.weight``, ``decoder.layers.<sub>.weight`` (homogeneous layers share a
  key and get a *prepended layer axis* ``(0, global_layer_index, num_layers)``),
  ``decoder.final_layernorm.weight``, ``output_layer.weight``;
* column-parallel weights are sharded on axis 0, row-parallel on axis 1 (after the prepended axis);
* the fused SwiGLU ``linear_fc1`` weight is stored as two shards (gate and up halves) so it can be
  re-split for another TP size;
* replicated tensors carry ``replica_id = tp_rank`` (only replica 0 is written); a weight tied across
  pipeline stages is a replica of the embedding key on the last stage.

On disk (the ``torch_dist`` backend Megatron uses: ``dist_checkpointing/serialization.py:288-311,410``,
``strategies/torch.py``): ``metadata.json`` (backend name and version), ``common.pt`` (non-tensor
state) and a ``torch.distributed.checkpoint`` directory — ``.metadata`` with every tensor's global
shape and chunk list plus ``__<rank>_<n>.distcp`` data files — so
``torch.distributed.checkpoint.FileSystemReader`` reads it.  The boxes are handed to DCP through two
small planners (one write item per :class:`ShardedTensor`, read items from DCP's own chunk
intersection), which is what makes a checkpoint written under one TP x PP x DP layout load under
another.

Optimizer state follows Megatron's model-space layout (``dist_checkpointing/optimizer.py``): for every
parameter shard ``optimizer.state.{exp_avg,exp_avg_sq,fp32_param}.<param key>`` with the parameter's
own box, gathered from the data-parallel shards of the flat AdamW buffers at save time and
re-scattered at load time, so it reshards with the model.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import torch

METADATA = {"sharded_backend": "torch_dist", "sharded_backend_version": 1, "common_backend": "torch",
            "common_backend_version": 1}


@dataclass
class ShardedTensor:
    key: str
    data: Optional[torch.Tensor]
    dtype: str
    local_shape: Tuple[int, ...]
    global_shape: Tuple[int, ...]
    global_offset: Tuple[int, ...]
    axis_fragmentations: Tuple[int, ...]
    replica_id: int = 0
    prepend_axis_num: int = 0

    def meta(self) -> dict:
        d = asdict(self)
        d.pop("data")
        return d


def _st(key, t, global_shape, offset, frags, replica=0, prepend=None) -> ShardedTensor:
    local = tuple(t.shape)
    pre = 0
    if prepend is not None:
        idx, n = prepend
        local, global_shape, offset, frags = (1,) + local, (n,) + tuple(global_shape), (idx,) + tuple(offset), \
            (n,) + tuple(frags)
        pre = 1
    return ShardedTensor(key, t, str(t.dtype).replace("torch.", ""), tuple(local), tuple(global_shape),
                         tuple(offset), tuple(frags), replica, pre)


def sharded_state_dict(model, tp_rank: int = 0, tp: int = 1, dp_rank: int = 0) -> List[ShardedTensor]:
    cfg = model.cfg
    L = cfg.num_layers
    out: List[ShardedTensor] = []
    rep = tp_rank + tp * dp_rank           # replicas beyond (tp 0, dp 0) are not written

    def col(key, w, layer=None, replica=0):           # sharded on axis 0
        g = (w.shape[0] * tp, w.shape[1])
        out.append(_st(key, w, g, (tp_rank * w.shape[0], 0), (tp, 1), dp_rank + replica, layer))

    def row(key, w, layer=None):           # sharded on axis 1
        g = (w.shape[0], w.shape[1] * tp)
        out.append(_st(key, w, g, (0, tp_rank * w.shape[1]), (1, tp), dp_rank, layer))

    def repl(key, w, layer=None):
        out.append(_st(key, w, tuple(w.shape), (0,) * w.dim(), (1,) * w.dim(), rep, layer))

    if model.embedding is not None:
        col("embedding.word_embeddings.weight", model.embedding.weight.data)
    for layer in model.decoder.layers:
        pre = (layer.layer_number, L)
        p = "decoder.layers."
        repl(p + "input_layernorm.weight", layer.input_norm.weight.data, pre)
        col(p + "self_attention.linear_qkv.weight", layer.qkv.weight.data, pre)
        if layer.qkv_post.qk_norm:
            repl(p + "self_attention.q_layernorm.weight", layer.qkv_post.q_norm_weight.data, pre)
            repl(p + "self_attention.k_layernorm.weight", layer.qkv_post.k_norm_weight.data, pre)
        row(p + "self_attention.linear_proj.weight", layer.proj.weight.data, pre)
        repl(p + "pre_mlp_layernorm.weight", layer.pre_mlp_norm.weight.data, pre)
        # SwiGLU: [gate | up] halves become two shards of one global [2F, H] tensor
        w = layer.fc1.weight.data
        f_local = w.shape[0] // 2
        for half, name in enumerate(("gate", "up")):
            part = w[half * f_local:(half + 1) * f_local]
            out.append(_st(p + "mlp.linear_fc1.weight", part, (2 * f_local * tp, w.shape[1]),
                           (half * f_local * tp + tp_rank * f_local, 0), (2 * tp, 1), dp_rank, pre))
        row(p + "mlp.linear_fc2.weight", layer.fc2.weight.data, pre)
    if model.post_process:
        repl("decoder.final_layernorm.weight", model.final_norm.weight.data)
        if not cfg.tie_embeddings:
            col("output_layer.weight", model.output_layer.weight.data)
        elif model.embedding is None:
            # tied weight whose other holder is the first pipeline stage: a replica of the embedding key
            # (never written, filled from the embedding on load)
            col("embedding.word_embeddings.weight", model.output_layer.weight.data, replica=1)
    return out


def _flat_key(s: ShardedTensor):
    return (s.key, tuple(int(o) for o in s.global_offset))


def _planners():
    """The two DCP planners, built lazily so importing this module does not import torch.distributed."""
    from torch.distributed.checkpoint.default_planner import DefaultLoadPlanner, DefaultSavePlanner
    from torch.distributed.checkpoint.metadata import ChunkStorageMetadata, MetadataIndex, TensorProperties
    from torch.distributed.checkpoint.planner import LoadPlan, SavePlan, TensorWriteData, WriteItem, WriteItemType
    from torch.distributed.checkpoint.planner_helpers import create_read_items_for_chunk_list

    class ShardSavePlanner(DefaultSavePlanner):
        """One SHARD write item per :class:`ShardedTensor` (replica 0 only)."""

        def __init__(self, shards: Sequence[ShardedTensor]):
            super().__init__(flatten_state_dict=False, flatten_sharded_tensors=False)
            self.shards = {_flat_key(s): s for s in shards}
            if len(self.shards) != len(shards):
                raise ValueError("two local shards share a key and offset")

        def create_local_plan(self):
            items = []
            for s in self.shards.values():
                t = s.data
                items.append(WriteItem(
                    index=MetadataIndex(s.key, torch.Size(s.global_offset)), type=WriteItemType.SHARD,
                    tensor_data=TensorWriteData(
                        chunk=ChunkStorageMetadata(offsets=torch.Size(s.global_offset), sizes=torch.Size(s.local_shape)),
                        properties=TensorProperties.create_from_tensor(t), size=torch.Size(s.global_shape))))
            self.plan = SavePlan(items)
            return self.plan

        def lookup_object(self, index):
            s = self.shards[(index.fqn, tuple(int(o) for o in index.offset))]
            return s.data.detach().reshape(s.local_shape).contiguous()

    class ShardLoadPlanner(DefaultLoadPlanner):
        """Read items for the wanted local boxes, by DCP's own chunk intersection."""

        def __init__(self, wants: Sequence[ShardedTensor], strict: bool = True):
            super().__init__(flatten_state_dict=False, flatten_sharded_tensors=False)
            self.wants, self.strict = list(wants), strict
            self.dest = {_flat_key(w): w.data.reshape(w.local_shape) for w in self.wants}
            for w in self.wants:
                if self.dest[_flat_key(w)].data_ptr() != w.data.data_ptr():
                    raise ValueError(f"{w.key}: destination must be contiguous")

        def create_local_plan(self):
            by_key: Dict[str, List[ShardedTensor]] = {}
            for w in self.wants:
                by_key.setdefault(w.key, []).append(w)
            reads = []
            for key, group in by_key.items():
                md = self.metadata.state_dict_metadata.get(key)
                if md is None:
                    if self.strict:
                        raise KeyError(f"checkpoint has no tensor {key!r}")
                    continue
                if tuple(md.size) != tuple(group[0].global_shape):
                    raise ValueError(f"{key}: checkpoint global shape {tuple(md.size)} != {group[0].global_shape}")
                chunks = [ChunkStorageMetadata(offsets=torch.Size(w.global_offset), sizes=torch.Size(w.local_shape))
                          for w in group]
                got = create_read_items_for_chunk_list(key, md, chunks)
                if self.strict:
                    filled: Dict[tuple, int] = {}
                    for r in got:
                        n = 1
                        for l in r.lengths:
                            n *= int(l)
                        k2 = tuple(int(o) for o in r.dest_index.offset)
                        filled[k2] = filled.get(k2, 0) + n
                    for w in group:
                        n = 1
                        for d in w.local_shape:
                            n *= d
                        if filled.get(tuple(w.global_offset), 0) != n:
                            raise KeyError(f"checkpoint covers {filled.get(tuple(w.global_offset), 0)} of {n} "
                                           f"elements of {w.key} at offset {w.global_offset}")
                reads += got
            return LoadPlan(reads)

        def lookup_tensor(self, index):
            return self.dest[(index.fqn, tuple(int(o) for o in index.offset))]

    return ShardSavePlanner, ShardLoadPlanner


# ----------------------------------------------------------------------------- optimizer state
OPT_STATES = ("exp_avg", "exp_avg_sq", "fp32_param")


def optimizer_shards(model_shards: Sequence[ShardedTensor], optimizer, full: Dict[str, torch.Tensor]) -> List[ShardedTensor]:
    """Model-space description of the AdamW state: for every parameter shard, the matching slices of
    the (data-parallel gathered) flat state buffers ``full[name]``, with the parameter's own box."""
    out: List[ShardedTensor] = []
    base, esz = optimizer.param_flat.data_ptr(), optimizer.param_flat.element_size()
    for s in model_shards:
        off = (s.data.data_ptr() - base) // esz
        n = s.data.numel()
        if not s.data.is_contiguous() or off < 0 or off + n > optimizer.total:
            raise ValueError(f"{s.key} is not a contiguous slice of the optimizer's flat parameter buffer")
        for name in OPT_STATES:
            t = full[name][off:off + n].view(s.data.shape)
            out.append(ShardedTensor(f"optimizer.state.{name}.{s.key}", t, str(t.dtype).replace("torch.", ""),
                                     s.local_shape, s.global_shape, s.global_offset, s.axis_fragmentations,
                                     s.replica_id, s.prepend_axis_num))
    return out


def _local_shards(model, tp_rank, tp, dp_rank, optimizer, for_load: bool):
    shards = sharded_state_dict(model, tp_rank, tp, dp_rank)
    full = None
    if optimizer is not None:
        full = optimizer.empty_full_state() if for_load else optimizer.gather_state()
        shards = shards + optimizer_shards(shards, optimizer, full)
    return shards, full


def save_group(ckpt_dir, members: Sequence[dict], common: Optional[dict] = None) -> None:
    """Write one checkpoint from several model shards held by THIS process (tests, conversion tools):
    ``members`` are keyword sets of :func:`save` (``model, rank, tp_rank, tp, dp_rank, optimizer``).  The
    planner/writer protocol of ``torch.distributed.checkpoint.save`` is run for every member in turn,
    member 0 acting as coordinator."""
    from torch.distributed.checkpoint import FileSystemWriter
    SavePlanner, _ = _planners()
    d = Path(ckpt_dir)
    d.mkdir(parents=True, exist_ok=True)
    writer = FileSystemWriter(str(d))
    planners, plans = [], []
    for i, m in enumerate(members):
        shards, _ = _local_shards(m["model"], m.get("tp_rank", 0), m.get("tp", 1), m.get("dp_rank", 0),
                                  m.get("optimizer"), False)
        pl = SavePlanner([s for s in shards if s.replica_id == 0])
        pl.set_up_planner({}, is_coordinator=(i == 0))
        writer.set_up_storage_writer(i == 0)
        planners.append(pl)
        plans.append(writer.prepare_local_plan(pl.create_local_plan()))
    global_plans, metadata = planners[0].create_global_plan(plans)
    global_plans = writer.prepare_global_plan(global_plans)
    results = []
    for pl, gp in zip(planners, global_plans):
        fut = writer.write_data(pl.finish_plan(gp), pl)
        fut.wait()
        results.append(fut.value())
    writer.finish(metadata, results)
    _write_common(d, common, members[0].get("optimizer"))


def _write_common(d: Path, common: Optional[dict], optimizer) -> None:
    (d / "metadata.json").write_text(json.dumps(METADATA))
    c = dict(common or {})
    if optimizer is not None:
        c["optimizer"] = {"step": optimizer.step_count}
    torch.save(c, d / "common.pt")


def save(model, ckpt_dir, rank: int = 0, tp_rank: int = 0, tp: int = 1, dp_rank: int = 0,
         common: Optional[dict] = None, optimizer=None, group=None) -> None:
    """Collective save: every rank of ``group`` (default: all ranks) calls it with its own coordinates.
    Without an initialised process group it writes a one-rank checkpoint."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1):
        save_group(ckpt_dir, [dict(model=model, rank=rank, tp_rank=tp_rank, tp=tp, dp_rank=dp_rank,
                                   optimizer=optimizer)], common)
        return
    import torch.distributed.checkpoint as dcp
    SavePlanner, _ = _planners()
    d = Path(ckpt_dir)
    if dist.get_rank(group) == 0:
        d.mkdir(parents=True, exist_ok=True)
    shards, _ = _local_shards(model, tp_rank, tp, dp_rank, optimizer, False)
    dcp.save({}, storage_writer=dcp.FileSystemWriter(str(d)),
             planner=SavePlanner([s for s in shards if s.replica_id == 0]), process_group=group)
    if dist.get_rank(group) == 0:
        _write_common(d, common, optimizer)
    dist.barrier(group=group)


def load(model, ckpt_dir, tp_rank: int = 0, tp: int = 1, strict: bool = True, optimizer=None, group=None,
         dp_rank: int = 0) -> dict:
    """Fill ``model``'s parameters (and ``optimizer``'s state) from a checkpoint written under any
    TP x PP x DP layout.  Every rank reads the boxes it needs by itself; no collective is involved."""
    import torch.distributed.checkpoint as dcp
    _, LoadPlanner = _planners()
    d = Path(ckpt_dir)
    meta = json.loads((d / "metadata.json").read_text())
    if meta.get("sharded_backend") != METADATA["sharded_backend"]:
        raise ValueError(f"unsupported checkpoint backend {meta}")
    wants, full = _local_shards(model, tp_rank, tp, dp_rank, optimizer, True)
    dcp.load({}, storage_reader=dcp.FileSystemReader(str(d)), planner=LoadPlanner(wants, strict), no_dist=True)
    common = torch.load(d / "common.pt", map_location="cpu", weights_only=True) if (d / "common.pt").exists() else {}
    if optimizer is not None:
        optimizer.scatter_state(full, step=int(common.get("optimizer", {}).get("step", 0)))
    return common
