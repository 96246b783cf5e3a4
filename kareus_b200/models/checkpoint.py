"""Distributed checkpoint in the Megatron layout.

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
* replicated tensors carry ``replica_id = tp_rank`` (only replica 0 is written).

``save`` writes ``metadata.json`` (``sharded_backend`` / version), ``common.pt`` (non-tensor state) and
one shard file per rank with its index; ``load`` assembles any requested local box from the saved
shards, so a checkpoint written under one TP×PP layout loads under another.
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

    def col(key, w, layer=None):           # sharded on axis 0
        g = (w.shape[0] * tp, w.shape[1])
        out.append(_st(key, w, g, (tp_rank * w.shape[0], 0), (tp, 1), dp_rank, layer))

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
        if not (cfg.tie_embeddings and model.embedding is not None):
            col("output_layer.weight", model.output_layer.weight.data)
    return out


def save(model, ckpt_dir, rank: int = 0, tp_rank: int = 0, tp: int = 1, dp_rank: int = 0,
         common: Optional[dict] = None, optimizer=None) -> None:
    d = Path(ckpt_dir)
    d.mkdir(parents=True, exist_ok=True)
    shards = [s for s in sharded_state_dict(model, tp_rank, tp, dp_rank) if s.replica_id == 0]
    torch.save({"index": [s.meta() for s in shards], "tensors": [s.data.detach().cpu().clone() for s in shards]},
               d / f"__{rank}_0.distcp")
    if optimizer is not None:
        torch.save({k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in optimizer.state_dict().items()},
                   d / f"optimizer_rank{rank}.pt")
    if rank == 0:
        (d / "metadata.json").write_text(json.dumps(METADATA))
        torch.save(common or {}, d / "common.pt")


def _intersect(off_a, shp_a, off_b, shp_b):
    lo = [max(a, b) for a, b in zip(off_a, off_b)]
    hi = [min(a + s, b + t) for a, s, b, t in zip(off_a, shp_a, off_b, shp_b)]
    if any(h <= l for l, h in zip(lo, hi)):
        return None
    return lo, hi


def load(model, ckpt_dir, tp_rank: int = 0, tp: int = 1, strict: bool = True) -> dict:
    """Fill ``model``'s parameters from a checkpoint written under any TP×PP layout."""
    d = Path(ckpt_dir)
    meta = json.loads((d / "metadata.json").read_text())
    if meta.get("sharded_backend") != METADATA["sharded_backend"]:
        raise ValueError(f"unsupported checkpoint backend {meta}")
    saved: Dict[str, List[Tuple[dict, torch.Tensor]]] = {}
    for f in sorted(d.glob("__*_0.distcp")):
        blob = torch.load(f, map_location="cpu")
        for m, t in zip(blob["index"], blob["tensors"]):
            saved.setdefault(m["key"], []).append((m, t))
    for want in sharded_state_dict(model, tp_rank, tp):
        srcs = saved.get(want.key, [])
        dst = want.data
        view = dst.reshape(want.local_shape) if want.prepend_axis_num else dst
        filled = 0
        for m, t in srcs:
            t = t.reshape(m["local_shape"])
            box = _intersect(want.global_offset, want.local_shape, m["global_offset"], m["local_shape"])
            if box is None:
                continue
            lo, hi = box
            dsl = tuple(slice(l - o, h - o) for l, h, o in zip(lo, hi, want.global_offset))
            ssl = tuple(slice(l - o, h - o) for l, h, o in zip(lo, hi, m["global_offset"]))
            view[dsl].copy_(t[ssl].to(view.dtype))
            n = 1
            for l, h in zip(lo, hi):
                n *= h - l
            filled += n
        if strict and filled != view.numel():
            raise KeyError(f"checkpoint covers {filled} of {view.numel()} elements of {want.key} "
                           f"at offset {want.global_offset}")
    return torch.load(d / "common.pt", map_location="cpu") if (d / "common.pt").exists() else {}
