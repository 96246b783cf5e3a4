"""Checkpoint layout (keys, prepended layer axis, TP axes, SwiGLU split), resharding load, utils."""
import json

import torch

from kareus_b200.config import ParallelConfig, get_model_config
from kareus_b200.models import checkpoint as ck
from kareus_b200.models.llama import GPTModel
from kareus_b200.utils.debug import nvtx_range, save_tensors
from kareus_b200.utils.timers import Timers


class _FakeComm:
    """CommFactory stand-in that reports a TP size without process groups."""
    heap = None

    def __init__(self, tp, rank):
        self.tp, self.rank = tp, rank

    def _args(self, axis):
        return (None, self.tp, self.rank) if axis == "tp" else (None, 1, 0)

    def make(self, cls, axis, name):
        g, w, r = self._args(axis)
        return cls(g, w, r, name=name)


def test_sharded_state_dict_contract():
    cfg = get_model_config("tiny")
    m = GPTModel(cfg, ParallelConfig(tp=2, tp_comm="sp"), comm=_FakeComm(2, 1), dtype="fp32")
    sd = ck.sharded_state_dict(m, tp_rank=1, tp=2)
    by = {}
    for s in sd:
        by.setdefault(s.key, []).append(s)
    q = by["decoder.layers.self_attention.linear_qkv.weight"]
    assert len(q) == cfg.num_layers and q[1].prepend_axis_num == 1
    assert q[1].global_shape[0] == cfg.num_layers and q[1].global_offset[0] == 1
    assert q[0].global_offset[1] == q[0].local_shape[1] and q[0].axis_fragmentations == (cfg.num_layers, 2, 1)
    pj = by["decoder.layers.self_attention.linear_proj.weight"][0]
    assert pj.axis_fragmentations == (cfg.num_layers, 1, 2) and pj.global_offset[2] == pj.local_shape[2]
    fc1 = by["decoder.layers.mlp.linear_fc1.weight"]
    assert len(fc1) == 2 * cfg.num_layers and fc1[0].axis_fragmentations == (cfg.num_layers, 4, 1)
    f_local = cfg.ffn_hidden_size // 2
    assert fc1[0].global_offset[1] == f_local and fc1[1].global_offset[1] == cfg.ffn_hidden_size + f_local
    assert by["decoder.final_layernorm.weight"][0].replica_id == 1
    assert "embedding.word_embeddings.weight" in by and "output_layer.weight" in by


def test_save_tp2_load_tp1_and_back(tmp_path):
    cfg = get_model_config("tiny")
    shards = [GPTModel(cfg, ParallelConfig(tp=2), comm=_FakeComm(2, r), dtype="fp32", seed=3) for r in range(2)]
    ck.save_group(tmp_path / "ckpt", [dict(model=m, rank=r, tp_rank=r, tp=2) for r, m in enumerate(shards)],
                  common={"step": 7})
    assert json.loads((tmp_path / "ckpt" / "metadata.json").read_text())["sharded_backend"] == "torch_dist"
    # a genuine torch.distributed.checkpoint directory: index + per-rank data files, readable by DCP's reader
    from torch.distributed.checkpoint import FileSystemReader
    md = FileSystemReader(str(tmp_path / "ckpt")).read_metadata()
    qkv_md = md.state_dict_metadata["decoder.layers.self_attention.linear_qkv.weight"]
    assert tuple(qkv_md.size)[0] == cfg.num_layers and len(qkv_md.chunks) == 2 * cfg.num_layers
    assert sorted(p.name for p in (tmp_path / "ckpt").glob("__*_0.distcp")) == ["__0_0.distcp", "__1_0.distcp"]
    full = GPTModel(cfg, ParallelConfig(tp=1), dtype="fp32", seed=99)
    common = ck.load(full, tmp_path / "ckpt", tp_rank=0, tp=1)
    assert common["step"] == 7
    l0 = full.decoder.layers[0]
    want_qkv = torch.cat([s.decoder.layers[0].qkv.weight for s in shards], 0)
    torch.testing.assert_close(l0.qkv.weight.data, want_qkv)
    gates = [s.decoder.layers[0].fc1.weight.chunk(2, 0)[0] for s in shards]
    ups = [s.decoder.layers[0].fc1.weight.chunk(2, 0)[1] for s in shards]
    torch.testing.assert_close(l0.fc1.weight.data, torch.cat(gates + ups, 0))
    torch.testing.assert_close(l0.proj.weight.data, torch.cat([s.decoder.layers[0].proj.weight for s in shards], 1))
    # and back: write TP1, load into a TP2 shard
    ck.save(full, tmp_path / "ckpt1", rank=0)
    again = GPTModel(cfg, ParallelConfig(tp=2), comm=_FakeComm(2, 1), dtype="fp32", seed=5)
    ck.load(again, tmp_path / "ckpt1", tp_rank=1, tp=2)
    torch.testing.assert_close(again.decoder.layers[1].fc2.weight.data, shards[1].decoder.layers[1].fc2.weight.data)
    torch.testing.assert_close(again.embedding.weight.data, shards[1].embedding.weight.data)


def test_debug_and_timers(tmp_path):
    with nvtx_range("x", enabled=True):
        pass
    p = save_tensors({"a": torch.ones(2)}, tmp_path, tp_rank=1, pp_rank=0)
    assert p.name == "tensors_tp1_pp0.pt" and torch.load(p)["a"].sum() == 2
    t = Timers(sync=False)
    t.on_instruction_begin("forward"); t.on_instruction_end("forward")
    out = t.export(tmp_path, 3, 1)
    assert out.name == "instructions-3-1.csv" and "forward-compute" in out.read_text()


def test_profiler_step_window():
    from kareus_b200.utils.debug import ProfilerStepWindow
    calls = []
    w = ProfilerStepWindow(2, 3, ranks=(0, 4), rank=4, start_fn=lambda: calls.append("start"),
                           stop_fn=lambda: calls.append("stop"))
    for step in range(6):
        w.on_step_begin()
        w.on_instruction_begin("forward"); w.on_instruction_end("forward")
        calls.append(("step", step, w.open))
        w.on_step_end()
    assert calls == [("step", 0, False), ("step", 1, False), "start", ("step", 2, True), ("step", 3, True), "stop",
                     ("step", 4, False), ("step", 5, False)]
    off = ProfilerStepWindow(0, 0, ranks=(0,), rank=1, start_fn=lambda: calls.append("x"))
    off.on_step_begin(); off.on_step_end()
    assert "x" not in calls


def test_yaml_run_config(tmp_path):
    from kareus_b200.config_yaml import load_run_config
    (tmp_path / "c.yaml").write_text("""
name: megatron_llama3.2_3b
trainer: {devices: 8, num_nodes: 2, precision: bf16, max_steps: 30, gradient_clip_val: 1.0}
model:
  micro_batch_size: 8
  global_batch_size: 64
  tensor_model_parallel_size: 8
  pipeline_model_parallel_size: 2
  context_parallel_size: 1
  cp_comm_type: all_gather
  num_layers_in_first_pipeline_stage: 15
  encoder_seq_length: 4096
  num_layers: 28
  hidden_size: 3072
  ffn_hidden_size: 8192
  num_attention_heads: 24
  kv_channels: 128
  num_query_groups: 8
  hidden_dropout: 0.1
  layernorm_epsilon: 1e-5
  enable_zeus_monitor: true
  enable_kareus_scheduler: false
  kareus_scheduler_kwargs: {solution_path: null}
  activations_checkpoint_granularity: full
  sequence_parallel: false
  nsys_profile: {enabled: true, start_step: 12, end_step: 14, ranks: [0, 8]}
  optim: {lr: 2e-4, weight_decay: 0.01, betas: [0.9, 0.98], sched: {warmup_steps: 500, min_lr: 2e-5}}
""")
    model, par, train, sw = load_run_config(tmp_path / "c.yaml", ["model.enable_kareus_scheduler=True",
                                                                 "model.kareus_scheduler_kwargs.solution_path=/p/s.py",
                                                                 "model.micro_batch_size=4"])
    assert (model.num_layers, model.hd, model.num_layers_in_first_pipeline_stage) == (28, 128, 15)
    assert (par.tp, par.pp, par.dp, par.recompute, par.tp_comm) == (8, 2, 1, True, "allreduce")
    assert train.micro_batch_size == 4 and train.num_microbatches(1) == 16 and train.betas == (0.9, 0.98)
    assert sw.enable_zeus_monitor and sw.enable_kareus_scheduler and sw.solution_path == "/p/s.py"
    assert (sw.nsys_profile, sw.nsys_start_step, sw.nsys_end_step, sw.nsys_ranks) == (True, 12, 14, (0, 8))


def _ckpt_trainer(tp, dp):
    from kareus_b200.config import TrainConfig
    from kareus_b200.parallel.mesh import Mesh
    from kareus_b200.train.trainer import Trainer
    cfg = get_model_config("tiny").replace(num_query_groups=4)
    tc = TrainConfig(micro_batch_size=2, global_batch_size=8, seq_len=32, lr=2e-3, warmup_steps=0, max_steps=10,
                     dtype="fp64")
    par = ParallelConfig(tp=tp, dp=dp, num_nanobatches=2, recompute=True)
    mesh = Mesh(tp=tp, dp=dp)
    return cfg, tc, mesh, Trainer(cfg, par, tc, mesh=mesh, dtype="fp64")


def _ckpt_step(cfg, tc, mesh, tr, seed):
    from kareus_b200.train.trainer import synthetic_batch
    full = synthetic_batch(cfg, tc, tc.num_microbatches(1), seed=seed, pin=False)
    share = tr.num_microbatches * tc.micro_batch_size
    lo = mesh.dp_rank * share
    return tr.train_step({k: v[lo:lo + share] for k, v in full.items()}, loss_denominator=float(full["loss_mask"].sum()))


def _save_worker(rank, world, path):
    cfg, tc, mesh, tr = _ckpt_trainer(2, 2)
    for i in range(2):
        _ckpt_step(cfg, tc, mesh, tr, 10 + i)
    tr.save_checkpoint(path)
    nxt = [_ckpt_step(cfg, tc, mesh, tr, 12 + i) for i in range(2)]
    if rank == 0:
        torch.save({"loss": nxt, "norm": float(tr.optimizer.last_grad_norm)}, path + "/expected.pt")


def _load_worker(rank, world, path):
    cfg, tc, mesh, tr = _ckpt_trainer(4, 1)
    common = tr.load_checkpoint(path)
    assert common["iteration"] == 2 and tr.optimizer.step_count == 2 and tr.step_index == 2
    got = [_ckpt_step(cfg, tc, mesh, tr, 12 + i) for i in range(2)]
    want = torch.load(path + "/expected.pt")
    # the second loss after the resume depends on the AdamW update, i.e. on both moments, the master
    # copy and the step counter
    # (losses are reported as fp32: one unit in the last place is 5e-7 here; a resume that lost the
    # moments would be off by about 1e-3)
    for a, b in zip(got, want["loss"]):
        assert abs(a - b) < 2e-6, (got, want)
    assert abs(float(tr.optimizer.last_grad_norm) - want["norm"]) < 1e-6


def test_resume_under_another_layout_continues_the_same_run(tmp_path):
    """Save model + AdamW state at TP2 x DP2 after two steps, resume at TP4 x DP1: the next two steps have
    the same losses and gradient norm as the uninterrupted run (fp64), so parameters, both moments, the
    fp32 master copy and the step counter all came back, resharded."""
    from dist_utils import run_distributed
    path = str(tmp_path / "ckpt")
    run_distributed(_save_worker, 4, path)
    from torch.distributed.checkpoint import FileSystemReader
    md = FileSystemReader(path).read_metadata().state_dict_metadata
    assert "optimizer.state.exp_avg.decoder.layers.mlp.linear_fc2.weight" in md
    assert "optimizer.state.fp32_param.embedding.word_embeddings.weight" in md
    run_distributed(_load_worker, 4, path)


def test_reference_run_configs_load():
    """The YAML files the reference ships (set KAREUS_REFERENCE_DIR) load as they are: model shape, layout,
    data section; the vocabulary follows the tokenizer they name."""
    import os
    from pathlib import Path
    import pytest
    from kareus_b200.config_yaml import load_run_config
    ref = Path(os.environ.get("KAREUS_REFERENCE_DIR", "/nonexistent")) / "tests" / "artifact" / "conf"
    if not ref.exists():
        pytest.skip("KAREUS_REFERENCE_DIR not set")
    m, p, t, sw = load_run_config(ref / "megatron_llama3.2_3b_config.yaml")
    assert (m.num_layers, m.hidden_size, m.ffn_hidden_size, m.vocab_size) == (28, 3072, 8192, 128256)
    assert (p.tp, p.pp, p.cp, p.recompute) == (8, 2, 1, True) and (t.micro_batch_size, t.global_batch_size) == (8, 64)
    assert sw.data_prefix.endswith("llama_dataset_text_document") and sw.data_split == "900,50,50"
    m, p, t, sw = load_run_config(ref / "megatron_qwen3_1.7b_config.yaml")
    assert m.qk_layernorm and m.tie_embeddings and m.vocab_size == 151936 and m.hidden_size == 2048
