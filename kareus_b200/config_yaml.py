"""Read the reference's Hydra/OmegaConf YAML run configs and CLI overrides.

The reference drives runs with ``tests/artifact/conf/*.yaml`` plus ``model.key=value`` overrides
(``tests/artifact/run_kareus.sh:434-446``).  This loader understands the same files (plain YAML,
``${...}`` interpolations of sibling keys are resolved for the keys we read) and maps the subset of
keys this runtime uses onto ``ModelConfig`` / ``ParallelConfig`` / ``TrainConfig`` and the energy
plane switches: ``enable_zeus_monitor, enable_power_monitor, enable_perseus_optimizer,
enable_kareus_scheduler, kareus_scheduler_kwargs.solution_path, enable_megatron_timers, cp_comm_type,
num_layers_in_first_pipeline_stage, sequence_parallel, nsys_profile.{enabled,start_step,end_step,ranks}``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, Optional, Tuple

import yaml

from .config import ModelConfig, ParallelConfig, TrainConfig


@dataclass
class RunSwitches:
    enable_zeus_monitor: bool = False
    enable_power_monitor: bool = False
    enable_perseus_optimizer: bool = False
    enable_kareus_scheduler: bool = False
    enable_megatron_timers: bool = False
    kareus_debug: bool = False
    solution_path: Optional[str] = None
    perseus_server_url: Optional[str] = None
    max_steps: int = 30
    nsys_profile: bool = False          # model.nsys_profile.{enabled,start_step,end_step,ranks}
    nsys_start_step: int = 10
    nsys_end_step: int = 10
    nsys_ranks: Tuple[int, ...] = (0,)
    # model.data.{data_prefix,splits_string,eod_mask_loss}: the (first) indexed token file of the blend
    data_prefix: Optional[str] = None
    data_blend: Tuple[str, ...] = ()       # the whole blend as `--data-path` takes it: (w0, prefix0, w1, prefix1, ...)
    data_split: str = "900,50,50"
    eod_mask_loss: bool = False


def _set_path(d: dict, dotted: str, value) -> None:
    keys = dotted.split(".")
    for k in keys[:-1]:
        d = d.setdefault(k, {})
    d[keys[-1]] = value


def _parse_scalar(text: str):
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


def apply_overrides(cfg: dict, overrides: Iterable[str]) -> dict:
    """``model.micro_batch_size=4``-style overrides (``+key=value`` and ``++key=value`` accepted)."""
    for o in overrides:
        if "=" not in o:
            raise ValueError(f"override must look like key=value, got {o!r}")
        k, v = o.lstrip("+").split("=", 1)
        _set_path(cfg, k, _parse_scalar(v))
    return cfg


def load_run_config(path, overrides: Iterable[str] = (), world_size: Optional[int] = None
                    ) -> Tuple[ModelConfig, ParallelConfig, TrainConfig, RunSwitches]:
    with open(path) as f:
        raw = yaml.safe_load(f)
    raw = apply_overrides(raw, overrides)
    m: Dict[str, Any] = raw.get("model", {})
    tr: Dict[str, Any] = raw.get("trainer", {})
    opt = m.get("optim", {}) or {}
    sched = opt.get("sched", {}) or {}
    heads = int(m["num_attention_heads"])
    # the reference's run configs carry no vocabulary size: it follows from the tokenizer they name
    tok_type = str((m.get("tokenizer") or {}).get("type", "")).lower()
    default_vocab = 151936 if "qwen" in tok_type else 128256
    model = ModelConfig(
        name=str(raw.get("name", "model")), hidden_size=int(m["hidden_size"]), num_attention_heads=heads,
        num_query_groups=int(m.get("num_query_groups") or heads), ffn_hidden_size=int(m["ffn_hidden_size"]),
        num_layers=int(m["num_layers"]), vocab_size=int(m.get("vocab_size") or default_vocab),
        head_dim=int(m["kv_channels"]) if m.get("kv_channels") else None,
        rope_theta=float(m.get("rotary_base", 500000.0)), norm_eps=float(m.get("layernorm_epsilon", 1e-5)),
        hidden_dropout=float(m.get("hidden_dropout", 0.0)), qk_layernorm=bool(m.get("qk_layernorm", False)),
        tie_embeddings=bool(m.get("share_embeddings_and_output_weights", False)),
        max_seq_len=int(m.get("encoder_seq_length", 4096)), init_std=float(m.get("init_method_std", 0.02)),
        num_layers_in_first_pipeline_stage=m.get("num_layers_in_first_pipeline_stage"))
    tp = int(m.get("tensor_model_parallel_size", 1))
    pp = int(m.get("pipeline_model_parallel_size", 1))
    cp = int(m.get("context_parallel_size", 1))
    ws = world_size or int(tr.get("devices", 1)) * int(tr.get("num_nodes", 1))
    dp = max(1, ws // (tp * pp * cp))
    cp_comm = {"all_gather": "all_gather", "p2p": "ring"}.get(str(m.get("cp_comm_type", "all_gather")), "all_gather")
    par = ParallelConfig(tp=tp, cp=cp, pp=pp, dp=dp, num_nanobatches=int(m.get("num_nanobatches", 2)),
                         tp_comm="sp" if m.get("sequence_parallel") else str(m.get("tp_comm", "allreduce")),
                         recompute=(m.get("activations_checkpoint_granularity") == "full"), cp_comm=cp_comm)
    betas = opt.get("betas", (0.9, 0.98))
    train = TrainConfig(micro_batch_size=int(m.get("micro_batch_size", 8)),
                        global_batch_size=int(m.get("global_batch_size", 64)),
                        seq_len=int(m.get("encoder_seq_length", 4096)), lr=float(opt.get("lr", 2e-4)),
                        min_lr=float(sched.get("min_lr", 2e-5)), weight_decay=float(opt.get("weight_decay", 0.01)),
                        betas=(float(betas[0]), float(betas[1])), grad_clip=float(tr.get("gradient_clip_val", 1.0)),
                        warmup_steps=int(sched.get("warmup_steps", 500)), max_steps=int(tr.get("max_steps", 30)),
                        seed=int(m.get("seed", 1234)),
                        dtype={"bf16": "bf16", "bf16-mixed": "bf16", 16: "fp16", 32: "fp32"}.get(tr.get("precision", "bf16"), "bf16"))
    sw = RunSwitches(enable_zeus_monitor=bool(m.get("enable_zeus_monitor", False)),
                     enable_power_monitor=bool(m.get("enable_power_monitor", False)),
                     enable_perseus_optimizer=bool(m.get("enable_perseus_optimizer", False)),
                     enable_kareus_scheduler=bool(m.get("enable_kareus_scheduler", False)),
                     enable_megatron_timers=bool(m.get("enable_megatron_timers", False)),
                     kareus_debug=bool(m.get("kareus_debug", False)),
                     solution_path=(m.get("kareus_scheduler_kwargs") or {}).get("solution_path"),
                     perseus_server_url=m.get("perseus_server_url"), max_steps=int(tr.get("max_steps", 30)))
    ns = m.get("nsys_profile") or {}
    if ns:
        sw.nsys_profile = bool(ns.get("enabled", False))
        sw.nsys_start_step = int(ns.get("start_step", 10))
        sw.nsys_end_step = int(ns.get("end_step", 10))
        sw.nsys_ranks = tuple(int(r) for r in (ns.get("ranks") or [0]))
    data = m.get("data") or {}
    prefix = data.get("data_prefix")
    if isinstance(prefix, (list, tuple)):
        # a blend is written [weight, prefix, weight, prefix, ...]
        paths = [p for p in prefix if isinstance(p, str)]
        if len(prefix) == 2 * len(paths) and paths:
            sw.data_blend = tuple(str(x) for x in prefix)
        prefix = paths[0] if paths else None
    if isinstance(prefix, dict):
        train_part = prefix.get("train")
        prefix = next((p for p in (train_part or []) if isinstance(p, str)), None)
    sw.data_prefix = str(prefix) if prefix else None
    sw.data_split = str(data.get("splits_string", sw.data_split))
    sw.eod_mask_loss = bool(data.get("eod_mask_loss", False))
    return model, par, train, sw
