"""Config-file entry point: the reference's ``kareus_gpt_pretraining.py`` (Hydra) equivalent.

    torchrun --nproc-per-node 8 -m kareus_b200.cli.pretrain --config conf/megatron_llama3.2_3b_config.yaml \
        model.micro_batch_size=8 model.enable_kareus_scheduler=True \
        model.kareus_scheduler_kwargs.solution_path=plans/scheds_pipeline_02495.py \
        +freqs=plans/freqs_pipeline_02495.py

Reads the reference's YAML layout (``kareus_b200.config_yaml``), applies ``key=value`` overrides and
runs ``run_train`` with the matching switches (energy monitor windows are always written on GPUs).
"""
from __future__ import annotations

import argparse


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--out", default="nemo_experiments")
    ap.add_argument("--method", default=None)
    ap.add_argument("--clock-mode", default="advisory", choices=["off", "advisory", "locked"])
    ap.add_argument("--eod-token", type=int, default=None, help="end-of-document id (for model.data.eod_mask_loss)")
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    import yaml
    from ..config import MODEL_REGISTRY
    from ..config_yaml import load_run_config
    from . import run_train
    extra = {}
    overrides = []
    for o in a.overrides:
        k, _, v = o.lstrip("+").partition("=")
        if k in ("freqs", "pfo_url"):
            extra[k] = v
        else:
            overrides.append(o)
    model, par, train, sw = load_run_config(a.config, overrides)
    MODEL_REGISTRY[model.name] = model          # make the configured model addressable by name
    method = a.method or ("kareus" if sw.enable_kareus_scheduler else
                          ("nanobatch_perseus" if sw.enable_perseus_optimizer and par.num_nanobatches > 1 else
                           ("perseus" if sw.enable_perseus_optimizer else
                            ("nanobatch" if par.num_nanobatches > 1 else "megatron"))))
    argv2 = ["--method", method, "--model", model.name, "--tp", str(par.tp), "--cp", str(par.cp), "--pp", str(par.pp),
             "--mbs", str(train.micro_batch_size), "--gbs", str(train.global_batch_size), "--seq", str(train.seq_len),
             "--steps", str(sw.max_steps), "--tp-comm", par.tp_comm, "--clock-mode", a.clock_mode, "--out", a.out]
    if sw.solution_path:
        argv2 += ["--scheds", sw.solution_path]
    if extra.get("freqs"):
        argv2 += ["--freqs", extra["freqs"]]
    if extra.get("pfo_url") or sw.perseus_server_url:
        argv2 += ["--pfo-url", extra.get("pfo_url") or sw.perseus_server_url]
    if sw.enable_power_monitor:
        argv2.append("--enable-power-monitor")
    if sw.nsys_profile:
        argv2 += ["--profile-start-step", str(sw.nsys_start_step), "--profile-end-step", str(sw.nsys_end_step),
                  "--profile-ranks", *map(str, sw.nsys_ranks)]
    if sw.enable_megatron_timers:
        argv2.append("--enable-timers")
    if not par.recompute:
        argv2.append("--no-recompute")
    if sw.data_prefix:
        from pathlib import Path
        blend = list(sw.data_blend) if len(sw.data_blend) > 2 else [sw.data_prefix]
        prefixes = blend[1::2] if len(blend) > 1 else blend
        if all(Path(p + ".idx").exists() for p in prefixes):
            argv2 += ["--data-path", *blend, "--data-split", sw.data_split, "--data-seed", str(train.seed)]
            if sw.eod_mask_loss and a.eod_token is not None:
                argv2 += ["--eod-token", str(a.eod_token)]
        else:
            print(f"model.data.data_prefix {sw.data_prefix}.idx not found: training on synthetic tokens", flush=True)
    return run_train.main(argv2)


if __name__ == "__main__":
    raise SystemExit(main())
