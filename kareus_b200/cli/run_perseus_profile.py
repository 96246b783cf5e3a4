"""Frequency-only baseline profile ("Megatron+Perseus" / "Nanobatching+Perseus").

Runs a few training steps at each clock of the GPU's grid, measures every pipeline instruction's
time and energy through the trainer's hooks and writes ``stage,instruction,frequency,time,energy``
(reference: ``tests/artifact/megatron_perseus_run_profiling.sh``, ``tests/perseus/
generate_profile_csv.py``).  ``run_optimization`` then plans with the frequency as the only knob.

    torchrun --nproc-per-node 8 -m kareus_b200.cli.run_perseus_profile --model llama3.2_3b --tp 8 \
        --method nanobatch_perseus --out perseus_profile.csv
"""
from __future__ import annotations

import argparse

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--method", default="perseus", choices=["perseus", "nanobatch_perseus"])
    ap.add_argument("--model", default="llama3.2_3b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--mbs", type=int, default=8)
    ap.add_argument("--gbs", type=int, default=64)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--skip", type=int, default=1)
    ap.add_argument("--gpu_type", default="B200")
    ap.add_argument("--freqs", type=int, nargs="*", default=None)
    ap.add_argument("--clock-mode", default="advisory", choices=["advisory", "locked"])
    ap.add_argument("--out", default="perseus_profile.csv")
    ap.add_argument("--route", default="windows", choices=["windows", "timers"],
                    help="windows: one measurement window per instruction; timers: the reference's route - "
                         "instruction timers + energy-counter poller files, integrated with a piecewise-linear model")
    ap.add_argument("--timer-dir", default="perseus_timers", help="where the timers route writes <freq>/timers/*.csv")
    a = ap.parse_args(argv)

    import torch.distributed as dist
    from ..compose.perseus import InstructionRecorder, profile_from_timer_files, write_frequency_profile
    from ..config import ParallelConfig, TrainConfig, get_freq_grid, get_model_config
    from ..energy import EnergyMonitor, FrequencyController
    from ..parallel.mesh import Mesh, init_distributed
    from ..train.trainer import Trainer, synthetic_batch

    rank, world, local = init_distributed()
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    dp = world // (a.tp * a.pp)
    par = ParallelConfig(tp=a.tp, pp=a.pp, dp=dp, num_nanobatches=2 if a.method == "nanobatch_perseus" else 1)
    mesh = Mesh(tp=a.tp, pp=a.pp, dp=dp)
    cfg = get_model_config(a.model)
    tc = TrainConfig(micro_batch_size=a.mbs, global_batch_size=a.gbs, seq_len=a.seq,
                     dtype="bf16" if cuda else "fp32")
    from ..energy.nvml import FakeNVML
    monitor = EnergyMonitor([local] if cuda else [0], nvml=None if cuda else FakeNVML(1))
    ctl = FrequencyController(local if cuda else 0, a.clock_mode, nvml=monitor.nvml)   # simulated NVML: one device
    trainer = Trainer(cfg, par, tc, mesh=mesh, device=device)
    if a.route == "timers":
        from pathlib import Path
        from ..energy.power import EnergyPoller
        from ..utils.timers import Timers
        for f in (a.freqs or get_freq_grid(a.gpu_type)):
            ctl.set_frequency(f)
            timers = Timers()
            trainer._hooks = [timers]
            poller = EnergyPoller(local if cuda else 0, period_s=0.005, nvml=monitor.nvml).start()
            poller.sample()
            for step in range(a.steps):
                trainer.train_step(synthetic_batch(cfg, tc, trainer.num_microbatches, seed=step),
                                   loss_denominator=float(a.gbs * a.seq))
            poller.sample()
            poller.stop()
            d = Path(a.timer_dir) / str(f)
            timers.export(d, rank, local)
            poller.dump(d / "timers" / f"time-energy-{rank}-{local}.csv")
        ctl.close()
        if world > 1:
            dist.barrier()
        if rank == 0:
            p = profile_from_timer_files(a.timer_dir, num_microbatches=trainer.num_microbatches,
                                         prof_iters=a.steps - a.skip, warmup_iters=a.skip,
                                         ranks_per_stage=a.tp, out=a.out)
            print(f"profile written: {p}")
        if world > 1:
            dist.destroy_process_group()
        return 0
    samples = {}
    for f in (a.freqs or get_freq_grid(a.gpu_type)):
        ctl.set_frequency(f)
        rec = InstructionRecorder(monitor, mesh.pp_rank, f)
        trainer._hooks = [rec]
        for step in range(a.steps):
            if step == a.skip:
                rec.samples.clear()
            trainer.train_step(synthetic_batch(cfg, tc, trainer.num_microbatches, seed=step),
                               loss_denominator=float(a.gbs * a.seq))
        samples.update(rec.samples)
    ctl.close()
    gathered = [None] * world
    if world > 1:
        dist.all_gather_object(gathered, samples)
    else:
        gathered = [samples]
    if rank == 0:
        merged = {}
        for g in gathered:
            for k, v in g.items():
                merged.setdefault(k, []).extend(v)
        print(f"profile written: {write_frequency_profile(a.out, merged)}")
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
