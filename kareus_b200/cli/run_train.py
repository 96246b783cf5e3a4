"""Phase 3: training run under a plan, with the reference's method names and output layout.

    torchrun --nproc-per-node 8 -m kareus_b200.cli.run_train --method kareus --model llama3.2_3b \
        --tp 8 --pp 1 --mbs 8 --seq 4096 --gbs 64 --steps 30 \
        --freqs plans/freqs_pipeline_02495.py --scheds plans/scheds_pipeline_02495.py

Methods: ``megatron`` (one nanobatch, no plan), ``nanobatch`` (two nanobatches, fixed schedule),
``perseus`` / ``nanobatch_perseus`` (frequency plan only), ``kareus`` (frequency + overlap plan).
Each rank writes ``<out>/<model>/<cp.._tp.._mbs.._seq..>/<method>/zeus_monitor_global_rank-G_local_rank-L.txt``
with the windows ``training_step`` and ``training_step_fwd_bwd_step_call``; rank 0 also appends one JSON object per
step (loss, learning rate, gradient norm, step time, tokens/s, consumed samples, validation loss) to
``metrics_global_rank-0.jsonl`` there.
"""
from __future__ import annotations

import argparse
import json
import os
import time
from pathlib import Path

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--method", default="kareus",
                    choices=["megatron", "nanobatch", "perseus", "nanobatch_perseus", "kareus"])
    ap.add_argument("--model", default="llama3.2_3b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--cp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--mbs", type=int, default=8)
    ap.add_argument("--gbs", type=int, default=64)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--tp-comm", default="sp_fused")
    ap.add_argument("--comm-backend", default="kernel")
    ap.add_argument("--freqs", default=None, help="freqs_pipeline_*.py (served in process, or by --pfo-url)")
    ap.add_argument("--scheds", default=None, help="scheds_pipeline_*.py")
    ap.add_argument("--pfo-url", default=None, help="http://MASTER_ADDR:7787 of a running plan server")
    ap.add_argument("--clock-mode", default="advisory", choices=["off", "advisory", "locked"])
    ap.add_argument("--out", default="nemo_experiments")
    ap.add_argument("--run-dir", default=None,
                    help="write this run's files exactly here instead of <out>/<model>/<layout>/<method> "
                         "(frontier runs: <method>/frontier/pipeline_NNNNN)")
    ap.add_argument("--enable-power-monitor", action="store_true")
    ap.add_argument("--enable-timers", action="store_true")
    ap.add_argument("--nano", type=int, default=None,
                    help="nanobatches per microbatch (default: 1 for megatron / perseus, 2 for the other methods)")
    ap.add_argument("--recompute-layers", type=int, default=4)
    ap.add_argument("--no-recompute", action="store_true",
                    help="keep all activations (the reference's activations_checkpoint_granularity: null); overlap plans "
                         "are then read in the per-microbatch (forward, backward) pair layout")
    ap.add_argument("--profile-start-step", type=int, default=None,
                    help="open the CUDA profiler capture range at this step (nsys --capture-range=cudaProfilerApi)")
    ap.add_argument("--profile-end-step", type=int, default=None)
    ap.add_argument("--profile-ranks", type=int, nargs="*", default=[0])
    ap.add_argument("--data-path", default=None, nargs="+",
                    help="prefix of a Megatron-format indexed token file (<prefix>.bin/.idx), or a weighted blend "
                         "`w0 prefix0 w1 prefix1 ...`; default: synthetic tokens")
    ap.add_argument("--data-split", default="949,50,1", help="train,validation,test weights over the documents")
    ap.add_argument("--data-seed", type=int, default=1234)
    ap.add_argument("--eod-token", type=int, default=None, help="mask the loss on this end-of-document token")
    ap.add_argument("--eval-interval", type=int, default=0,
                    help="every N steps report the loss on held-out batches (validation documents of --data-path, "
                         "or synthetic tokens of other seeds); 0: never")
    ap.add_argument("--eval-iters", type=int, default=1, help="global batches per evaluation")
    ap.add_argument("--save", default=None, help="write a distributed checkpoint (model + optimizer) here at the end")
    ap.add_argument("--save-interval", type=int, default=0, help="also save every N steps")
    ap.add_argument("--load", default=None, help="resume from this distributed checkpoint (any TP x PP x DP layout)")
    ap.add_argument("--keep-process-group", action="store_true",
                    help="leave torch.distributed initialised (when called from another driver)")
    a = ap.parse_args(argv)

    import torch.distributed as dist
    from ..config import ParallelConfig, TrainConfig, get_model_config
    from ..energy import EnergyMonitor, FrequencyController, PipelineFrequencyOptimizer, PointSolution, PowerMonitor
    from ..parallel.mesh import Mesh, init_distributed
    from ..plan import PipelineCommScheduler, parse_schedule_file
    from ..train.optimizer import cosine_lr
    from ..train.trainer import Trainer, synthetic_batch
    from ..utils.timers import Timers

    rank, world, local = init_distributed()
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    dp = world // (a.tp * a.cp * a.pp)
    nano = a.nano if a.nano else (1 if a.method in ("megatron", "perseus") else 2)
    if a.mbs % nano and a.seq % nano:
        raise SystemExit(f"{nano} nanobatches divide neither the micro batch ({a.mbs}) nor the sequence ({a.seq})")
    tp_comm = a.tp_comm if a.tp > 1 else "allreduce"
    par = ParallelConfig(tp=a.tp, cp=a.cp, pp=a.pp, dp=dp, num_nanobatches=nano, tp_comm=tp_comm,
                         comm_backend=a.comm_backend if cuda else "nccl", recompute=not a.no_recompute)
    mesh = Mesh(tp=a.tp, cp=a.cp, dp=dp, pp=a.pp)
    cfg = get_model_config(a.model)
    tc = TrainConfig(micro_batch_size=a.mbs, global_batch_size=a.gbs, seq_len=a.seq,
                     dtype="bf16" if cuda else "fp32")
    tag = f"cp{a.cp}_tp{a.tp}_mbs{a.mbs}_seq{a.seq}"
    out = Path(a.run_dir) if a.run_dir else Path(a.out) / a.model / tag / a.method
    out.mkdir(parents=True, exist_ok=True)
    # without a GPU the windows are still written, against the simulated NVML (the flow of drivers, the
    # comparison tool and the tests need the files; the joules then mean nothing)
    sim = None
    if not cuda:
        from ..energy.nvml import FakeNVML
        sim = FakeNVML(1)
    monitor = EnergyMonitor([local] if cuda else [0], nvml=sim,
                            log_file=str(out / f"zeus_monitor_global_rank-{rank}_local_rank-{local}.txt"))
    M = tc.num_microbatches(dp)
    ctl = FrequencyController(local, a.clock_mode)
    freq_client = None
    if a.method in ("perseus", "nanobatch_perseus", "kareus") and (a.freqs or a.pfo_url):
        tpr, tpd = mesh.folded_tp_rank()
        freq_client = PipelineFrequencyOptimizer(rank, mesh.dp_rank, mesh.pp_rank, tpr, local, dp, a.pp, tpd, world, ctl,
                                                 server_url=a.pfo_url,
                                                 solution=PointSolution.from_file(a.freqs) if a.freqs else None)
    sched = None
    if a.method == "kareus" and a.scheds:
        parsed = [None]
        if rank == 0:
            parsed[0] = parse_schedule_file(a.scheds, not a.no_recompute, a.cp > 1)
        if world > 1:
            dist.broadcast_object_list(parsed, src=0)      # rank 0 parses, everyone receives
        sched = PipelineCommScheduler.from_parsed(parsed[0], mesh.pp_rank, M, not a.no_recompute, a.cp > 1)
    heap = None
    if cuda and a.tp > 1 and (par.comm_backend == "kernel" or par.tp_comm == "sp_fused"):
        from ..parallel.symm_heap import SymmetricHeap
        heap = SymmetricHeap.create(mesh.group("tp"), device)
        if os.environ.get("KAREUS_NVLS", "0") == "1":
            heap.enable_nvls(int(os.environ.get("KAREUS_NVLS_BYTES", str(3 << 30))))
    trainer = Trainer(cfg, par, tc, mesh=mesh, device=device, monitor=monitor, freq_client=freq_client,
                      comm_scheduler=sched, heap=heap, recompute_layers=a.recompute_layers)
    timers = Timers() if a.enable_timers else None
    if timers is not None:
        trainer._hooks.append(timers)
    if a.profile_start_step is not None:
        from ..utils.debug import ProfilerStepWindow
        end = a.profile_end_step if a.profile_end_step is not None else a.profile_start_step
        trainer._hooks.append(ProfilerStepWindow(a.profile_start_step, end, a.profile_ranks, rank))
    power = PowerMonitor(local).start() if (a.enable_power_monitor and cuda) else None
    first = 0
    if a.load:
        trainer.load_checkpoint(a.load)
        first = trainer.step_index
        if rank == 0:
            print(f"resumed from {a.load} at step {first}", flush=True)
    batches = None
    if a.data_path:
        from ..data import PretrainingBatches
        from ..data.factory import TRAIN, VALIDATION, TokenData
        try:
            data = TokenData(a.data_path, a.data_split, a.seq, a.data_seed, a.eod_token, cfg.vocab_size)
        except ValueError as e:
            raise SystemExit(str(e))
        ds = data.dataset(TRAIN, a.steps * a.gbs)
        # the run resumes at the sample where the checkpointed step count left off
        batches = PretrainingBatches(ds, a.mbs, M, dp_rank=mesh.dp_rank, dp_size=dp, consumed_samples=first * a.gbs,
                                     cp=a.cp, cp_rank=mesh.cp_rank)
        if rank == 0:
            for line in data.describe():
                print("data: " + line, flush=True)
    val_ds = None
    if a.data_path and a.eval_interval > 0:
        if data.has_share(VALIDATION):
            # the same held-out batches at every evaluation, in file order
            val_ds = data.dataset(VALIDATION, a.eval_iters * a.gbs, shuffle=False)
        elif rank == 0:
            print("the validation share of --data-split is empty: evaluating on synthetic tokens", flush=True)

    metrics_file = open(out / f"metrics_global_rank-{rank}.jsonl", "a") if rank == 0 else None

    def log_metrics(**kv) -> None:
        """One JSON object per line: per-step training metrics and evaluation results of this run."""
        if metrics_file is not None:
            metrics_file.write(json.dumps(kv) + "\n")
            metrics_file.flush()

    def evaluate(step: int) -> None:
        losses = []
        if val_ds is not None:
            with PretrainingBatches(val_ds, a.mbs, M, dp_rank=mesh.dp_rank, dp_size=dp, cp=a.cp,
                                    cp_rank=mesh.cp_rank) as vb:
                for vbatch in vb:
                    losses.append(trainer.evaluate(vbatch))
        else:
            for k in range(a.eval_iters):
                losses.append(trainer.evaluate(synthetic_batch(cfg, tc, M, seed=1_000_000 + k, cp=a.cp,
                                                               cp_rank=mesh.cp_rank)))
        if rank == 0 and losses:
            print(f"step {step} validation loss {sum(losses) / len(losses):.4f} ({len(losses)} batches)", flush=True)
            log_metrics(step=step, validation_loss=sum(losses) / len(losses), validation_batches=len(losses))

    try:
        for step in range(first, a.steps):
            batch = next(batches) if batches is not None else \
                synthetic_batch(cfg, tc, M, seed=step, cp=a.cp, cp_rank=mesh.cp_rank)
            t0 = time.perf_counter()
            loss = trainer.train_step(batch, loss_denominator=float(a.gbs * a.seq))     # reads the loss: synchronises
            dt = time.perf_counter() - t0
            if rank == 0:
                print(f"step {step} loss {loss:.4f}", flush=True)
                norm = trainer.optimizer.last_grad_norm
                log_metrics(step=step, loss=loss, lr=cosine_lr(step, tc),
                            grad_norm=float(norm) if norm is not None else None, step_time_s=dt,
                            tokens_per_s=a.gbs * a.seq / dt, consumed_samples=(step + 1) * a.gbs)
            if a.eval_interval > 0 and (step + 1) % a.eval_interval == 0:
                evaluate(step)
            if a.save and a.save_interval and (step + 1) % a.save_interval == 0 and step + 1 < a.steps:
                trainer.save_checkpoint(a.save)
        if a.save:
            trainer.save_checkpoint(a.save)
    finally:
        if metrics_file is not None:
            metrics_file.close()
        if batches is not None:
            batches.close()
        ctl.close()
        if power is not None:
            power.stop()
            power.dump(out / f"power_monitor_global_rank-{rank}_local_rank-{local}.txt")
        if timers is not None:
            timers.export(out, rank, local)
        if heap is not None and heap.nvls is not None:
            heap.nvls.close(collective=False)     # unbind switch-multicast memory before this rank leaves
            heap.nvls = None
        if world > 1:
            dist.barrier()
            if not a.keep_process_group:
                dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
