"""Phase 1: Bayesian profiling of one partition (or of the non-partition parts).

    torchrun --nproc-per-node 8 -m kareus_b200.cli.run_bayesian --partition fwd_attn \
        -m llama3.2_3b -w 8 -tp 8 -cp 1 -b 8 -s 4096 --gpu_type B200

Writes ``<out>/logs/<model>/cp<C>-tp<T>-bs<B>-seq<S>/<partition>/eval_results.jsonl`` (+ result CSVs),
or ``.../nonpartition/<freq>/*_energy.csv`` with ``--nonpartition``.  Clocks are only *recorded*
unless ``--clock-mode locked`` is given (locking clocks changes the GPU for every process on it).
"""
from __future__ import annotations

import argparse
import os

import torch


def env_freq_grid():
    """``FREQ_START`` / ``FREQ_END`` / ``FREQ_STEP`` (MHz) of the reference's driver scripts, highest clock first;
    ``None`` unless start and end are set."""
    lo, hi = os.environ.get("FREQ_START"), os.environ.get("FREQ_END")
    if not lo or not hi:
        return None
    step = abs(int(os.environ.get("FREQ_STEP", "30"))) or 30
    a, b = sorted((int(lo), int(hi)))
    return list(range(b, a - 1, -step))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--partition", default="fwd_attn",
                    help="partition key, or 'all': every partition of the chosen --tp-comm flavour in one process")
    ap.add_argument("--nonpartition", action="store_true")
    ap.add_argument("-m", "--model_name", default="llama3.2_3b")
    ap.add_argument("-w", "--world_size", type=int, default=None)
    ap.add_argument("-tp", "--tensor_parallel_size", type=int, default=1)
    ap.add_argument("-cp", "--context_parallel_size", type=int, default=1)
    ap.add_argument("-b", "--batch_size", type=int, default=8)
    ap.add_argument("-s", "--seq_len", type=int, default=4096)
    ap.add_argument("--gpu_type", default=os.environ.get("GPU_TYPE", "B200"))
    ap.add_argument("--out", default=".")
    ap.add_argument("--tp-comm", default="allreduce")
    ap.add_argument("--comm-backend", default="kernel")
    ap.add_argument("--clock-mode", default="advisory", choices=["off", "advisory", "locked"])
    ap.add_argument("--n-init", type=int, default=None)
    ap.add_argument("--batches", type=int, default=None)
    ap.add_argument("--acq-batch", type=int, default=None)
    ap.add_argument("--measure-s", type=float, default=5.0)
    ap.add_argument("--cooldown-s", type=float, default=5.0)
    ap.add_argument("--nano", type=int, nargs="*", default=[2])
    ap.add_argument("--freqs", type=int, nargs="*", default=None,
                    help="restrict the clock grid (default: the GPU type's full grid)")
    a = ap.parse_args(argv)

    import torch.distributed as dist
    from ..config import ParallelConfig, get_freq_grid, get_model_config, get_p2p_power
    from ..energy import EnergyMonitor, FrequencyController
    from ..parallel.collectives import CommFactory
    from ..parallel.mesh import Mesh, init_distributed
    from ..profile.bo import run_bo_search
    from ..profile.hardware import HardwareEvaluator
    from ..profile.partition_executor import PartitionExecutor
    from ..profile.space import partition_space
    from ..compose.composer import run_dir

    rank, world, local = init_distributed()
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    tp, cp = a.tensor_parallel_size, a.context_parallel_size
    mesh = Mesh(tp=tp, cp=cp, dp=world // (tp * cp))
    cfg = get_model_config(a.model_name)
    heap = None
    if cuda and world > 1 and a.comm_backend == "kernel":
        from ..parallel.symm_heap import SymmetricHeap
        heap = SymmetricHeap.create(mesh.group("tp"), device)
    base = run_dir(a.out, a.model_name, cp, tp, a.batch_size, a.seq_len)
    from ..energy.nvml import FakeNVML
    monitor = EnergyMonitor([local] if cuda else [0], nvml=None if cuda else FakeNVML(1))
    ctl = FrequencyController(local if cuda else 0, a.clock_mode, nvml=monitor.nvml)
    freqs = list(a.freqs) if a.freqs else env_freq_grid() or get_freq_grid(a.gpu_type)

    if a.nonpartition:
        from ..models.llama import GPTModel
        from ..profile.nonpartition import build_cases, profile_nonpartition
        par = ParallelConfig(tp=tp, cp=cp, tp_comm=a.tp_comm, comm_backend=a.comm_backend)
        model = GPTModel(cfg, par, mesh=mesh, comm=CommFactory(mesh, a.comm_backend, heap), device=device,
                         layer_range=range(0))
        profile_nonpartition(build_cases(model, a.batch_size, a.seq_len // cp, device), freqs, base, monitor, ctl,
                             world_size=world, measurement_duration=a.measure_s, cooldown_duration=a.cooldown_s)
        ctl.close()
        return 0

    import copy
    from ..profile.space import CP_PARTITIONS, SP_FUSED_PARTITIONS, TP_PARTITIONS
    if a.partition == "all":
        if tp == 1:
            raise SystemExit("--partition all needs tensor parallelism: the partitions are the segments of a layer around "
                             "its tensor-parallel collectives (context-parallel partitions are profiled together with "
                             "them, as in the reference's TP x CP configurations)")
        if cp > 1 and a.tp_comm != "allreduce":
            raise SystemExit("--partition all with context parallelism profiles the all-reduce flavour of tensor "
                             "parallelism (the reference's TP x CP layouts): pass --tp-comm allreduce")
        parts = CP_PARTITIONS if cp > 1 else (SP_FUSED_PARTITIONS if a.tp_comm in ("sp", "sp_fused") else TP_PARTITIONS)
    else:
        parts = (a.partition,)
    for part in parts:
        kind, space = partition_space(part, a.tp_comm)
        space = copy.deepcopy(space)
        space.nano_values = list(a.nano)

        def make_executor(nano: int, part=part):
            par = ParallelConfig(tp=tp, cp=cp, num_nanobatches=nano, tp_comm=a.tp_comm, comm_backend=a.comm_backend,
                                 recompute=False)
            return PartitionExecutor(cfg, par, part, a.batch_size, a.seq_len, mesh=mesh,
                                     comm=CommFactory(mesh, a.comm_backend, heap), device=device)

        ev = HardwareEvaluator(make_executor, monitor, ctl, world_size=world, measurement_duration=a.measure_s,
                               cooldown_duration=a.cooldown_s)
        logs = base / part
        if rank == 0:
            print(f"[{part}] {kind}; grid {len(space.grid(freqs))} configurations → {logs}", flush=True)
        # every rank runs the search with the same seed so all ranks measure the same configurations;
        # only rank 0's files are kept
        res = run_bo_search(space, freqs, ev, logs if rank == 0 else logs / f".rank{rank}", get_p2p_power(a.gpu_type),
                            n_init=a.n_init, batches=a.batches, acq_batch=a.acq_batch,
                            log=(print if rank == 0 else (lambda s: None)))
        ev.close()
        if rank == 0:
            print(f"[{part}] {len(res.records)} measurements, {len(res.pareto_effective)} on the effective frontier",
                  flush=True)
    ctl.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
