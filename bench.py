"""Headline benchmark: Llama-3.2-3B training throughput (tokens/s) and energy (J/iteration).

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 3 --warmup 3

Config (the reference's headline run, ``tests/artifact/conf/megatron_llama3.2_3b_config.yaml``):
Llama-3.2-3B, bf16, micro batch 8, sequence 4096, global batch 64 (8 microbatches per step),
activation recompute, AdamW with fp32 master weights, TP = number of GPUs, synthetic uniform-random
tokens and random-init weights.  The global batch is fixed, so scaling over GPUs is strong scaling.

Two measurements are reported: ``value`` times K steps on the device (CUDA events, inputs staged
on the device beforehand, max over ranks); ``e2e`` times K calls of ``Trainer.train_step`` with
pinned host inputs copied every step and the loss read back every step.

A third, shorter region re-times the same model in the reference-like configuration (all-reduce
tensor parallelism over NCCL, cuBLAS GEMMs, flash-attention wheel, no launch lists) in the same
process and reports it as ``nccl_cublas_baseline``, because the reference's own stack cannot be
installed here.  Other layouts of the same engine: ``--tp/--pp/--cp`` (product = number of GPUs
times 1/dp), ``--model``, ``--seq``, ``--mbs``, ``--gbs``, ``--cp-comm``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

BASELINE_TOKENS_PER_S = 60200.0   # planner-predicted max-throughput plan of the reference, 16 x A100


def _reference_arm(args) -> int:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference's kareus package installs only with --no-deps (pure Python); its training "
                       "path imports megatron.core, transformer_engine, nemo, apex, mscclpp, cupy and zeus, none "
                       "of which is in the image or the offline wheelhouse",
    }))
    return 0


class ClockSampler(threading.Thread):
    """Samples SM clock, power and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index: int, period_s: float = 0.2):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.power = [], set(), []
        self.max_mhz = None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    _NAMES = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
              0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost"}

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self._NAMES.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(self.period)

    def energy_mj(self):
        try:
            return self.nv.nvmlDeviceGetTotalEnergyConsumption(self.h)
        except Exception:
            return None

    def stop(self):
        self._stop_evt.set()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "power_w_max": max(self.power) if self.power else None, "reasons": sorted(self.reasons)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3.2_3b")
    ap.add_argument("--mbs", type=int, default=8)
    ap.add_argument("--gbs", type=int, default=64)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--nano", type=int, default=int(os.environ.get("KAREUS_NANOBATCHES", "2")))
    ap.add_argument("--tp-comm", default=os.environ.get("KAREUS_TP_COMM"),
                    help="allreduce | sp | sp_fused (default: sp_fused, the fused GEMM+collective kernels)")
    ap.add_argument("--comm-backend", default=os.environ.get("KAREUS_COMM_BACKEND"),
                    help="nccl | kernel (default: kernel, peer-memory collectives of this package)")
    ap.add_argument("--recompute-layers", type=int, default=int(os.environ.get("KAREUS_RECOMPUTE_LAYERS", "4")))
    ap.add_argument("--comm-sm", type=int, default=int(os.environ.get("KAREUS_COMM_SM", "16")),
                    help="CTAs given to a collective (plan knob sm_num) when no plan file is loaded")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--tp", type=int, default=0, help="tensor-parallel size (default: all GPUs not used by pp/cp)")
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--cp", type=int, default=1)
    ap.add_argument("--cp-comm", default="all_gather", choices=["all_gather", "ring"])
    ap.add_argument("--baseline-steps", type=int, default=int(os.environ.get("KAREUS_BASELINE_STEPS", "5")),
                    help="timed steps of the NCCL + cuBLAS + flash-attention configuration (0: skip)")
    args = ap.parse_args()
    if args.impl == "reference":
        return _reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    from kareus_b200.config import ParallelConfig, TrainConfig, get_model_config
    from kareus_b200.kernels import cuda as KC, launch_count
    from kareus_b200.parallel.mesh import Mesh, init_distributed
    from kareus_b200.train.trainer import Trainer, synthetic_batch

    rank, world, local = init_distributed()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    KC.lib()

    # Defaults for N > 1: the product path (fused all-gather→GEMM / GEMM→reduce-scatter kernels over
    # peer memory).  `--tp-comm allreduce --comm-backend nccl` is the reference-like NCCL baseline.
    if args.tp_comm is None:
        args.tp_comm = "sp_fused"
    if args.comm_backend is None:
        args.comm_backend = "kernel"
    tp = args.tp or max(1, world // (args.pp * args.cp))
    if world > 1:
        # a peer's matching kernel can sit behind a full-GPU GEMM of the other nanobatch: allow for it
        os.environ.setdefault("KAREUS_PEER_WAIT_MS", "8000")
    if tp > 1 and args.tp_comm == "sp_fused":
        os.environ.setdefault("KAREUS_SYNC", "lazy")
        if tp >= 4:
            # two nanobatches' fused kernels side by side, each on half of the SMs
            os.environ.setdefault("KAREUS_COMM_STREAMS", "per_nanobatch")
            os.environ.setdefault("KAREUS_FUSED_SMS", "72")
            if "KAREUS_COMM_SM" not in os.environ:
                args.comm_sm = 12
    cfg = get_model_config(args.model)
    tc = TrainConfig(micro_batch_size=args.mbs, global_batch_size=args.gbs, seq_len=args.seq, dtype="bf16")
    if world % (tp * args.pp * args.cp):
        raise SystemExit(f"tp {tp} x pp {args.pp} x cp {args.cp} does not divide {world} GPUs")
    dp = world // (tp * args.pp * args.cp)
    mesh = Mesh(tp=tp, cp=args.cp, dp=dp, pp=args.pp)
    heap = heap_cp = None
    if tp > 1 and (args.comm_backend == "kernel" or args.tp_comm == "sp_fused"):
        from kareus_b200.parallel.symm_heap import SymmetricHeap
        heap = SymmetricHeap.create(mesh.group("tp"), device)
        if os.environ.get("KAREUS_NVLS", "0") == "1":
            # fused kernels and heap collectives go through the NVLink switch (multimem) where supported
            heap.enable_nvls(int(os.environ.get("KAREUS_NVLS_BYTES", str(3 << 30))))
    if args.cp > 1 and args.cp_comm == "ring":
        from kareus_b200.parallel.symm_heap import SymmetricHeap
        heap_cp = SymmetricHeap.create(mesh.group("cp"), device, size_bytes=2 << 30)

    import atexit

    def _release_heaps():
        # a rank that leaves on an error must still unbind its switch-multicast memory (no barriers here)
        for h in (heap, heap_cp):
            if h is not None and not h.closed:
                try:
                    h.close(collective=False)
                except Exception:
                    pass
    atexit.register(_release_heaps)

    def make_trainer(tp_comm, comm_backend):
        par = ParallelConfig(tp=tp, cp=args.cp, dp=dp, pp=args.pp, num_nanobatches=args.nano,
                             tp_comm=tp_comm if tp > 1 else "allreduce", comm_backend=comm_backend, recompute=True,
                             cp_comm=args.cp_comm)
        t = Trainer(cfg, par, tc, mesh=mesh, device=device, heap=heap if comm_backend == "kernel" or tp_comm == "sp_fused" else None,
                    heap_cp=heap_cp, recompute_layers=args.recompute_layers,
                    sync=os.environ.get("KAREUS_SYNC", "partition_end"))
        t.model.decoder.engine.default_shape = (args.comm_sm, 1024)
        return t, par

    trainer, par = make_trainer(args.tp_comm, args.comm_backend)
    M = trainer.num_microbatches
    host_batches = [synthetic_batch(cfg, tc, M, seed=1000 + i + 17 * mesh.dp_rank, cp=args.cp, cp_rank=mesh.cp_rank)
                    for i in range(2)]
    tokens_per_step = args.gbs * args.seq
    denom = float(tokens_per_step)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ------------------------------------------------------------- device-timed region
    dev_batches = [trainer.to_device(b) for b in host_batches]
    first_loss = None
    for i in range(args.warmup):
        trainer.optimizer.zero_grad()
        l = trainer.forward_backward(dev_batches[i % 2], denom)
        if first_loss is None:
            first_loss = trainer.reduce_loss(l)       # random-init model: about ln(vocab)
        trainer.model.finalize_grads()
        trainer.optimizer.step()
    sync_all()
    KC.check_status()
    if args.pp > 1 and trainer.p2p is not None:
        from kareus_b200.parallel.pipeline import P2PStats
        trainer.p2p.stats = P2PStats()
    sampler = ClockSampler(local)
    sampler.start()
    e0 = sampler.energy_mj()
    l0 = launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    h0 = time.perf_counter()
    for i in range(args.steps):
        trainer.optimizer.zero_grad()
        loss = trainer.forward_backward(dev_batches[i % 2], denom)
        trainer.model.finalize_grads()
        trainer.optimizer.step()
    end.record()
    host_ms = (time.perf_counter() - h0) * 1000.0      # time the host needed to enqueue the K steps
    sync_all()
    e1 = sampler.energy_mj()
    launches = launch_count() - l0
    sampler.stop()
    KC.check_status()
    ms = start.elapsed_time(end)
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    en = torch.tensor([(e1 - e0) / 1000.0 if (e0 is not None and e1 is not None) else 0.0], device=device,
                      dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(en, op=dist.ReduceOp.SUM)
    ms = float(t.item())
    value = tokens_per_step * args.steps / (ms / 1000.0)
    final_loss = trainer.reduce_loss(loss)
    p2p = None
    if args.pp > 1 and trainer.p2p is not None and trainer.p2p.stats is not None:
        st = trainer.p2p.stats.summary()
        trainer.p2p.stats = None
        v = torch.tensor([st["stall_ms"], float(st["received_bytes"]), float(st["receives"])], device=device,
                         dtype=torch.float64)
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        # per step, worst stage: time the compute stream waited for a neighbour's activations or gradients
        # (unhidden transfer + pipeline bubble), next to the time the bytes need at the measured peer-copy rate
        p2p = {"recv_stall_ms_per_step": float(v[0]) / args.steps, "recv_bytes_per_step": float(v[1]) / args.steps,
               "receives_per_step": float(v[2]) / args.steps,
               "transfer_ms_at_770GBs_per_step": float(v[1]) / args.steps / 770e9 * 1e3}

    # ------------------------------------------------------------- end-to-end region
    e2e = None
    if not args.skip_e2e:
        for i in range(2):
            trainer.train_step(host_batches[i % 2], loss_denominator=denom)
        sync_all()
        t0 = time.perf_counter()
        for i in range(args.steps):
            final_loss = trainer.train_step(host_batches[i % 2], loss_denominator=denom)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        tt = torch.tensor([dt], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
        h2d = sum(v.numel() * v.element_size() for v in host_batches[0].values())
        e2e = {"value": tokens_per_step * args.steps / dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": 4, "ms_per_step": dt * 1000.0 / args.steps}
        KC.check_status()

    # ------------------------------------------------------------- reference-like configuration, same process
    baseline = None
    if args.baseline_steps > 0:
        replayed = trainer.model.decoder.engine.replayed_regions
        del trainer, dev_batches
        torch.cuda.empty_cache()
        os.environ["KAREUS_B200_LIBRARY_BASELINE"] = "1"
        streams_mode = os.environ.get("KAREUS_COMM_STREAMS")
        os.environ["KAREUS_COMM_STREAMS"] = "shared"          # one ordered side stream, like the reference
        try:
            bt, _ = make_trainer("allreduce", "nccl")
            bt.model.decoder.engine.replay = False
            bdev = [bt.to_device(b) for b in host_batches]

            def bstep(i):
                bt.optimizer.zero_grad()
                l_ = bt.forward_backward(bdev[i % 2], denom)
                bt.model.finalize_grads()
                bt.optimizer.step()
                return l_

            for i in range(3):
                bstep(i)
            sync_all()
            be0 = sampler.energy_mj()
            bs, be = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            bs.record()
            for i in range(args.baseline_steps):
                bl = bstep(i)
            be.record()
            sync_all()
            be1 = sampler.energy_mj()
            bt_ms = torch.tensor([bs.elapsed_time(be)], device=device, dtype=torch.float64)
            ben = torch.tensor([(be1 - be0) / 1000.0 if (be0 is not None and be1 is not None) else 0.0],
                               device=device, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(bt_ms, op=dist.ReduceOp.MAX)
                dist.all_reduce(ben, op=dist.ReduceOp.SUM)
            bms = float(bt_ms.item())
            baseline = {"value": tokens_per_step * args.baseline_steps / (bms / 1000.0), "unit": "tokens/s",
                        "ms_per_step": bms / args.baseline_steps, "steps": args.baseline_steps, "warmup": 3,
                        "energy_j_per_step": float(ben.item()) / args.baseline_steps, "loss": bt.reduce_loss(bl),
                        "config": "same model, batch and layout; all-reduce tensor parallelism over NCCL, cuBLAS "
                                  "GEMMs, flash-attention wheel, interpreter-driven launches"}
            del bt, bdev
        finally:
            os.environ.pop("KAREUS_B200_LIBRARY_BASELINE", None)
            if streams_mode is None:
                os.environ.pop("KAREUS_COMM_STREAMS", None)
            else:
                os.environ["KAREUS_COMM_STREAMS"] = streams_mode
    else:
        replayed = trainer.model.decoder.engine.replayed_regions

    layout = "".join(f"{k}{v}" for k, v in (("tp", tp), ("pp", args.pp), ("cp", args.cp), ("dp", dp)) if v > 1) or "tp1"
    if rank == 0:
        out = {
            "metric": f"tokens/s ({cfg.name} training throughput)" if args.model != "llama3.2_3b" else
                      "tokens/s (Llama-3.2-3B training throughput)", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": value / BASELINE_TOKENS_PER_S,
            "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
            "config": {"model": args.model, "global_batch": args.gbs, "micro_batch": args.mbs, "seq_len": args.seq,
                       "parallelism": layout, "nanobatches": args.nano, "tp_comm": par.tp_comm,
                       "cp_comm": args.cp_comm if args.cp > 1 else None,
                       "comm_backend": par.comm_backend, "comm_sm": args.comm_sm,
                       "ag_drivers": ("as comm_sm" if os.environ.get("KAREUS_AG_AUTO", "1") == "0" else
                                      "comm_sm x3 up to N=768, x2 up to N=1280, at most a third of the kernel's SMs"),
                       "sync": os.environ.get("KAREUS_SYNC", "partition_end"),
                       "comm_streams": os.environ.get("KAREUS_COMM_STREAMS", "shared"),
                       "fused_sms": os.environ.get("KAREUS_FUSED_SMS", "0"), "recompute": f"full, {args.recompute_layers} layers per chunk",
                       "optimizer": "AdamW fp32 master, in the timed region",
                       "l2": "inputs larger than L2 (6.4 GB of weights and multi-GB activations per step)"},
            "energy_j_per_step": float(en.item()) / args.steps,
            "clocks": sampler.summary(), "e2e": e2e, "gpu_launches": launches, "loss": final_loss,
            "first_step_loss": first_loss, "launches_per_step": launches / args.steps,
            "host_enqueue_ms_per_step": host_ms / args.steps,
            "host_us_per_launch": host_ms * 1000.0 / max(1, launches),
            "launch_list_regions_replayed": replayed,
            "nccl_cublas_baseline": baseline, "pipeline_p2p": p2p,
            "impl": "ours",
        }
        print(json.dumps(out))
    for h in (heap, heap_cp):
        if h is not None:
            h.close()          # collective: unbinds switch multicast memory before any rank leaves
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
