"""Static ("blocked in a p2p wait") power probe.

Rank 0 blocks in a receive for ``duration_s`` while its board power is integrated; the mean power
is the ``P_p2p`` constant the planner subtracts to get effective energy (reference
``tests/data/profile_p2p.py:27-88``; A100 85 W, A40 70 W in ``tests/bayesian/common/
model_config.py:14-15``).  The B200 value has to be measured on the box in use.
"""
from __future__ import annotations

import time
from typing import Optional

from .monitor import EnergyMonitor


def probe_p2p_power(duration_s: float = 60.0, monitor: Optional[EnergyMonitor] = None, device=None,
                    sleep_fn=time.sleep) -> float:
    """Run on 2 ranks.  Returns watts on rank 0 (0.0 elsewhere)."""
    import torch
    import torch.distributed as dist
    rank = dist.get_rank()
    dev = device if device is not None else ("cuda" if torch.cuda.is_available() and dist.get_backend() == "nccl" else "cpu")
    buf = torch.zeros(1 << 20, device=dev)
    if rank == 0:
        monitor = monitor or EnergyMonitor([torch.cuda.current_device()] if dev != "cpu" else [0])
        monitor.begin_window("p2p_wait", sync=False)
        dist.recv(buf, src=1)                 # blocks until rank 1 sends, `duration_s` later
        if dev != "cpu":
            torch.cuda.synchronize()
        m = monitor.end_window("p2p_wait", sync=False, cancel=True)
        return m.total_energy / max(m.time, 1e-9)
    if rank == 1:
        sleep_fn(duration_s)
        dist.send(buf, dst=0)
    return 0.0


def main(argv=None) -> int:
    """``torchrun --nproc-per-node 2 -m kareus_b200.energy.p2p_probe --duration 20`` prints one JSON line
    with the measured watts (rank 0's GPU, blocked in an NCCL receive)."""
    import argparse
    import json
    import torch
    import torch.distributed as dist
    from ..parallel.mesh import init_distributed
    ap = argparse.ArgumentParser()
    ap.add_argument("--duration", type=float, default=20.0)
    a = ap.parse_args(argv)
    rank, world, local = init_distributed()
    if world < 2:
        raise SystemExit("the probe needs two ranks")
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
        # make sure the communicator exists before the measured wait
        t = torch.zeros(1, device="cuda")
        dist.all_reduce(t)
        torch.cuda.synchronize()
    monitor = None
    if not torch.cuda.is_available():
        # no GPU: the run only shows that the probe works; its watts come from the simulated NVML
        from .nvml import FakeNVML
        monitor = EnergyMonitor([0], nvml=FakeNVML(1))
    watts = probe_p2p_power(a.duration, monitor=monitor)
    if rank == 0:
        line = {"p2p_wait_power_w": watts, "duration_s": a.duration,
                "gpu": torch.cuda.get_device_name(local) if torch.cuda.is_available() else "cpu"}
        if monitor is not None:
            line["simulated"] = True
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
