"""Window-based time/energy measurement from the NVML total-energy counter.

Semantics follow what the reference gets from ``ZeusMonitor`` (zeus 0.15.1; call sites
``3rdparty/NeMo/.../megatron_base_model.py:350-363``, ``kareus/nemo/.../megatron_gpt_model.py:
612-613,683-689,843-844``; consumer ``tests/artifact/compare_method.py:85-100``):
``begin_window(name)`` / ``end_window(name)`` synchronise the GPUs, read the wall clock and the
energy counter (mJ) and return ``Measurement(time, gpu_energy{idx: J}, total_energy)``; windows
nest; with ``log_file`` every finished window appends a CSV row with the columns
``start_time,window_name,elapsed_time,gpu<N>_energy``.

``measure()`` is the repeated-call profiler the Bayesian search uses
(``zeus.profile.measure``; ``tests/bayesian/common/hardware.py:118-132``).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Dict, List, Optional, Sequence

from .nvml import get_nvml


@dataclass
class Measurement:
    time: float
    gpu_energy: Dict[int, float]

    @property
    def total_energy(self) -> float:
        return sum(self.gpu_energy.values())


def _cuda_sync(indices: Sequence[int]) -> None:
    try:
        import torch
        if torch.cuda.is_available():
            for i in indices:
                if i < torch.cuda.device_count():
                    torch.cuda.synchronize(i)
    except Exception:
        pass


class EnergyMonitor:
    def __init__(self, gpu_indices: Optional[Sequence[int]] = None, log_file: Optional[str] = None,
                 nvml=None, sync_fn: Optional[Callable[[Sequence[int]], None]] = None,
                 time_fn: Callable[[], float] = time.monotonic, nvml_indices: Optional[Sequence[int]] = None):
        """``gpu_indices`` are CUDA device indices (for synchronisation and column names);
        ``nvml_indices`` the matching NVML indices when ``CUDA_VISIBLE_DEVICES`` remaps them."""
        self.nvml = nvml or get_nvml()
        self.gpu_indices = list(gpu_indices) if gpu_indices is not None else [0]
        nv_idx = list(nvml_indices) if nvml_indices is not None else _visible_to_nvml(self.gpu_indices)
        self.handles = {g: self.nvml.handle(n) for g, n in zip(self.gpu_indices, nv_idx)}
        self.sync_fn = sync_fn or _cuda_sync
        self.time_fn = time_fn
        self._open: Dict[str, tuple] = {}
        self.history: List[tuple] = []
        self.log_file = Path(log_file) if log_file else None
        if self.log_file is not None:
            self.log_file.parent.mkdir(parents=True, exist_ok=True)
            with self.log_file.open("w") as f:
                f.write("start_time,window_name,elapsed_time," +
                        ",".join(f"gpu{g}_energy" for g in self.gpu_indices) + "\n")

    def _read(self) -> Dict[int, int]:
        return {g: self.nvml.total_energy_mj(h) for g, h in self.handles.items()}

    def begin_window(self, name: str, sync: bool = True) -> None:
        if name in self._open:
            raise ValueError(f"measurement window {name!r} is already open")
        if sync:
            self.sync_fn(self.gpu_indices)
        self._open[name] = (self.time_fn(), time.time(), self._read())

    def end_window(self, name: str, sync: bool = True, cancel: bool = False) -> Measurement:
        if name not in self._open:
            raise ValueError(f"measurement window {name!r} was never opened")
        if sync:
            self.sync_fn(self.gpu_indices)
        t0, wall0, e0 = self._open.pop(name)
        t1, e1 = self.time_fn(), self._read()
        m = Measurement(t1 - t0, {g: (e1[g] - e0[g]) / 1000.0 for g in self.gpu_indices})
        if cancel:
            return m
        self.history.append((name, m))
        if self.log_file is not None:
            with self.log_file.open("a") as f:
                f.write(f"{wall0},{name},{m.time}," + ",".join(str(m.gpu_energy[g]) for g in self.gpu_indices) + "\n")
        return m


def _visible_to_nvml(cuda_indices: Sequence[int]) -> List[int]:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if not vis:
        return list(cuda_indices)
    try:
        mapping = [int(x) for x in vis.split(",") if x.strip() != ""]
        return [mapping[i] if i < len(mapping) else i for i in cuda_indices]
    except ValueError:      # UUID form: NVML order equals CUDA order for the visible set
        return list(cuda_indices)


@dataclass
class Trial:
    iterations: int
    time_per_iter: float
    energy_per_iter: float
    total_time: float
    total_energy: float


def measure(target_function: Callable[[], None], monitor: EnergyMonitor, measurement_duration: float = 5.0,
            cooldown_duration: float = 5.0, group=None, min_iterations: int = 1,
            sleep_fn: Callable[[float], None] = time.sleep) -> Trial:
    """Run ``target_function`` back to back for about ``measurement_duration`` seconds inside one
    window.  Collective when ``group``/the default process group exists: every rank runs the same
    number of iterations (rank 0 decides when to stop) and ``energy_per_iter`` is the sum over ranks,
    as callers of the reference's ``zeus.profile.measure`` expect (they divide by the world size)."""
    dist = _dist()
    world = dist.get_world_size(group) if dist is not None else 1
    target_function()                      # warm-up outside the window
    monitor.begin_window("__measure__")
    t0 = monitor.time_fn()
    iters = 0
    while True:
        target_function()
        iters += 1
        stop = (monitor.time_fn() - t0) >= measurement_duration and iters >= min_iterations
        if world > 1:
            import torch
            flag = torch.tensor([1 if stop else 0], dtype=torch.int32,
                                device="cuda" if torch.cuda.is_available() and dist.get_backend(group) == "nccl" else "cpu")
            dist.broadcast(flag, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
            stop = bool(flag.item())
        if stop:
            break
    m = monitor.end_window("__measure__", cancel=True)
    energy = m.total_energy
    if world > 1:
        import torch
        dev = "cuda" if torch.cuda.is_available() and dist.get_backend(group) == "nccl" else "cpu"
        e = torch.tensor([energy], dtype=torch.float64, device=dev)
        dist.all_reduce(e, group=group)
        energy = float(e.item())
    if cooldown_duration > 0:
        sleep_fn(cooldown_duration)
    return Trial(iters, m.time / iters, energy / iters, m.time, energy)


def _dist():
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return dist
    except Exception:
        pass
    return None
