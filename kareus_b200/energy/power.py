"""Background samplers: instantaneous power timeline, SM clock / throttle change points, and the
cumulative energy-counter poller.

Reference: ``PowerMonitor(update_period=0.05)`` and the forked ``gpu_stats_monitor``
(``3rdparty/NeMo/.../megatron_base_model.py:163-263,774-836``), and the Timers energy poller that
writes ``timers/time-energy-G-L.csv`` (``3rdparty/Megatron-LM/megatron/core/timers.py:311-340``).
Samplers are threads (NVML calls release the GIL) rather than forked processes.
"""
from __future__ import annotations

import threading
import time
from pathlib import Path
from typing import Callable, List, Optional, Tuple

from .nvml import decode_throttle, get_nvml


class _Sampler:
    def __init__(self, period_s: float):
        self.period_s = period_s
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def start(self):
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        self._thread.join(timeout=2.0)

    def _run(self):
        while not self._stop.is_set():
            self.sample()
            self._stop.wait(self.period_s)

    def sample(self):  # pragma: no cover - abstract
        raise NotImplementedError


class PowerMonitor(_Sampler):
    """``timeline`` is a list of ``(unix time, watts)``; ``dump`` writes ``timestamp,power``."""

    def __init__(self, nvml_index: int = 0, update_period: float = 0.05, nvml=None):
        super().__init__(update_period)
        self.nvml = nvml or get_nvml()
        self.h = self.nvml.handle(nvml_index)
        self.timeline: List[Tuple[float, float]] = []

    def sample(self):
        self.timeline.append((time.time(), self.nvml.power_w(self.h)))

    def get_power_timeline(self) -> List[Tuple[float, float]]:
        return list(self.timeline)

    def dump(self, path) -> None:
        p = Path(path)
        p.parent.mkdir(parents=True, exist_ok=True)
        with p.open("w") as f:
            f.write("timestamp,power\n")
            for t, w in self.timeline:
                f.write(f"{t},{w}\n")


class GpuStatsMonitor(_Sampler):
    """Logs SM clock and throttle reasons, change points only (``frequency_monitor_*.txt`` /
    ``throttle_monitor_*.txt`` in the reference)."""

    def __init__(self, nvml_index: int = 0, period_s: float = 0.05, nvml=None):
        super().__init__(period_s)
        self.nvml = nvml or get_nvml()
        self.h = self.nvml.handle(nvml_index)
        self.clock_changes: List[Tuple[float, int]] = []
        self.throttle_changes: List[Tuple[float, List[str]]] = []
        self._last_clock, self._last_mask = None, None

    def sample(self):
        now = time.time()
        c = self.nvml.sm_clock(self.h)
        if c != self._last_clock:
            self.clock_changes.append((now, c))
            self._last_clock = c
        m = self.nvml.throttle_mask(self.h)
        if m != self._last_mask:
            self.throttle_changes.append((now, decode_throttle(m)))
            self._last_mask = m

    def dump(self, freq_path, throttle_path) -> None:
        for path, rows, hdr in ((freq_path, self.clock_changes, "timestamp,sm_clock_mhz"),
                                (throttle_path, self.throttle_changes, "timestamp,reasons")):
            p = Path(path)
            p.parent.mkdir(parents=True, exist_ok=True)
            with p.open("w") as f:
                f.write(hdr + "\n")
                for t, v in rows:
                    f.write(f"{t},{'|'.join(v) if isinstance(v, list) else v}\n")


class EnergyPoller(_Sampler):
    """Polls the cumulative energy counter; ``dump`` writes ``time,energy`` (unix seconds, joules), the
    ``timers/time-energy-<global rank>-<local rank>.csv`` file of the reference's energy poller."""

    def __init__(self, nvml_index: int = 0, period_s: float = 0.01, nvml=None):
        super().__init__(period_s)
        self.nvml = nvml or get_nvml()
        self.h = self.nvml.handle(nvml_index)
        self.samples: List[Tuple[float, int]] = []

    def sample(self):
        self.samples.append((time.time(), self.nvml.total_energy_mj(self.h)))

    def dump(self, path) -> None:
        p = Path(path)
        p.parent.mkdir(parents=True, exist_ok=True)
        with p.open("w") as f:
            f.write("time,energy\n")
            for t, e in self.samples:
                f.write(f"{t},{e / 1000.0}\n")
