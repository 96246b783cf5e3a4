"""Measure configurations on real GPUs: clock → settle → repeated-run measurement → cool-down.

Reference ``tests/bayesian/common/hardware.py:52-192``: a world of ranks per batch of candidates;
rank 0 locks the SM clock (2 s settle), all ranks barrier, ``measure`` runs the partition for 5 s
and cools down 5 s; ``energy_j`` is the per-GPU mean, ``time_s`` the shared time per iteration.
Clock control goes through :class:`FrequencyController` whose mode defaults to ``"advisory"``:
intended clocks are recorded next to every sample but no GPU setting is changed unless the
operator passes ``clock_mode="locked"``.  The achieved SM clock and throttle reasons are stored
with every sample (on a power-limited part the requested clock is often not the one held).
"""
from __future__ import annotations

import time
from typing import Callable, List, Optional, Sequence, Tuple

from ..energy.freq_controller import FrequencyController
from ..energy.monitor import EnergyMonitor, measure
from ..energy.nvml import decode_throttle
from .space import Config


class HardwareEvaluator:
    def __init__(self, make_executor: Callable[[int], object], monitor: EnergyMonitor,
                 controller: Optional[FrequencyController] = None, world_size: int = 1,
                 measurement_duration: float = 5.0, cooldown_duration: float = 5.0, settle_s: float = 2.0,
                 group=None, sleep_fn=time.sleep):
        self.make_executor, self.monitor = make_executor, monitor
        self.controller = controller or FrequencyController(mode="advisory")
        self.world_size, self.group = world_size, group
        self.duration, self.cooldown, self.settle_s = measurement_duration, cooldown_duration, settle_s
        self.sleep_fn = sleep_fn
        self._executors = {}
        self.samples: List[dict] = []

    def _executor(self, nano: int):
        if nano not in self._executors:
            ex = self.make_executor(nano)
            for _ in range(3):          # first calls pay for lazy initialisation (buffers, function attributes)
                ex.execute(("first", "none"), (16, 1024))
            self._executors[nano] = ex
        return self._executors[nano]

    def __call__(self, configs: Sequence[Config]) -> List[Tuple[float, float]]:
        out = []
        for c in configs:
            ex = self._executor(c.nano)
            self.controller.set_frequency(c.freq)
            if self.controller.mode == "locked":
                self.controller.wait_idle()
                self.sleep_fn(self.settle_s)
            trial = measure(lambda: ex.execute(c.overlap, (c.sm, c.block)), self.monitor, self.duration,
                            self.cooldown, group=self.group, sleep_fn=self.sleep_fn)
            nv, h = self.monitor.nvml, next(iter(self.monitor.handles.values()))
            self.samples.append({"config": c.key(), "sm_clock": nv.sm_clock(h),
                                 "throttle": decode_throttle(nv.throttle_mask(h)), "iterations": trial.iterations})
            out.append((trial.time_per_iter, trial.energy_per_iter / self.world_size))
        return out

    def close(self) -> None:
        self.controller.close()
