"""NVML access behind one small interface, with a simulated implementation for tests.

The real backend uses ``pynvml`` (``nvidia-ml-py``).  Everything that *changes* a GPU setting
(locked clocks) lives in :class:`kareus_b200.energy.freq_controller.FrequencyController`, is off
unless explicitly enabled, and is exercised in the test-suite only against :class:`FakeNVML`.
Reads (energy counter, power, clocks, throttle reasons) are always safe.

Reference usage: ``nvmlDeviceSetGpuLockedClocks`` / energy counters through zeus
(``tests/bayesian/common/hardware.py:52-73,113-126``), the clock/throttle logger
(``3rdparty/NeMo/.../megatron_base_model.py:163-263``) and the energy poller
(``3rdparty/Megatron-LM/megatron/core/timers.py:311-340``).
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional, Sequence

THROTTLE_BITS = {
    0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
    0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
    0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
}


def decode_throttle(mask: int) -> List[str]:
    return [n for b, n in THROTTLE_BITS.items() if mask & b]


class NVMLError(RuntimeError):
    pass


class RealNVML:
    """Thin adapter over pynvml; one instance per process."""

    def __init__(self):
        try:
            import pynvml
        except Exception as e:  # pragma: no cover - image always has it
            raise NVMLError(f"pynvml is not importable: {e}")
        self.nv = pynvml
        try:
            pynvml.nvmlInit()
        except Exception as e:
            raise NVMLError(f"nvmlInit failed: {e}")

    def device_count(self) -> int:
        return self.nv.nvmlDeviceGetCount()

    def handle(self, index: int):
        return self.nv.nvmlDeviceGetHandleByIndex(index)

    def name(self, h) -> str:
        n = self.nv.nvmlDeviceGetName(h)
        return n.decode() if isinstance(n, bytes) else n

    def total_energy_mj(self, h) -> int:
        return int(self.nv.nvmlDeviceGetTotalEnergyConsumption(h))

    def power_w(self, h) -> float:
        return self.nv.nvmlDeviceGetPowerUsage(h) / 1000.0

    def sm_clock(self, h) -> int:
        return int(self.nv.nvmlDeviceGetClockInfo(h, self.nv.NVML_CLOCK_SM))

    def max_sm_clock(self, h) -> int:
        return int(self.nv.nvmlDeviceGetMaxClockInfo(h, self.nv.NVML_CLOCK_SM))

    def supported_sm_clocks(self, h) -> List[int]:
        mem = self.nv.nvmlDeviceGetSupportedMemoryClocks(h)
        out = set()
        for m in mem[:1]:
            out.update(self.nv.nvmlDeviceGetSupportedGraphicsClocks(h, m))
        return sorted(out, reverse=True)

    def throttle_mask(self, h) -> int:
        fn = getattr(self.nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            self.nv.nvmlDeviceGetCurrentClocksThrottleReasons
        return int(fn(h))

    def set_locked_clocks(self, h, lo: int, hi: int) -> None:
        try:
            self.nv.nvmlDeviceSetGpuLockedClocks(h, int(lo), int(hi))
        except Exception as e:
            raise NVMLError(f"nvmlDeviceSetGpuLockedClocks({lo},{hi}) failed: {e}")

    def reset_locked_clocks(self, h) -> None:
        try:
            self.nv.nvmlDeviceResetGpuLockedClocks(h)
        except Exception as e:
            raise NVMLError(f"nvmlDeviceResetGpuLockedClocks failed: {e}")


class FakeNVML:
    """Simulated GPUs: power is ``static + k·f³·load`` and the energy counter integrates it.

    ``deny_clock_control`` makes ``set_locked_clocks`` raise like an unprivileged NVML call;
    ``calls`` records every setting change so tests can assert on what would have been done.
    """

    def __init__(self, n: int = 8, max_clock: int = 1965, min_clock: int = 210, step: int = 15,
                 static_w: float = 190.0, peak_w: float = 1000.0, time_fn: Callable[[], float] = time.monotonic,
                 deny_clock_control: bool = False):
        self.n, self.max_clock, self.min_clock, self.step = n, max_clock, min_clock, step
        self.static_w, self.peak_w = static_w, peak_w
        self.time_fn = time_fn
        self.deny = deny_clock_control
        self.locked: Dict[int, Optional[int]] = {i: None for i in range(n)}
        self.load: Dict[int, float] = {i: 1.0 for i in range(n)}
        self._e: Dict[int, float] = {i: 0.0 for i in range(n)}
        self._t: Dict[int, float] = {i: time_fn() for i in range(n)}
        self.calls: List[tuple] = []
        self._lock = threading.Lock()

    def device_count(self) -> int:
        return self.n

    def handle(self, index: int):
        if not 0 <= index < self.n:
            raise NVMLError(f"invalid device index {index}")
        return index

    def name(self, h) -> str:
        return "Fake B200"

    def _clock(self, h) -> int:
        return self.locked[h] if self.locked[h] is not None else self.max_clock

    def power_w(self, h) -> float:
        f = self._clock(h) / self.max_clock
        return self.static_w + (self.peak_w - self.static_w) * (f ** 3) * self.load[h]

    def _integrate(self, h) -> None:
        now = self.time_fn()
        self._e[h] += self.power_w(h) * (now - self._t[h])
        self._t[h] = now

    def total_energy_mj(self, h) -> int:
        with self._lock:
            self._integrate(h)
            return int(self._e[h] * 1000.0)

    def sm_clock(self, h) -> int:
        return self._clock(h)

    def max_sm_clock(self, h) -> int:
        return self.max_clock

    def supported_sm_clocks(self, h) -> List[int]:
        return list(range(self.max_clock, self.min_clock - 1, -self.step))

    def throttle_mask(self, h) -> int:
        return 0x4 if self.power_w(h) > 0.99 * self.peak_w else 0

    def set_load(self, h, load: float) -> None:
        with self._lock:
            self._integrate(h)
            self.load[h] = load

    def set_locked_clocks(self, h, lo: int, hi: int) -> None:
        if self.deny:
            raise NVMLError("insufficient permissions (simulated)")
        with self._lock:
            self._integrate(h)
            self.locked[h] = int(hi)
            self.calls.append(("lock", h, int(lo), int(hi)))

    def reset_locked_clocks(self, h) -> None:
        if self.deny:
            raise NVMLError("insufficient permissions (simulated)")
        with self._lock:
            self._integrate(h)
            self.locked[h] = None
            self.calls.append(("reset", h))


_DEFAULT = None


def get_nvml(fake: Optional[FakeNVML] = None):
    """The process-wide NVML backend (``fake`` overrides it, used by tests)."""
    global _DEFAULT
    if fake is not None:
        return fake
    if _DEFAULT is None:
        _DEFAULT = RealNVML()
    return _DEFAULT
