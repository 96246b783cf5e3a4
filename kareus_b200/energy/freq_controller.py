"""Asynchronous SM-clock controller.

``FrequencyController.set_frequency(mhz)`` never blocks the training thread: a worker thread per
GPU takes the newest requested clock from a one-slot mailbox and applies NVML locked clocks
``(f, f)``.  This is the behaviour of the frequency-controller worker inside zeus'
``PipelineFrequencyOptimizer`` that the reference drives at every pipeline instruction
(``3rdparty/Megatron-LM/megatron/core/pipeline_parallel/schedules.py:282-284,407-409``).

Changing clocks alters a GPU for every process that shares it, so this class has three modes:

* ``"off"``      — default; requests are ignored;
* ``"advisory"`` — requests are recorded (``history``) but no setting is touched;
* ``"locked"``   — NVML locked clocks are applied; ``close()`` (also run at interpreter exit and on
  ``__exit__``) resets them.  If the first NVML call is refused the controller drops to advisory.
"""
from __future__ import annotations

import atexit
import threading
import time
from typing import List, Optional, Tuple

from .nvml import NVMLError, get_nvml

MODES = ("off", "advisory", "locked")


class FrequencyController:
    def __init__(self, nvml_index: int = 0, mode: str = "off", nvml=None, settle_s: float = 0.0):
        if mode not in MODES:
            raise ValueError(f"mode must be one of {MODES}")
        self.mode = mode
        self.nvml = nvml if nvml is not None else (get_nvml() if mode == "locked" else None)
        self.index = nvml_index
        self.handle = self.nvml.handle(nvml_index) if self.nvml is not None else None
        self.settle_s = settle_s
        self.history: List[Tuple[float, int]] = []
        self.applied: Optional[int] = None
        self.errors: List[str] = []
        self._want: Optional[int] = None
        self._cv = threading.Condition()
        self._stop = False
        self._dirty = False
        self._thread: Optional[threading.Thread] = None
        if mode == "locked":
            self._thread = threading.Thread(target=self._worker, name=f"freqctl-{nvml_index}", daemon=True)
            self._thread.start()
            atexit.register(self.close)

    # ------------------------------------------------------------------ API
    def set_frequency(self, mhz: int) -> None:
        if self.mode == "off":
            return
        self.history.append((time.monotonic(), int(mhz)))
        if self.mode != "locked":
            return
        with self._cv:
            self._want = int(mhz)
            self._dirty = True
            self._cv.notify()

    def wait_idle(self, timeout: float = 5.0) -> bool:
        """Block until the worker has applied the latest request (tests, profilers)."""
        end = time.monotonic() + timeout
        with self._cv:
            while self._dirty and time.monotonic() < end:
                self._cv.wait(0.01)
            return not self._dirty

    def close(self) -> None:
        if self._thread is None:
            return
        with self._cv:
            self._stop = True
            self._cv.notify()
        self._thread.join(timeout=5.0)
        self._thread = None
        if self.applied is not None:
            try:
                self.nvml.reset_locked_clocks(self.handle)
            except NVMLError as e:
                self.errors.append(str(e))
            self.applied = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ------------------------------------------------------------------ worker
    def _worker(self) -> None:
        while True:
            with self._cv:
                while not self._dirty and not self._stop:
                    self._cv.wait()
                if self._stop:
                    return
                f = self._want
            if f != self.applied:
                try:
                    self.nvml.set_locked_clocks(self.handle, f, f)
                    self.applied = f
                    if self.settle_s:
                        time.sleep(self.settle_s)
                except NVMLError as e:
                    self.errors.append(str(e))
                    self.mode = "advisory"       # no permission: keep recording, stop touching NVML
            with self._cv:
                if self._want == f:
                    self._dirty = False
                self._cv.notify_all()
            if self.mode != "locked":
                with self._cv:
                    self._dirty = False
                    self._cv.notify_all()
                return
