"""Host-side failure detection: a per-rank watchdog that flags a training step exceeding its deadline.

The reference has only the 3-minute collective timeout of ``init_process_group`` (``train.py:94``) and a
post-mortem grep of the job log (``template/base_job.slurm:82-94``). The watchdog adds an in-job signal:
a daemon thread that, if a step does not finish within ``timeout_s``, records the event (``fired``),
prints a diagnostic with the step index and -- when ``abort`` is set -- terminates the process with exit
code 124 so that the launcher (``torchrun --max_restarts``) or the Slurm wrapper can classify the job
as ``timeout`` and resume from the latest checkpoint. Nothing here touches the GPU.
"""
from __future__ import annotations

import contextlib
import os
import sys
import threading
import time
from typing import Callable, Optional


class StepWatchdog:
    def __init__(self, timeout_s: float = 0.0, abort: bool = False, on_timeout: Optional[Callable[[int], None]] = None):
        self.timeout_s = timeout_s
        self.abort = abort
        self.on_timeout = on_timeout
        self.fired = False
        self.fired_step: Optional[int] = None
        self._deadline: Optional[float] = None
        self._step = -1
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        if timeout_s > 0:
            self._thread = threading.Thread(target=self._run, name="step-watchdog", daemon=True)
            self._thread.start()

    def _run(self):
        while not self._stop.wait(min(0.05, self.timeout_s / 4)):
            with self._lock:
                expired = self._deadline is not None and time.monotonic() > self._deadline
                step = self._step
                if expired:
                    self._deadline = None
            if expired:
                self.fired, self.fired_step = True, step
                sys.stderr.write(f"[watchdog] Timeout: step {step} exceeded {self.timeout_s:.1f}s on rank "
                                 f"{os.environ.get('RANK', '0')}\n")
                sys.stderr.flush()
                if self.on_timeout is not None:
                    self.on_timeout(step)
                if self.abort:
                    os._exit(124)

    @contextlib.contextmanager
    def step(self, step_idx: int):
        if self.timeout_s > 0:
            with self._lock:
                self._step = step_idx
                self._deadline = time.monotonic() + self.timeout_s
        try:
            yield
        finally:
            with self._lock:
                self._deadline = None

    def close(self):
        self._stop.set()
