"""Tracing and profiling hooks: NVTX ranges, per-phase timers on the device clock, a ``torch.profiler`` window.

The reference has no tracing at all: only ``VERBOSE=1`` prints of pipeline/ring messages
(``pp_communications.py:6``, ``cp_communications.py:8``) and ``torch.cuda.memory_reserved()`` in the step line
(``train.py:257``). Three tools are provided here, all off by default and all free when off:

* :func:`nvtx_range` -- named ranges (optimizer step, micro-batches, pipeline phases, decoder layers) that show up
  in Nsight Systems / Nsight Compute timelines. Enabled with ``logging.nvtx`` in the config or ``PICOTRON_NVTX=1``.
* :class:`PhaseTimer` -- accumulates the time of named phases of a step. On a CUDA device a phase is bracketed by
  two events recorded on the current stream (no host synchronisation while the step runs); the events are resolved
  once, when the summary is read. On the CPU it is ``time.perf_counter``.
* :class:`ProfilerWindow` -- runs ``torch.profiler`` for a window of steps given by ``logging.profile`` and writes a
  Chrome trace per rank. ``logging.profile`` may be ``true`` (steps 3..4) or ``{"start_step", "num_steps", "dir"}``.
"""
from __future__ import annotations

import contextlib
import os
import time
from typing import Any, Dict, List, Optional, Tuple

import torch

_NVTX = os.environ.get("PICOTRON_NVTX", "0") == "1"


def enable_nvtx(on: bool = True) -> None:
    global _NVTX
    _NVTX = bool(on)


def nvtx_enabled() -> bool:
    return _NVTX and torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str):
    """``with nvtx_range("optimizer"):`` -- a pushed/popped NVTX range when enabled, nothing otherwise."""
    if not nvtx_enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


class PhaseTimer:
    """Accumulated time per named phase, measured on the device clock where there is one."""

    def __init__(self, device: Optional[torch.device] = None, enabled: bool = True):
        self.enabled = enabled
        self.cuda = bool(device is not None and torch.device(device).type == "cuda" and torch.cuda.is_available())
        self._pending: List[Tuple[str, Any, Any]] = []       # (phase, start event, end event) not yet resolved
        self._ms: Dict[str, float] = {}
        self._count: Dict[str, int] = {}

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        with nvtx_range(name):
            if self.cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                try:
                    yield
                finally:
                    e1.record()
                    self._pending.append((name, e0, e1))
            else:
                t0 = time.perf_counter()
                try:
                    yield
                finally:
                    self._add(name, (time.perf_counter() - t0) * 1e3)

    def _add(self, name: str, ms: float) -> None:
        self._ms[name] = self._ms.get(name, 0.0) + ms
        self._count[name] = self._count.get(name, 0) + 1

    def summary(self, reset: bool = True) -> Dict[str, float]:
        """Milliseconds per phase since the last reset. Resolving CUDA events waits for the last one to complete."""
        if self._pending:
            self._pending[-1][2].synchronize()
            for name, e0, e1 in self._pending:
                self._add(name, e0.elapsed_time(e1))
            self._pending.clear()
        out = dict(self._ms)
        if reset:
            self._ms.clear()
            self._count.clear()
        return out


# Timer that library code outside the trainer (the pipeline schedules) reports its phases to; the trainer installs its own
# PhaseTimer here when ``logging.phase_timers`` is set. Disabled timers cost one attribute test per phase.
_ACTIVE_TIMER = PhaseTimer(enabled=False)


def set_active_timer(timer: Optional[PhaseTimer]) -> None:
    global _ACTIVE_TIMER
    _ACTIVE_TIMER = timer if timer is not None else PhaseTimer(enabled=False)


def timed_phase(name: str):
    """``with timed_phase("pp/forward"):`` -- a phase of the active timer (see :func:`set_active_timer`)."""
    return _ACTIVE_TIMER.phase(name)


class ProfilerWindow:
    """``torch.profiler`` over ``num_steps`` steps starting at ``start_step``; one Chrome trace per rank.

    ``step()`` is called once per optimizer step (after it). Outside the window, and when ``spec`` is falsy, every
    method is a no-op, so the training loop can call them unconditionally.
    """

    def __init__(self, spec: Any, rank: int = 0, default_dir: str = "./profile"):
        self.prof = None
        self.path: Optional[str] = None
        if not spec:
            return
        if spec is True:
            spec = {}
        start = int(spec.get("start_step", 3))
        num = int(spec.get("num_steps", 2))
        out_dir = spec.get("dir", default_dir)
        os.makedirs(out_dir, exist_ok=True)
        self.path = os.path.join(out_dir, f"trace_rank{rank}.json")
        activities = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            activities.append(torch.profiler.ProfilerActivity.CUDA)
        # steps are counted from 1 by the trainer: skip `start - 1` steps, then record `num`
        self.prof = torch.profiler.profile(
            activities=activities,
            schedule=torch.profiler.schedule(wait=max(start - 1, 0), warmup=0, active=num, repeat=1),
            on_trace_ready=lambda p: p.export_chrome_trace(self.path),
            record_shapes=bool(spec.get("record_shapes", False)), with_stack=bool(spec.get("with_stack", False)))
        self.prof.__enter__()

    def step(self) -> None:
        if self.prof is not None:
            self.prof.step()

    def close(self) -> None:
        if self.prof is not None:
            self.prof.__exit__(None, None, None)
            self.prof = None
