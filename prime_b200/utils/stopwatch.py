"""Named, nestable wall-clock timers that also open profiler / NVTX ranges
(reference: src/zeroband/utils/stopwatch.py:9-130). Ranges are always emitted (they are what a
torch.profiler or Nsight trace shows); the lap log lines are only produced at DEBUG level."""
from __future__ import annotations

import time
from contextlib import contextmanager

import torch
from torch.autograd.profiler import record_function

_NVTX = torch.cuda.is_available()


class _RecordBlockContext:
    def __init__(self, sw_ref: "Stopwatch", prof_name: str):
        self.sw_ref = sw_ref
        self.rf = record_function(prof_name)
        self.name = prof_name

    def __enter__(self):
        self.rf.__enter__()
        if _NVTX:
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        if _NVTX:
            torch.cuda.nvtx.range_pop()
        self.rf.__exit__(exc_type, exc_value, traceback)
        self.sw_ref.stop()


class Stopwatch:
    def __init__(self, config=None):
        self.timers: dict[str, dict[str, float]] = {}
        self.stack: list[str] = []
        self.disabled = (config.log_level != "DEBUG") if config else False
        self.logger = None

    def _log(self, msg: str):
        if self.logger is None:
            from .logger import get_logger
            self.logger = get_logger()
        self.logger.debug(msg)

    def record_block(self, message: str | None = None, name: str | None = None) -> _RecordBlockContext:
        self.start(message, name)
        return _RecordBlockContext(self, message or name or "block")

    def start(self, message: str | None = None, name: str | None = None) -> None:
        if self.disabled:
            return
        name = name or message or f"_sw_{len(self.timers)}"
        self.timers[name] = {"start_time": time.perf_counter(), "last_lap_time": time.perf_counter()}
        self.timers[name]["message"] = message
        self.stack.append(name)
        if message:
            self._log(f"Starting {message}")

    def lap(self, message: str | None = None, name: str | None = None) -> float:
        if self.disabled:
            return 0.0
        name = name or (self.stack[-1] if self.stack else None)
        if name is None or name not in self.timers:
            raise ValueError(f"Timer {name!r} was never started")
        now = time.perf_counter()
        t = self.timers[name]
        lap = now - t["last_lap_time"]
        t["last_lap_time"] = now
        if message:
            self._log(f"{message} took {lap:.4f} s")
        return lap

    def elapsed(self, name: str | None = None) -> float:
        if self.disabled:
            return 0.0
        name = name or (self.stack[-1] if self.stack else None)
        if name is None or name not in self.timers:
            raise ValueError(f"Timer {name!r} was never started")
        return time.perf_counter() - self.timers[name]["start_time"]

    def stop(self, name: str | None = None) -> float:
        if self.disabled:
            return 0.0
        if name is None:
            if not self.stack:
                return 0.0
            name = self.stack.pop()
        elif name in self.stack:
            self.stack.remove(name)
        t = self.timers.pop(name)
        total = time.perf_counter() - t["start_time"]
        if t.get("message"):
            self._log(f"Finished {t['message']} in {total:.4f} s")
        return total

    @contextmanager
    def timed(self, message: str):
        self.start(message)
        try:
            yield
        finally:
            self.stop()
