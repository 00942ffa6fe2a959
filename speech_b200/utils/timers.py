"""Named wall-clock timers with optional CUDA synchronisation and a device-side event timer.

``NamedTimer`` mirrors ``nemo/utils/timers.py:28`` (start/stop by name, rolling buffer, mean /
sum / last reductions).  ``CudaEventTimer`` times a region on the launching stream with CUDA
events, which is how every throughput number in this framework is taken.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch


class NamedTimer:
    _REDUCTION_TYPE = ["mean", "sum", "min", "max", "none"]

    def __init__(self, reduction: str = "mean", sync_cuda: bool = False, buffer_size: int = 1):
        if reduction not in self._REDUCTION_TYPE:
            raise ValueError(f"Unknown reduction={reduction} please use one of {self._REDUCTION_TYPE}")
        self._reduction, self._sync_cuda, self._buffer_size = reduction, sync_cuda, buffer_size
        self.timers: Dict[str, Dict] = {}

    @property
    def buffer_size(self) -> int:
        return self._buffer_size

    def __getitem__(self, k: str):
        return self.get(k)

    def reset(self, name: Optional[str] = None):
        if name is None:
            self.timers = {}
        else:
            self.timers[name] = {}

    def is_active(self, name: str) -> bool:
        return self.timers.get(name, {}).get("start", None) is not None

    def _sync(self):
        if self._sync_cuda and torch.cuda.is_available() and torch.cuda.is_initialized():
            torch.cuda.synchronize()

    def start(self, name: str = ""):
        t = self.timers.setdefault(name, {})
        if t.get("start") is not None:
            raise RuntimeError(f"Cannot start timer = '{name}' since it is already active")
        self._sync()
        t["start"] = time.time()

    def stop(self, name: str = ""):
        t = self.timers.get(name)
        if t is None or t.get("start") is None:
            raise RuntimeError(f"Cannot end timer = '{name}' since it is not active")
        self._sync()
        dt = time.time() - t.pop("start")
        buf: List[float] = t.setdefault("dt", [])
        buf.append(dt)
        if self._buffer_size > 0:
            del buf[: max(0, len(buf) - self._buffer_size)]
        t["start"] = None

    def active_timers(self):
        return [k for k, v in self.timers.items() if v.get("start") is not None]

    def get(self, name: str = ""):
        dt = self.timers.get(name, {}).get("dt", [])
        r = self._reduction
        if r == "none":
            return dt
        if not dt:
            return 0.0
        return {"mean": sum(dt) / len(dt), "sum": sum(dt), "min": min(dt), "max": max(dt)}[r]

    def export(self):
        return {k: self.get(k) for k in self.timers}


class SimpleTimer:
    def __init__(self):
        self.reset()

    def reset(self):
        self._t0, self.total = None, 0.0

    def start(self, device=None):
        if device is not None and torch.cuda.is_available():
            torch.cuda.synchronize(device)
        self._t0 = time.perf_counter()

    def stop(self, device=None):
        if device is not None and torch.cuda.is_available():
            torch.cuda.synchronize(device)
        self.total += time.perf_counter() - self._t0
        self._t0 = None

    def total_sec(self) -> float:
        return self.total


class CudaEventTimer:
    """Device time of a region: ``with CudaEventTimer() as t: ...; t.ms``."""

    def __init__(self, stream: Optional[torch.cuda.Stream] = None):
        self.stream = stream
        self.ms = 0.0

    def __enter__(self):
        self._a = torch.cuda.Event(enable_timing=True)
        self._b = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        self._a.record(self.stream)
        return self

    def __exit__(self, *exc):
        self._b.record(self.stream)
        torch.cuda.synchronize()
        self.ms = self._a.elapsed_time(self._b)
        return False
