"""Lightweight region timers (reference: clt/training/profiler.py:13-240).

Same region names as the reference so dashboards keep working (``data_loading``, ``forward_pass``,
``loss_computation``, ``backward_pass``, ``optimizer_step``, ...).  CUDA regions are timed with event
pairs that are resolved lazily when a summary is requested, so enabling the profiler does not insert a
device synchronisation into every region (the reference synchronises on every timer exit).  Regions are
also emitted as NVTX ranges.
"""
from __future__ import annotations

import logging
import time
from collections import defaultdict
from contextlib import contextmanager
from typing import Any, Dict, List, Optional

import torch

logger = logging.getLogger(__name__)


class _Region:
    __slots__ = ("elapsed", "_start", "_end", "_t0")

    def __init__(self):
        self.elapsed: Optional[float] = None
        self._start = self._end = None
        self._t0 = 0.0


class TrainingProfiler:
    def __init__(self, enabled: bool = True, log_interval: int = 100):
        self.enabled = enabled
        self.log_interval = log_interval
        self.timings: Dict[str, List[float]] = defaultdict(list)
        self._pending: List[Any] = []  # (name, start_event, end_event)
        self.step_count = 0
        self._cuda = torch.cuda.is_available()

    @contextmanager
    def timer(self, name: str):
        region = _Region()
        if not self.enabled:
            yield region
            return
        if self._cuda:
            torch.cuda.nvtx.range_push(name)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            t0 = time.perf_counter()
            try:
                yield region
            finally:
                end.record()
                torch.cuda.nvtx.range_pop()
                self._pending.append((name, start, end))
                region.elapsed = time.perf_counter() - t0  # host-side time; device time is resolved lazily
        else:
            t0 = time.perf_counter()
            try:
                yield region
            finally:
                region.elapsed = time.perf_counter() - t0
                self.timings[name].append(region.elapsed)

    def record(self, name: str, duration: float) -> None:
        """Accepted for API compatibility: ``timer`` already records its region."""
        return None

    def _resolve(self) -> None:
        if not self._pending:
            return
        torch.cuda.synchronize()
        for name, start, end in self._pending:
            self.timings[name].append(start.elapsed_time(end) / 1e3)
        self._pending.clear()

    def step(self) -> None:
        if not self.enabled:
            return
        self.step_count += 1
        if self.step_count % self.log_interval == 0:
            self.log_summary()

    def get_summary(self) -> Dict[str, Dict[str, float]]:
        if self._cuda:
            self._resolve()
        out = {}
        for name, vals in self.timings.items():
            if vals:
                out[name] = {"avg": sum(vals) / len(vals), "min": min(vals), "max": max(vals), "total": sum(vals), "count": len(vals)}
        return out

    def log_summary(self, reset: bool = True) -> None:
        if not self.enabled:
            return
        summary = self.get_summary()
        if not summary:
            return
        total = sum(v["total"] for v in summary.values()) or 1.0
        lines = [f"Performance profile (step {self.step_count}):"]
        for name, s in sorted(summary.items(), key=lambda kv: -kv[1]["total"]):
            lines.append(
                f"  {name:<28s} avg {s['avg'] * 1e3:9.3f} ms  min {s['min'] * 1e3:9.3f}  max {s['max'] * 1e3:9.3f}  {100 * s['total'] / total:5.1f}%"
            )
        logger.info("\n".join(lines))
        if reset:
            self.timings.clear()


class CUDAMemoryProfiler:
    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self.snapshots: List[Dict[str, Any]] = []

    def snapshot(self, name: str) -> None:
        if not self.enabled:
            return
        snap = {
            "name": name,
            "allocated_gb": torch.cuda.memory_allocated() / 1e9,
            "reserved_gb": torch.cuda.memory_reserved() / 1e9,
            "peak_allocated_gb": torch.cuda.max_memory_allocated() / 1e9,
        }
        self.snapshots.append(snap)
        logger.debug("memory[%s]: %.2f GB allocated, %.2f GB reserved", name, snap["allocated_gb"], snap["reserved_gb"])

    def log_summary(self) -> None:
        if self.enabled and self.snapshots:
            peak = max(s["peak_allocated_gb"] for s in self.snapshots)
            logger.info("CUDA memory: peak allocated %.2f GB over %d snapshots", peak, len(self.snapshots))


class DistributedProfiler:
    """Wall-clock timing of collectives bracketed by device syncs (opt-in, for debugging only)."""

    def __init__(self, enabled: bool = True, rank: int = 0):
        self.enabled = enabled
        self.rank = rank
        self.timings: Dict[str, List[float]] = defaultdict(list)

    @contextmanager
    def profile_op(self, name: str):
        if not self.enabled:
            yield
            return
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self.timings[name].append(time.perf_counter() - t0)

    def log_summary(self) -> None:
        if not self.enabled or self.rank != 0:
            return
        for name, vals in self.timings.items():
            logger.info("dist op %s: avg %.3f ms over %d calls", name, 1e3 * sum(vals) / len(vals), len(vals))
