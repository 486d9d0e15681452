"""Structured counters and timers keyed by (domain, name, phase, device, tags); JSON / CSV / table export.

Same record schema as the reference collector (reference: src/v2/utils/PerfStatsCollector.h:37-118,
PerfStatsCollector.cpp:115-189).  Host timers use `perf_counter`; device timers take CUDA event pairs on the
current stream and are resolved lazily at export so that recording never synchronises.
"""
from __future__ import annotations

import atexit
import csv
import io
import json
import threading
import time
from contextlib import contextmanager
from dataclasses import dataclass, field

from .env import debug_env


@dataclass
class Record:
    domain: str
    name: str
    phase: str = ""
    device: str = ""
    tags: tuple = ()
    count: int = 0
    total_ms: float = 0.0
    min_ms: float = float("inf")
    max_ms: float = 0.0
    value: float = 0.0          # counters / gauges

    def add_time(self, ms: float) -> None:
        self.count += 1
        self.total_ms += ms
        self.min_ms = min(self.min_ms, ms)
        self.max_ms = max(self.max_ms, ms)

    def row(self) -> dict:
        return {"domain": self.domain, "name": self.name, "phase": self.phase, "device": self.device,
                "tags": ",".join(self.tags), "count": self.count, "total_ms": round(self.total_ms, 4),
                "mean_ms": round(self.total_ms / self.count, 4) if self.count else 0.0,
                "min_ms": 0.0 if self.min_ms == float("inf") else round(self.min_ms, 4), "max_ms": round(self.max_ms, 4), "value": self.value}


class PerfStats:
    def __init__(self, enabled: bool | None = None):
        self.enabled = debug_env().profiling if enabled is None else enabled
        self._rec: dict[tuple, Record] = {}
        self._pending: list[tuple[Record, object, object]] = []      # unresolved CUDA event pairs
        self._lock = threading.Lock()
        self._phase = threading.local()

    # -- phases (thread-local, inherited explicitly by worker threads) ---------------------------------------
    def set_phase(self, phase: str) -> None:
        self._phase.value = phase

    def phase(self) -> str:
        return getattr(self._phase, "value", "")

    def _get(self, domain, name, device, tags) -> Record:
        key = (domain, name, self.phase(), device, tuple(tags))
        with self._lock:
            r = self._rec.get(key)
            if r is None:
                r = self._rec[key] = Record(domain, name, self.phase(), device, tuple(tags))
            return r

    # -- recording ------------------------------------------------------------------------------------------
    def count(self, domain: str, name: str, value: float = 1.0, device: str = "", tags=()) -> None:
        if self.enabled:
            r = self._get(domain, name, device, tags)
            r.value += value
            r.count += 1

    def gauge(self, domain: str, name: str, value: float, device: str = "", tags=()) -> None:
        if self.enabled:
            self._get(domain, name, device, tags).value = value

    @contextmanager
    def timer(self, domain: str, name: str, device: str = "", tags=()):
        if not self.enabled:
            yield
            return
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self._get(domain, name, device, tags).add_time((time.perf_counter() - t0) * 1e3)

    @contextmanager
    def cuda_timer(self, domain: str, name: str, device="cuda", tags=()):
        """Device time between entry and exit on the current stream (skipped while a CUDA graph is being captured)."""
        import torch
        if not self.enabled or not torch.cuda.is_available() or torch.cuda.is_current_stream_capturing():
            yield
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            with self._lock:
                self._pending.append((self._get(domain, name, str(device), tags), a, b))

    def resolve(self) -> None:
        with self._lock:
            pend, self._pending = self._pending, []
        for rec, a, b in pend:
            b.synchronize()
            rec.add_time(a.elapsed_time(b))

    # -- export -----------------------------------------------------------------------------------------------
    def rows(self, flt: str = "") -> list[dict]:
        self.resolve()
        rows = [r.row() for r in self._rec.values()]
        if flt:
            rows = [r for r in rows if flt in r["domain"] or flt in r["name"]]
        return sorted(rows, key=lambda r: (r["domain"], r["name"], r["phase"], r["device"]))

    def to_json(self, flt: str = "") -> str:
        return json.dumps(self.rows(flt), indent=1)

    def to_csv(self, flt: str = "") -> str:
        rows = self.rows(flt)
        buf = io.StringIO()
        if rows:
            w = csv.DictWriter(buf, fieldnames=list(rows[0]))
            w.writeheader()
            w.writerows(rows)
        return buf.getvalue()

    def table(self, flt: str = "") -> str:
        rows = self.rows(flt)
        head = f"{'domain':14s} {'name':28s} {'phase':10s} {'device':8s} {'count':>8s} {'total ms':>12s} {'mean ms':>10s} {'max ms':>10s} {'value':>12s}"
        lines = [head, "-" * len(head)]
        for r in rows:
            lines.append(f"{r['domain']:14s} {r['name']:28s} {r['phase']:10s} {r['device']:8s} {r['count']:8d} {r['total_ms']:12.3f} "
                         f"{r['mean_ms']:10.4f} {r['max_ms']:10.3f} {r['value']:12.1f}")
        return "\n".join(lines)

    def reset(self) -> None:
        with self._lock:
            self._rec.clear()
            self._pending.clear()

    def export_from_env(self) -> None:
        env = debug_env()
        flt = env.perf_stats_filter
        if env.perf_stats_json:
            with open(env.perf_stats_json, "w") as f:
                f.write(self.to_json(flt))
        if env.perf_stats_csv:
            with open(env.perf_stats_csv, "w") as f:
                f.write(self.to_csv(flt))
        if env.perf_stats_table:
            print(self.table(flt))


_global = PerfStats()
atexit.register(lambda: _global.export_from_env() if _global.enabled else None)


def perf_stats() -> PerfStats:
    return _global
