"""Failure detection between ranks: heartbeats through the rendezvous store, a step watchdog, coordinated abort.

The reference wakes peers that are blocked in a collective by aborting the communicator when one tensor-parallel
worker fails, and bounds how long it waits for workers (reference: src/v2/execution/local_execution/orchestrators/
RankOrchestrator.cpp:1610-1616, :1697-1719; src/v2/collective/LocalTPContext.cpp:529-571;
src/v2/collective/coordinators/NCCLCoordinator.h:92-103).  With one process per GPU the same roles are:

* `Heartbeat`: each rank writes a monotonically increasing beat (and, on failure, an error text) to a key-value
  store (`torch.distributed.TCPStore` / `FileStore` / any object with set/get); a monitor thread reads the peers'
  beats and calls ``on_failure(rank, reason)`` when one is stale or has posted an error.
* `StepWatchdog`: a timer armed around each engine step; if the step does not finish in time (a peer died inside
  a collective), it posts the failure and calls ``abort`` (by default `abort_process_group`).
* `vote_all_ok`: the initialisation vote -- every rank contributes success/failure, all ranks get the minimum, so
  a failure on one rank fails start-up everywhere (reference: OrchestrationRunner.cpp:746-765).

No part of this touches a GPU: faults are detected on the host, and the device-side waits of the fused kernels are
bounded and report through a status word (`parallel.symm.SymmetricArena.check_status`).
"""
from __future__ import annotations

import threading
import time

import torch
import torch.distributed as dist

from ..utils.env import debug_env


class RankFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} failed: {reason}")
        self.rank, self.reason = rank, reason


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float | None = None, timeout_s: float | None = None,
                 on_failure=None, prefix: str = "hb"):
        env = debug_env()
        self.store, self.rank, self.world = store, rank, world
        self.interval = env.heartbeat_s if interval_s is None else interval_s
        self.timeout = env.watchdog_timeout_s if timeout_s is None else timeout_s
        self.on_failure = on_failure
        self.prefix = prefix
        self.failed: dict[int, str] = {}
        self._stop = threading.Event()
        self._beat = 0
        self._seen: dict[int, tuple[int, float]] = {}
        self._thread: threading.Thread | None = None
        self.paused = False                       # test hook: stop beating without stopping the monitor
        self._own_step_errors: dict[int, str] = {}
        self._last_ok_step = -1
        self._peer_step_seen: dict[int, str] = {}

    def _key(self, r: int, what: str) -> str:
        return f"{self.prefix}/{what}/{r}"

    def start(self) -> "Heartbeat":
        self._write_beat()
        self._thread = threading.Thread(target=self._run, name=f"heartbeat-{self.rank}", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.interval * 4 + 1)

    def post_error(self, reason: str) -> None:
        self.store.set(self._key(self.rank, "err"), reason[:2000])

    def post_step_error(self, step: int, reason: str) -> None:
        """Record that replicated command number ``step`` raised on this rank.  Ranks replay the same commands, so an
        error that every rank raises for the same command is harmless (rank 0 fails the affected requests); one that
        only some ranks raise leaves the engines out of step.  The monitor of every rank compares the peers' records
        with its own (`poll_once`) and reports a rank whose record has no local counterpart as failed."""
        self._own_step_errors[step] = reason[:200]
        while len(self._own_step_errors) > 64:
            self._own_step_errors.pop(next(iter(self._own_step_errors)))
        self.store.set(self._key(self.rank, "steperr"), f"{step}|{reason[:500]}")

    def note_step_ok(self, step: int) -> None:
        """The command number ``step`` completed on this rank without an error (kept locally, nothing is sent)."""
        self._last_ok_step = max(self._last_ok_step, step)

    def _write_beat(self) -> None:
        self._beat += 1
        self.store.set(self._key(self.rank, "beat"), str(self._beat))

    def _read(self, key: str) -> str | None:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            v = self.store.get(key)
            return v.decode() if isinstance(v, (bytes, bytearray)) else str(v)
        except Exception:
            return None

    def poll_once(self, now: float | None = None) -> dict[int, str]:
        """One monitor pass; returns newly failed ranks -> reason."""
        now = time.monotonic() if now is None else now
        new: dict[int, str] = {}
        for r in range(self.world):
            if r == self.rank or r in self.failed:
                continue
            err = self._read(self._key(r, "err"))
            if err:
                new[r] = err
                continue
            se = self._read(self._key(r, "steperr"))
            if se and se != self._peer_step_seen.get(r):
                step_s, _, why = se.partition("|")
                step = int(step_s) if step_s.lstrip("-").isdigit() else -1
                if step in self._own_step_errors:
                    self._peer_step_seen[r] = se            # the same command failed here too: the ranks are still in step
                elif step <= self._last_ok_step:
                    self._peer_step_seen[r] = se
                    new[r] = f"command {step} failed on rank {r} only: {why}"
                    continue
                # else: this rank has not run that command yet; look again at the next pass
            b = self._read(self._key(r, "beat"))
            beat = int(b) if b else 0
            last = self._seen.get(r)
            if last is None or beat != last[0]:
                self._seen[r] = (beat, now)
            elif now - last[1] > self.timeout:
                new[r] = f"no heartbeat for {now - last[1]:.1f} s"
        for r, why in new.items():
            self.failed[r] = why
            if self.on_failure is not None:
                self.on_failure(r, why)
        return new

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                if not self.paused:
                    self._write_beat()
                self.poll_once()
            except Exception:
                pass

    def raise_if_failed(self) -> None:
        for r, why in self.failed.items():
            raise RankFailure(r, why)


def abort_process_group(group=None) -> None:
    """Tear down the communicators so that ranks blocked in a collective return with an error."""
    try:
        pg = group if group is not None else dist.group.WORLD
        backend = pg._get_backend(torch.device("cuda")) if torch.cuda.is_available() else None
        if backend is not None and hasattr(backend, "abort"):
            backend.abort()
            return
    except Exception:
        pass
    try:
        dist.destroy_process_group()
    except Exception:
        pass


class StepWatchdog:
    """Arms a timer around a step; on expiry posts the failure and calls ``abort`` once."""

    def __init__(self, timeout_s: float | None = None, abort=abort_process_group, heartbeat: Heartbeat | None = None):
        self.timeout = debug_env().step_timeout_s if timeout_s is None else timeout_s
        self.abort, self.heartbeat = abort, heartbeat
        self.expired = False
        self._timer: threading.Timer | None = None

    def _fire(self, what: str) -> None:
        self.expired = True
        if self.heartbeat is not None:
            self.heartbeat.post_error(f"{what} exceeded {self.timeout:.1f} s")
        self.abort()

    def __call__(self, what: str = "step"):
        return _Armed(self, what)


class _Armed:
    def __init__(self, wd: StepWatchdog, what: str):
        self.wd, self.what = wd, what

    def __enter__(self):
        if self.wd.timeout > 0:
            self.wd._timer = threading.Timer(self.wd.timeout, self.wd._fire, args=(self.what,))
            self.wd._timer.daemon = True
            self.wd._timer.start()
        return self.wd

    def __exit__(self, *exc):
        if self.wd._timer is not None:
            self.wd._timer.cancel()
            self.wd._timer = None
        return False


def vote_all_ok(ok: bool, group=None, device="cpu") -> bool:
    """All ranks learn whether every rank succeeded (MIN all-reduce of a flag)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return ok
    t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    return bool(int(t.item()))
