"""Background thread that owns the engine: requests come in through a queue, tokens go out through per-request
queues.  Several HTTP handlers can be in flight at once (up to `--batch-size` lanes decode together); the
reference serialises requests behind one inference mutex (reference: src/v2/app/modes/ServerMode.cpp:126-160).
A failure inside a step fails the requests that were running, is reported to their handlers, and leaves the
loop alive for the next request.
"""
from __future__ import annotations

import queue
import threading
import traceback
from dataclasses import dataclass, field


@dataclass
class Ticket:
    prompt: list[int]
    params: object
    events: "queue.Queue" = field(default_factory=queue.Queue)     # ("tokens", [ids], logprobs | None) / ("done", reason) / ("error", msg, status)
    rid: int | None = None
    cancelled: bool = False
    prefix_hit_tokens: int = 0


class EngineLoop:
    def __init__(self, engine, on_step=None):
        self.engine = engine
        self._in: "queue.Queue" = queue.Queue()
        self._tickets: dict[int, Ticket] = {}
        self._stop = threading.Event()
        self._wake = threading.Event()
        self.on_step = on_step
        self.errors = 0
        # counters for /metrics (written by the engine thread only)
        self.counters = {"requests_submitted": 0, "requests_finished": 0, "requests_cancelled": 0, "requests_rejected": 0,
                         "prompt_tokens": 0, "generated_tokens": 0, "prefix_hit_tokens": 0, "engine_steps": 0,
                         # Prometheus summary pairs: mean = sum / count
                         "ttft_seconds_sum": 0.0, "ttft_seconds_count": 0, "request_seconds_sum": 0.0, "request_seconds_count": 0}
        self._thread = threading.Thread(target=self._run, name="engine-loop", daemon=True)
        self._thread.start()

    # -- called from handler threads -----------------------------------------------------------------
    def submit(self, prompt: list[int], params) -> Ticket:
        t = Ticket(list(prompt), params)
        self._in.put(("add", t))
        self._wake.set()
        return t

    def force_token(self, ticket: Ticket, token: int) -> None:
        self._in.put(("force", ticket, token))
        self._wake.set()

    def cancel(self, ticket: Ticket) -> None:
        ticket.cancelled = True
        self._in.put(("cancel", ticket))
        self._wake.set()

    def metrics(self) -> dict:
        """Counters plus the current queue state (read from handler threads; plain ints, no locking needed)."""
        m = dict(self.counters)
        m["engine_errors"] = self.errors
        m["requests_running"] = len(self._tickets)
        m["requests_waiting"] = len(getattr(self.engine, "waiting", ()))
        m["preemptions"] = int(getattr(self.engine, "stats", {}).get("preemptions", 0))
        alloc = getattr(getattr(self.engine, "kv", None), "allocator", None)
        if alloc is not None:
            m["kv_pages_free"] = int(alloc.n_free)
        return m

    def shutdown(self) -> None:
        self._stop.set()
        self._wake.set()
        self._thread.join(timeout=10)

    # -- engine thread ---------------------------------------------------------------------------------
    def _drain_commands(self) -> None:
        while True:
            try:
                cmd = self._in.get_nowait()
            except queue.Empty:
                return
            kind, t = cmd[0], cmd[1]
            if kind == "add":
                try:
                    r = self.engine.add_request(t.prompt, t.params)
                    t.rid = r.rid
                    self._tickets[r.rid] = t
                    self.counters["requests_submitted"] += 1
                    self.counters["prompt_tokens"] += len(t.prompt)
                except Exception as exc:                       # e.g. prompt longer than the context window
                    self.counters["requests_rejected"] += 1
                    t.events.put(("error", str(exc), 400))
            elif kind == "force" and t.rid is not None:
                self.engine.force_token(t.rid, cmd[2])
            elif kind == "cancel" and t.rid is not None:
                self.engine.abort(t.rid)
                if self._tickets.pop(t.rid, None) is not None:
                    self.counters["requests_cancelled"] += 1
                self.engine.requests.pop(t.rid, None)

    def _run(self) -> None:
        eng = self.engine
        while not self._stop.is_set():
            self._drain_commands()
            if not eng.has_unfinished():
                self._wake.wait(timeout=0.05)
                self._wake.clear()
                continue
            try:
                outs = eng.step()
                self.counters["engine_steps"] += 1
            except Exception as exc:                           # fail the running requests, keep serving
                self.errors += 1
                msg = f"{type(exc).__name__}: {exc}"
                traceback.print_exc()
                for rid, t in list(self._tickets.items()):
                    t.events.put(("error", msg, 500))
                    try:
                        eng.abort(rid)
                    except Exception:
                        pass
                    eng.requests.pop(rid, None)
                self._tickets.clear()
                eng.waiting.clear()
                continue
            for o in outs:
                t = self._tickets.get(o.rid)
                if t is None:
                    continue
                req = eng.requests.get(o.rid)
                if req is not None:
                    t.prefix_hit_tokens = req.prefix_hit_tokens
                if o.new_tokens:
                    self.counters["generated_tokens"] += len(o.new_tokens)
                    t.events.put(("tokens", list(o.new_tokens), getattr(o, "logprobs", None)))
                if o.finished:
                    self.counters["requests_finished"] += 1
                    if req is not None and req.t_first_token is not None:
                        import time
                        self.counters["ttft_seconds_sum"] += req.t_first_token - req.t_arrival
                        self.counters["ttft_seconds_count"] += 1
                        self.counters["request_seconds_sum"] += time.perf_counter() - req.t_arrival
                        self.counters["request_seconds_count"] += 1
                    self.counters["prefix_hit_tokens"] += int(t.prefix_hit_tokens or 0)
                    t.events.put(("done", o.finish_reason))
                    self._tickets.pop(o.rid, None)
                    eng.requests.pop(o.rid, None)
            if self.on_step is not None:
                self.on_step(outs)
