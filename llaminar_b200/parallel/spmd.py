"""Command replication for multi-process serving: rank 0 owns the HTTP front end and the scheduler decisions,
every other rank mirrors the engine calls so that all ranks issue identical kernels and collectives.

The reference does the same with an `MPI_Bcast` of a command tag + payload and a worker loop on the non-root
ranks (reference: src/v2/execution/runner/OrchestrationRunner.cpp:13352-13485, src/v2/app/modes/ServerMode.cpp:89-101).
Here the control channel is a gloo broadcast of a small Python object; the data plane stays on NCCL / NVLink.
"""
from __future__ import annotations

import torch.distributed as dist

ADD, STEP, ABORT, FORCE, CLEAR, SHUTDOWN = "add", "step", "abort", "force", "clear", "shutdown"


class ControlChannel:
    def __init__(self, world_group=None, timeout_s: float = 1800.0):
        import datetime
        # a CPU (gloo) group over the same ranks carries the commands
        self.group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
        self.rank = dist.get_rank()

    def bcast(self, obj=None):
        box = [obj]
        dist.broadcast_object_list(box, src=0, group=self.group)
        return box[0]


class ReplicatedEngine:
    """Rank-0 proxy: forwards each call to the local engine after broadcasting it to the workers."""

    def __init__(self, engine, channel: ControlChannel):
        self._e, self._ch = engine, channel
        self._n = 0                                   # commands sent so far; the workers count the same way

    def _run(self, fn):
        """Run one replicated command locally; its outcome goes on record for the cross-rank comparison of step errors
        (`parallel.watchdog.Heartbeat.post_step_error`)."""
        n, self._n = self._n, self._n + 1
        hb = getattr(self._e, "heartbeat", None)
        try:
            out = fn()
        except Exception as exc:
            if hb is not None:
                hb.post_step_error(n, f"{type(exc).__name__}: {exc}")
            raise
        if hb is not None:
            hb.note_step_ok(n)
        return out

    def __getattr__(self, name):
        return getattr(self._e, name)

    def add_request(self, prompt, params):
        self._ch.bcast((ADD, list(prompt), params))
        return self._run(lambda: self._e.add_request(prompt, params))

    def step(self):
        self._ch.bcast((STEP,))
        wd = getattr(self._e, "step_watchdog", None)
        if wd is None:
            return self._run(self._e.step)
        with wd("engine step"):
            return self._run(self._e.step)

    def abort(self, rid):
        self._ch.bcast((ABORT, rid))
        return self._run(lambda: self._e.abort(rid))

    def force_token(self, rid, token):
        self._ch.bcast((FORCE, rid, token))
        return self._run(lambda: self._e.force_token(rid, token))

    def clear_cache(self):
        self._ch.bcast((CLEAR,))
        return self._run(self._e.clear_cache)

    def shutdown_workers(self):
        self._ch.bcast((SHUTDOWN,))


def worker_loop(engine, channel: ControlChannel) -> None:
    """Non-root ranks: replay the commands of rank 0 until told to stop.  A command that raises here is put on record
    through the heartbeat: if rank 0 raised for the same command the ranks are still in step (rank 0 fails the affected
    requests), otherwise the monitors report this rank as failed and the process group is torn down."""
    n = -1
    hb = getattr(engine, "heartbeat", None)
    while True:
        cmd = channel.bcast()
        op = cmd[0]
        if op == SHUTDOWN:
            return
        n += 1
        try:
            if op == ADD:
                engine.add_request(cmd[1], cmd[2])
            elif op == STEP:
                wd = getattr(engine, "step_watchdog", None)
                if wd is None:
                    engine.step()
                else:
                    with wd("engine step"):
                        engine.step()
                for rid in [r for r, q in engine.requests.items() if q.state == "finished"]:
                    engine.requests.pop(rid, None)
            elif op == ABORT:
                engine.abort(cmd[1])
                engine.requests.pop(cmd[1], None)
            elif op == FORCE:
                engine.force_token(cmd[1], cmd[2])
            elif op == CLEAR:
                engine.clear_cache()
            if hb is not None:
                hb.note_step_ok(n)
        except Exception as exc:
            import traceback
            traceback.print_exc()
            if hb is not None:
                hb.post_step_error(n, f"{type(exc).__name__}: {exc}")
