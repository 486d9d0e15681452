"""Debug aid: verify that every rank of a group issues the same collectives in the same order.

A mismatch in collective order across ranks is the classic source of silent deadlocks.  In check mode every
collective issued through `TPContext` is recorded as (sequence number, op, shape, dtype); every ``interval``
records the ranks exchange a digest of their logs over the control group and raise on the first divergence,
naming the entry (reference: src/v2/collective/CollectiveOrderChecker.h; enabled there by
LLAMINAR_COLLECTIVE_ORDER_CHECK).  The exchange itself uses ``all_gather_object`` on a host (gloo) group so
it cannot interleave with the device collectives it audits.
"""
from __future__ import annotations

import hashlib

import torch.distributed as dist


class CollectiveOrderMismatch(RuntimeError):
    pass


class CollectiveOrderChecker:
    def __init__(self, control_group=None, interval: int = 64, keep: int = 256):
        self.group = control_group
        self.interval, self.keep = interval, keep
        self.log: list[tuple[int, str, tuple, str]] = []
        self.seq = 0
        self.checked = 0

    def record(self, op: str, tensor=None, extra: str = "") -> None:
        shape = tuple(tensor.shape) if tensor is not None else ()
        dtype = str(tensor.dtype) if tensor is not None else extra
        self.log.append((self.seq, op, shape, dtype))
        self.seq += 1
        if len(self.log) > self.keep:
            del self.log[:len(self.log) - self.keep]
        if self.seq % self.interval == 0:
            self.verify()

    def digest(self) -> str:
        h = hashlib.blake2b(digest_size=12)
        for e in self.log:
            h.update(repr(e).encode())
        return h.hexdigest()

    def verify(self) -> None:
        """Collective over the control group: all ranks must call it at the same sequence number."""
        if not dist.is_initialized():
            return
        size = dist.get_world_size(self.group)
        if size == 1:
            return
        mine = (self.seq, self.digest())
        box = [None] * size
        dist.all_gather_object(box, mine, group=self.group)
        self.checked += 1
        if all(b == mine for b in box):
            return
        logs = [None] * size
        dist.all_gather_object(logs, list(self.log), group=self.group)
        rank = dist.get_rank(self.group)
        for r, other in enumerate(logs):
            if other == self.log:
                continue
            for a, b in zip(self.log, other):
                if a != b:
                    raise CollectiveOrderMismatch(f"collective order diverged: rank {rank} issued {a}, rank {r} issued {b}")
            raise CollectiveOrderMismatch(f"collective count diverged: rank {rank} has {self.seq}, rank {r} has {box[r][0]}")
