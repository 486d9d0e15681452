"""Symmetric peer-memory arena for the fused tensor-parallel kernels.

Every rank allocates the same buffer through ``torch.distributed._symmetric_memory`` and learns the device
addresses of all peers' copies (NVLink peer access inside one node).  The buffer holds, per rank,

    flags   [n_tiles_cap] uint32   per-output-tile arrival counters (monotone, never reset)
    inbox   [2 parities][world][rows_cap][n_cap] float32   partial output tiles pushed by the peers

and a small device-resident descriptor (`TpFuse` in ops/csrc/tp_fuse.cuh) lists all peers' addresses so the
GEMV / GEMM epilogues can store to them directly.  The reference has no counterpart: its collectives are
NCCL calls between kernels (reference: src/v2/collective/backends/NCCLBackend.cpp:504).
"""
from __future__ import annotations

import struct

import torch
import torch.distributed as dist

ROWS_CAP = 64
TP_MAX_RANKS = 8


class SymmetricArena:
    def __init__(self, group, device, n_cap: int, rows_cap: int = ROWS_CAP, spin_limit: int | None = None):
        import torch.distributed._symmetric_memory as symm_mem
        from ..utils.env import debug_env
        spin_limit = debug_env().tp_spin_limit if spin_limit is None else spin_limit
        self.group, self.device = group, torch.device(device)
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        if self.size > TP_MAX_RANKS:
            raise ValueError(f"fused tensor parallelism supports at most {TP_MAX_RANKS} ranks")
        self.n_cap, self.rows_cap = n_cap, rows_cap
        n_tiles = n_cap // 128
        self.flag_bytes = (n_tiles * 4 + 255) // 256 * 256
        self.inbox_bytes = 2 * self.size * rows_cap * n_cap * 4
        total = self.flag_bytes + self.inbox_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm_mem.rendezvous(self.buf, group.group_name)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.epoch = torch.zeros(n_tiles, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        # struct TpFuse { float* inbox[8]; unsigned* flags[8]; unsigned* epoch; int* status; int rank, size, rows_cap, n_cap; unsigned spin_limit; }
        inbox = [p + self.flag_bytes for p in ptrs] + [0] * (TP_MAX_RANKS - self.size)
        flags = ptrs + [0] * (TP_MAX_RANKS - self.size)
        blob = struct.pack("<8Q8QQQiiiiI4x", *inbox, *flags, self.epoch.data_ptr(), self.status.data_ptr(),
                           self.rank, self.size, rows_cap, n_cap, spin_limit)
        self.desc = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(self.device)
        dist.barrier(group=group)

    @staticmethod
    def create(group, device, n_cap: int = 8192) -> "SymmetricArena":
        return SymmetricArena(group, device, n_cap)

    def supports(self, lin, rows: int) -> bool:
        from ..ops.layout import PackedWeight
        if rows > self.rows_cap or len(lin.parts) != 1:
            return False
        w = lin.parts[0][0]
        return isinstance(w, PackedWeight) and w.n_tiles * 128 <= self.n_cap

    def fused_row_parallel(self, lin, x: torch.Tensor, h: torch.Tensor, model, small: bool) -> None:
        """h += all-reduce(x @ W_shard^T), one kernel: the epilogue exchanges tiles over peer memory."""
        from .. import ops
        w = lin.parts[0][0]
        if small:
            ops.gemv(w, x, h, epi=ops.EPI_RESID, bias=lin.bias, scratch=model.scratch, tp=self.desc)
        else:
            ops.gemm(w, x, h, epi=ops.EPI_RESID, bias=lin.bias, scratch=model.scratch, tp=self.desc)

    def check_status(self) -> None:
        s = int(self.status[0])
        if s != 0:
            self.status.zero_()
            raise RuntimeError(f"a fused tensor-parallel kernel gave up waiting for a peer (status {s})")
