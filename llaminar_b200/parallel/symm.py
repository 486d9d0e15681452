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
CANARY_BYTE = 0xA5


def tp_fuse_blob(*, inbox, flags, epoch_ptr: int, status_ptr: int, rank: int, size: int, rows_cap: int, n_cap: int,
                 spin_limit: int, two_phase_min_rows: int = 0, rs=None, ag=None, flags2=None, epoch2_ptr: int = 0) -> bytes:
    """The bytes of a `TpFuse` descriptor (ops/csrc/tp_fuse.cuh) from explicit device addresses, one list entry per rank.
    `SymmetricArena` fills it with the peers' symmetric-memory addresses; a single-GPU test can fill it with local
    buffers standing in for a peer that never answers."""
    def pad(xs):
        xs = list(xs or [])
        return xs + [0] * (TP_MAX_RANKS - len(xs))
    # the kernels read epoch, epoch2 and status on every call, and inbox / flags of every rank below `size`
    if not (epoch_ptr and epoch2_ptr and status_ptr) or len(inbox) < size or len(flags) < size or not all(inbox[:size]) or not all(flags[:size]):
        raise ValueError("TpFuse descriptor with a null pointer the kernels dereference (epoch, epoch2, status, inbox, flags)")
    if two_phase_min_rows > 0 and not (rs and ag and flags2 and all(rs[:size]) and all(ag[:size]) and all(flags2[:size])):
        raise ValueError("two-phase TpFuse descriptor without its reduce-scatter / all-gather buffers")
    # struct TpFuse { float* inbox[8]; unsigned* flags[8]; unsigned* epoch; int* status; int rank, size, rows_cap, n_cap;
    #                 unsigned spin_limit; int two_phase_min_rows; float* rs_inbox[8]; float* ag_inbox[8]; unsigned* flags2[8];
    #                 unsigned* epoch2; }
    return struct.pack("<8Q8QQQiiiiIi8Q8Q8QQ", *pad(inbox), *pad(flags), epoch_ptr, status_ptr, rank, size, rows_cap, n_cap,
                       spin_limit, two_phase_min_rows, *pad(rs), *pad(ag), *pad(flags2), epoch2_ptr)


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
        self.rs_bytes = 2 * rows_cap * n_cap * 4          # [2][size][rows_cap][n_cap / size]
        self.ag_bytes = 2 * rows_cap * n_cap * 4          # [2][rows_cap][n_cap]
        # guard words behind every region that peers write into: a store that runs past its region lands on a canary
        # and `check_canaries` (debug runs: LLAMINAR_VERIFY_COLLECTIVES) names the region instead of a later wrong sum
        self.guard_bytes = 256
        total = 2 * self.flag_bytes + self.inbox_bytes + self.rs_bytes + self.ag_bytes + 4 * self.guard_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm_mem.rendezvous(self.buf, group.group_name)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.epoch = torch.zeros(2 * n_tiles, dtype=torch.int32, device=self.device)      # one-shot counters, then two-phase counters
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        g = self.guard_bytes
        o_inbox = 2 * self.flag_bytes + g
        o_rs, o_ag = o_inbox + self.inbox_bytes + g, o_inbox + self.inbox_bytes + g + self.rs_bytes + g
        self._guards = {"flags": 2 * self.flag_bytes, "inbox": o_inbox + self.inbox_bytes, "rs_inbox": o_rs + self.rs_bytes,
                        "ag_inbox": o_ag + self.ag_bytes}
        for off in self._guards.values():
            self.buf[off:off + g].fill_(CANARY_BYTE)
        torch.cuda.synchronize(self.device)
        two_phase_min_rows = 16 if (self.size >= 4 and 128 % self.size == 0) else 0
        blob = tp_fuse_blob(inbox=[p + o_inbox for p in ptrs], flags=ptrs, epoch_ptr=self.epoch.data_ptr(),
                            status_ptr=self.status.data_ptr(), rank=self.rank, size=self.size, rows_cap=rows_cap, n_cap=n_cap,
                            spin_limit=spin_limit, two_phase_min_rows=two_phase_min_rows, rs=[p + o_rs for p in ptrs],
                            ag=[p + o_ag for p in ptrs], flags2=[p + self.flag_bytes for p in ptrs],
                            epoch2_ptr=self.epoch.data_ptr() + n_tiles * 4)
        self.desc = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(self.device)
        dist.barrier(group=group)

    @staticmethod
    def create(group, device, n_cap: int = 8192) -> "SymmetricArena":
        return SymmetricArena(group, device, n_cap)

    def supports(self, lin, rows: int) -> bool:
        from ..ops.layout import PackedWeight
        if rows > min(self.rows_cap, 32) or len(lin.parts) != 1:      # GEMV up to 4 rows, small-batch GEMM up to 32
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

    def check_canaries(self) -> None:
        """Raise if a peer (or this rank) wrote past one of the arena's regions (debug aid; one small device read per region)."""
        for name, off in self._guards.items():
            if not bool((self.buf[off:off + self.guard_bytes] == CANARY_BYTE).all()):
                raise RuntimeError(f"symmetric arena: the guard words behind '{name}' were overwritten on rank {self.rank}")

    def resync(self) -> None:
        """Collective: bring the arrival counters and call counters of every rank back to zero.  After a wait that ran out
        (or a call that one rank skipped) the ranks' epochs disagree and every later fused call would wait for arrivals
        that were counted already or never come; all ranks call this between steps, with no fused kernel in flight."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.buf[:2 * self.flag_bytes].zero_()
        self.epoch.zero_()
        self.status.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)


class AllGatherArena:
    """Buffers of the fused all-gather -> GEMM (`ops.gemm_allgather`).

    Symmetric (peer-visible) per rank: eight arrival counters and two parities of the rows this rank owns,
    ``[rows_cap, k_cap]`` bf16; the producer of the activations writes there (`own_rows`).  Local, ordinary device memory:
    the staging buffer ``x[m, k]`` that the kernel's copier CTAs fill from all owners and that the GEMM's tensor map
    reads (TMA reads of symmetric-memory mappings measured ~10 % slower, so the operand is staged in ordinary memory).
    A call uses parity ``epoch & 1``; a rank can run at most one call ahead of its peers (it needs their rows to finish
    a call), so two parities suffice.  The epoch is a host counter passed as a kernel argument, so these launches are
    not meant for CUDA-graph capture (prefill runs eagerly).  The reference has no counterpart: its column-parallel
    projections read a replicated input (reference: src/v2/compute_stages/stages/FusedQKVGEMMStage.cpp).
    """

    def __init__(self, group, device, rows_cap: int, k_cap: int, copy_ctas: int = 16, spin_limit: int | None = None):
        import torch.distributed._symmetric_memory as symm_mem
        from ..utils.env import debug_env
        self.group, self.device = group, torch.device(device)
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        self.rows_cap, self.k_cap, self.copy_ctas = rows_cap, k_cap, copy_ctas
        self.spin_limit = debug_env().tp_spin_limit if spin_limit is None else spin_limit
        self.row_bytes = rows_cap * k_cap * 2
        self.flag_bytes = 256
        self.buf = symm_mem.empty(self.flag_bytes + 2 * self.row_bytes, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm_mem.rendezvous(self.buf, group.group_name)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.stage = torch.zeros(self.size * rows_cap * k_cap, dtype=torch.bfloat16, device=self.device)
        self.staged = torch.zeros(4096, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.epoch = 0
        dist.barrier(group=group)

    def own_rows(self, rows: int, k: int) -> torch.Tensor:
        """View of this rank's row buffer for the NEXT call; the producer writes its [rows, k] bf16 activations here."""
        assert rows <= self.rows_cap and k <= self.k_cap
        off = self.flag_bytes + (self.epoch & 1) * self.row_bytes
        return self.buf[off:off + rows * k * 2].view(torch.bfloat16).view(rows, k)

    def gathered(self, m_total: int, k: int) -> torch.Tensor:
        """The staging buffer as [m_total, k] (all rows are present once a call has run)."""
        return self.stage[:m_total * k].view(m_total, k)

    def gemm(self, pw, m_total: int, rows_per_rank: int, out: torch.Tensor, *, epi: int = 0, bias=None) -> None:
        """out[m_total, n] = x[m_total, k] @ W^T where rank r owns (and has written) rows [r * rows_per_rank, ...) of x."""
        from .. import ops
        assert pw.k <= self.k_cap and m_total <= self.size * rows_per_rank and rows_per_rank <= self.rows_cap
        par = self.epoch & 1
        src = [p + self.flag_bytes + par * self.row_bytes for p in self.ptrs] + [0] * (TP_MAX_RANKS - self.size)
        avail = list(self.ptrs) + [0] * (TP_MAX_RANKS - self.size)
        desc = torch.tensor(src + avail + [self.stage.data_ptr(), self.staged.data_ptr(), self.size, self.rank, rows_per_rank,
                                          self.copy_ctas, self.epoch, self.spin_limit], dtype=torch.int64)
        ops.gemm_allgather(pw, m_total, out, desc, epi=epi, bias=bias, status=self.status)
        self.epoch += 1

    def check_status(self) -> None:
        if int(self.status[0]) != 0:
            self.status.zero_()
            raise RuntimeError("the fused all-gather GEMM gave up waiting for a peer's rows")


class SeqShardArena:
    """Buffers of the sequence-sharded tensor-parallel prefill path: fused GEMM -> reduce-scatter and all-gather -> GEMM.

    Between the row-parallel projections (attention output, FFN down) and the next column-parallel ones (QKV, gate|up) the
    residual stream is sharded by rows: rank o owns rows ``[o * Tw, (o + 1) * Tw)`` of a chunk of T rows, ``Tw`` a multiple
    of 64.  The row-parallel GEMM pushes bf16 partial tiles into the owners' inboxes from its epilogue
    (`ops.gemm_reduce_scatter`), the owner sums them into its fp32 residual rows and writes the next RMSNorm as bf16 into
    the all-gather arena (`ops.rs_reduce_norm`), and the column-parallel GEMM pulls all rows from their owners while it
    already multiplies (`AllGatherArena.gemm`).  Per layer that is two reduce-scatters and two all-gathers of bf16 rows that
    overlap the GEMMs tile by tile, instead of two fp32 all-reduces between kernels.

    Symmetric memory per rank: two parities of arrival counters and of ``[world][rows_cap][d]`` bf16 inbox rows.  A call uses
    parity ``calls & 1``; the owner clears the counters of a parity after it has consumed them.  A rank reaches call c + 2
    only after every peer has finished call c + 1's reduce, which is stream-ordered after that peer's reduce of call c, so
    two parities suffice.  The reference has no counterpart (its residual stream is replicated and all-reduced:
    src/v2/models/qwen/QwenGraphBase.cpp:2937-3014).
    """

    FLAGS_PER_PARITY = 64

    def __init__(self, group, device, rows_cap: int, d: int, spin_limit: int | None = None):
        import torch.distributed._symmetric_memory as symm_mem
        from ..utils.env import debug_env
        self.group, self.device = group, torch.device(device)
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        if self.size > TP_MAX_RANKS:
            raise ValueError(f"fused tensor parallelism supports at most {TP_MAX_RANKS} ranks")
        self.rows_cap = (rows_cap + 63) // 64 * 64
        self.d = d
        self.spin_limit = debug_env().tp_spin_limit if spin_limit is None else spin_limit
        self.flag_bytes = 2 * self.FLAGS_PER_PARITY * 4
        self.inbox_bytes = 2 * self.size * self.rows_cap * d * 2
        self.buf = symm_mem.empty(self.flag_bytes + self.inbox_bytes, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm_mem.rendezvous(self.buf, group.group_name)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.flags_view = self.buf[:self.flag_bytes].view(torch.int32).view(2, self.FLAGS_PER_PARITY)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.ag = AllGatherArena(group, device, self.rows_cap, d, spin_limit=self.spin_limit)
        self.calls = 0
        dist.barrier(group=group)

    def rows_per_rank(self, T: int) -> int:
        """Rows every rank owns of a chunk of T rows (a multiple of 64; the last owners may hold fewer or none)."""
        tw = ((T + self.size - 1) // self.size + 63) // 64 * 64
        if tw > self.rows_cap:
            raise ValueError(f"a chunk of {T} rows needs {tw} rows per rank, the arena holds {self.rows_cap}")
        return tw

    def my_rows(self, T: int, tw: int) -> tuple[int, int]:
        """(first global row, number of rows) this rank owns."""
        r0 = self.rank * tw
        return r0, max(0, min(T - r0, tw))

    def gemm_reduce_scatter(self, pw, x: torch.Tensor, tw: int) -> None:
        """Partial x @ W_shard^T of all T rows, pushed to the owners of the rows from the GEMM's epilogue."""
        from .. import ops
        par = self.calls & 1
        inbox = [p + self.flag_bytes for p in self.ptrs] + [0] * (TP_MAX_RANKS - self.size)
        flags = list(self.ptrs) + [0] * (TP_MAX_RANKS - self.size)
        desc = torch.tensor(inbox + flags + [self.size, self.rank, tw, self.d, par, self.FLAGS_PER_PARITY], dtype=torch.int64)
        ops.gemm_reduce_scatter(pw, x, desc, status=self.status)

    def reduce_norm(self, h_local: torch.Tensor, T: int, tw: int, n_out: int, norm_w, xn_out, eps: float) -> None:
        """h_local[row] += the ranks' partial rows of this call (rank order); xn_out[row] = RMSNorm(h_local[row]) * norm_w."""
        from .. import ops
        par = self.calls & 1
        rows = h_local.shape[0]
        if rows:
            bm = int(ops.ext().gemm_tc_rs_block_m(T, tw))
            n_tiles = (n_out + 127) // 128
            inbox_ptr = self.ptrs[self.rank] + self.flag_bytes + par * self.size * tw * self.d * 2
            flags_ptr = self.ptrs[self.rank] + par * self.FLAGS_PER_PARITY * 4
            ops.rs_reduce_norm(inbox_ptr, flags_ptr, n_tiles * self.size, self.size, tw, self.d, bm, h_local, norm_w, xn_out, eps,
                               self.spin_limit, self.status)
        self.flags_view[par].zero_()          # stream-ordered after the reduce; the next writers of this parity come a call later
        self.calls += 1

    def check_status(self) -> None:
        if int(self.status[0]) != 0:
            self.status.zero_()
            raise RuntimeError("a fused reduce-scatter gave up waiting for a peer's partial rows")
        self.ag.check_status()
