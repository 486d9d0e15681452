"""Tensor-parallel context: one process per GPU, `torch.distributed` for the plumbing.

Two implementations of the row-parallel "GEMM + all-reduce + residual add" step exist side by side:

* the baseline issues the partial GEMM/GEMV, an NCCL (or gloo, on CPU) all-reduce and an add, which is what
  the reference does per layer (reference: src/v2/compute_stages/stages/TPAllreduceStage.cpp ->
  src/v2/collective/LocalTPContext.cpp:726 -> ncclAllReduce; two [tokens x d_model] all-reduces per layer,
  src/v2/models/qwen/QwenGraphBase.cpp:2992-3010, :2119-2139);
* the fused path (GPU, `fused=True`) lets the GEMV/GEMM epilogue push its partial tile straight into every
  peer's inbox over NVLink (peer stores on symmetric memory), signal a per-tile flag, wait (bounded) for the
  other ranks' tiles and add the sum to the residual stream, all inside the one kernel.

Logits are vocab-parallel; `all_gather_vocab` assembles full rows for sampling.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..utils.env import debug_env


@dataclass
class TPContext:
    group: object
    rank: int
    size: int
    device: torch.device
    fused: bool = False
    symm: object = None                 # parallel.symm.SymmetricArena when fused kernels are available
    stats: dict = field(default_factory=lambda: {"allreduce_calls": 0, "allreduce_bytes": 0, "fused_calls": 0})
    order_check: object = None          # parallel.collective_check.CollectiveOrderChecker in debug mode
    moe_mode: str = "expert-parallel"   # --moe-expert-mode: expert-parallel | replicated
    skip_allreduce: bool = False        # debug switch LLAMINAR_SKIP_ALLREDUCE (isolates compute time; results are wrong)
    verify_checksums: bool = False      # debug switch LLAMINAR_VERIFY_COLLECTIVES: every rank must hold the same reduced values
    allreduce_precision: str = "auto"   # LLAMINAR_ALLREDUCE_PRECISION: fp32 | bf16 | fp16 | auto (reference: LocalTPContext.cpp:835-989)

    @staticmethod
    def create(group=None, device=None, fused: bool | None = None) -> "TPContext":
        group = group if group is not None else dist.group.WORLD
        rank, size = dist.get_rank(group), dist.get_world_size(group)
        device = torch.device(device if device is not None else "cpu")
        ctx = TPContext(group, rank, size, device)
        ctx.skip_allreduce = debug_env().skip_allreduce
        ctx.verify_checksums = debug_env().verify_collectives
        ctx.allreduce_precision = str(debug_env().allreduce_precision).lower()
        if ctx.allreduce_precision not in ("auto", "fp32", "bf16", "fp16"):
            raise ValueError(f"LLAMINAR_ALLREDUCE_PRECISION={ctx.allreduce_precision!r}: expected fp32, bf16, fp16 or auto")
        if debug_env().collective_order_check:
            from .collective_check import CollectiveOrderChecker
            ctx.order_check = CollectiveOrderChecker(None)
        want_fused = fused if fused is not None else (device.type == "cuda" and size > 1
                                                      and debug_env().tp_fused)
        if want_fused and device.type == "cuda" and size > 1:
            from .symm import SymmetricArena
            try:
                ctx.symm = SymmetricArena.create(group, device)
                ctx.fused = True
            except Exception as exc:        # no peer access / symmetric memory unavailable: keep the NCCL path
                if fused:
                    raise
                ctx.fused = False
                ctx.stats["fused_unavailable"] = str(exc)
        return ctx

    # -- collectives (baseline) -------------------------------------------------------------------
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        if self.order_check is not None:
            self.order_check.record("all_reduce", x)
        if self.skip_allreduce:
            return x
        dist.all_reduce(x, group=self.group)
        self.stats["allreduce_calls"] += 1
        self.stats["allreduce_bytes"] += x.numel() * x.element_size()
        if self.verify_checksums:
            self.verify_replicated(x, "all_reduce")
        return x

    def verify_replicated(self, x: torch.Tensor, what: str) -> None:
        """Debug check that ``x`` is bit-identical on every rank of the group (an all-reduce result, or the residual
        stream after a fused reduce epilogue): the ranks exchange a 64-bit checksum of the bytes plus NaN / Inf counts and
        raise on a mismatch.  Counterpart of the reference's LLAMINAR_MPI_VERIFY_CHECKSUMS (src/v2/utils/DebugEnv.h)."""
        flat = x.detach().contiguous().view(-1).view(torch.uint8).to(torch.int64)
        weights = torch.arange(1, flat.numel() + 1, dtype=torch.int64, device=flat.device) % 65521
        mine = torch.stack([(flat * weights).sum(), flat.sum(),
                            torch.isnan(x).sum().to(torch.int64) if x.is_floating_point() else flat.new_zeros(()),
                            torch.isinf(x).sum().to(torch.int64) if x.is_floating_point() else flat.new_zeros(())])
        everyone = torch.empty(self.size * 4, dtype=torch.int64, device=mine.device)
        dist.all_gather_into_tensor(everyone, mine, group=self.group)
        everyone = everyone.view(self.size, 4).cpu()
        self.stats["verified_collectives"] = self.stats.get("verified_collectives", 0) + 1
        bad = [r for r in range(self.size) if not torch.equal(everyone[r, :2], everyone[0, :2])]
        if bad:
            raise RuntimeError(f"{what}: ranks {bad} hold different bytes than rank 0 (checksums {everyone[:, 0].tolist()})")
        if int(everyone[0, 2]) or int(everyone[0, 3]):
            raise RuntimeError(f"{what}: result has {int(everyone[0, 2])} NaN and {int(everyone[0, 3])} Inf values")

    def all_gather_vocab(self, logits: torch.Tensor, vocab: int) -> torch.Tensor:
        """[rows, vocab_local] shards (rank order, last shard may be short) -> [rows, vocab]."""
        if self.size == 1:
            return logits
        if self.order_check is not None:
            self.order_check.record("all_gather_vocab", logits)
        rows = logits.shape[0]
        from .tp_plan import VOCAB_UNIT, _split
        n_units = (vocab + VOCAB_UNIT - 1) // VOCAB_UNIT
        widths = []
        for r in range(self.size):
            u0, u1 = _split(n_units, self.size, r)
            widths.append(min(u1 * VOCAB_UNIT, vocab) - u0 * VOCAB_UNIT)
        wmax = max(widths)
        send = logits
        if logits.shape[1] != wmax:
            send = torch.zeros(rows, wmax, dtype=logits.dtype, device=logits.device)
            send[:, :logits.shape[1]] = logits
        flat = torch.empty(self.size * rows, wmax, dtype=logits.dtype, device=logits.device)
        dist.all_gather_into_tensor(flat, send.contiguous(), group=self.group)
        out = flat.view(self.size, rows, wmax)
        if all(w == wmax for w in widths):
            return out.permute(1, 0, 2).reshape(rows, self.size * wmax)
        return torch.cat([out[r, :, :w] for r, w in enumerate(widths)], dim=1)

    def all_gather_flat(self, out: torch.Tensor, inp: torch.Tensor) -> torch.Tensor:
        """out[rank] = inp for every rank (small fixed-size records, e.g. per-shard argmax candidates)."""
        if self.order_check is not None:
            self.order_check.record("all_gather_flat", inp)
        dist.all_gather_into_tensor(out, inp, group=self.group)
        return out

    def broadcast_object(self, obj, src: int = 0):
        box = [obj]
        dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, src) if self.group is not dist.group.WORLD else src,
                                   group=self.group)
        return box[0]

    def barrier(self) -> None:
        if self.size > 1:
            dist.barrier(group=self.group)

    # -- row-parallel linear + all-reduce + residual ---------------------------------------------------
    def row_parallel_resid(self, lin, x: torch.Tensor, h: torch.Tensor, model) -> None:
        """h += sum over ranks of (x @ W_shard^T)."""
        from .. import ops
        T = x.shape[0]
        small = T <= ops.GEMV_MAX_ROWS
        if self.fused and self.symm is not None and self.symm.supports(lin, T):
            self.symm.fused_row_parallel(lin, x, h, model, small)
            self.stats["fused_calls"] += 1
            return
        part = model.ws_partial[:T]
        lin(x, part, scratch=model.scratch, xn=None if small else x)
        dt = self.payload_dtype(T)
        if dt is torch.float32 or self.device.type != "cuda":
            self.all_reduce(part)
            h += part
        else:
            # reduced-precision payload: half the bytes on the wire for the bandwidth-bound prefill all-reduce; every rank
            # receives the same reduced bits, so the residual streams stay identical
            low = part.to(dt)
            self.all_reduce(low)
            h += low

    def payload_dtype(self, rows: int) -> torch.dtype:
        """Element type of the NCCL all-reduce payload for a call of ``rows`` activation rows (the policy the reference
        sets per layer or through LLAMINAR_ALLREDUCE_PRECISION; reference: src/v2/collective/LocalTPContext.cpp:835-989)."""
        p = self.allreduce_precision
        if p == "auto":
            p = "bf16" if rows > 32 else "fp32"
        return {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[p]
