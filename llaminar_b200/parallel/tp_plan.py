"""Per-rank tensor-parallel slicing plan (pure arithmetic, no devices involved).

Megatron-style split as in the reference: Q/K/V, gate/up and the LM head are column-parallel
(weight rows are split), Wo and down are row-parallel (weight columns are split, outputs are
summed), norms are replicated, experts are range-partitioned (reference:
src/v2/loaders/WeightTypes.h:39-46).  When there are fewer KV heads than ranks the KV heads are
replicated and Q heads are dealt out so that every rank's Q heads share one KV head (reference:
src/v2/config/TensorParallelConfig.cpp:348-395).  The FFN width is split on 256-column
boundaries so that the row-parallel down projection is cut between quantisation super-blocks;
ranks may therefore own slightly different widths.
"""
from __future__ import annotations

from dataclasses import dataclass

FF_UNIT = 256
VOCAB_UNIT = 128


def _split(n_units: int, parts: int, idx: int) -> tuple[int, int]:
    return n_units * idx // parts, n_units * (idx + 1) // parts


@dataclass(frozen=True)
class TPPlan:
    tp: int
    rank: int
    q_head_start: int
    q_head_stop: int
    kv_head_start: int
    kv_head_stop: int
    kv_replicas: int            # how many ranks hold a copy of each of this rank's KV heads
    ff_start: int
    ff_stop: int
    vocab_start: int
    vocab_stop: int
    expert_start: int
    expert_stop: int
    # linear-attention value heads of a hybrid model (key heads stay replicated: value head j reads key head j mod n_k, and
    # the q / k work is a small share of the block; reference: the head mapping comment in
    # src/v2/models/qwen35/Qwen35Graph.cpp:888-900)
    gdn_v_start: int = 0
    gdn_v_stop: int = 0

    @property
    def n_heads_local(self) -> int:
        return self.q_head_stop - self.q_head_start

    @property
    def n_kv_local(self) -> int:
        return self.kv_head_stop - self.kv_head_start

    @staticmethod
    def validate(cfg, tp: int) -> list[str]:
        """Human-readable reasons why ``cfg`` cannot be split ``tp`` ways (empty list: fine)."""
        errs = []
        if tp < 1:
            errs.append("tensor-parallel degree must be >= 1")
            return errs
        if cfg.n_heads % tp:
            errs.append(f"n_heads={cfg.n_heads} is not divisible by tp={tp}")
        if cfg.n_kv_heads >= tp:
            if cfg.n_kv_heads % tp:
                errs.append(f"n_kv_heads={cfg.n_kv_heads} is not divisible by tp={tp}")
        elif tp % cfg.n_kv_heads:
            errs.append(f"tp={tp} is not a multiple of n_kv_heads={cfg.n_kv_heads} (needed to replicate KV heads)")
        if not cfg.is_moe and cfg.d_ff // FF_UNIT < tp:
            errs.append(f"d_ff={cfg.d_ff} has fewer than tp={tp} blocks of {FF_UNIT} columns")
        if cfg.is_moe and cfg.n_experts < tp:
            errs.append(f"n_experts={cfg.n_experts} < tp={tp}")
        if getattr(cfg, "is_hybrid", False) and cfg.ssm_v_heads % tp:
            errs.append(f"ssm value heads={cfg.ssm_v_heads} are not divisible by tp={tp}")
        if (cfg.q_dim // tp) % 32 and tp > 1:
            errs.append(f"per-rank attention width {cfg.q_dim // tp} is not a multiple of 32 (smallest quantisation block)")
        return errs

    @staticmethod
    def build(cfg, tp: int = 1, rank: int = 0, moe_mode: str = "expert-parallel") -> "TPPlan":
        errs = TPPlan.validate(cfg, tp)
        if errs:
            raise ValueError("; ".join(errs))
        qs, qe = _split(cfg.n_heads, tp, rank)
        group = cfg.n_heads // cfg.n_kv_heads
        if cfg.n_kv_heads >= tp:
            ks, ke = _split(cfg.n_kv_heads, tp, rank)
            rep = 1
        else:
            ks = qs // group
            ke = ks + 1
            rep = tp // cfg.n_kv_heads
            assert (qe - 1) // group == ks, "a rank's Q heads must share one KV head"
        if cfg.is_moe:
            fs, fe = 0, 0
        else:
            u0, u1 = _split(cfg.d_ff // FF_UNIT, tp, rank)
            fs, fe = u0 * FF_UNIT, u1 * FF_UNIT
            if rank == tp - 1:
                fe = cfg.d_ff
        n_vu = (cfg.vocab_size + VOCAB_UNIT - 1) // VOCAB_UNIT
        v0, v1 = _split(n_vu, tp, rank)
        vs, ve = v0 * VOCAB_UNIT, min(v1 * VOCAB_UNIT, cfg.vocab_size)
        if moe_mode == "tensor-parallel":
            raise ValueError("--moe-expert-mode tensor-parallel (every expert split across ranks) is not built; "
                             "use expert-parallel or replicated")
        if cfg.is_moe and moe_mode == "replicated":
            es, ee = 0, cfg.n_experts           # every rank holds and computes all experts: no exchange after the MoE block
        else:
            es, ee = _split(cfg.n_experts, tp, rank) if cfg.is_moe else (0, 0)
        gs, ge = _split(cfg.ssm_v_heads, tp, rank) if getattr(cfg, "is_hybrid", False) else (0, 0)
        return TPPlan(tp, rank, qs, qe, ks, ke, rep, fs, fe, vs, ve, es, ee, gs, ge)

    def describe(self) -> str:
        return (f"rank {self.rank}/{self.tp}: q heads [{self.q_head_start},{self.q_head_stop}) "
                f"kv heads [{self.kv_head_start},{self.kv_head_stop}) x{self.kv_replicas} "
                f"ffn [{self.ff_start},{self.ff_stop}) vocab [{self.vocab_start},{self.vocab_stop}) "
                f"experts [{self.expert_start},{self.expert_stop})")
