"""Python surface of the sm_100a kernels.

Everything here launches hand-written CUDA from ``csrc/`` on the current torch stream.  There is
no silent fallback: on a machine with a GPU the extension must load, otherwise these calls raise.
The pure-PyTorch execution path used on CPU lives in :mod:`llaminar_b200.models.reference`.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import build as _build
from .layout import FMT_IDS, PackedWeight, can_pack, pack_experts, pack_matrix  # noqa: F401

EPI_STORE, EPI_RESID, EPI_SWIGLU, EPI_MOE_COMBINE = 0, 1, 2, 3
GEMV_MAX_ROWS = 4
PAGE_SIZE = 64

_launches = 0          # kernels of this extension launched by the current process (bench evidence)


_ext_ready = False


def ext():
    global _ext_ready
    mod = _build.load()
    if not _ext_ready:
        from ..utils.env import debug_env
        mod.set_pdl(bool(debug_env().pdl))       # programmatic dependent launch of the decode-path kernels
        _ext_ready = True
    return mod


def bounds_status(reset: bool = True) -> int:
    """Status word of the bounds-check build (LLAMINAR_BOUNDS_CHECK=1): non-zero after a kernel met an index outside its
    table (it used index 0 instead and went on).  Always 0 in the production build."""
    return int(ext().bounds_status(bool(reset)))


def launch_count() -> int:
    return _launches


def _count(n: int = 1) -> None:
    global _launches
    _launches += n


@dataclass
class Scratch:
    """Per-device reusable scratch: split-K accumulators, arrival counters, attention split partials.

    All buffers are returned to zero by the kernels that use them, so they can be shared by every
    call on one stream (calls on different streams need separate instances).
    """
    accum: torch.Tensor
    tickets: torch.Tensor
    part_o: torch.Tensor
    part_ml: torch.Tensor
    attn_tickets: torch.Tensor
    status: torch.Tensor
    partials: torch.Tensor          # small-batch GEMM: per-CTA slots for the partial sums of split tiles

    @staticmethod
    def create(device, accum_rows: int = 256, accum_cols: int = 65536, attn_slots: int = 1 << 22) -> "Scratch":
        z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=device)
        return Scratch(accum=z(accum_rows, accum_cols), tickets=z(8192, dt=torch.int32),
                       part_o=z(attn_slots), part_ml=z(attn_slots // 32), attn_tickets=z(8192, dt=torch.int32),
                       status=z(4, dt=torch.int32), partials=z(148 * 2 * 128 * 32))


    def reset(self) -> None:
        """Return the split-K accumulators and counters to zero (after a kernel reported a timed-out wait)."""
        for t in (self.accum, self.tickets, self.attn_tickets, self.status):
            t.zero_()


_scratch: dict[str, Scratch] = {}


def scratch_for(device) -> Scratch:
    key = str(device)
    if key not in _scratch:
        _scratch[key] = Scratch.create(device)
    return _scratch[key]


def _accum_args(pw: PackedWeight, rows: int, sc: Scratch | None):
    if sc is None or pw.n_tiles * 128 > sc.accum.shape[1] or rows > sc.accum.shape[0]:
        return None, None
    return sc.accum, sc.tickets


def gemv(pw: PackedWeight, x: torch.Tensor, out: torch.Tensor, *, norm_w: torch.Tensor | None = None, eps: float = 1e-6,
         epi: int = EPI_STORE, bias: torch.Tensor | None = None, scratch: Scratch | None = None, ksplit: int = 0,
         tp: torch.Tensor | None = None, tuned: bool = True, stream: bool = True) -> None:
    """out[m, :] (+)= x[m, :] @ W^T for m <= 4 rows.  x: fp32 residual rows when ``norm_w`` is given, else bf16.
    Plain dense calls run the streaming kernel (persistent CTAs, chunks by bulk copy; ``stream=False`` keeps the
    register-path kernel, which also serves the fused tensor-parallel epilogue and the expert work lists).
    ``tp``: device copy of the tensor-parallel descriptor; with EPI_RESID the epilogue all-reduces across ranks.
    ``ksplit`` 0 lets the tuning table (``ops/tuning.py``), then the kernel's heuristic, pick the split-K factor."""
    rows = x.shape[0]
    assert 1 <= rows <= GEMV_MAX_ROWS
    if ksplit == 0 and tuned and tp is None:          # the fused all-reduce epilogue keeps the kernel's own choice
        from .tuning import table
        ksplit = table().ksplit("gemv", pw.fmt, pw.n, pw.k, rows)
    accum, tickets = _accum_args(pw, rows, scratch)
    if tickets is None and scratch is not None and pw.n_tiles <= scratch.tickets.numel():
        tickets = scratch.tickets          # wider than the split-K accumulator (the LM head): the streaming kernel needs the counters only
    ext().gemv(pw.data, pw.fmt, pw.n, pw.k, x, norm_w, eps, out, epi, bias, accum, tickets, ksplit, None, 0, 1, rows, 1, tp,
               scratch.partials if scratch is not None else None, scratch.status if scratch is not None else None,
               stream and tp is None)
    _count()


def gemv_experts(pw: PackedWeight, x: torch.Tensor, out: torch.Tensor, expert_ids: torch.Tensor, slots_per_row: int, *,
                 epi: int = EPI_STORE, scratch: Scratch | None = None) -> None:
    """One GEMV per (token, expert slot): out[z] = W[expert_ids[z]] @ x[z // slots_per_row]."""
    z = expert_ids.numel()
    accum, tickets = _accum_args(pw, z, scratch)
    if tickets is not None and z * pw.n_tiles > tickets.numel():
        accum, tickets = None, None
    stride = pw.n_tiles * pw.k_blocks * pw.chunk_bytes
    ext().gemv(pw.data, pw.fmt, pw.n, pw.k, x, None, 0.0, out, epi, None, accum, tickets, 0, expert_ids, stride,
               slots_per_row, 1, z, None, None, None, False)
    _count()


MOE_ITEM_INTS = 6          # struct MoeItem { int expert, m, slot[4]; }


def moe_route(h, norm_w, eps, router, top_k, renorm, e0, n_local, ids, wts, items, n_items, ticket, counts=None) -> None:
    """Fused RMSNorm + router projection + softmax top-k + grouped work list of the local experts."""
    ext().moe_route(h, norm_w, eps, router, top_k, bool(renorm), e0, n_local, ids, wts, items, n_items, ticket, counts)
    _count()


def moe_route_only(h, norm_w, eps, router, top_k, renorm, ids, wts, xn_out=None) -> None:
    """RMSNorm + router projection + softmax top-k for any number of tokens; ``xn_out`` receives the normalised rows (bf16)."""
    ext().moe_route_only(h, norm_w, eps, router, top_k, bool(renorm), ids, wts, xn_out)
    _count()


def moe_combine_sorted(h, y, pos, wts, top_k: int) -> None:
    """h[t] += sum_s wts[t, s] * y[pos[t, s]] (slot order; zero-weight slots skipped)."""
    ext().moe_combine_sorted(h, y, pos, wts, top_k)
    _count()


def gemm_grouped(pw: PackedWeight, x: torch.Tensor, out: torch.Tensor, row_off: torch.Tensor, tile_off: torch.Tensor, block_m: int, *,
                 epi: int = EPI_STORE, scratch: Scratch | None = None) -> None:
    """Expert GEMMs of one chunk in one launch: rows of ``x`` / ``out`` are sorted by expert, ``row_off`` / ``tile_off``
    (device int32 [experts + 1]) give every expert's first row and first m-tile of height ``block_m``."""
    stride = pw.n_tiles * pw.k_blocks * pw.chunk_bytes
    ext().gemm_tc_grouped(pw.data, pw.fmt, pw.n, pw.k, pw.n_experts, stride, x, out, epi, row_off, tile_off, block_m,
                          scratch.status if scratch is not None else None)
    _count()


def moe_gate_up(pw: PackedWeight, h, norm_w, eps, act, items, n_items, top_k, z_max, scratch: Scratch | None = None) -> None:
    """Grouped expert gate|up GEMV with fused RMSNorm prologue and SwiGLU epilogue: act[pair] for every local pair."""
    accum, tickets = _accum_args(pw, 4 * z_max, scratch)
    if tickets is not None and z_max * pw.n_tiles > tickets.numel():
        accum, tickets = None, None
    stride = pw.n_tiles * pw.k_blocks * pw.chunk_bytes
    ext().moe_gemv(pw.data, pw.fmt, pw.n, pw.k, stride, h, norm_w, eps, act, EPI_SWIGLU, items, n_items, top_k, z_max,
                   accum, tickets, None, None, top_k, 0, 0, None, None, None)
    _count()


def moe_down_combine(pw: PackedWeight, act, yslot, items, n_items, z_max, ids, wts, top_k, e0, n_local, h, tile_tickets,
                     scratch: Scratch | None = None, tp=None) -> None:
    """Grouped expert down GEMV; the last CTA of each column tile combines the weighted pairs, all-reduces the tile
    across expert-parallel ranks over peer memory (when ``tp`` is given) and adds it to the residual stream."""
    accum, tickets = _accum_args(pw, 4 * z_max, scratch)
    if tickets is not None and z_max * pw.n_tiles > tickets.numel():
        accum, tickets = None, None
    stride = pw.n_tiles * pw.k_blocks * pw.chunk_bytes
    ext().moe_gemv(pw.data, pw.fmt, pw.n, pw.k, stride, act, None, 0.0, yslot, EPI_MOE_COMBINE, items, n_items, 1, z_max,
                   accum, tickets, ids, wts, top_k, e0, n_local, h, tile_tickets, tp)
    _count()


def gemm(pw: PackedWeight, x: torch.Tensor, out: torch.Tensor, *, epi: int = EPI_STORE, bias: torch.Tensor | None = None,
         scratch: Scratch | None = None, ksplit: int = 0, debug_ptr: int = 0, flags: int = 0,
         tp: torch.Tensor | None = None) -> None:
    """Tensor-core path: out[M, N] (+)= x[M, K] @ dequant(W)^T, any M."""
    accum, tickets = _accum_args(pw, x.shape[0], scratch)
    ext().gemm_tc(pw.data, pw.fmt, pw.n, pw.k, x, out, epi, bias, accum, tickets, ksplit if accum is not None else 1,
                  scratch.status if scratch is not None else None, debug_ptr, flags, tp,
                  scratch.partials if scratch is not None else None)
    _count()


def gemm_allgather(pw: PackedWeight, m_total: int, out: torch.Tensor, desc: torch.Tensor, *, epi: int = EPI_STORE,
                   bias: torch.Tensor | None = None, status: torch.Tensor | None = None) -> None:
    """Column-parallel GEMM with the all-gather of its row-sharded input fused into the launch (see AgFuse in gemm_tc.h)."""
    ext().gemm_tc_allgather(pw.data, pw.fmt, pw.n, pw.k, m_total, out, epi, bias, status, desc)
    _count()


def gemm_reduce_scatter(pw: PackedWeight, x: torch.Tensor, desc: torch.Tensor, *, status: torch.Tensor | None = None) -> None:
    """Row-parallel GEMM whose bf16 partial tiles go straight to the owners of their rows (see RsFuse in gemm_tc.h)."""
    ext().gemm_tc_rs(pw.data, pw.fmt, pw.n, pw.k, x, status, desc)
    _count()


def rs_reduce_norm(inbox_ptr: int, flags_ptr: int, target: int, world: int, rows_per_rank: int, n_cap: int, block_m: int,
                   h: torch.Tensor, norm_w: torch.Tensor | None, xn: torch.Tensor | None, eps: float, spin_limit: int,
                   status: torch.Tensor | None) -> None:
    """Owner side of the fused reduce-scatter: h[row] += sum of the ranks' partial rows; xn[row] = RMSNorm(h[row]) * norm_w."""
    ext().rs_reduce_norm(inbox_ptr, flags_ptr, target, world, rows_per_rank, n_cap, block_m, h, norm_w, xn, eps, spin_limit, status)
    _count()


def dequant(pw: PackedWeight, out: torch.Tensor | None = None) -> torch.Tensor:
    if out is None:
        out = torch.empty(pw.n, pw.k, dtype=torch.bfloat16, device=pw.data.device)
    ext().dequant(pw.data, pw.fmt, pw.n, pw.k, out)
    _count()
    return out


def gather_rows(pw: PackedWeight, rows: torch.Tensor, out: torch.Tensor) -> None:
    ext().gather_rows(pw.data, pw.fmt, pw.k, rows, out)
    _count()


def rmsnorm(h: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    ext().rmsnorm(h, w, out, eps)
    _count()


def mtp_concat_norm(emb, hidden, enorm, hnorm, out, eps: float) -> None:
    """out[row] = [RMSNorm(emb[row]) * enorm | RMSNorm(hidden[row]) * hnorm] in bf16 (input of the NextN eh_proj)."""
    ext().mtp_concat_norm(emb, hidden, enorm, hnorm, out, eps)
    _count()


def rope_kv(qkv, q_out, kv, q_norm, k_norm, positions, seq_ids, block_table, n_heads, n_kv_heads, head_dim, theta, eps) -> None:
    ext().rope_kv(qkv, q_out, kv, q_norm, k_norm, positions, seq_ids, block_table, n_heads, n_kv_heads, head_dim, theta, eps)
    _count()


def attn_decode(q, kv, out, block_table, seq_lens, n_heads, n_kv_heads, head_dim, rows_per_seq, scale, n_splits,
                scratch: Scratch) -> None:
    ext().attn_decode(q, kv, out, block_table, seq_lens, scratch.part_o, scratch.part_ml, scratch.attn_tickets,
                      n_heads, n_kv_heads, head_dim, rows_per_seq, scale, n_splits)
    _count()


def attn_prefill(q, kv, out, block_table, cu_q, ctx_lens, n_heads, n_kv_heads, head_dim, scale, max_q_len,
                 tensor_core: bool | None = None, scratch: "Scratch | None" = None) -> None:
    """Causal GQA attention of a prefill chunk over the paged cache.  ``tensor_core`` picks the tcgen05 kernel (head_dim 128),
    otherwise the mma.sync kernel runs.  Default: the tcgen05 kernel for chunks of at least ATTN_TC_MIN_ROWS query rows per
    sequence (measured 283 vs 246 TFLOP/s at 2048 rows, 323 vs 234 at 4096, but 223 vs 237 at 1024, where its per-CTA
    start-up weighs more); LLAMINAR_ATTN_TC=0 turns it off."""
    if tensor_core is None:
        tensor_core = head_dim == 128 and max_q_len >= ATTN_TC_MIN_ROWS and _attn_tc_default()
    status = scratch.status if (tensor_core and scratch is not None) else None
    ext().attn_prefill(q, kv, out, block_table, cu_q, ctx_lens, n_heads, n_kv_heads, head_dim, scale, max_q_len, bool(tensor_core), status)
    _count()


def kv_dequant_pages(kv8: torch.Tensor, block_table: torch.Tensor, n_tokens: torch.Tensor, n_kv_heads: int, head_dim: int,
                     staging: torch.Tensor) -> None:
    """8-bit KV pages of the sequences in ``block_table`` -> bf16 pages: page j of sequence s lands at staging page
    ``s * block_table.shape[1] + j`` (only pages that hold one of the sequence's ``n_tokens[s]`` tokens are written)."""
    ext().kv_dequant_pages(kv8, block_table, n_tokens, n_kv_heads, head_dim, staging)
    _count()


def gdn_step(inp: torch.Tensor, C: int, z_off: int, ab_off: int, conv_w: torch.Tensor, ssm_a: torch.Tensor, dt_bias: torch.Tensor,
             norm_w: torch.Tensor, conv_state: torch.Tensor, rec: torch.Tensor, slots: torch.Tensor, y: torch.Tensor,
             out: torch.Tensor, n_k: int, v_head_offset: int, eps: float) -> None:
    """One new token per row of a Gated-DeltaNet block, between its input and output projections (two launches).
    ``inp`` [rows, >= C + ...] bf16 is the input projection's output: q | k | v in columns [0, C), the gate z from
    ``z_off``, (alpha | b) from ``ab_off``.  conv_state [slots, C, K-1] and rec [slots, n_v, d, d] are the layer's fp32 state
    pools, ``slots`` [rows] int32 picks each row's slot; y [rows, C] fp32 is scratch; out [rows, n_v * d] bf16."""
    ext().gdn_conv_step(inp, conv_w, conv_state, slots, y)
    ext().gdn_recurrent_step(y, inp, z_off, ab_off, ssm_a, dt_bias, norm_w, rec, slots, out, n_k, v_head_offset, eps)
    _count(2)


ATTN_TC_MIN_ROWS = 1536
_ATTN_TC = None


def _attn_tc_default() -> bool:
    global _ATTN_TC
    if _ATTN_TC is None:
        from ..utils.env import debug_env
        _ATTN_TC = bool(debug_env().attn_tc)
    return _ATTN_TC


def argmax(logits: torch.Tensor, tokens: torch.Tensor | None, pairs: torch.Tensor | None = None, idx_offset: int = 0) -> None:
    """Row argmax (ties -> lower index).  ``pairs`` [rows, 2] int32 receives (value bits, idx_offset + index) for the
    cross-rank merge of a vocabulary-sharded head."""
    ext().argmax(logits, tokens, pairs, idx_offset)
    _count()


def argmax_merge(gathered: torch.Tensor, ranks: int, rows: int, tokens: torch.Tensor) -> None:
    """gathered [ranks, rows, 2] int32 of per-shard (value bits, global index) -> tokens[rows]."""
    ext().argmax_merge(gathered, ranks, rows, tokens)
    _count()


def sample(logits, temperature, top_k, top_p, seeds, step, tokens, probs_out=None) -> None:
    ext().sample(logits, temperature, top_k, top_p, seeds, step, tokens, probs_out)
    _count()


def sample_candidates(logits, idx_offset: int, pairs) -> None:
    """Pass 1 of sampling over a vocabulary-sharded head: pairs[rows, k, 2] (int32) receive this shard's k best entries as
    (float bits, global token id), best first."""
    ext().sample_candidates(logits, idx_offset, pairs)
    _count()


def sample_merged(gathered, temperature, top_k, top_p, seeds, step, tokens) -> None:
    """Pass 2: draw from the all-gathered pairs [ranks, rows, k, 2]; the token equals the one `sample` draws from the full row."""
    ext().sample_merged(gathered, temperature, top_k, top_p, seeds, step, tokens)
    _count()


def penalties_dense(logits, counts, presence, frequency) -> None:
    """logits[row, t] -= presence[row] * (counts[row, t] > 0) + frequency[row] * counts[row, t] (int16 count table per lane)."""
    ext().penalties_dense(logits, counts, presence, frequency)
    _count()


def count_tokens(counts, tokens, v0: int, vocab: int) -> None:
    """counts[row, tokens[row] - v0] += 1 where the token falls into [v0, v0 + vocab): the sampled tokens join the history."""
    ext().count_tokens(counts, tokens, v0, vocab)
    _count()


def nan_scan(x: torch.Tensor) -> tuple[int, int]:
    counts = torch.zeros(2, dtype=torch.int32, device=x.device)
    ext().nan_scan(x.contiguous(), counts)
    _count()
    c = counts.tolist()
    return c[0], c[1]


def spec_verify_greedy(draft, target, n_accept, out_tokens) -> None:
    ext().spec_verify_greedy(draft, target, n_accept, out_tokens)
    _count()


def spec_verify_reject(p_target, p_draft, draft, seeds, step, n_accept, out_tokens) -> None:
    ext().spec_verify_reject(p_target, p_draft, draft, seeds, step, n_accept, out_tokens)
    _count()


def moe_topk(logits, k, renorm, ids, weights, counts=None) -> None:
    ext().moe_topk(logits, k, renorm, ids, weights, counts)
    _count()
