"""Mixture-of-experts FFN on the GPU runner.

Routing follows the reference (softmax over all experts, top-k with lower-id tie-break, weights
renormalised over the top-k: src/v2/kernels/cuda/moe/CUDAMoEKernels.cu ``softmax_topk_kernel``,
src/v2/models/qwen35moe/Qwen35MoEGraphConfigBuilder.cpp:37-45).  Small batches run one expert GEMV per
(token, slot) straight from the expert slab (device-resident expert ids, no host round trip, so the
step stays graph-capturable); larger batches group tokens by expert and run the tensor-core GEMM per
expert.  Under expert parallelism a rank only computes the slots routed to its experts and the
partial outputs are summed across ranks.

Decode-sized batches take the fused path: `moe_route` (RMSNorm + router + top-k + grouped work list, one launch),
a grouped gate|up GEMV with SwiGLU epilogue and a grouped down GEMV whose last CTA per column tile does the weighted
combine, the all-reduce across the expert-parallel ranks over peer memory and the residual add
(the reference runs route, count, scan, scatter, per-expert GEMMs, gather-scale-add and an NCCL all-reduce as
separate stages: src/v2/compute_stages/stages/MoEExpertComputeStage.cpp, src/v2/models/qwen35moe/Qwen35MoEGraph.cpp:1766-1779).
Because the residual stream is replicated across the ranks of a tensor-parallel group, "dispatch" needs no transfer:
every rank gathers the rows routed to its own experts from its local copy.
"""
from __future__ import annotations

import torch

from .. import ops

SMALL_SLOTS = 256


FUSED_MAX_PAIRS = 4096        # tokens * top_k the in-kernel work-list builder accepts
FUSED_MAX_TOKENS = 64         # rows of the peer-memory inbox used by the fused combine


class _FusedWS:
    """Persistent buffers of the fused decode path (allocated once per token count: CUDA-graph safe)."""

    def __init__(self, model, T: int, n_local: int):
        c, dev = model.cfg, model.device
        k = c.n_experts_used
        z = lambda *s, dt: torch.zeros(*s, dtype=dt, device=dev)
        self.z_max = n_local + (T * k + 3) // 4
        self.ids, self.wts = z(T, k, dt=torch.int32), z(T, k, dt=torch.float32)
        self.items = z(self.z_max * ops.MOE_ITEM_INTS, dt=torch.int32)
        self.n_items, self.ticket = z(1, dt=torch.int32), z(1, dt=torch.int32)
        self.counts = z(max(n_local, 1), dt=torch.int32)
        self.act = z(T * k, c.expert_ff, dt=torch.bfloat16)
        self.yslot = z(T * k, c.d_model, dt=torch.float32)
        self.tile_tickets = z((c.d_model + 127) // 128, dt=torch.int32)


def _record_routing(model, L, ids: torch.Tensor) -> None:
    """Router statistics for the load-aware expert placement (models/expert_placement.py); eager steps only."""
    stats = getattr(model, "expert_stats", None)
    if stats is not None and not torch.cuda.is_current_stream_capturing():
        stats.record(L.index, ids)


def fused_supported(model, L, T: int) -> bool:
    c = model.cfg
    if not hasattr(ops, "moe_route") or T * c.n_experts_used > FUSED_MAX_PAIRS or c.n_experts > 256 or c.d_model % 256:
        return False
    ep = model.tp is not None and model.tp.size > 1 and getattr(model.tp, "moe_mode", "expert-parallel") != "replicated"
    if ep:
        symm = getattr(model.tp, "symm", None)
        if not (model.tp.fused and symm is not None and T <= symm.rows_cap and c.d_model <= symm.n_cap):
            return T <= FUSED_MAX_TOKENS * 4          # fused kernels + NCCL all-reduce of the combined rows
    return True


def moe_forward_fused(model, L, h: torch.Tensor, T: int) -> None:
    """Three launches per layer: route (+ work list), grouped gate|up + SwiGLU, grouped down + combine + all-reduce + residual."""
    c, sc = model.cfg, model.scratch
    slab = L.experts
    k = c.n_experts_used
    cache = model.__dict__.setdefault("_moe_ws", {})
    ws = cache.get(T)
    if ws is None:
        ws = cache[T] = _FusedWS(model, T, slab.n_local)
    ops.moe_route(h, L.ffn_norm, c.rms_eps, L.router, k, c.norm_topk_prob, slab.e0, slab.n_local, ws.ids, ws.wts,
                  ws.items, ws.n_items, ws.ticket, ws.counts)
    _record_routing(model, L, ws.ids)
    ops.moe_gate_up(slab.gate_up, h, L.ffn_norm, c.rms_eps, ws.act, ws.items, ws.n_items, k, ws.z_max, scratch=sc)
    ep = model.tp is not None and model.tp.size > 1 and getattr(model.tp, "moe_mode", "expert-parallel") != "replicated"
    symm = getattr(model.tp, "symm", None) if ep else None
    in_kernel = ep and model.tp.fused and symm is not None and T <= symm.rows_cap and c.d_model <= symm.n_cap
    if ep and not in_kernel:
        target = model.ws_partial[:T]
        target.zero_()
        ops.moe_down_combine(slab.down, ws.act, ws.yslot, ws.items, ws.n_items, ws.z_max, ws.ids, ws.wts, k, slab.e0, slab.n_local,
                             target, ws.tile_tickets, scratch=sc)
        model.tp.all_reduce(target)
        h += target
        return
    ops.moe_down_combine(slab.down, ws.act, ws.yslot, ws.items, ws.n_items, ws.z_max, ws.ids, ws.wts, k, slab.e0, slab.n_local,
                         h, ws.tile_tickets, scratch=sc, tp=symm.desc if in_kernel else None)
    if in_kernel:
        model.tp.stats["fused_calls"] += 1


def grouped_supported(model, L, T: int) -> bool:
    c = model.cfg
    return (hasattr(ops, "gemm_grouped") and getattr(model, "moe_grouped", True) and c.n_experts <= 256 and c.d_model % 256 == 0
            and c.expert_ff % 256 == 0 and L.experts.n_local >= 1)


def moe_forward_grouped(model, L, h: torch.Tensor, T: int) -> None:
    """Prefill-sized batches, entirely on the device: route (RMSNorm + router + top-k, one launch), sort the (token, slot)
    pairs by expert with device-side torch ops (no host round trip), ONE grouped tensor-core GEMM for gate|up + SwiGLU and
    one for down over all local experts, and an ordered weighted combine.  The reference's grouped prefill path does the
    same in its count / scan / scatter kernels, per-expert grouped GEMMs and ordered weighted scatter
    (reference: src/v2/kernels/cuda/moe/CUDAMoEKernels.cu:1242, :1537, :1707, :1826)."""
    c, sc, dev = model.cfg, model.scratch, model.device
    k, slab = c.n_experts_used, L.experts
    P = T * k
    xn = model.ws_xn[:T]
    ids = torch.empty(T, k, dtype=torch.int32, device=dev)
    wts = torch.empty(T, k, dtype=torch.float32, device=dev)
    ops.moe_route_only(h, L.ffn_norm, c.rms_eps, L.router, k, c.norm_topk_prob, ids, wts, xn)
    _record_routing(model, L, ids)
    flat = ids.view(-1)
    local = (flat >= slab.e0) & (flat < slab.e0 + slab.n_local)
    key = torch.where(local, flat - slab.e0, torch.full_like(flat, slab.n_local)).long()
    order = torch.argsort(key, stable=True)                  # pairs of other ranks' experts sort to the end and stay unused
    counts = torch.zeros(slab.n_local + 1, dtype=torch.int32, device=dev).index_add_(0, key, torch.ones(P, dtype=torch.int32, device=dev))
    avg = P // max(c.n_experts, 1)
    bm = 256 if avg >= 192 else (128 if avg >= 96 else 64)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    row_off = torch.cat([zero, torch.cumsum(counts[:slab.n_local], 0, dtype=torch.int32)])
    tile_off = torch.cat([zero, torch.cumsum((counts[:slab.n_local] + (bm - 1)) // bm, 0, dtype=torch.int32)])
    xg = xn.index_select(0, order // k)                      # activation rows in expert order
    act = torch.empty(P, c.expert_ff, dtype=torch.bfloat16, device=dev)
    y = torch.empty(P, c.d_model, dtype=torch.float32, device=dev)
    ops.gemm_grouped(slab.gate_up, xg, act, row_off, tile_off, bm, epi=ops.EPI_SWIGLU, scratch=sc)
    ops.gemm_grouped(slab.down, act, y, row_off, tile_off, bm, scratch=sc)
    pos = torch.empty(P, dtype=torch.int32, device=dev)
    pos[order] = torch.arange(P, dtype=torch.int32, device=dev)
    w_eff = torch.where(local.view(T, k), wts, torch.zeros_like(wts))
    ep = model.tp is not None and model.tp.size > 1 and getattr(model.tp, "moe_mode", "expert-parallel") != "replicated"
    target = model.ws_partial[:T] if ep else h
    if ep:
        target.zero_()
    ops.moe_combine_sorted(target, y, pos, w_eff, k)
    if ep:
        model.tp.all_reduce(target)
        h += target


def a2a_supported(model, L, T: int) -> bool:
    tp = model.tp
    # prefill-sized batches only: the split sizes of the exchange are read on the host, which a captured decode step cannot do
    return (tp is not None and tp.size > 1 and getattr(tp, "moe_mode", "") == "expert-parallel-a2a" and grouped_supported(model, L, T)
            and model.cfg.n_experts == L.experts.n_local * tp.size and T * model.cfg.n_experts_used > FUSED_MAX_PAIRS
            and not torch.cuda.is_current_stream_capturing())


def moe_forward_a2a(model, L, h: torch.Tensor, T: int) -> None:
    """Token-sharded expert parallelism through NCCL all-to-all (`--moe-expert-mode expert-parallel-a2a`), prefill-sized batches.

    Rank r routes only its own T / W tokens, sends every (token, slot) row to the rank that owns the expert
    (`all_to_all_single`, rows sorted by expert so that they arrive grouped), runs the grouped tensor-core expert GEMMs on what
    it received, sends the results back, combines them with the routing weights for its own tokens and all-gathers the token
    rows (the residual stream stays replicated for the tensor-parallel attention).  This is the dispatch / return form of the
    reference (reference: src/v2/execution/moe/MoEOverlaySparseCollective.cpp) and the baseline that the default mode is
    measured against: with a replicated residual it moves top_k * d per token and direction (bf16 out, fp32 back) where the
    default mode's dense all-reduce moves about 2 * d fp32, and NCCL's variable split sizes cost one host synchronisation per
    layer, so it is not the default."""
    import torch.distributed as dist
    c, sc, dev, tp = model.cfg, model.scratch, model.device, model.tp
    W, r, k, slab, d = tp.size, tp.rank, c.n_experts_used, L.experts, c.d_model
    nl = slab.n_local
    t0, t1 = T * r // W, T * (r + 1) // W
    To = t1 - t0
    xn = model.ws_xn[:To]
    ids = torch.empty(To, k, dtype=torch.int32, device=dev)
    wts = torch.empty(To, k, dtype=torch.float32, device=dev)
    ops.moe_route_only(h[t0:t1], L.ffn_norm, c.rms_eps, L.router, k, c.norm_topk_prob, ids, wts, xn)
    flat = ids.view(-1).long()
    order = torch.argsort(flat, stable=True)                 # by expert, hence by destination rank
    sorted_e = flat[order]
    send_counts = torch.bincount(sorted_e // nl, minlength=W)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=tp.group)
    sc_l, rc_l = send_counts.tolist(), recv_counts.tolist()  # NCCL wants the split sizes on the host
    R = sum(rc_l)
    send_rows = xn.index_select(0, order // k)
    send_eid = (sorted_e % nl).to(torch.int32)
    recv_rows = torch.empty(R, d, dtype=torch.bfloat16, device=dev)
    recv_eid = torch.empty(R, dtype=torch.int32, device=dev)
    dist.all_to_all_single(recv_rows, send_rows, rc_l, sc_l, group=tp.group)
    dist.all_to_all_single(recv_eid, send_eid, rc_l, sc_l, group=tp.group)
    y_arr = torch.empty(R, d, dtype=torch.float32, device=dev)
    if R > 0:
        key = recv_eid.long()
        order2 = torch.argsort(key, stable=True)             # arrival order is by source rank; the GEMMs want it by expert
        counts = torch.bincount(key, minlength=nl).to(torch.int32)
        avg = R // max(nl, 1)
        bm = 256 if avg >= 192 else (128 if avg >= 96 else 64)
        zero = torch.zeros(1, dtype=torch.int32, device=dev)
        row_off = torch.cat([zero, torch.cumsum(counts, 0, dtype=torch.int32)])
        tile_off = torch.cat([zero, torch.cumsum((counts + (bm - 1)) // bm, 0, dtype=torch.int32)])
        xg = recv_rows.index_select(0, order2)
        act = torch.empty(R, c.expert_ff, dtype=torch.bfloat16, device=dev)
        y = torch.empty(R, d, dtype=torch.float32, device=dev)
        ops.gemm_grouped(slab.gate_up, xg, act, row_off, tile_off, bm, epi=ops.EPI_SWIGLU, scratch=sc)
        ops.gemm_grouped(slab.down, act, y, row_off, tile_off, bm, scratch=sc)
        y_arr[order2] = y                                    # back to arrival order
    back = torch.empty(To * k, d, dtype=torch.float32, device=dev)
    dist.all_to_all_single(back, y_arr, sc_l, rc_l, group=tp.group)
    # `back` is in this rank's by-expert order of its own pairs
    Tmax = (T + W - 1) // W
    own = torch.zeros(Tmax, d, dtype=torch.float32, device=dev)
    if To > 0:
        pos = torch.empty(To * k, dtype=torch.int32, device=dev)
        pos[order] = torch.arange(To * k, dtype=torch.int32, device=dev)
        ops.moe_combine_sorted(own[:To], back, pos, wts, k)
    full = torch.empty(W, Tmax, d, dtype=torch.float32, device=dev)
    dist.all_gather_into_tensor(full, own, group=tp.group)
    for q in range(W):
        q0, q1 = T * q // W, T * (q + 1) // W
        if q1 > q0:
            h[q0:q1] += full[q, :q1 - q0]
    tp.stats["a2a_calls"] = tp.stats.get("a2a_calls", 0) + 1
    tp.stats["a2a_bytes"] = tp.stats.get("a2a_bytes", 0) + sum(sc_l) * d * 2 + R * d * 4


def moe_forward(model, L, h: torch.Tensor, T: int) -> None:
    c, sc = model.cfg, model.scratch
    dev = model.device
    k = c.n_experts_used
    if a2a_supported(model, L, T):
        return moe_forward_a2a(model, L, h, T)
    if T * k <= SMALL_SLOTS * 2 and fused_supported(model, L, T):
        return moe_forward_fused(model, L, h, T)
    if T * k > SMALL_SLOTS and grouped_supported(model, L, T):
        return moe_forward_grouped(model, L, h, T)
    xn = model.ws_xn[:T]
    ops.rmsnorm(h, L.ffn_norm, xn, c.rms_eps)
    logits = (xn @ L.router.T).float()
    ids = torch.empty(T, k, dtype=torch.int32, device=dev)
    wts = torch.empty(T, k, dtype=torch.float32, device=dev)
    ops.moe_topk(logits, k, c.norm_topk_prob, ids, wts)
    _record_routing(model, L, ids)
    slab = L.experts
    local = (ids >= slab.e0) & (ids < slab.e0 + slab.n_local)
    lids = torch.where(local, ids - slab.e0, torch.zeros_like(ids)).contiguous()
    w_eff = torch.where(local, wts, torch.zeros_like(wts))
    ff, d = c.expert_ff, c.d_model
    ep = model.tp is not None and model.tp.size > 1 and getattr(model.tp, "moe_mode", "expert-parallel") != "replicated"
    target = model.ws_partial[:T] if ep else h
    if ep:
        target.zero_()
    if T * k <= SMALL_SLOTS:
        act = torch.empty(T * k, ff, dtype=torch.bfloat16, device=dev)
        y = torch.empty(T * k, d, dtype=torch.bfloat16, device=dev)
        flat = lids.view(-1)
        ops.gemv_experts(slab.gate_up, xn, act, flat, k, epi=ops.EPI_SWIGLU, scratch=sc)
        ops.gemv_experts(slab.down, act, y, flat, 1, scratch=sc)
        target += (y.float().view(T, k, d) * w_eff.unsqueeze(-1)).sum(dim=1)
    else:
        # group (token, slot) pairs by expert; one tensor-core GEMM pair per expert that received tokens
        flat_e = torch.where(local, lids, torch.full_like(lids, slab.n_local)).view(-1)
        order = torch.argsort(flat_e, stable=True)
        counts = torch.bincount(flat_e, minlength=slab.n_local + 1)[:slab.n_local].tolist()
        tok_of = (order // k)
        w_sorted = w_eff.view(-1)[order]
        start = 0
        gu_stride = slab.gate_up.data.shape[1] if slab.gate_up.data.dim() == 2 else 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            rows = tok_of[start:start + n]
            xe = xn.index_select(0, rows).contiguous()
            act = torch.empty(n, ff, dtype=torch.bfloat16, device=dev)
            ye = torch.empty(n, d, dtype=torch.float32, device=dev)
            ops.gemm(_expert_view(slab.gate_up, e), xe, act, epi=ops.EPI_SWIGLU, scratch=sc)
            ops.gemm(_expert_view(slab.down, e), act, ye, scratch=sc)
            target.index_add_(0, rows, ye * w_sorted[start:start + n].unsqueeze(-1))
            start += n
    if ep:
        model.tp.all_reduce(target)
        h += target


def _expert_view(pw, e: int):
    from ..ops.layout import PackedWeight
    return PackedWeight(pw.fmt, pw.qtype, pw.n, pw.k, pw.n_tiles, pw.k_blocks, pw.data[e])
