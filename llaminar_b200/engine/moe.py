"""Mixture-of-experts FFN on the GPU runner.

Routing follows the reference (softmax over all experts, top-k with lower-id tie-break, weights
renormalised over the top-k: src/v2/kernels/cuda/moe/CUDAMoEKernels.cu ``softmax_topk_kernel``,
src/v2/models/qwen35moe/Qwen35MoEGraphConfigBuilder.cpp:37-45).  Small batches run one expert GEMV per
(token, slot) straight from the expert slab (device-resident expert ids, no host round trip, so the
step stays graph-capturable); larger batches group tokens by expert and run the tensor-core GEMM per
expert.  Under expert parallelism a rank only computes the slots routed to its experts and the
partial outputs are summed across ranks.
"""
from __future__ import annotations

import torch

from .. import ops

SMALL_SLOTS = 256


def moe_forward(model, L, h: torch.Tensor, T: int) -> None:
    c, sc = model.cfg, model.scratch
    dev = model.device
    k = c.n_experts_used
    xn = model.ws_xn[:T]
    ops.rmsnorm(h, L.ffn_norm, xn, c.rms_eps)
    logits = (xn @ L.router.T).float()
    ids = torch.empty(T, k, dtype=torch.int32, device=dev)
    wts = torch.empty(T, k, dtype=torch.float32, device=dev)
    ops.moe_topk(logits, k, c.norm_topk_prob, ids, wts)
    slab = L.experts
    local = (ids >= slab.e0) & (ids < slab.e0 + slab.n_local)
    lids = torch.where(local, ids - slab.e0, torch.zeros_like(ids)).contiguous()
    w_eff = torch.where(local, wts, torch.zeros_like(wts))
    ff, d = c.expert_ff, c.d_model
    ep = model.tp is not None and model.tp.size > 1
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
