"""Small, self-contained launches of the hot kernels for profiling and timing.

    python -m llaminar_b200.ops.profile_cases --case gemm_small --iters 5

Each case builds inputs larger than the L2 cache (so DRAM counters mean something) but well under a few GB, runs the
kernel a handful of times and prints the CUDA-event time of the last launches with the achieved bandwidth / FLOP rate.
The cases are the shapes of the Qwen3-32B (dense) and Qwen3-30B-A3B (MoE) decode and prefill steps.
"""
from __future__ import annotations

import argparse
import json
import math

import torch


def _rand_weight(ops, qt, n, k, dev, seed=1):
    from ..gguf.constants import BLOCK_GEOMETRY
    e, b = BLOCK_GEOMETRY[qt]
    g = torch.Generator(device=dev).manual_seed(seed)
    raw = torch.randint(0, 256, (n * k // e * b,), dtype=torch.uint8, device=dev, generator=g)
    raw.view(torch.int16).bitwise_and_(0x1FFF)            # keep every fp16 scale field finite and small (|d| < 0.0079)
    return ops.pack_matrix(raw, qt, n, k), raw.numel()


def _time(fn, iters):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    return sorted(ts)[len(ts) // 2]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=["gemm_small", "gemv", "gemm_large", "attn_decode", "attn_prefill", "moe"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--fmt", default="Q4_K")
    ap.add_argument("--m", type=int, default=0, help="rows of activations (GEMM cases; default: the case's own)")
    ap.add_argument("--n", type=int, default=51200)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--seq", type=int, default=2048, help="tokens per sequence of the attn_prefill case")
    args = ap.parse_args()
    from .. import ops
    from ..gguf import GGMLType
    dev = torch.device("cuda")
    sc = ops.scratch_for(dev)
    qt = GGMLType[args.fmt]
    g = torch.Generator(device=dev).manual_seed(0)
    rec = {"case": args.case}
    if args.case in ("gemm_small", "gemv", "gemm_large"):
        n, k = args.n, args.k                               # default: gate|up of the Qwen3-32B shape, 147 MB of Q4_K, larger than L2
        m = args.m or {"gemm_small": 32, "gemv": 1, "gemm_large": 1024}[args.case]
        pws = [_rand_weight(ops, qt, n, k, dev, s) for s in (1, 2)]
        x = (torch.randn(m, k, device=dev, generator=g) * 0.1).to(torch.bfloat16)
        out = torch.empty(m, n // 2, dtype=torch.bfloat16, device=dev)
        i = [0]

        def fn():
            i[0] += 1
            pw = pws[i[0] & 1][0]
            (ops.gemv if m <= 4 else ops.gemm)(pw, x, out, epi=ops.EPI_SWIGLU, scratch=sc)
        us = _time(fn, args.iters)
        wbytes = pws[0][1]
        rec.update(m=m, n=n, k=k, fmt=args.fmt, us=round(us, 1), weight_gbs=round(wbytes / us / 1e3, 1),
                   tflops=round(2.0 * m * n * k / us / 1e6, 1))
    elif args.case == "attn_decode":
        B, ctx, nq, nkv, D = 32, 2048, 64, 8, 128
        pages = (ctx + 63) // 64
        kv = (torch.randn(B * pages + 1, 2, nkv, 64, D, device=dev, generator=g) * 0.3).to(torch.bfloat16)
        bt = (torch.arange(B * pages, dtype=torch.int32, device=dev) + 1).view(B, pages)
        q = (torch.randn(B, nq, D, device=dev, generator=g) * 0.3).to(torch.bfloat16)
        out = torch.empty_like(q)
        lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        fn = lambda: ops.attn_decode(q, kv, out, bt, lens, nq, nkv, D, 1, 1.0 / math.sqrt(D), 1, sc)
        us = _time(fn, args.iters)
        kv_bytes = B * ctx * 2 * nkv * D * 2
        rec.update(batch=B, ctx=ctx, heads=f"{nq}/{nkv}", us=round(us, 1), kv_gbs=round(kv_bytes / us / 1e3, 1))
    elif args.case == "attn_prefill":
        B, L, nq, nkv, D = 4, args.seq, 32, 8, 128
        pages = (L + 63) // 64
        kv = (torch.randn(B * pages + 1, 2, nkv, 64, D, device=dev, generator=g) * 0.3).to(torch.bfloat16)
        bt = (torch.arange(B * pages, dtype=torch.int32, device=dev) + 1).view(B, pages)
        q = (torch.randn(B * L, nq, D, device=dev, generator=g) * 0.3).to(torch.bfloat16)
        out = torch.empty_like(q)
        cu = torch.arange(0, (B + 1) * L, L, dtype=torch.int32, device=dev)
        ctxl = torch.zeros(B, dtype=torch.int32, device=dev)
        flops = 4.0 * B * nq * D * L * L / 2                 # causal: half of the score matrix
        rec.update(batch=B, seq=L, heads=f"{nq}/{nkv}")
        for name, tc in (("mma_sync", False), ("tcgen05", True)):
            fn = lambda: ops.attn_prefill(q, kv, out, bt, cu, ctxl, nq, nkv, D, 1.0 / math.sqrt(D), L, tensor_core=tc)
            us = _time(fn, args.iters)
            rec[name] = {"us": round(us, 1), "tflops": round(flops / us / 1e6, 1)}
    else:  # moe: Qwen3-30B-A3B layer, 64 tokens, all 128 experts local (259 MB of IQ3_S expert weights)
        from ..ops.layout import pack_experts
        from ..gguf.constants import BLOCK_GEOMETRY
        T, E, kk, d, ff = 64, 128, 8, 2048, 768
        q3 = GGMLType.IQ3_S
        e_, b_ = BLOCK_GEOMETRY[q3]

        def slab(n, k):
            raw = torch.randint(0, 256, (E * n * k // e_ * b_,), dtype=torch.uint8, device=dev, generator=g)
            raw.view(torch.int16).bitwise_and_(0x1FFF)
            return pack_experts(raw, q3, E, n, k), raw.numel()
        (gate_up, b1), (down, b2) = slab(2 * ff, d), slab(d, ff)
        h = torch.randn(T, d, device=dev, generator=g)
        norm_w = torch.ones(d, device=dev)
        router = (torch.randn(E, d, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        z_max = E + (T * kk + 3) // 4
        zi = lambda *s, dt=torch.int32: torch.zeros(*s, dtype=dt, device=dev)
        ids, wts = zi(T, kk), zi(T, kk, dt=torch.float32)
        items, n_items, ticket = zi(z_max * ops.MOE_ITEM_INTS), zi(1), zi(1)
        act, yslot, tt = zi(T * kk, ff, dt=torch.bfloat16), zi(T * kk, d, dt=torch.float32), zi(d // 128)

        def fn():
            ops.moe_route(h, norm_w, 1e-6, router, kk, True, 0, E, ids, wts, items, n_items, ticket)
            ops.moe_gate_up(gate_up, h, norm_w, 1e-6, act, items, n_items, kk, z_max, scratch=sc)
            ops.moe_down_combine(down, act, yslot, items, n_items, z_max, ids, wts, kk, 0, E, h, tt, scratch=sc)
        us = _time(fn, args.iters)
        parts = [round(_time(lambda: ops.moe_route(h, norm_w, 1e-6, router, kk, True, 0, E, ids, wts, items, n_items, ticket), args.iters), 1),
                 round(_time(lambda: ops.moe_gate_up(gate_up, h, norm_w, 1e-6, act, items, n_items, kk, z_max, scratch=sc), args.iters), 1),
                 round(_time(lambda: ops.moe_down_combine(down, act, yslot, items, n_items, z_max, ids, wts, kk, 0, E, h, tt, scratch=sc), args.iters), 1)]
        touched = int(torch.unique(ids).numel())
        rec.update(tokens=T, experts=E, top_k=kk, us_three_launches=round(us, 1), us_route_gateup_down=parts, experts_touched=touched,
                   expert_weight_gbs=round((b1 + b2) * touched / E / us / 1e3, 1))
    print(json.dumps(rec), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
