"""Microbenchmark of the fused row-parallel GEMM/GEMV + all-reduce against GEMM + NCCL all-reduce + add.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        -m llaminar_b200.parallel.bench_fused --rows 1 32 --shape 5120x8192 5120x25600

Every number is the device time of one call (CUDA events on the launching stream, L2 made cold by rotating through
weight copies larger than the cache), maximum over ranks.  The roofline printed beside it is the slower of the
weight bytes over the measured HBM bandwidth and the bytes that must cross NVLink over the measured peer bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, nargs="+", default=[1, 4, 32])
    ap.add_argument("--shape", nargs="+", default=["5120x8192", "5120x25600"], help="N x K of the full (unsharded) weight")
    ap.add_argument("--fmt", default="Q4_K")
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--hbm-gbs", type=float, default=6455.6)
    ap.add_argument("--nvlink-gbs", type=float, default=770.0)
    ap.add_argument("--bf16-tflops", type=float, default=1428.7)
    ap.add_argument("--mode", default="rowpar", choices=["rowpar", "allgather"],
                    help="rowpar: GEMM -> all-reduce (+ residual); allgather: all-gather -> column-parallel GEMM")
    ap.add_argument("--ag-rows", type=int, nargs="+", default=[2048, 8192], help="allgather mode: total rows over all ranks")
    ap.add_argument("--copy-ctas", type=int, default=8)
    args = ap.parse_args()
    from .. import ops
    from ..gguf import GGMLType
    from ..gguf.constants import BLOCK_GEOMETRY
    from .tp import TPContext
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tp = TPContext.create(device=dev, fused=True) if world > 1 else None
    qt = GGMLType[args.fmt]
    elems, bpb = BLOCK_GEOMETRY[qt]
    sc = ops.scratch_for(dev)
    out = []

    def timed(fn, iters):
        for _ in range(3):
            fn(0)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        for i, (a, b) in enumerate(evs):
            a.record()
            fn(i)
            b.record()
        torch.cuda.synchronize()
        ts = sorted(a.elapsed_time(b) * 1e3 for a, b in evs)
        t = torch.tensor([ts[len(ts) // 2]], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    if args.mode == "allgather":
        from .symm import AllGatherArena
        for shp in args.shape:
            n_full, k = (int(v) for v in shp.split("x"))
            n = n_full // world                                      # column-parallel: this rank's output columns
            wbytes = n * k // elems * bpb
            g = torch.Generator(device=dev).manual_seed(1 + rank)
            raw = torch.randint(0, 256, (wbytes,), dtype=torch.uint8, device=dev, generator=g)
            raw.view(torch.int16).bitwise_and_(0x1FFF)
            pw = ops.pack_matrix(raw, qt, n, k)
            for m_total in args.ag_rows:
                rpr = (m_total + world - 1) // world
                arena = AllGatherArena(dist.group.WORLD, dev, rows_cap=rpr, k_cap=k, copy_ctas=args.copy_ctas)
                x_own = (torch.randn(rpr, k, device=dev, generator=g) * 0.1).to(torch.bfloat16)
                x_all = torch.empty(world * rpr, k, dtype=torch.bfloat16, device=dev)
                out = torch.empty(m_total, n, dtype=torch.bfloat16, device=dev)

                def nccl(i):
                    dist.all_gather_into_tensor(x_all, x_own)
                    ops.gemm(pw, x_all[:m_total], out, scratch=sc)

                def gemm_only(i):
                    ops.gemm(pw, x_all[:m_total], out, scratch=sc)

                def fused(i):
                    arena.own_rows(rpr, k).copy_(x_own)              # stands for the producer writing its rows in place
                    arena.gemm(pw, m_total, rpr, out)

                def copy_only(i):
                    arena.own_rows(rpr, k).copy_(x_own)

                def gemm_symm(i):                                     # same GEMM, activations read from symmetric memory
                    ops.gemm(pw, x_symm, out, scratch=sc)

                arena.own_rows(rpr, k).copy_(x_own)
                arena.gemm(pw, m_total, rpr, out)
                x_symm = arena.gathered(m_total, k)
                rec = {"mode": "allgather", "shape": shp, "n_local": n, "rows_total": m_total, "fmt": args.fmt, "world": world,
                       "gemm_only_us": round(timed(gemm_only, args.iters), 1), "gemm_on_symmetric_memory_us": round(timed(gemm_symm, args.iters), 1),
                       "allgather_then_gemm_us": round(timed(nccl, args.iters), 1),
                       "fused_us": round(timed(fused, args.iters) - timed(copy_only, args.iters), 1)}
                arena.check_status()
                flops = 2.0 * m_total * n * k
                link_bytes = (world - 1) * rpr * k * 2               # rows this rank must pull from its peers
                roof = max(flops / (args.bf16_tflops * 1e6), link_bytes / (args.nvlink_gbs * 1e3), wbytes / (args.hbm_gbs * 1e3))
                rec.update(roofline_us=round(roof, 1), fused_frac_of_roofline=round(roof / rec["fused_us"], 3),
                           speedup_vs_nccl=round(rec["allgather_then_gemm_us"] / rec["fused_us"], 2),
                           tflops_fused=round(flops / rec["fused_us"] / 1e6, 1))
                if rank == 0:
                    print(json.dumps(rec), flush=True)
                del arena
        dist.destroy_process_group()
        return 0
    for shp in args.shape:
        n, k_full = (int(v) for v in shp.split("x"))
        k = k_full // world
        wbytes = n * k // elems * bpb
        copies = max(2, int(400e6 // wbytes) + 1)                   # rotate through > 3x the L2 capacity
        g = torch.Generator(device=dev).manual_seed(1 + rank)
        raws = [torch.randint(0, 256, (wbytes,), dtype=torch.uint8, device=dev, generator=g) for _ in range(copies)]
        # random bytes are valid blocks for timing purposes except for fp16 scale fields that could decode to inf/nan;
        # clear the exponent's top bit of every 16-bit word so all scales stay finite
        pws = []
        for r in raws:
            r.view(torch.int16).bitwise_and_(0x1FFF)
            pws.append(ops.pack_matrix(r, qt, n, k))
        for rows in args.rows:
            x = (torch.randn(rows, k, device=dev, generator=g) * 0.1).to(torch.bfloat16)
            h = torch.zeros(rows, n, device=dev)
            part = torch.zeros(rows, n, device=dev)
            small = rows <= ops.GEMV_MAX_ROWS
            call = ops.gemv if small else ops.gemm

            def plain(i):
                call(pws[i % copies], x, h, epi=ops.EPI_RESID, scratch=sc)

            def nccl(i):
                call(pws[i % copies], x, part, epi=ops.EPI_STORE, scratch=sc)
                dist.all_reduce(part)
                h.add_(part)

            def fused(i):
                call(pws[i % copies], x, h, epi=ops.EPI_RESID, scratch=sc, tp=tp.symm.desc)

            rec = {"shape": shp, "rows": rows, "fmt": args.fmt, "world": world, "k_local": k,
                   "gemm_only_us": round(timed(plain, args.iters), 2)}
            if world > 1:
                rec["gemm_nccl_add_us"] = round(timed(nccl, args.iters), 2)
                rec["fused_us"] = round(timed(fused, args.iters), 2)
                tp.symm.check_status()
                link_bytes = rows * n * 4 * (world - 1)              # this rank's partial tile rows go to every peer
                roof = max(wbytes / (args.hbm_gbs * 1e3), link_bytes / (args.nvlink_gbs * 1e3))
                rec["roofline_us"] = round(roof, 2)
                rec["fused_frac_of_roofline"] = round(roof / rec["fused_us"], 3)
                rec["speedup_vs_nccl"] = round(rec["gemm_nccl_add_us"] / rec["fused_us"], 2)
            out.append(rec)
            if rank == 0:
                print(json.dumps(rec), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
