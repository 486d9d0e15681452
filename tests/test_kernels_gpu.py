"""CUDA kernels against plain PyTorch fp32 references of the same op."""
import math

import pytest
import torch

from llaminar_b200.gguf import GGMLType, dequantize, quantize
from llaminar_b200.models.reference import rmsnorm as ref_rmsnorm, rope_split_half

pytestmark = pytest.mark.gpu
DEV = "cuda"
FORMATS = [GGMLType.Q4_K, GGMLType.Q5_K, GGMLType.Q6_K, GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.IQ3_S]


def _weight(qt, n, k, seed=0):
    from llaminar_b200 import ops
    g = torch.Generator(device=DEV).manual_seed(seed)
    w = torch.randn(n, k, generator=g, device=DEV) * 0.05
    raw = quantize(w, qt)
    wf = dequantize(raw, qt, (n, k))
    return ops.pack_matrix(raw, qt, n, k), wf


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12)).item()


@pytest.mark.parametrize("qt", FORMATS)
def test_dequant_matches_codec(qt):
    from llaminar_b200 import ops
    pw, wf = _weight(qt, 200, 512)
    out = ops.dequant(pw)
    torch.cuda.synchronize()
    assert _rel(out, wf) < 6e-3          # bf16 rounding only
    rows = torch.tensor([3, 199, 128, 0, 77], dtype=torch.int32, device=DEV)
    g32 = torch.empty(5, 512, dtype=torch.float32, device=DEV)
    ops.gather_rows(pw, rows, g32)
    assert _rel(g32, wf[rows.long()]) < 6e-3


@pytest.mark.parametrize("qt", FORMATS)
@pytest.mark.parametrize("m", [1, 2, 3, 4])
def test_gemv_plain_and_norm(qt, m):
    from llaminar_b200 import ops
    n, k = 384, 1024
    pw, wf = _weight(qt, n, k, seed=m)
    sc = ops.scratch_for(DEV)
    x = torch.randn(m, k, device=DEV)
    xb = x.to(torch.bfloat16)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    bias = torch.randn(n, device=DEV)
    sc.status.zero_()
    for stream in (True, False):            # the streaming kernel (bulk-copy ring) and the register-path kernel
        for ks in (1, 0, 2):
            out.zero_()
            ops.gemv(pw, xb, out, bias=bias, scratch=sc, ksplit=ks, stream=stream)
            ref = xb.float() @ wf.T + bias
            assert _rel(out, ref) < 2e-2, (qt, m, ks, stream)
        # fused RMSNorm prologue + residual epilogue
        gain = torch.rand(k, device=DEV) + 0.5
        h = torch.randn(m, n, device=DEV)
        h0 = h.clone()
        ops.gemv(pw, x, h, norm_w=gain, eps=1e-6, epi=ops.EPI_RESID, scratch=sc, stream=stream)
        ref = h0 + ref_rmsnorm(x, gain, 1e-6) @ wf.T
        assert _rel(h, ref) < 2e-2, stream
    assert int(sc.status[0]) == 0, "a bounded wait of the streaming kernel ran out"
    assert int(sc.tickets.abs().sum()) == 0 and float(sc.accum.abs().sum()) == 0.0


@pytest.mark.parametrize("shape", [(5120, 8192), (1000, 25600), (10240, 5120), (128, 256), (384, 512)])
@pytest.mark.parametrize("m", [1, 3])
def test_gemv_streaming_split_tiles_match_the_register_path(shape, m):
    """Shapes whose tiles are split between CTAs (long K), ranges that wrap over a tile end, a ragged last tile and problems
    smaller than the grid: the streaming kernel equals the fp32 reference, repeats bit for bit, and leaves its counters at zero."""
    from llaminar_b200 import ops
    n, k = shape
    pw, wf = _weight(GGMLType.Q4_K, n, k, seed=11)
    sc = ops.scratch_for(DEV)
    sc.status.zero_()
    xb = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    ref = xb.float() @ wf.T
    outs = []
    for rep in range(3):
        out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
        ops.gemv(pw, xb, out, scratch=sc)
        outs.append(out)
    old = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    ops.gemv(pw, xb, old, scratch=sc, stream=False)
    torch.cuda.synchronize()
    assert int(sc.status[0]) == 0
    assert _rel(outs[0], ref) < 2e-2
    assert _rel(outs[0], old) < 1e-4              # same int8 activations and dp4a sums, different summation order over chunks
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert int(sc.tickets.abs().sum()) == 0


@pytest.mark.parametrize("qt", [GGMLType.Q4_K, GGMLType.Q8_0])
def test_gemv_swiglu(qt):
    from llaminar_b200 import ops
    from llaminar_b200.ops.layout import interleave_gate_up
    d_ff, k = 256, 512
    g = torch.Generator(device=DEV).manual_seed(5)
    wg = torch.randn(d_ff, k, generator=g, device=DEV) * 0.05
    wu = torch.randn(d_ff, k, generator=g, device=DEV) * 0.05
    rg, ru = quantize(wg, qt), quantize(wu, qt)
    raw, _, n2, _ = interleave_gate_up(rg, ru, qt, d_ff, k)
    pw = ops.pack_matrix(raw, qt, n2, k)
    x = torch.randn(2, k, device=DEV).to(torch.bfloat16)
    out = torch.empty(2, d_ff, dtype=torch.bfloat16, device=DEV)
    gf, uf = dequantize(rg, qt, (d_ff, k)), dequantize(ru, qt, (d_ff, k))
    ref = torch.nn.functional.silu(x.float() @ gf.T) * (x.float() @ uf.T)
    for stream in (True, False):
        out.zero_()
        ops.gemv(pw, x, out, epi=ops.EPI_SWIGLU, scratch=ops.scratch_for(DEV), stream=stream)
        assert _rel(out, ref) < 3e-2, stream


@pytest.mark.parametrize("qt", FORMATS)
@pytest.mark.parametrize("m", [5, 32, 100, 300])
def test_gemm_tc(qt, m):
    from llaminar_b200 import ops
    n, k = 384, 1024
    pw, wf = _weight(qt, n, k, seed=7)
    sc = ops.scratch_for(DEV)
    sc.status.zero_()
    x = (torch.randn(m, k, device=DEV)).to(torch.bfloat16)
    ref = x.float() @ wf.T
    for ks in (1, 2, 0):
        out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
        ops.gemm(pw, x, out, scratch=sc, ksplit=ks)
        torch.cuda.synchronize()
        assert int(sc.status[0]) == 0, "pipeline wait timed out"
        assert _rel(out, ref) < 1.2e-2, (qt, m, ks)
    h = torch.randn(m, n, device=DEV)
    h0 = h.clone()
    bias = torch.randn(n, device=DEV)
    ops.gemm(pw, x, h, epi=ops.EPI_RESID, bias=bias, scratch=sc)
    assert _rel(h, h0 + ref + bias) < 1.2e-2
    assert int(sc.tickets.abs().sum()) == 0 and float(sc.accum.abs().sum()) == 0.0


@pytest.mark.parametrize("qt,m,n,k,ks", [(GGMLType.Q4_K, 2048, 8192, 1024, 1), (GGMLType.Q6_K, 1024, 4096, 2048, 1),
                                          (GGMLType.Q8_0, 600, 2048, 1024, 1), (GGMLType.Q4_K, 48, 4096, 4096, 0),
                                          (GGMLType.IQ3_S, 130, 3072, 768, 0)])
def test_gemm_tc_many_ctas_per_sm(qt, m, n, k, ks):
    """Grids with several waves of CTAs: the producer sets run far ahead of the MMA consumer here."""
    from llaminar_b200 import ops
    pw, wf = _weight(qt, n, k, seed=3)
    sc = ops.scratch_for(DEV)
    sc.status.zero_()
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    for _ in range(3):
        ops.gemm(pw, x, out, scratch=sc, ksplit=ks)
    torch.cuda.synchronize()
    assert int(sc.status[0]) == 0
    assert _rel(out, x.float() @ wf.T) < 1.2e-2


@pytest.mark.parametrize("m", [16, 200])
def test_gemm_tc_swiglu_large_k(m):
    from llaminar_b200 import ops
    from llaminar_b200.ops.layout import interleave_gate_up
    qt, d_ff, k = GGMLType.Q4_K, 512, 4096
    g = torch.Generator(device=DEV).manual_seed(11)
    wg = torch.randn(d_ff, k, generator=g, device=DEV) * 0.03
    wu = torch.randn(d_ff, k, generator=g, device=DEV) * 0.03
    rg, ru = quantize(wg, qt), quantize(wu, qt)
    raw, _, n2, _ = interleave_gate_up(rg, ru, qt, d_ff, k)
    pw = ops.pack_matrix(raw, qt, n2, k)
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    out = torch.empty(m, d_ff, dtype=torch.bfloat16, device=DEV)
    ops.gemm(pw, x, out, epi=ops.EPI_SWIGLU, scratch=ops.scratch_for(DEV))
    gf, uf = dequantize(rg, qt, (d_ff, k)), dequantize(ru, qt, (d_ff, k))
    ref = torch.nn.functional.silu(x.float() @ gf.T) * (x.float() @ uf.T)
    assert _rel(out, ref) < 2e-2


@pytest.mark.parametrize("rows,d", [(37, 1024), (3, 5120), (5, 12288)])
def test_rmsnorm(rows, d):
    """Rows up to 8192 values stay in registers across the reduction; longer rows are read twice."""
    from llaminar_b200 import ops
    h = torch.randn(rows, d, device=DEV)
    w = torch.rand(d, device=DEV) + 0.5
    out = torch.empty(rows, d, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(h, w, out, 1e-6)
    assert _rel(out, ref_rmsnorm(h, w, 1e-6)) < 5e-3


def _paged_setup(B, ctx_lens, n_kv, D, extra_pages=3):
    pages_per = [(c + 63) // 64 for c in ctx_lens]
    max_pages = max(pages_per) + 1
    n_pages = sum(pages_per) + extra_pages + B
    perm = torch.randperm(n_pages)[: B * max_pages].reshape(B, max_pages).to(torch.int32).to(DEV)
    kv = torch.zeros(n_pages, 2, n_kv, 64, D, dtype=torch.bfloat16, device=DEV)
    return kv, perm, max_pages


@pytest.mark.parametrize("D,nq,nkv", [(128, 32, 8), (64, 4, 2), (128, 64, 8)])
def test_rope_kv_and_attention(D, nq, nkv):
    from llaminar_b200 import ops
    torch.manual_seed(0)
    B = 3
    q_lens = [70, 129, 5]
    kv, btab, max_pages = _paged_setup(B, [l + 3 for l in q_lens], nkv, D)
    T = sum(q_lens)
    qkv = (torch.randn(T, (nq + 2 * nkv) * D, device=DEV) * 0.5).to(torch.bfloat16)
    qn = torch.rand(D, device=DEV) + 0.5
    kn = torch.rand(D, device=DEV) + 0.5
    pos = torch.cat([torch.arange(l) for l in q_lens]).to(torch.int32).to(DEV)
    sid = torch.cat([torch.full((l,), i) for i, l in enumerate(q_lens)]).to(torch.int32).to(DEV)
    q_out = torch.empty(T, nq, D, dtype=torch.bfloat16, device=DEV)
    ops.rope_kv(qkv.clone(), q_out, kv, qn, kn, pos, sid, btab, nq, nkv, D, 1e6, 1e-6)
    # reference
    x = qkv.float().view(T, nq + 2 * nkv, D)
    qr = rope_split_half(ref_rmsnorm(x[:, :nq], qn, 1e-6), pos, 1e6)
    kr = rope_split_half(ref_rmsnorm(x[:, nq:nq + nkv], kn, 1e-6), pos, 1e6)
    vr = x[:, nq + nkv:]
    assert _rel(q_out, qr) < 6e-3
    # prefill attention
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    ctx = torch.zeros(B, dtype=torch.int32, device=DEV)
    out = torch.empty(T, nq, D, dtype=torch.bfloat16, device=DEV)
    scale = 1.0 / math.sqrt(D)
    ops.attn_prefill(q_out, kv, out, btab, cu, ctx, nq, nkv, D, scale, max(q_lens))
    g = nq // nkv
    s0 = 0
    for b, L in enumerate(q_lens):
        qb, kb, vb = qr[s0:s0 + L], kr[s0:s0 + L].repeat_interleave(g, 1), vr[s0:s0 + L].repeat_interleave(g, 1)
        sc = torch.einsum("thd,shd->hts", qb, kb) * scale
        mask = torch.ones(L, L, device=DEV).tril().bool()
        sc = sc.masked_fill(~mask[None], float("-inf"))
        ref = torch.einsum("hts,shd->thd", sc.softmax(-1), vb)
        assert _rel(out[s0:s0 + L], ref) < 2e-2, (b, L)
        s0 += L
    # decode: one new token per sequence on top of the cached prompt, R rows
    for R in (1, 2 if g * 2 <= 16 else 1):
        newq = (torch.randn(B * R, (nq + 2 * nkv) * D, device=DEV) * 0.5).to(torch.bfloat16)
        pos2 = torch.cat([torch.arange(L, L + R) for L in q_lens]).to(torch.int32).to(DEV)
        sid2 = torch.arange(B).repeat_interleave(R).to(torch.int32).to(DEV)
        kv2 = kv.clone()
        qd = torch.empty(B * R, nq, D, dtype=torch.bfloat16, device=DEV)
        ops.rope_kv(newq.clone(), qd, kv2, qn, kn, pos2, sid2, btab, nq, nkv, D, 1e6, 1e-6)
        seq_lens = torch.tensor([L + R for L in q_lens], dtype=torch.int32, device=DEV)
        xd = newq.float().view(B * R, nq + 2 * nkv, D)
        qd_ref = rope_split_half(ref_rmsnorm(xd[:, :nq], qn, 1e-6), pos2, 1e6)
        kd_ref = rope_split_half(ref_rmsnorm(xd[:, nq:nq + nkv], kn, 1e-6), pos2, 1e6)
        vd_ref = xd[:, nq + nkv:]
        for splits in (1, 2, 3):
            od = torch.empty(B * R, nq, D, dtype=torch.bfloat16, device=DEV)
            ops.attn_decode(qd, kv2, od, btab, seq_lens, nq, nkv, D, R, scale, splits, ops.scratch_for(DEV))
            s0 = 0
            for b, L in enumerate(q_lens):
                for r in range(R):
                    K = torch.cat([kr[s0:s0 + L], kd_ref[b * R:b * R + r + 1]]).repeat_interleave(g, 1)
                    V = torch.cat([vr[s0:s0 + L], vd_ref[b * R:b * R + r + 1]]).repeat_interleave(g, 1)
                    sc = torch.einsum("hd,shd->hs", qd_ref[b * R + r], K) * scale
                    ref = torch.einsum("hs,shd->hd", sc.softmax(-1), V)
                    assert _rel(od[b * R + r], ref) < 2e-2, (R, splits, b, r)
                s0 += L
        assert int(ops.scratch_for(DEV).attn_tickets.abs().sum()) == 0


@pytest.mark.parametrize("D,nq,nkv", [(128, 32, 8), (64, 4, 2)])
def test_kv_cache_8bit_against_the_bf16_cache(D, nq, nkv):
    """8-bit KV pages (int8 + one fp16 scale per 32 values): the quantising append, the expansion into bf16 staging pages that
    the prefill kernels read, and decode attention straight from the 8-bit pages, each against the bf16 cache."""
    from llaminar_b200 import ops
    torch.manual_seed(1)
    B, q_lens = 3, [70, 129, 5]
    kv, btab, max_pages = _paged_setup(B, [l + 3 for l in q_lens], nkv, D)
    data = 2 * nkv * 64 * D
    kv8 = torch.zeros(kv.shape[0], data + data // 16, dtype=torch.uint8, device=DEV)
    T = sum(q_lens)
    qkv = (torch.randn(T, (nq + 2 * nkv) * D, device=DEV) * 0.5).to(torch.bfloat16)
    qn, kn = torch.rand(D, device=DEV) + 0.5, torch.rand(D, device=DEV) + 0.5
    pos = torch.cat([torch.arange(l) for l in q_lens]).to(torch.int32).to(DEV)
    sid = torch.cat([torch.full((l,), i) for i, l in enumerate(q_lens)]).to(torch.int32).to(DEV)
    q_a = torch.empty(T, nq, D, dtype=torch.bfloat16, device=DEV)
    q_b = torch.empty_like(q_a)
    ops.rope_kv(qkv.clone(), q_a, kv, qn, kn, pos, sid, btab, nq, nkv, D, 1e6, 1e-6)
    ops.rope_kv(qkv.clone(), q_b, kv8, qn, kn, pos, sid, btab, nq, nkv, D, 1e6, 1e-6)
    assert torch.equal(q_a, q_b)
    # expansion of the sequences' pages: staging page s * max_pages + j holds page btab[s, j]
    n_tok = torch.tensor(q_lens, dtype=torch.int32, device=DEV)
    staging = torch.zeros(B * max_pages, 2, nkv, 64, D, dtype=torch.bfloat16, device=DEV)
    ops.kv_dequant_pages(kv8, btab, n_tok, nkv, D, staging)
    for b, L in enumerate(q_lens):
        for j in range((L + 63) // 64):
            ref = kv[int(btab[b, j])].float()
            got = staging[b * max_pages + j].float()
            assert _rel(got, ref) < 8e-3, (b, j)                     # half a step of 1/127 of each block's largest value
    # prefill attention over the staging pool against the bf16 cache
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    ctx = torch.zeros(B, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    o_a = torch.empty(T, nq, D, dtype=torch.bfloat16, device=DEV)
    o_b = torch.empty_like(o_a)
    bt2 = torch.arange(B * max_pages, dtype=torch.int32, device=DEV).view(B, max_pages)
    ops.attn_prefill(q_a, kv, o_a, btab, cu, ctx, nq, nkv, D, scale, max(q_lens))
    ops.attn_prefill(q_a, staging, o_b, bt2, cu, ctx, nq, nkv, D, scale, max(q_lens))
    assert _rel(o_b, o_a.float()) < 1.5e-2
    # decode straight from the 8-bit pages, one and two rows per sequence, with and without splits
    g = nq // nkv
    for R in (1, 2 if g * 2 <= 16 else 1):
        newq = (torch.randn(B * R, (nq + 2 * nkv) * D, device=DEV) * 0.5).to(torch.bfloat16)
        pos2 = torch.cat([torch.arange(L, L + R) for L in q_lens]).to(torch.int32).to(DEV)
        sid2 = torch.arange(B).repeat_interleave(R).to(torch.int32).to(DEV)
        kv_a, kv_b = kv.clone(), kv8.clone()
        qd = torch.empty(B * R, nq, D, dtype=torch.bfloat16, device=DEV)
        ops.rope_kv(newq.clone(), qd, kv_a, qn, kn, pos2, sid2, btab, nq, nkv, D, 1e6, 1e-6)
        ops.rope_kv(newq.clone(), qd, kv_b, qn, kn, pos2, sid2, btab, nq, nkv, D, 1e6, 1e-6)
        seq_lens = torch.tensor([L + R for L in q_lens], dtype=torch.int32, device=DEV)
        for splits in (1, 3):
            od_a = torch.empty(B * R, nq, D, dtype=torch.bfloat16, device=DEV)
            od_b = torch.empty_like(od_a)
            ops.attn_decode(qd, kv_a, od_a, btab, seq_lens, nq, nkv, D, R, scale, splits, ops.scratch_for(DEV))
            ops.attn_decode(qd, kv_b, od_b, btab, seq_lens, nq, nkv, D, R, scale, splits, ops.scratch_for(DEV))
            assert _rel(od_b, od_a.float()) < 1.5e-2, (R, splits)
    assert int(ops.scratch_for(DEV).attn_tickets.abs().sum()) == 0


@pytest.mark.parametrize("nq,nkv,q_lens,ctx_lens", [(8, 2, [70, 129, 5], [0, 0, 0]), (4, 4, [300, 128], [0, 64]),
                                                     (16, 2, [257, 40, 1], [200, 131, 513])])
def test_prefill_attention_tcgen05(nq, nkv, q_lens, ctx_lens):
    """tcgen05 prefill attention (head_dim 128) against an fp32 reference, with and without a cached prefix."""
    from llaminar_b200 import ops
    torch.manual_seed(2)
    D, B = 128, len(q_lens)
    tot = [c + l for c, l in zip(ctx_lens, q_lens)]
    max_pages = max((t + 63) // 64 for t in tot) + 1
    n_pages = B * max_pages + 3
    btab = torch.randperm(n_pages)[: B * max_pages].reshape(B, max_pages).to(torch.int32).to(DEV)
    kv = torch.zeros(n_pages, 2, nkv, 64, D, dtype=torch.bfloat16, device=DEV)
    # fill the cache with every sequence's keys / values (prefix and this chunk)
    ks = [(torch.randn(t, nkv, D, device=DEV) * 0.7) for t in tot]
    vs = [(torch.randn(t, nkv, D, device=DEV) * 0.7) for t in tot]
    for b in range(B):
        for t in range(tot[b]):
            page = int(btab[b, t // 64])
            kv[page, 0, :, t % 64] = ks[b][t].to(torch.bfloat16)
            kv[page, 1, :, t % 64] = vs[b][t].to(torch.bfloat16)
    T = sum(q_lens)
    q = (torch.randn(T, nq, D, device=DEV) * 0.7).to(torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    ctx = torch.tensor(ctx_lens, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    sc = ops.scratch_for(DEV)
    out_tc = torch.zeros(T, nq, D, dtype=torch.bfloat16, device=DEV)
    out_old = torch.zeros_like(out_tc)
    ops.attn_prefill(q, kv, out_tc, btab, cu, ctx, nq, nkv, D, scale, max(q_lens), tensor_core=True, scratch=sc)
    ops.attn_prefill(q, kv, out_old, btab, cu, ctx, nq, nkv, D, scale, max(q_lens), tensor_core=False)
    torch.cuda.synchronize()
    assert int(sc.status[0]) == 0
    g = nq // nkv
    s0 = 0
    for b, L in enumerate(q_lens):
        C = ctx_lens[b]
        kb = ks[b].to(torch.bfloat16).float().repeat_interleave(g, 1)
        vb = vs[b].to(torch.bfloat16).float().repeat_interleave(g, 1)
        qb = q[s0:s0 + L].float()
        scr = torch.einsum("thd,shd->hts", qb, kb) * scale
        mask = (torch.arange(C + L, device=DEV)[None, :] <= (C + torch.arange(L, device=DEV))[:, None])
        scr = scr.masked_fill(~mask[None], float("-inf"))
        ref = torch.einsum("hts,shd->thd", scr.softmax(-1), vb)
        assert _rel(out_old[s0:s0 + L], ref) < 2e-2, ("mma.sync", b, L)
        assert _rel(out_tc[s0:s0 + L], ref) < 2e-2, ("tcgen05", b, L, _rel(out_tc[s0:s0 + L], ref))
        s0 += L


def test_sampling_kernels():
    from llaminar_b200 import ops
    torch.manual_seed(0)
    rows, vocab = 6, 5000
    logits = torch.randn(rows, vocab, device=DEV) * 3
    tok = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.argmax(logits, tok)
    assert tok.tolist() == logits.argmax(-1).tolist()
    temp = torch.tensor([0.0, 1.0, 0.7, 1.0, 1.0, 1.0], device=DEV)
    top_k = torch.tensor([0, 1, 5, 50, 0, 40], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1.0, 1.0, 1.0, 0.5, 0.9, 0.9], device=DEV)
    seeds = torch.arange(rows, dtype=torch.int64, device=DEV) + 123
    probs = torch.empty(rows, vocab, device=DEV)
    counts = torch.zeros(rows, vocab, device=DEV)
    for step in range(200):
        st = torch.full((rows,), step, dtype=torch.int32, device=DEV)
        ops.sample(logits, temp, top_k, top_p, seeds, st, tok, probs)
        counts[torch.arange(rows), tok.long()] += 1
    am = logits.argmax(-1)
    assert counts[0, am[0]] == 200 and counts[1, am[1]] == 200          # greedy rows
    assert (counts[2] > 0).sum() <= 5                                   # top-k 5
    top5 = logits[2].topk(5).indices
    assert counts[2, top5].sum() == 200
    # distribution returned for row 2 equals softmax over the top-5 at temperature 0.7
    ref = torch.zeros(vocab, device=DEV)
    ref[top5] = torch.softmax(logits[2, top5] / 0.7, -1)
    assert torch.allclose(probs[2], ref, atol=1e-4)
    assert abs(probs[3].sum().item() - 1) < 1e-4 and abs(probs[4].sum().item() - 1) < 1e-4
    # top-p 0.5 over top-50: kept set is the smallest prefix reaching 0.5 mass
    srt = torch.softmax(logits[3].topk(50).values, -1)
    n_keep = int((srt.cumsum(0) - srt < 0.5).sum())
    assert int((probs[3] > 0).sum()) == n_keep
    emp = counts[5] / 200
    assert (emp - probs[5]).abs().max() < 0.15


def test_sharded_sampling_draws_the_same_token_as_the_full_row():
    """Per-shard candidates + merged draw (what tensor-parallel ranks do) against one launch over the whole vocabulary."""
    from llaminar_b200 import ops
    torch.manual_seed(1)
    rows, vocab, shards = 5, 6000, 4
    logits = torch.randn(rows, vocab, device=DEV) * 2
    logits[0, 17] = logits[0, 4000] = logits[0].max() + 1          # a tie across two shards: the lower token id must win
    temp = torch.tensor([0.0, 1.0, 0.8, 1.0, 1.3], device=DEV)
    top_k = torch.tensor([0, 0, 7, 50, 1000], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1.0, 0.9, 1.0, 0.6, 0.95], device=DEV)
    seeds = torch.arange(rows, dtype=torch.int64, device=DEV) + 7
    per = vocab // shards
    kc = 1024
    full, merged = torch.empty(rows, dtype=torch.int32, device=DEV), torch.empty(rows, dtype=torch.int32, device=DEV)
    gathered = torch.zeros(shards, rows, kc, 2, dtype=torch.int32, device=DEV)
    for step in range(40):
        st = torch.full((rows,), step, dtype=torch.int32, device=DEV)
        ops.sample(logits, temp, top_k, top_p, seeds, st, full)
        for s in range(shards):
            ops.sample_candidates(logits[:, s * per:(s + 1) * per], s * per, gathered[s])
        ops.sample_merged(gathered, temp, top_k, top_p, seeds, st, merged)
        assert merged.tolist() == full.tolist(), step
    assert full[0].item() == 17
    # the candidates of a shard are its best entries, best first, with global token ids
    vals = gathered[1, 2, :, 0].view(torch.float32)
    ref = logits[2, per:2 * per].topk(kc)
    assert torch.equal(vals, ref.values) and gathered[1, 2, :8, 1].tolist() == (ref.indices[:8] + per).tolist()


def test_spec_verify_and_moe_topk_and_nan_scan():
    from llaminar_b200 import ops
    draft = torch.tensor([[5, 6], [5, 9], [1, 2]], dtype=torch.int32, device=DEV)
    target = torch.tensor([[5, 6, 7], [5, 6, 7], [9, 9, 9]], dtype=torch.int32, device=DEV)
    na = torch.empty(3, dtype=torch.int32, device=DEV)
    ot = torch.empty(3, 3, dtype=torch.int32, device=DEV)
    ops.spec_verify_greedy(draft, target, na, ot)
    assert na.tolist() == [2, 1, 0]
    assert ot.tolist() == [[5, 6, 7], [5, 6, -1], [9, -1, -1]]
    # rejection sampling: identical distributions always accept; disjoint support always rejects
    B, d, V = 4, 2, 300
    pt = torch.softmax(torch.randn(B, d + 1, V, device=DEV), -1)
    pd = pt[:, :d].clone().contiguous()
    dr = pd.argmax(-1).to(torch.int32)
    seeds = torch.arange(B, dtype=torch.int64, device=DEV)
    step = torch.zeros(B, dtype=torch.int32, device=DEV)
    na = torch.empty(B, dtype=torch.int32, device=DEV)
    ot = torch.empty(B, d + 1, dtype=torch.int32, device=DEV)
    ops.spec_verify_reject(pt.contiguous(), pd, dr, seeds, step, na, ot)
    assert na.tolist() == [d] * B and (ot[:, :d] == dr).all() and (ot[:, d] >= 0).all()
    pd2 = torch.zeros(B, d, V, device=DEV); pd2[:, :, 0] = 1.0
    pt2 = torch.zeros(B, d + 1, V, device=DEV); pt2[:, :, 7] = 1.0
    dr2 = torch.zeros(B, d, dtype=torch.int32, device=DEV)
    ops.spec_verify_reject(pt2, pd2, dr2, seeds, step, na, ot)
    assert na.tolist() == [0] * B and ot[:, 0].tolist() == [7] * B
    # MoE router
    from llaminar_b200.models.reference import moe_route
    lg = torch.randn(33, 128, device=DEV)
    lg[0, 5] = lg[0, 9] = 10.0          # tie -> lower id first
    ids = torch.empty(33, 8, dtype=torch.int32, device=DEV)
    wts = torch.empty(33, 8, device=DEV)
    cnt = torch.zeros(128, dtype=torch.int32, device=DEV)
    ops.moe_topk(lg, 8, True, ids, wts, cnt)
    rid, rw = moe_route(lg, 8, True)
    assert (ids.long() == rid).all() and torch.allclose(wts, rw, atol=1e-5) and int(cnt.sum()) == 33 * 8
    x = torch.randn(1000, device=DEV); x[3] = float("nan"); x[10] = float("inf"); x[11] = -float("inf")
    assert ops.nan_scan(x) == (1, 2)
    assert ops.nan_scan(torch.ones(64, device=DEV).to(torch.bfloat16)) == (0, 0)


@pytest.mark.parametrize("tokens,qt_name", [(1, "IQ3_S"), (7, "IQ3_S"), (64, "IQ3_S"), (33, "Q4_K")])
def test_moe_fused_route_gate_up_down_combine(tokens, qt_name):
    """Router + grouped expert GEMVs + weighted combine against a plain fp32 restatement (single rank: no all-reduce)."""
    from llaminar_b200 import ops
    from llaminar_b200.models.reference import moe_route
    from llaminar_b200.ops.layout import interleave_gate_up, pack_experts
    dev = torch.device("cuda")
    E, k, d, ff = 128, 8, 2048, 768
    e0, n_local = 32, 48                                  # this "rank" owns experts 32..79
    qt = GGMLType[qt_name]
    g = torch.Generator(device=dev).manual_seed(7)
    h = torch.randn(tokens, d, device=dev, generator=g)
    norm_w = 1.0 + 0.1 * torch.randn(d, device=dev, generator=g)
    router = (torch.randn(E, d, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    wg = torch.randn(n_local, ff, d, device=dev, generator=g) * 0.05
    wu = torch.randn(n_local, ff, d, device=dev, generator=g) * 0.05
    wd = torch.randn(n_local, d, ff, device=dev, generator=g) * 0.05
    gu_raw, dn_raw, wg_q, wu_q, wd_q = [], [], [], [], []
    for e in range(n_local):
        rg, ru, rd = quantize(wg[e], qt), quantize(wu[e], qt), quantize(wd[e], qt)
        wg_q.append(dequantize(rg, qt, (ff, d))); wu_q.append(dequantize(ru, qt, (ff, d))); wd_q.append(dequantize(rd, qt, (d, ff)))
        gu_raw.append(interleave_gate_up(rg, ru, qt, ff, d)[0])
        dn_raw.append(rd)
    gate_up = pack_experts(torch.cat(gu_raw), qt, n_local, 2 * ff, d)
    down = pack_experts(torch.cat(dn_raw), qt, n_local, d, ff)
    z_max = n_local + (tokens * k + 3) // 4
    zi = lambda *s, dt=torch.int32: torch.zeros(*s, dtype=dt, device=dev)
    ids, wts = zi(tokens, k), zi(tokens, k, dt=torch.float32)
    items, n_items, ticket, counts = zi(z_max * ops.MOE_ITEM_INTS), zi(1), zi(1), zi(n_local)
    act = zi(tokens * k, ff, dt=torch.bfloat16)
    yslot = zi(tokens * k, d, dt=torch.float32)
    tile_tickets = zi(d // 128)
    sc = ops.scratch_for(dev)
    eps = 1e-6
    for rep in range(2):                                  # second pass: tickets and counters were returned to zero
        hh = h.clone()
        ops.moe_route(hh, norm_w, eps, router, k, True, e0, n_local, ids, wts, items, n_items, ticket, counts)
        ops.moe_gate_up(gate_up, hh, norm_w, eps, act, items, n_items, k, z_max, scratch=sc)
        ops.moe_down_combine(down, act, yslot, items, n_items, z_max, ids, wts, k, e0, n_local, hh, tile_tickets, scratch=sc)
        torch.cuda.synchronize()
        xn = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * norm_w
        logits = xn @ router.float().T
        rid, rw = moe_route(logits, k, True)
        same = (rid.sort(-1).values == ids.long().sort(-1).values).float().mean().item()
        assert same > 0.98                                # a near-tie at the k-th place may resolve differently
        assert torch.allclose(wts.sum(-1), torch.ones(tokens, device=dev), atol=1e-4)
        # expert math on the kernel's own routing
        ref = h.clone()
        for t in range(tokens):
            for j in range(k):
                e = int(ids[t, j]) - e0
                if 0 <= e < n_local:
                    a = torch.nn.functional.silu(wg_q[e] @ xn[t]) * (wu_q[e] @ xn[t])
                    ref[t] += float(wts[t, j]) * (wd_q[e] @ a)
        delta, rdelta = hh - h, ref - h
        assert (delta - rdelta).norm() / rdelta.norm().clamp_min(1e-6) < 3e-2
        local_pairs = int(((ids >= e0) & (ids < e0 + n_local)).sum())
        assert int(counts.sum()) == local_pairs
        assert int(n_items) >= max(1, (local_pairs + 3) // 4) and int(ticket) == 0 and int(tile_tickets.sum()) == 0


@pytest.mark.parametrize("rows", [2, 32])
def test_fused_allreduce_wait_runs_out_and_reports(rows):
    """The bounded wait of the fused tensor-parallel epilogue, made to run out on ONE GPU: a descriptor of two ranks whose
    'peer' buffers are local memory that nothing ever signals.  The kernel must come back by itself with STATUS_TIMEOUT in
    the status word, leave the residual rows alone, and the same engine-side check that runs after every step must raise
    and reset the scratch; an ordinary call afterwards is clean."""
    from llaminar_b200 import ops
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.parallel.symm import tp_fuse_blob
    n, k, n_cap, rows_cap = 256, 1024, 256, 32
    pw, wf = _weight(GGMLType.Q4_K, n, k, seed=3)
    sc = ops.scratch_for(DEV)
    sc.reset()
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=DEV)
    inbox = [z(2 * 2 * rows_cap * n_cap) for _ in range(2)]
    flags = [z(64, dt=torch.int32) for _ in range(2)]
    epoch, status = z(64, dt=torch.int32), z(4, dt=torch.int32)
    blob = tp_fuse_blob(inbox=[t.data_ptr() for t in inbox], flags=[t.data_ptr() for t in flags], epoch_ptr=epoch.data_ptr(),
                        status_ptr=status.data_ptr(), rank=0, size=2, rows_cap=rows_cap, n_cap=n_cap, spin_limit=20000,
                        epoch2_ptr=epoch.data_ptr() + 32 * 4)
    desc = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(DEV)
    x = torch.randn(rows, k, device=DEV).to(torch.bfloat16)
    h0 = torch.randn(rows, n, device=DEV)
    h = h0.clone()
    (ops.gemv if rows <= 4 else ops.gemm)(pw, x, h, epi=ops.EPI_RESID, scratch=sc, tp=desc)
    torch.cuda.synchronize()
    assert int(status[0]) == 1                                   # STATUS_TIMEOUT
    assert torch.equal(h, h0)                                    # no tile was added without its peer's share
    assert int(flags[0][0]) == 1 and int(flags[1][0]) == 1       # this rank did signal both inboxes, once per tile

    class _Model:                                                # the part of an engine that the health check reads
        scratch = sc

    class _Symm:
        pass
    eng = LLMEngine.__new__(LLMEngine)
    eng.is_cuda, eng.device, eng.model = True, torch.device(DEV), _Model()
    eng.tp = type("TP", (), {"symm": _Symm(), "size": 1, "group": None})()
    eng.tp.symm.status = status
    sc.status.zero_()
    with pytest.raises(RuntimeError, match="bounded wait"):
        eng.check_health()
    assert int(status[0]) == 0 and int(sc.tickets.abs().sum()) == 0 and float(sc.accum.abs().sum()) == 0.0
    eng.check_health()                                           # nothing left to report
    out = torch.zeros(rows, n, dtype=torch.bfloat16, device=DEV)
    (ops.gemv if rows <= 4 else ops.gemm)(pw, x, out, scratch=sc)
    torch.cuda.synchronize()
    assert _rel(out.float(), x.float() @ wf.T) < 2e-2 and int(sc.status[0]) == 0


@pytest.mark.parametrize("tokens,qt_name", [(300, "IQ3_S"), (1000, "Q4_K"), (70, "IQ3_S")])
def test_moe_grouped_prefill_matches_fp32_reference(tokens, qt_name):
    """Prefill-sized MoE block on the device-side grouped path (route, sort by expert, two grouped tensor-core GEMMs, ordered
    combine; no host round trip) against an fp32 evaluation of the same routing decisions on the dequantised experts."""
    from llaminar_b200 import ops
    from llaminar_b200.engine.cuda_model import CudaModel, _expert_view_for_tests
    from llaminar_b200.engine import moe as moe_mod
    from llaminar_b200.models.config import SHAPES, QuantRecipe
    from llaminar_b200.models.synth import synthesize
    cfg = SHAPES["tiny-qwen3moe"].with_(d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, expert_ff=256, n_experts=16,
                                        n_experts_used=4, n_layers=1)
    recipe = QuantRecipe(GGMLType.Q4_K, {"_exps": GGMLType[qt_name], "output.weight": GGMLType.Q6_K, "ffn_gate_inp": GGMLType.F32}, "test")
    w = synthesize(cfg, recipe, seed=3)
    model = CudaModel(w, DEV, max_tokens=1024)
    L = model.layers[0]
    k, ff, d = cfg.n_experts_used, cfg.expert_ff, cfg.d_model
    h0 = torch.randn(tokens, d, device=DEV)
    h = h0.clone()
    moe_mod.moe_forward_grouped(model, L, h, tokens)
    # the same routing, evaluated in fp32
    ids = torch.empty(tokens, k, dtype=torch.int32, device=DEV)
    wts = torch.empty(tokens, k, dtype=torch.float32, device=DEV)
    xn = torch.empty(tokens, d, dtype=torch.bfloat16, device=DEV)
    ops.moe_route_only(h0, L.ffn_norm, cfg.rms_eps, L.router, k, cfg.norm_topk_prob, ids, wts, xn)
    ref = torch.zeros(tokens, d, device=DEV)
    x32 = xn.float()
    for e in range(cfg.n_experts):
        gu = ops.dequant(_expert_view_for_tests(L.experts.gate_up, e)).float().view(2 * ff // 32, 2, 16, d)     # 16 gate rows, 16 up rows
        gate, up = gu[:, 0].reshape(ff, d), gu[:, 1].reshape(ff, d)
        dn = ops.dequant(_expert_view_for_tests(L.experts.down, e)).float()
        sel = (ids == e)
        rows = sel.any(1).nonzero().view(-1)
        if rows.numel() == 0:
            continue
        xe = x32[rows]
        act = (torch.nn.functional.silu(xe @ gate.T) * (xe @ up.T)).to(torch.bfloat16).float()
        ye = act @ dn.T
        ref[rows] += ye * (wts * sel)[rows].sum(1, keepdim=True)
    torch.cuda.synchronize()
    assert _rel(h - h0, ref) < 2e-2
    assert torch.isfinite(h).all()
