"""Tensor parallelism on real GPUs: fused peer-memory all-reduce epilogues against NCCL and a dense reference."""
import pytest
import torch

from tests.mp_utils import run_ranks_gpu

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _fused_kernels(rank, world, qt_name, rows):
    """Row-parallel x @ W^T with K split over ranks; h += sum of partials through the fused epilogue."""
    import torch.distributed as dist
    from llaminar_b200 import ops
    from llaminar_b200.gguf import GGMLType, dequantize, quantize
    from llaminar_b200.parallel.tp import TPContext
    dev = torch.device("cuda", rank)
    tp = TPContext.create(device=dev, fused=True)
    qt = GGMLType[qt_name]
    n, k = 640, 1024 * world
    g = torch.Generator(device=dev).manual_seed(1)          # same seed -> identical tensors on every rank
    w = torch.randn(n, k, device=dev, generator=g) * 0.05
    x = torch.randn(rows, k, device=dev, generator=g).to(torch.bfloat16)
    h0 = torch.randn(rows, n, device=dev, generator=g)
    ks, ke = rank * 1024, (rank + 1) * 1024
    raw = quantize(w[:, ks:ke].contiguous(), qt)
    pw = ops.pack_matrix(raw, qt, n, 1024)
    wf_full = torch.cat([dequantize(quantize(w[:, r * 1024:(r + 1) * 1024].contiguous(), qt), qt, (n, 1024)) for r in range(world)], 1)
    ref = h0 + x.float() @ wf_full.T
    sc = ops.scratch_for(dev)
    errs = []
    xs = x[:, ks:ke].contiguous()
    for call in range(5):                                       # several calls: epochs / parities advance
        h = h0.clone()
        if rows <= 4:
            ops.gemv(pw, xs, h, epi=ops.EPI_RESID, scratch=sc, tp=tp.symm.desc)
        else:
            ops.gemm(pw, xs, h, epi=ops.EPI_RESID, scratch=sc, tp=tp.symm.desc)
        torch.cuda.synchronize()
        tp.symm.check_status()
        errs.append(((h - ref).norm() / ref.norm()).item())
        # every rank must hold bit-identical results
        gathered = [torch.empty_like(h) for _ in range(world)]
        dist.all_gather(gathered, h)
        assert all(torch.equal(gathered[0], t) for t in gathered)
    return max(errs)


@pytest.mark.parametrize("qt_name,rows", [("Q4_K", 1), ("Q6_K", 4), ("Q4_K", 32), ("Q8_0", 17)])
def test_fused_row_parallel_allreduce_2gpu(qt_name, rows):
    _need(2)
    errs = run_ranks_gpu(_fused_kernels, 2, qt_name, rows)
    assert max(errs) < 2e-2


def _engine_tokens(rank, world, fused):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.tp import TPContext
    dev = torch.device("cuda", rank)
    cfg = SHAPES["tiny-qwen3"].with_(d_model=1024, n_heads=8, n_kv_heads=2, head_dim=128, d_ff=2048, n_layers=2)
    w = synthesize(cfg, "Q4_K_M", seed=0)
    tp = TPContext.create(device=dev, fused=fused)
    eng = LLMEngine(w, device=dev, max_batch=8, max_context=256, tp=tp)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (40, 9, 70, 21, 64, 5)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    return outs, dict(tp.stats)


def test_engine_tp2_fused_equals_nccl_baseline():
    _need(2)
    fused = run_ranks_gpu(_engine_tokens, 2, True)
    base = run_ranks_gpu(_engine_tokens, 2, False)
    assert fused[0][0] == fused[1][0] and base[0][0] == base[1][0]
    assert fused[0][1]["fused_calls"] > 0 and base[0][1]["fused_calls"] == 0
    agree = sum(a == b for fo, bo in zip(fused[0][0], base[0][0]) for a, b in zip(fo, bo))
    assert agree >= 0.9 * 48            # different summation order may flip a near-tie


def _engine_sampled_tokens(rank, world):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.tp import TPContext
    dev = torch.device("cuda", rank)
    cfg = SHAPES["tiny-qwen3"].with_(d_model=1024, n_heads=8, n_kv_heads=2, head_dim=128, d_ff=2048, n_layers=2)
    w = synthesize(cfg, "Q4_K_M", seed=0)
    tp = TPContext.create(device=dev, fused=True)
    eng = LLMEngine(w, device=dev, max_batch=8, max_context=256, tp=tp)
    calls = [0]
    inner = eng._sharded_sample
    def counted(*a, **k):
        calls[0] += 1
        return inner(*a, **k)
    eng._sharded_sample = counted
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (30, 12, 50)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.9, top_k=40, top_p=0.95, seed=11, max_tokens=12, ignore_eos=True))
    eng.check_health()
    return outs, calls[0], cfg.vocab_size


def test_engine_tp2_sampled_decode_uses_candidate_merge():
    _need(2)
    res = run_ranks_gpu(_engine_sampled_tokens, 2)
    assert res[0][0] == res[1][0]                       # every rank drew the same tokens
    assert res[0][1] > 0                                # through the per-shard candidate path (graph capture calls it)
    assert all(0 <= t < res[0][2] for o in res[0][0] for t in o) and all(len(o) == 12 for o in res[0][0])


def _moe_engine_tokens(rank, world, fused, moe_mode="expert-parallel", lens=(40, 9, 70, 21, 64, 5)):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.tp import TPContext
    dev = torch.device("cuda", rank)
    cfg = SHAPES["tiny-qwen3moe"].with_(d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, expert_ff=256, n_experts=16,
                                        n_experts_used=4, n_layers=2)
    w = synthesize(cfg, "Q4_K_M", seed=0)
    tp = TPContext.create(device=dev, fused=fused)
    tp.moe_mode = moe_mode
    eng = LLMEngine(w, device=dev, max_batch=8, max_context=max(256, max(lens) + 64), max_prefill_tokens=4096, tp=tp)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    eng.check_health()
    return outs, dict(tp.stats)


def test_engine_moe_all_to_all_dispatch_matches_the_dense_all_reduce_2gpu():
    """`--moe-expert-mode expert-parallel-a2a`: token-sharded routing, NCCL all-to-all dispatch and return, grouped expert
    GEMMs on the received rows; the tokens agree with the default expert-parallel mode (dense all-reduce of partial rows)."""
    _need(2)
    lens = (400, 90, 700, 210)                       # 1400 prompt rows x top-4 = 5600 pairs in one prefill chunk: above the threshold
    a2a = run_ranks_gpu(_moe_engine_tokens, 2, False, "expert-parallel-a2a", lens)
    base = run_ranks_gpu(_moe_engine_tokens, 2, False, "expert-parallel", lens)
    assert a2a[0][0] == a2a[1][0]
    assert a2a[0][1].get("a2a_calls", 0) > 0 and base[0][1].get("a2a_calls", 0) == 0
    agree = sum(x == y for fo, bo in zip(a2a[0][0], base[0][0]) for x, y in zip(fo, bo))
    assert agree >= 0.85 * 32


def test_engine_moe_expert_parallel_fused_combine_2gpu():
    """Expert parallelism over 2 GPUs: the grouped down-projection's epilogue combines and all-reduces over peer memory."""
    _need(2)
    fused = run_ranks_gpu(_moe_engine_tokens, 2, True)
    base = run_ranks_gpu(_moe_engine_tokens, 2, False)
    assert fused[0][0] == fused[1][0] and base[0][0] == base[1][0]
    assert fused[0][1]["fused_calls"] > base[0][1]["fused_calls"]
    agree = sum(a == b for fo, bo in zip(fused[0][0], base[0][0]) for a, b in zip(fo, bo))
    assert agree >= 0.85 * 48


def _allgather_gemm(rank, world, qt_name, m_total, n, k):
    """Column-parallel GEMM on row-sharded input: every rank must get gather(x) @ W_shard^T for all rows."""
    import torch.distributed as dist
    from llaminar_b200 import ops
    from llaminar_b200.gguf import GGMLType, dequantize, quantize
    from llaminar_b200.parallel.symm import AllGatherArena
    dev = torch.device("cuda", rank)
    qt = GGMLType[qt_name]
    rows_per_rank = (m_total + world - 1) // world
    arena = AllGatherArena(dist.group.WORLD, dev, rows_cap=rows_per_rank, k_cap=k, copy_ctas=4)
    g = torch.Generator(device=dev).manual_seed(11)                  # same seed: every rank can build the reference
    x_full = (torch.randn(m_total, k, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    g2 = torch.Generator(device=dev).manual_seed(100 + rank)         # each rank owns different weight columns
    w = torch.randn(n, k, device=dev, generator=g2) * 0.05
    raw = quantize(w, qt)
    pw = ops.pack_matrix(raw, qt, n, k)
    wq = dequantize(raw, qt, (n, k))
    errs = []
    for call in range(4):                                            # parities alternate, epochs advance
        xs = (x_full.float() * (1.0 + 0.25 * call)).to(torch.bfloat16)
        r0, r1 = rank * rows_per_rank, min(m_total, (rank + 1) * rows_per_rank)
        arena.own_rows(r1 - r0, k).copy_(xs[r0:r1])
        out = torch.zeros(m_total, n, device=dev)
        arena.gemm(pw, m_total, rows_per_rank, out)
        torch.cuda.synchronize()
        arena.check_status()
        ref = xs.float() @ wq.T
        errs.append(((out - ref).norm() / ref.norm()).item())
    return max(errs)


@pytest.mark.parametrize("qt_name,m_total,n,k", [("Q4_K", 512, 640, 1024), ("Q6_K", 333, 256, 512), ("Q4_K", 2048, 1280, 2048)])
def test_allgather_gemm_2gpu(qt_name, m_total, n, k):
    _need(2)
    errs = run_ranks_gpu(_allgather_gemm, 2, qt_name, m_total, n, k)
    assert max(errs) < 2e-2


@pytest.mark.parametrize("qt_name,rows", [("Q4_K", 32), ("Q6_K", 17), ("Q4_K", 2)])
def test_fused_row_parallel_allreduce_4gpu_two_phase(qt_name, rows):
    """Groups of four: batches of >= 16 rows take the reduce-scatter + all-gather epilogue, small ones the one-shot push."""
    _need(4)
    errs = run_ranks_gpu(_fused_kernels, 4, qt_name, rows)
    assert max(errs) < 2e-2


def _skipped_call(rank, world):
    """Rank 1 leaves out one fused call between steps: rank 0's bounded wait runs out and returns with a status (no rank
    exits, nothing faults); after `resync()` the next fused call is correct on both ranks."""
    import torch.distributed as dist
    from llaminar_b200 import ops
    from llaminar_b200.gguf import GGMLType, dequantize, quantize
    from llaminar_b200.parallel.symm import SymmetricArena
    dev = torch.device("cuda", rank)
    arena = SymmetricArena(dist.group.WORLD, dev, n_cap=1024, spin_limit=200_000)     # a fraction of a second
    qt = GGMLType.Q4_K
    n, rows = 640, 8
    g = torch.Generator(device=dev).manual_seed(1)
    w = torch.randn(n, 1024 * world, device=dev, generator=g) * 0.05
    x = torch.randn(rows, 1024 * world, device=dev, generator=g).to(torch.bfloat16)
    h0 = torch.randn(rows, n, device=dev, generator=g)
    ks = rank * 1024
    pw = ops.pack_matrix(quantize(w[:, ks:ks + 1024].contiguous(), qt), qt, n, 1024)
    wf = torch.cat([dequantize(quantize(w[:, r * 1024:(r + 1) * 1024].contiguous(), qt), qt, (n, 1024)) for r in range(world)], 1)
    ref = h0 + x.float() @ wf.T
    xs = x[:, ks:ks + 1024].contiguous()
    sc = ops.scratch_for(dev)

    def call():
        h = h0.clone()
        ops.gemm(pw, xs, h, epi=ops.EPI_RESID, scratch=sc, tp=arena.desc)
        torch.cuda.synchronize()
        return h
    ok0 = ((call() - ref).norm() / ref.norm()).item()
    dist.barrier()
    timed_out = False
    if rank == 0:                                   # rank 1 skips this call
        h = call()
        timed_out = int(arena.status[0]) == 1 and torch.equal(h, h0)
    dist.barrier()
    arena.resync()
    sc.reset()
    ok1 = ((call() - ref).norm() / ref.norm()).item()
    return ok0, timed_out, ok1, int(arena.status[0])


def test_skipped_fused_call_times_out_and_resync_recovers_2gpu(monkeypatch):
    _need(2)
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    res = run_ranks_gpu(_skipped_call, 2)
    assert res[0][0] < 2e-2 and res[1][0] < 2e-2
    assert res[0][1] is True                        # rank 0 gave up its wait and left the residual alone
    assert res[0][2] < 2e-2 and res[1][2] < 2e-2 and res[0][3] == 0 and res[1][3] == 0


def _reduce_scatter_layer(rank, world, qt_name, T, n, k_total):
    """Row-parallel GEMM with the reduce-scatter in its epilogue, then the owner-side reduce + residual + RMSNorm, then the
    all-gather GEMM on the normed rows: every stage against an fp32 reference, over several calls (parities alternate)."""
    import torch.distributed as dist
    from llaminar_b200 import ops
    from llaminar_b200.gguf import GGMLType, dequantize, quantize
    from llaminar_b200.parallel.symm import SeqShardArena
    dev = torch.device("cuda", rank)
    qt = GGMLType[qt_name]
    kl = k_total // world
    arena = SeqShardArena(dist.group.WORLD, dev, rows_cap=(T + world - 1) // world, d=n)
    g = torch.Generator(device=dev).manual_seed(5)                   # same seed: every rank can build the reference
    w = torch.randn(n, k_total, device=dev, generator=g) * 0.05
    w2 = torch.randn(256, n, device=dev, generator=g) * 0.05         # the next column-parallel weight (replicated here)
    x = (torch.randn(T, k_total, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    h0 = torch.randn(T, n, device=dev, generator=g)
    gain = torch.rand(n, device=dev, generator=g) + 0.5
    raws = [quantize(w[:, r * kl:(r + 1) * kl].contiguous(), qt) for r in range(world)]
    pw = ops.pack_matrix(raws[rank], qt, n, kl)
    wq = torch.cat([dequantize(raws[r], qt, (n, kl)) for r in range(world)], 1)
    raw2 = quantize(w2, GGMLType.Q8_0)
    pw2 = ops.pack_matrix(raw2, GGMLType.Q8_0, 256, n)
    w2q = dequantize(raw2, GGMLType.Q8_0, (256, n))
    tw = arena.rows_per_rank(T)
    r0, mine = arena.my_rows(T, tw)
    errs = []
    for call in range(3):
        xs = (x.float() * (1.0 + 0.5 * call)).to(torch.bfloat16)
        ref_h = h0 + xs.float() @ wq.T
        ref_xn = ref_h * torch.rsqrt((ref_h * ref_h).mean(-1, keepdim=True) + 1e-6) * gain
        h = h0[r0:r0 + mine].clone()
        arena.gemm_reduce_scatter(pw, xs[:, rank * kl:(rank + 1) * kl].contiguous(), tw)
        arena.reduce_norm(h, T, tw, n, gain, arena.ag.own_rows(tw, n)[:mine] if mine else None, 1e-6)
        out = torch.zeros(T, 256, device=dev)
        arena.ag.gemm(pw2, T, tw, out)
        torch.cuda.synchronize()
        arena.check_status()
        if mine:
            errs.append(((h - ref_h[r0:r0 + mine]).norm() / ref_h[r0:r0 + mine].norm()).item())
        ref_out = ref_xn.to(torch.bfloat16).float() @ w2q.T
        errs.append(((out - ref_out).norm() / ref_out.norm()).item())
    return max(errs)


@pytest.mark.parametrize("qt_name,T,n,k_total", [("Q4_K", 512, 1024, 2048), ("Q6_K", 300, 512, 1024), ("Q4_K", 2048, 1024, 1024)])
def test_fused_reduce_scatter_norm_allgather_2gpu(qt_name, T, n, k_total):
    _need(2)
    errs = run_ranks_gpu(_reduce_scatter_layer, 2, qt_name, T, n, k_total)
    assert max(errs) < 2e-2


@pytest.mark.parametrize("qt_name,T,n,k_total", [("Q4_K", 640, 1024, 2048), ("Q4_K", 2048, 1024, 4096)])
def test_fused_reduce_scatter_norm_allgather_4gpu(qt_name, T, n, k_total):
    _need(4)
    errs = run_ranks_gpu(_reduce_scatter_layer, 4, qt_name, T, n, k_total)
    assert max(errs) < 2e-2


def _engine_prefill_tokens(rank, world, fused):
    """Prompts long enough for the sequence-sharded prefill path (fused reduce-scatter / all-gather GEMMs)."""
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.tp import TPContext
    dev = torch.device("cuda", rank)
    cfg = SHAPES["tiny-qwen3"].with_(d_model=1024, n_heads=8, n_kv_heads=2, head_dim=128, d_ff=2048, n_layers=2)
    w = synthesize(cfg, "Q4_K_M", seed=0)
    tp = TPContext.create(device=dev, fused=fused)
    eng = LLMEngine(w, device=dev, max_batch=8, max_context=1024, tp=tp, max_prefill_tokens=1024)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (400, 190, 700, 333)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    eng.check_health()
    arena = getattr(eng.model, "_ss_arena", None)
    if arena is not None:
        arena.check_status()
    return outs, dict(tp.stats), arena is not None and arena.calls > 0


def test_engine_tp2_sequence_sharded_prefill_equals_nccl_baseline():
    _need(2)
    fused = run_ranks_gpu(_engine_prefill_tokens, 2, True)
    base = run_ranks_gpu(_engine_prefill_tokens, 2, False)
    assert fused[0][0] == fused[1][0] and base[0][0] == base[1][0]
    assert fused[0][2] and not base[0][2]                          # the fused run went through the reduce-scatter arena
    agree = sum(a == b for fo, bo in zip(fused[0][0], base[0][0]) for a, b in zip(fo, bo))
    assert agree >= 0.85 * 24            # bf16 partial sums and another summation order may flip a near-tie


def _group_failure_case(rank, world):
    """A status word set on ONE rank: every rank's health check raises in the same step (MAX over the group), the arrival
    counters are resynchronised by all of them together, and the next requests run through the fused kernels again."""
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.tp import TPContext
    dev = torch.device("cuda", rank)
    cfg = SHAPES["tiny-qwen3"].with_(d_model=1024, n_heads=8, n_kv_heads=2, head_dim=128, d_ff=2048, n_layers=2)
    w = synthesize(cfg, "Q4_K_M", seed=0)
    tp = TPContext.create(device=dev, fused=True)
    eng = LLMEngine(w, device=dev, max_batch=4, max_context=256, tp=tp)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (40, 9)]
    ps = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    first = eng.generate(prompts, ps)
    if rank == 0:
        tp.symm.status[0] = 1                      # as a wait of this rank that ran out would leave it
    raised, text = False, ""
    try:
        eng.check_health()
    except RuntimeError as e:
        raised, text = True, str(e)
    again = eng.generate(prompts, ps)
    eng.check_health()
    return raised, "another rank" in text, first == again, int(tp.symm.status[0])


def test_a_failure_on_one_rank_is_seen_and_resynchronised_by_all():
    _need(2)
    out = run_ranks_gpu(_group_failure_case, 2)
    assert out[0][0] and out[1][0]                  # both ranks raised
    assert not out[0][1] and out[1][1]              # rank 1 had nothing in its own words
    assert out[0][2] and out[1][2]                  # the fused path works again afterwards, same tokens
    assert out[0][3] == 0 and out[1][3] == 0


def _pp2_gpu_case(rank, world):
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.pp import build_pipeline_engine
    dev = torch.device("cuda", rank)
    cfg = SHAPES["tiny-qwen3"].with_(d_model=1024, n_heads=8, n_kv_heads=2, head_dim=128, d_ff=2048, n_layers=4)
    w = synthesize(cfg, "Q4_K_M", seed=0)
    layout = {"pp": 2, "tp": 1, "world": 2, "stages": [(f"s{i}", [f"cuda:{i}"], None, None) for i in range(2)]}
    eng = build_pipeline_engine(w, layout, rank, microbatch_tokens=64, device=dev, max_batch=4, max_context=256)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (40, 130, 9)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    sampled = eng.generate(prompts[:2], SamplingParams(temperature=0.8, top_k=20, seed=5, max_tokens=6, ignore_eos=True))
    eng.check_health()
    return outs, sampled, dict(eng.model.stats), str(eng.model.payload_dtype)


def test_pipeline_stages_on_two_gpus_exchange_bf16_rows_and_token_ids():
    """PP = 2 on GPUs: the residual stream crosses as bf16, only sampled token ids come back (no full-vocabulary rows), both
    stages end up with the same tokens for greedy and for sampled requests."""
    _need(2)
    out = run_ranks_gpu(_pp2_gpu_case, 2)
    assert out[0][0] == out[1][0] and out[0][1] == out[1][1]
    assert all(len(o) == 8 for o in out[0][0]) and all(len(o) == 6 for o in out[0][1])
    assert out[0][3] == "torch.bfloat16"
    s0, s1 = out[0][2], out[1][2]
    assert s0["sent_bytes"] > 0 and s0["sent_bytes"] == s1["recv_bytes"]
    assert s0["token_syncs"] > 0 and s0["bcast_bytes"] == s1["bcast_bytes"] < 4096
