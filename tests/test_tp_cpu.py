"""Tensor parallelism on CPU ranks (gloo): sharded runner + engine must reproduce the single-rank tokens."""
import torch

from llaminar_b200.models.config import SHAPES
from llaminar_b200.parallel.tp_plan import TPPlan
from tests.mp_utils import run_ranks


def _tp_generate(rank, world, shape, recipe, n_new):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.tp import TPContext
    w = synthesize(SHAPES[shape], recipe, seed=0)
    tp = TPContext.create(device="cpu")
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=128, tp=tp)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (17, 40)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    return outs, tp.stats["allreduce_calls"]


def _single(shape, recipe, n_new):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.synth import synthesize
    w = synthesize(SHAPES[shape], recipe, seed=0)
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=128)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (17, 40)]
    return eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))


def test_tp2_dense_matches_single_rank():
    ref = _single("tiny-qwen3", "Q8_0", 6)
    res = run_ranks(_tp_generate, 2, "tiny-qwen3", "Q8_0", 6)
    assert res[0][0] == ref and res[1][0] == ref
    assert res[0][1] > 0                         # the row-parallel layers really all-reduced


def test_tp2_moe_expert_parallel_matches_single_rank():
    ref = _single("tiny-qwen3moe", "Q8_0", 5)
    res = run_ranks(_tp_generate, 2, "tiny-qwen3moe", "Q8_0", 5)
    assert res[0][0] == ref and res[1][0] == ref


def test_tp_plan_rules():
    c = SHAPES["qwen3-32b"]
    plans = [TPPlan.build(c, 8, r) for r in range(8)]
    assert [p.n_heads_local for p in plans] == [8] * 8 and [p.n_kv_local for p in plans] == [1] * 8
    assert sum(p.ff_stop - p.ff_start for p in plans) == c.d_ff and all((p.ff_start % 256) == 0 for p in plans)
    assert plans[-1].vocab_stop == c.vocab_size and plans[0].vocab_start == 0
    moe = SHAPES["qwen3-30b-a3b"]
    p = TPPlan.build(moe, 8, 5)
    assert p.kv_replicas == 2 and p.n_kv_local == 1 and p.kv_head_start == 5 * 4 // 8      # 4 KV heads over 8 ranks
    assert (p.expert_start, p.expert_stop) == (80, 96)
    assert TPPlan.validate(SHAPES["qwen3-8b"], 3)        # 32 heads are not divisible by 3
    assert not TPPlan.validate(SHAPES["qwen3-8b"], 8)


def _tp_generate_replicated(rank, world):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.tp import TPContext
    w = synthesize(SHAPES["tiny-qwen3moe"], "Q8_0", seed=0)
    tp = TPContext.create(device="cpu")
    tp.moe_mode = "replicated"
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=128, tp=tp)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (17, 40)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    return outs, eng.model.plan.expert_stop - eng.model.plan.expert_start


def test_tp2_moe_replicated_experts_matches_single_rank():
    ref = _single("tiny-qwen3moe", "Q8_0", 5)
    res = run_ranks(_tp_generate_replicated, 2)
    assert res[0][0] == ref and res[1][0] == ref
    assert res[0][1] == SHAPES["tiny-qwen3moe"].n_experts


def test_moe_tensor_parallel_mode_is_rejected_by_name():
    import pytest
    with pytest.raises(ValueError, match="tensor-parallel"):
        TPPlan.build(SHAPES["tiny-qwen3moe"], 2, 0, "tensor-parallel")


def _verify_worker(rank, world):
    from llaminar_b200.parallel.tp import TPContext
    tp = TPContext.create(device="cpu")
    tp.verify_checksums = True
    x = torch.full((4, 8), float(rank + 1))
    tp.all_reduce(x)                                    # verified inside: every rank holds 3.0
    ok_calls = tp.stats["verified_collectives"]
    diverged = torch.full((4, 8), 1.0)
    if rank == 1:
        diverged[2, 3] = 1.0000001                      # one rank differs in one element
    caught = ""
    try:
        tp.verify_replicated(diverged, "residual stream")
    except RuntimeError as exc:
        caught = str(exc)
    bad = torch.full((4,), float("nan"))
    nan_msg = ""
    try:
        tp.verify_replicated(bad, "logits")
    except RuntimeError as exc:
        nan_msg = str(exc)
    return float(x[0, 0]), ok_calls, caught, nan_msg


def test_collective_checksum_verification_catches_divergence_and_nans():
    res = run_ranks(_verify_worker, 2)
    for val, calls, caught, nan_msg in res:
        assert val == 3.0 and calls == 1
        assert "ranks [1] hold different bytes" in caught and "residual stream" in caught
        assert "4 NaN" in nan_msg


def _placed_generate(rank, world, loads):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.expert_placement import apply_placement
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.tp import TPContext
    w = synthesize(SHAPES["tiny-qwen3moe"], "Q8_0", seed=0)
    if loads is not None:
        apply_placement(w, loads, world)
    tp = TPContext.create(device="cpu")
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=128, tp=tp)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (17, 40)]
    return eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))


def test_expert_placement_balances_ranks_and_keeps_the_model_function(tmp_path):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.expert_placement import ExpertStats, balanced_permutation, range_loads
    from llaminar_b200.models.synth import synthesize
    cfg = SHAPES["tiny-qwen3moe"]
    # 1. measure router statistics on one rank
    w = synthesize(cfg, "Q8_0", seed=0)
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=128)
    eng.model.expert_stats = ExpertStats(cfg.n_layers, cfg.n_experts)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (17, 40)]
    base = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    f = tmp_path / "stats.json"
    eng.model.expert_stats.dump(str(f), cfg.name)
    loads = ExpertStats.load(str(f))
    assert set(loads) == set(range(cfg.n_layers)) and sum(loads[0]) == (17 + 40 + 2 * 5) * cfg.n_experts_used
    # 2. the permutation balances the two contiguous ranges at least as well as the checkpoint's numbering
    perm = balanced_permutation(loads[0], 2)
    assert sorted(perm) == list(range(cfg.n_experts))
    before, after = range_loads(loads[0], list(range(cfg.n_experts)), 2), range_loads(loads[0], perm, 2)
    assert max(after) - min(after) <= max(before) - min(before)
    skew = [100.0, 90.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0]
    p2 = balanced_permutation(skew, 2)
    assert (0 in p2[:4]) != (1 in p2[:4]) and max(range_loads(skew, p2, 2)) < 110
    # 3. renumbered experts compute the same function: same greedy tokens on 2 expert-parallel ranks
    placed = run_ranks(_placed_generate, 2, loads)
    plain = run_ranks(_placed_generate, 2, None)
    assert placed[0] == placed[1] == plain[0] == base


def _tp_preempt(rank, world):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.tp import TPContext
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    tp = TPContext.create(device="cpu")
    eng = LLMEngine(w, device="cpu", max_batch=3, max_context=256, kv_pages=7, tp=tp)
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 1024, (50,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(temperature=0.7, top_k=20, top_p=0.9, seed=4, max_tokens=100, ignore_eos=True, logprobs=1)
    reqs = [eng.add_request(p, sp) for p in prompts]
    while eng.has_unfinished():
        eng.step()
    return [r.output for r in reqs], eng.stats["preemptions"], [[round(lp, 4) for _, lp, _ in r.logprobs] for r in reqs]


def test_tp2_ranks_stay_in_step_through_preemptions_and_sampled_logprobs():
    """Scheduling decisions (who is preempted, when it returns) depend only on replicated state, so both ranks issue
    the same collectives in the same order and end with the same sampled tokens and log-probabilities."""
    res = run_ranks(_tp_preempt, 2)
    assert res[0] == res[1] and res[0][1] >= 1
    assert all(len(o) == 100 for o in res[0][0])
