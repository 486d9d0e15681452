"""Scheduler / paged-KV engine on the CPU backend against the contiguous-KV fp32 oracle."""
import torch

from llaminar_b200.engine.engine import LLMEngine
from llaminar_b200.engine.sampling import SamplingParams, dry_match_lengths, sample_row
from llaminar_b200.models.config import SHAPES
from llaminar_b200.models.reference import ReferenceModel
from llaminar_b200.models.synth import synthesize

GREEDY = SamplingParams(temperature=0.0, max_tokens=32, ignore_eos=True)


def _prompt(n, seed=1, vocab=1024):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def test_config1_tiny_qwen3_q8_greedy_matches_oracle(tmp_path):
    """64 random prompt tokens, 32 greedy tokens, Q8_0 GGUF round trip, logits vs the fp32 oracle."""
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    path = str(tmp_path / "tiny.gguf")
    w.save_gguf(path)
    eng = LLMEngine.from_gguf(path, device="cpu", max_batch=2, max_context=256)
    prompt = _prompt(64)
    out = eng.generate([prompt], GREEDY)[0]
    ref_tokens, _ = ReferenceModel(w).generate_greedy(torch.tensor(prompt), 32)
    assert out == ref_tokens


def test_continuous_batching_equals_single_requests():
    w = synthesize(SHAPES["tiny-qwen2"], "Q4_K_M", seed=3)
    eng = LLMEngine(w, device="cpu", max_batch=3, max_context=256, max_prefill_tokens=80)
    prompts = [_prompt(n, seed=n) for n in (5, 70, 33, 130, 64)]
    p = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    outs = eng.generate(prompts, p)
    ref = ReferenceModel(w)
    for pr, o in zip(prompts, outs):
        assert o == ref.generate_greedy(torch.tensor(pr), 12)[0]
    assert eng.kv.allocator.n_free == eng.kv.n_pages - 1       # every page returned


def test_moe_and_stop_conditions():
    w = synthesize(SHAPES["tiny-qwen3moe"], "Q8_0", seed=5)
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=128, eos_token_id=None)
    prompt = _prompt(20, seed=9)
    ref = ReferenceModel(w).generate_greedy(torch.tensor(prompt), 8)[0]
    assert eng.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8))[0] == ref
    stop = ref[3]
    out = eng.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8, stop_token_ids=(stop,)))[0]
    assert out == ref[:ref.index(stop) + 1]
    r = eng.add_request(prompt, SamplingParams(temperature=0.0, max_tokens=4))
    eng.step()
    eng.force_token(r.rid, 7)
    eng.step()
    assert r.output[1] == 7


def test_sampler_reference():
    logits = torch.tensor([0.0, 5.0, 4.0, -1.0])
    assert sample_row(logits, SamplingParams(temperature=0.0)) == 1
    assert sample_row(logits, SamplingParams(temperature=1.0, top_k=1, top_p=1.0)) == 1
    g = torch.Generator().manual_seed(0)
    picks = {sample_row(logits, SamplingParams(temperature=1.0, top_k=2, top_p=1.0), g) for _ in range(50)}
    assert picks <= {1, 2}
    # DRY: history "a b c a b" -> emitting c would extend a repeat of length 2
    assert dry_match_lengths([1, 2, 3, 1, 2]) == {3: 2}


def test_parity_report_against_the_oracle(tmp_path):
    """The parity tool: per-layer cosine / logit gates of the runtime model against the fp32 oracle, CSV output, and a
    failing gate when the runtime model is broken on purpose."""
    from llaminar_b200 import parity
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    out = tmp_path / "p.csv"
    assert parity.main(["--synthetic", "tiny-qwen3", "--synthetic-recipe", "Q8_0", "-d", "cpu", "--prompt-tokens", "24",
                        "--decode-steps", "2", "--csv", str(out)]) == 0
    lines = out.read_text().splitlines()
    assert lines[0].startswith("phase,stage,cosine") and len(lines) == 1 + 3 * (2 + 1)
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    rows, failed = parity.compare(w, "cpu", prompt_tokens=16, decode_steps=1)
    assert not failed and all(r["cosine"] > 0.9999 for r in rows if r["stage"] != "logits")
    m = parity.logit_metrics(torch.tensor([[0.0, 5.0, 1.0, 0.5, 0.2, 0.1]]), torch.tensor([[5.0, 0.0, 1.0, 0.5, 0.2, 0.1]]))
    assert m["top1"] == 0.0 and m["kl"] > 1.0 and abs(m["top5_overlap"] - 0.8) < 1e-9


def test_logprobs_follow_the_models_distribution():
    """The chosen token's log-probability and the k likeliest alternatives, per output token, against the oracle's
    logits; a request without the option in the same batch is unaffected."""
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=256)
    prompt = _prompt(40, seed=4)
    with_lp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, logprobs=3)
    plain = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    a, b = eng.add_request(prompt, with_lp), eng.add_request(prompt, plain)
    steps = []
    while eng.has_unfinished():
        steps += eng.step()
    ref_tokens, ref_logits = ReferenceModel(w).generate_greedy(torch.tensor(prompt), 6)
    assert a.output == ref_tokens and b.output == ref_tokens
    assert b.logprobs == [] and all(o.logprobs is None for o in steps if o.rid == b.rid)
    assert sum(len(o.logprobs) for o in steps if o.rid == a.rid) == 6
    ref_lp = torch.log_softmax(ref_logits.float(), -1)
    for i, (tok, lp, top) in enumerate(a.logprobs):
        assert tok == ref_tokens[i] and abs(lp - float(ref_lp[i, tok])) < 2e-2
        assert len(top) == 3 and top[0][0] == tok                      # greedy: the emitted token leads the list
        assert [t for t, _ in top] == ref_lp[i].topk(3).indices.tolist()
        assert all(x[1] >= y[1] for x, y in zip(top, top[1:]))
    # sampled requests report the probability of the token that was drawn, not of the likeliest one
    sp = SamplingParams(temperature=1.5, top_k=0, top_p=1.0, seed=11, max_tokens=8, ignore_eos=True, logprobs=0)
    r = eng.add_request(prompt, sp)
    while eng.has_unfinished():
        eng.step()
    assert [t for t, _, _ in r.logprobs] == r.output and all(top == [] and lp <= 0.0 for _, lp, top in r.logprobs)


def test_preemption_when_the_kv_cache_runs_out_continues_the_same_output():
    """Three long generations in a cache that holds about half of them: the youngest sequences are preempted (pages freed,
    tokens folded into the prompt, prefix recomputed later) instead of failing the step; greedy outputs equal those of an
    engine with room for everything, logprobs stay aligned, and every page comes back."""
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    prompts = [_prompt(60, seed=s) for s in (1, 2, 3)]
    sp = SamplingParams(temperature=0.0, max_tokens=150, ignore_eos=True, logprobs=0)
    big = LLMEngine(w, device="cpu", max_batch=3, max_context=256)
    want = big.generate(prompts, sp)
    assert big.stats["preemptions"] == 0
    small = LLMEngine(w, device="cpu", max_batch=3, max_context=256, kv_pages=8)       # 7 usable pages of 64 tokens
    reqs = [small.add_request(p, sp) for p in prompts]
    while small.has_unfinished():
        small.step()
    assert small.stats["preemptions"] >= 1
    for r, ref in zip(reqs, want):
        assert r.output == ref and [t for t, _, _ in r.logprobs] == r.output and r.n_tokens == 60 + 150
    assert small.kv.allocator.n_free == small.kv.n_pages - 1
    # a single sequence that outgrows the whole cache ends with what it has (finish reason "length"); the engine goes on
    tiny = LLMEngine(w, device="cpu", max_batch=1, max_context=256, kv_pages=3)          # 2 usable pages: 128 tokens
    a = tiny.add_request(prompts[0], sp)
    b = tiny.add_request(prompts[1][:20], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    outs = []
    while tiny.has_unfinished():
        outs += tiny.step()
    assert a.finish_reason == "length" and 60 + len(a.output) == 129           # 128 cached positions + the token not fed yet
    assert any(o.rid == a.rid and o.finished and o.finish_reason == "length" for o in outs)
    assert b.finish_reason == "length" and len(b.output) == 5                       # the next request was served normally
    assert tiny.kv.allocator.n_free == tiny.kv.n_pages - 1


def test_forward_batch_index_check_names_every_out_of_range_input():
    """The host-side check behind LLAMINAR_VALIDATE_TENSORS: well-formed prefill and decode batches pass; a page id, a
    sequence id, a token, a length or a query partition outside its range is reported by name before anything launches."""
    from llaminar_b200.engine.cuda_model import ForwardBatch
    it = lambda x: torch.tensor(x, dtype=torch.int32)
    ok_prefill = ForwardBatch(tokens=it([5, 6, 7, 8]), positions=it([64, 65, 0, 1]), seq_ids=it([0, 0, 1, 1]),
                              block_table=it([[3, 4], [2, 0]]), cu_q=it([0, 2, 4]), ctx_lens=it([64, 0]), max_q_len=2,
                              logit_rows=it([1, 3]))
    assert ok_prefill.index_errors(vocab=1024, n_pages=8, max_positions=4096) == []
    ok_decode = ForwardBatch(tokens=it([5, 6]), positions=it([70, 3]), seq_ids=it([0, 1]), block_table=it([[3, 4], [2, 0]]),
                             seq_lens=it([71, 4]))
    assert ok_decode.index_errors(1024, 8, 4096) == []
    import dataclasses
    bad = {
        "tokens": dataclasses.replace(ok_decode, tokens=it([5, 1024])),
        "block_table": dataclasses.replace(ok_decode, block_table=it([[3, 9], [2, 0]])),
        "seq_ids": dataclasses.replace(ok_decode, seq_ids=it([0, 2])),
        "seq_lens": dataclasses.replace(ok_decode, seq_lens=it([129, 4])),
        "positions": dataclasses.replace(ok_prefill, positions=it([64, 65, 0, -1])),
        "cu_q": dataclasses.replace(ok_prefill, cu_q=it([0, 3, 2])),
        "max_q_len": dataclasses.replace(ok_prefill, max_q_len=1),
        "context + query": dataclasses.replace(ok_prefill, ctx_lens=it([127, 0])),
        "logit_rows": dataclasses.replace(ok_prefill, logit_rows=it([4])),
    }
    for name, fb in bad.items():
        errs = fb.index_errors(1024, 8, 4096)
        assert errs and any(name in e for e in errs), (name, errs)


def test_a_prompt_larger_than_the_whole_cache_is_ended_and_the_queue_goes_on():
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=256, kv_pages=3)            # 2 usable pages: 128 tokens
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    big, small = eng.add_request(_prompt(200, seed=1), sp), eng.add_request(_prompt(30, seed=2), sp)
    outs = []
    while eng.has_unfinished():
        outs += eng.step()
    assert big.finish_reason == "cache_full" and big.output == []
    assert any(o.rid == big.rid and o.finished and o.finish_reason == "cache_full" for o in outs)
    assert small.finish_reason == "length" and len(small.output) == 4
    assert eng.kv.allocator.n_free == eng.kv.n_pages - 1


def test_filtered_sampling_distribution_matches_the_transformers_logits_warpers():
    """temperature -> top-k -> top-p as `transformers` applies them (its warpers, then softmax) against `filtered_probs`, the
    distribution the samplers here draw from (the GPU kernel is tested against the same function)."""
    pytest = __import__("pytest")
    tf = pytest.importorskip("transformers")
    from transformers import TemperatureLogitsWarper, TopKLogitsWarper, TopPLogitsWarper
    from llaminar_b200.engine.sampling import filtered_probs
    g = torch.Generator().manual_seed(0)
    for temp, k, p in ((0.7, 40, 0.9), (1.3, 5, 0.5), (0.6, 20, 0.95), (1.0, 200, 1.0), (0.8, 0, 0.3)):
        logits = torch.randn(1, 2000, generator=g) * 3
        x = TemperatureLogitsWarper(temp)(None, logits.clone())
        if k:
            x = TopKLogitsWarper(k)(None, x)
        else:
            x = TopKLogitsWarper(1024)(None, x)                  # top_k = 0 means "the best 1024" here
        if p < 1.0:
            x = TopPLogitsWarper(p)(None, x)
        want = torch.softmax(x, dim=-1)[0]
        got = filtered_probs(logits[0], SamplingParams(temperature=temp, top_k=k, top_p=p))
        assert torch.equal(got > 0, want > 0), (temp, k, p)
        assert torch.allclose(got, want, atol=1e-6)
