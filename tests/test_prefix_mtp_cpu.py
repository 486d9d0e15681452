"""Prefix cache (tiers, eviction, terminal state) and NextN speculative decoding on the CPU runner."""
import dataclasses

import pytest
import torch

from llaminar_b200.engine.engine import LLMEngine
from llaminar_b200.engine.mtp import DepthController, MTPConfig, MTPDecoder
from llaminar_b200.engine.prefix_cache import PrefixCache, PrefixCacheConfig, chain_hashes
from llaminar_b200.engine.sampling import SamplingParams
from llaminar_b200.models.config import SHAPES
from llaminar_b200.models.synth import synthesize

GREEDY = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)


@pytest.fixture(scope="module")
def weights():
    return synthesize(dataclasses.replace(SHAPES["tiny-qwen3"], nextn_layers=1), "Q8_0", seed=1)


def _prompts():
    g = torch.Generator().manual_seed(3)
    return [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (70, 33, 150)]


def test_chain_hashes_depend_on_parent_and_salt():
    a = chain_hashes(list(range(200)), b"s1")
    b = chain_hashes(list(range(64)) + [7] * 64 + list(range(128, 200)), b"s1")
    assert len(a) == 3 and a[0] == b[0] and a[1] != b[1] and a[2] != b[2]      # a changed block poisons its successors
    assert chain_hashes(list(range(200)), b"s2")[0] != a[0]


def test_prefix_hit_reuses_pages_and_matches(weights):
    base = LLMEngine(weights, device="cpu", max_batch=4, max_context=512)
    ref = base.generate(_prompts(), GREEDY)
    eng = LLMEngine(weights, device="cpu", max_batch=4, max_context=512,
                    prefix_cache=PrefixCache(PrefixCacheConfig(terminal_state="off"), "fp"))
    assert eng.generate(_prompts(), GREEDY) == ref
    before = eng.stats["prefill_tokens"]
    assert eng.generate(_prompts(), GREEDY) == ref
    # second pass: 64 + 0 + 128 tokens came from the cache
    assert eng.stats["prefill_tokens"] - before == sum(len(p) for p in _prompts()) - 192
    shared = _prompts()[2][:128] + [9, 8, 7]
    assert eng.generate([shared], GREEDY) == base.generate([shared], GREEDY)
    assert eng.prefix_cache.stats()["hit_tokens"] >= 192 + 128


def test_terminal_state_skips_forward(weights):
    base = LLMEngine(weights, device="cpu", max_batch=4, max_context=512)
    p = _prompts()[2]
    ref = base.generate([p], GREEDY)
    eng = LLMEngine(weights, device="cpu", max_batch=4, max_context=512, prefix_cache=PrefixCache(PrefixCacheConfig(), "fp"))
    assert eng.generate([p], GREEDY) == ref
    n = eng.stats["prefill_tokens"]
    assert eng.generate([p], GREEDY) == ref
    assert eng.stats["prefill_tokens"] == n and eng.prefix_cache.stats()["terminal_hits"] == 1


def test_eviction_spills_to_ram_and_disk_and_promotes(weights, tmp_path):
    base = LLMEngine(weights, device="cpu", max_batch=2, max_context=512)
    pc = PrefixCache(PrefixCacheConfig(storage="tiered", vram_budget_mb=0, ram_budget_mb=0, disk_budget_mb=64,
                                       disk_dir=str(tmp_path), terminal_state="off"), "fp")
    eng = LLMEngine(weights, device="cpu", max_batch=2, max_context=512, prefix_cache=pc)
    pc.cfg.vram_budget_mb = 0
    g = torch.Generator().manual_seed(9)
    ps = [torch.randint(0, 1024, (130,), generator=g).tolist() for _ in range(3)]
    refs = [base.generate([p], GREEDY)[0] for p in ps]
    for p, r in zip(ps, refs):
        assert eng.generate([p], GREEDY)[0] == r
    st = pc.stats()
    assert st["evicted_to_disk"] > 0 and st["device_blocks"] <= 1
    for p, r in zip(ps, refs):                        # blocks come back from disk
        assert eng.generate([p], GREEDY)[0] == r
    assert pc.stats()["promoted"] > 0
    pc2 = PrefixCache(PrefixCacheConfig(disk_budget_mb=64, disk_dir=str(tmp_path)), "fp")
    LLMEngine(weights, device="cpu", max_batch=2, max_context=512, prefix_cache=pc2)   # the scan runs once the page geometry is known
    assert pc2.stats()["disk_blocks"] > 0           # a new process finds the persisted blocks
    pc3 = PrefixCache(PrefixCacheConfig(disk_budget_mb=64, disk_dir=str(tmp_path)), "another model")
    LLMEngine(weights, device="cpu", max_batch=2, max_context=512, prefix_cache=pc3)
    assert pc3.stats()["disk_blocks"] == 0          # and nothing that another fingerprint wrote
    pc.clear()
    assert all(r <= 1 for r in eng.kv.allocator.refs)


@pytest.mark.parametrize("k", [1, 2, 3])
def test_mtp_greedy_is_lossless(weights, k):
    base = LLMEngine(weights, device="cpu", max_batch=4, max_context=512)
    ref = base.generate(_prompts(), GREEDY)
    eng = LLMEngine(weights, device="cpu", max_batch=4, max_context=512, mtp=MTPDecoder(MTPConfig(draft_tokens=k)))
    assert eng.generate(_prompts(), GREEDY) == ref
    assert eng.mtp.stats()["drafted"] > 0


def test_mtp_accepts_correct_drafts(weights, monkeypatch):
    """Drafts that equal the trunk's continuation are all accepted: k + 1 tokens per step."""
    base = LLMEngine(weights, device="cpu", max_batch=1, max_context=512)
    p = _prompts()[0]
    ref = base.generate([p], GREEDY)[0]
    dec = MTPDecoder(MTPConfig(draft_tokens=2))
    eng = LLMEngine(weights, device="cpu", max_batch=1, max_context=512, mtp=dec)
    def oracle(engine, logits, reqs, sampling, p_draft, j):
        r = reqs[0]
        i = len(r.output) + j
        return [ref[i] if i < len(ref) else 0]
    monkeypatch.setattr(dec, "_draft_tokens", oracle)
    assert eng.generate([p], GREEDY)[0] == ref
    st = dec.stats()
    assert st["acceptance_rate"] > 0.8 and st["tokens_per_step"] > 2.0


def test_mtp_speculative_sampling_runs_and_is_seeded(weights):
    sp = SamplingParams(max_tokens=10, temperature=0.8, top_k=20, seed=11, ignore_eos=True)
    outs = []
    for _ in range(2):
        eng = LLMEngine(weights, device="cpu", max_batch=2, max_context=512,
                        mtp=MTPDecoder(MTPConfig(draft_tokens=2, verify_mode="speculative-sampling")))
        outs.append(eng.generate(_prompts()[:2], sp))
    assert outs[0] == outs[1] and all(len(o) == 10 for o in outs[0])


def test_mtp_with_prefix_cache_and_forced_tokens(weights):
    base = LLMEngine(weights, device="cpu", max_batch=2, max_context=512)
    p = _prompts()[2]
    ref = base.generate([p], GREEDY)[0]
    eng = LLMEngine(weights, device="cpu", max_batch=2, max_context=512, mtp=MTPDecoder(MTPConfig(draft_tokens=2)),
                    prefix_cache=PrefixCache(PrefixCacheConfig(), "fp+mtp"))
    assert eng.generate([p], GREEDY)[0] == ref
    assert eng.generate([p], GREEDY)[0] == ref          # terminal-state hit feeds the draft head its hidden row
    r = eng.add_request(p, GREEDY)
    eng.step()
    eng.force_token(r.rid, 5)
    eng.step()
    assert r.output[1] == 5


def test_depth_controller_demotes_and_promotes():
    cfg = MTPConfig(draft_tokens=3, depth_policy="dynamic", depth_window=4, depth_min_samples=2, depth_cooldown=1, depth_promote_windows=2)
    c = DepthController(cfg)
    for _ in range(4):
        c.observe(0, 3)
        c.end_step()
    assert c.depth < 3
    low = c.depth
    for _ in range(40):
        c.observe(c.depth, c.depth)
        c.end_step()
    assert c.depth > low and c.history
    fixed = DepthController(MTPConfig(draft_tokens=2))
    for _ in range(20):
        fixed.observe(0, 2)
        fixed.end_step()
    assert fixed.depth == 2


def test_preemption_with_a_prefix_cache_keeps_outputs_and_page_accounting():
    """Cache exhaustion with the prefix cache on: cached pages are evicted first, then sequences are preempted; the
    outputs equal those of a roomy engine and no page is lost (free + held by the cache == all pages)."""
    from llaminar_b200.engine.sampling import SamplingParams
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    g = torch.Generator().manual_seed(5)
    shared = torch.randint(0, 1024, (64,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 1024, (10 + i,), generator=g).tolist() for i in range(3)]
    sp = SamplingParams(temperature=0.0, max_tokens=140, ignore_eos=True)
    want = LLMEngine(w, device="cpu", max_batch=3, max_context=256).generate(prompts, sp)
    pc = PrefixCache(PrefixCacheConfig(terminal_state="off"), "fp")
    eng = LLMEngine(w, device="cpu", max_batch=3, max_context=256, kv_pages=9, prefix_cache=pc)
    got = eng.generate(prompts, sp)
    assert got == want and eng.stats["preemptions"] >= 1
    held = len(pc.device)
    assert eng.kv.allocator.n_free + held == eng.kv.n_pages - 1
    assert all(r <= 1 for r in eng.kv.allocator.refs)


def test_preemption_under_speculative_decoding_stays_lossless(weights):
    """Speculation reserves pages for its draft rows; when they run out the youngest sequence is preempted, its
    speculative state dropped and rebuilt by the re-prefill: greedy outputs still equal plain decoding."""
    sp = SamplingParams(max_tokens=120, temperature=0.0, ignore_eos=True)
    prompts = _prompts()[:2] + [_prompts()[0][:40]]
    ref = LLMEngine(weights, device="cpu", max_batch=3, max_context=512).generate(prompts, sp)
    eng = LLMEngine(weights, device="cpu", max_batch=3, max_context=512, kv_pages=8, mtp=MTPDecoder(MTPConfig(draft_tokens=2)))
    got = eng.generate(prompts, sp)
    assert eng.stats["preemptions"] >= 1 and got == ref
    assert eng.kv.allocator.n_free == eng.kv.n_pages - 1 and not eng.mtp.seq


def test_logprobs_under_speculative_decoding_fall_back_to_plain_steps(weights):
    sp = SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True, logprobs=2)
    ref = LLMEngine(weights, device="cpu", max_batch=2, max_context=512)
    a = ref.add_request(_prompts()[0], sp)
    while ref.has_unfinished():
        ref.step()
    eng = LLMEngine(weights, device="cpu", max_batch=2, max_context=512, mtp=MTPDecoder(MTPConfig(draft_tokens=2)))
    b = eng.add_request(_prompts()[0], sp)
    c = eng.add_request(_prompts()[1], GREEDY)                # rides along; speculation resumes once b is done
    while eng.has_unfinished():
        eng.step()
    assert b.output == a.output and [t for t, _, _ in b.logprobs] == b.output
    assert all(abs(x[1] - y[1]) < 1e-4 for x, y in zip(a.logprobs, b.logprobs))
    assert len(c.output) == 12 and c.logprobs == [] and eng.mtp.stats()["drafted"] > 0


def test_lookup_keeps_its_pages_while_later_blocks_are_promoted(weights):
    """A tight cache: promoting a block from the RAM tier must not evict (and hand back) a page that the same lookup
    has already returned.  Every page of a lookup result is distinct and the prefix is restored bit for bit."""
    base = LLMEngine(weights, device="cpu", max_batch=1, max_context=512)
    g = torch.Generator().manual_seed(21)
    p = torch.randint(0, 1024, (64 * 4 + 5,), generator=g).tolist()
    ref = base.generate([p], GREEDY)[0]
    pc = PrefixCache(PrefixCacheConfig(storage="tiered", vram_budget_mb=1, terminal_state="off"), "fp")
    eng = LLMEngine(weights, device="cpu", max_batch=1, max_context=512, prefix_cache=pc, kv_pages=7)
    assert eng.generate([p], GREEDY)[0] == ref
    # move the two oldest blocks of the chain to the RAM tier, keep the others on the device
    hs = chain_hashes(p, pc.salt)
    for h in hs[:2]:
        page = pc.device.pop(h)
        pc._spill(h, eng.kv.export_page(page))
        eng.kv.allocator.release(page)
    # leave exactly one free page: promoting the second block has to evict
    spare = [eng.kv.allocator.alloc() for _ in range(eng.kv.allocator.n_free - 1)]
    held, covered = pc.lookup(p)
    assert len(set(held)) == len(held) and covered == len(held) * 64
    assert all(eng.kv.allocator.refs[pg] >= 1 for pg in held)
    pc.release_pages(held)
    for pg in spare:
        eng.kv.allocator.release(pg)
    assert eng.generate([p], GREEDY)[0] == ref
    pc.clear()
    assert all(r <= 1 for r in eng.kv.allocator.refs)
