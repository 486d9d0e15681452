"""Failure detection without touching a GPU: host-made faults among gloo ranks and against an in-memory store."""
import datetime
import time

import pytest
import torch

from llaminar_b200.parallel.watchdog import Heartbeat, RankFailure, StepWatchdog, vote_all_ok
from tests.mp_utils import run_ranks


class DictStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_heartbeat_detects_silent_and_failed_ranks():
    store = DictStore()
    seen = []
    a = Heartbeat(store, 0, 3, interval_s=0.05, timeout_s=1.0, on_failure=lambda r, why: seen.append((r, why)))
    b = Heartbeat(store, 1, 3, interval_s=0.05, timeout_s=1.0)
    c = Heartbeat(store, 2, 3, interval_s=0.05, timeout_s=1.0)
    for h in (a, b, c):
        h._write_beat()
    assert a.poll_once(now=100.0) == {}
    b._write_beat()                                    # rank 1 keeps beating, rank 2 is silent
    assert a.poll_once(now=100.5) == {}
    b._write_beat()
    new = a.poll_once(now=101.6)
    assert list(new) == [2] and "no heartbeat" in new[2]
    b.post_error("CUDA error in step 7")
    new = a.poll_once(now=101.7)
    assert new == {1: "CUDA error in step 7"} and [r for r, _ in seen] == [2, 1]
    with pytest.raises(RankFailure):
        a.raise_if_failed()


def test_heartbeat_threads_over_a_dropped_beat():
    store = DictStore()
    fails = []
    a = Heartbeat(store, 0, 2, interval_s=0.02, timeout_s=0.3, on_failure=lambda r, w: fails.append(r)).start()
    b = Heartbeat(store, 1, 2, interval_s=0.02, timeout_s=0.3).start()
    time.sleep(0.2)
    assert not fails
    b.paused = True                                    # the test drops rank 1's heartbeats
    time.sleep(0.8)
    a.stop()
    b.stop()
    assert fails == [1]


def test_step_watchdog_fires_abort_once():
    calls = []
    wd = StepWatchdog(timeout_s=0.1, abort=lambda: calls.append("abort"))
    with wd("fast"):
        pass
    time.sleep(0.2)
    assert not calls and not wd.expired
    with wd("slow"):
        time.sleep(0.3)
    assert calls == ["abort"] and wd.expired


def _vote(rank, world):
    return vote_all_ok(rank != 1)


def test_init_vote_fails_everywhere():
    assert run_ranks(_vote, 3) == [False, False, False]


def _rank_raises_in_step(rank, world):
    """Rank 1 raises inside its step; the others learn of it through the store before their next collective."""
    import torch.distributed as dist
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=2.0).start()
    x = torch.ones(4)
    out = "ok"
    try:
        for step in range(50):
            hb.poll_once()
            hb.raise_if_failed()
            if rank == 1 and step == 3:
                raise ValueError("injected failure in step 3")
            dist.all_reduce(x)
            time.sleep(0.02)
    except ValueError as exc:
        hb.post_error(str(exc))
        out = "raised"
        time.sleep(1.0)                              # stay alive so the store outlives the peers' polls
    except RankFailure as exc:
        out = f"peer {exc.rank}: {exc.reason}"
    except RuntimeError as exc:                      # a collective the dead rank never joined ends with an error
        out = f"collective error: {type(exc).__name__}"
    hb.stop()
    return out


def _entry_short_timeout(rank, world):
    return _rank_raises_in_step(rank, world)


def test_peers_stop_when_a_rank_raises():
    res = run_ranks(_entry_short_timeout, 3, timeout=120)
    assert res[1] == "raised"
    assert all(r.startswith("peer 1") or r.startswith("collective error") for r in (res[0], res[2])), res


def test_server_answers_500_and_keeps_serving():
    """A step that raises fails the request with HTTP 500; the next request is served."""
    import http.client
    import json
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.serve.chat_handler import ChatCompletionHandler
    from llaminar_b200.serve.engine_loop import EngineLoop
    from llaminar_b200.serve.server import Server
    from llaminar_b200.tokenizer.bpe import BPETokenizer
    from llaminar_b200.tokenizer.chat_template import ChatTemplate
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=256)
    tok = BPETokenizer.from_metadata(w.metadata)
    real_step, boom = eng.step, {"n": 1}
    def flaky_step():
        if boom["n"]:
            boom["n"] -= 1
            raise RuntimeError("injected step failure")
        return real_step()
    eng.step = flaky_step
    chat = ChatCompletionHandler(EngineLoop(eng), tok, ChatTemplate.resolve(None, tok.chat_template), "qwen3", 256, model_name="tiny")
    srv = Server(chat, "127.0.0.1", 0)
    srv.start_background()
    try:
        def post():
            c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=60)
            c.request("POST", "/v1/chat/completions", body=json.dumps({"messages": [{"role": "user", "content": "x"}], "max_tokens": 3}))
            r = c.getresponse()
            return r.status, json.loads(r.read())
        st, body = post()
        assert st == 500 and "injected" in body["error"]["message"]
        st, body = post()
        assert st == 200 and body["choices"][0]["message"]["role"] == "assistant"
    finally:
        srv.stop()


def test_step_errors_of_one_rank_only_are_reported_and_shared_ones_are_not():
    """Ranks replay the same commands.  A command that raises on every rank keeps them in step; one that raises on a
    single rank does not, and the other ranks' monitors report that rank."""
    store = DictStore()
    seen = []
    a = Heartbeat(store, 0, 2, interval_s=0.05, timeout_s=10.0, on_failure=lambda r, why: seen.append((r, why)))
    b = Heartbeat(store, 1, 2, interval_s=0.05, timeout_s=10.0)
    a._write_beat(); b._write_beat()
    # command 3 fails on both ranks (say, a prompt longer than the context window)
    a.post_step_error(3, "ValueError: prompt too long")
    b.post_step_error(3, "ValueError: prompt too long")
    assert a.poll_once(now=1.0) == {}
    # command 5 fails on rank 1 only; rank 0 has not finished it yet: no verdict so far
    b.post_step_error(5, "RuntimeError: a kernel gave up a bounded wait")
    a.note_step_ok(4)
    assert a.poll_once(now=1.1) == {}
    a.note_step_ok(5)
    new = a.poll_once(now=1.2)
    assert list(new) == [1] and "command 5 failed on rank 1 only" in new[1] and seen[0][0] == 1
    assert a.poll_once(now=1.3) == {}                   # reported once


def _worker_error_case(rank, world):
    """The worker's engine raises in a step that rank 0 completes: rank 0's heartbeat monitor learns of it."""
    import torch.distributed as dist
    from llaminar_b200.parallel.spmd import ControlChannel, ReplicatedEngine, worker_loop
    from llaminar_b200.parallel.watchdog import Heartbeat

    class Eng:
        def __init__(self, bad):
            self.requests, self.bad, self.n = {}, bad, 0

        def step(self):
            self.n += 1
            if self.bad and self.n == 2:
                raise RuntimeError("status word set")
            return []

    failed = []
    store = dist.distributed_c10d._get_default_store()
    eng = Eng(bad=(rank == 1))
    eng.heartbeat = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=30.0, on_failure=lambda r, why: failed.append((r, why))).start()
    ch = ControlChannel()
    if rank == 0:
        drive = ReplicatedEngine(eng, ch)
        for _ in range(3):
            drive.step()
        deadline = time.time() + 5.0
        while not failed and time.time() < deadline:
            time.sleep(0.05)
        drive.shutdown_workers()
    else:
        worker_loop(eng, ch)
    eng.heartbeat.stop()
    return failed


def test_worker_only_step_error_reaches_rank_zero():
    out = run_ranks(_worker_error_case, 2)
    assert out[0] and out[0][0][0] == 1 and "command 1 failed on rank 1 only" in out[0][0][1]
    assert out[1] == []


def _kv_pages_case(rank, world):
    import dataclasses
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.tp import TPContext
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=1)
    tp = TPContext.create(device="cpu")
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=256, tp=tp, kv_pages=40 + 7 * rank)
    return eng.kv.n_pages, eng.kv_pages_per_rank


def test_ranks_agree_on_the_smallest_kv_page_count():
    out = run_ranks(_kv_pages_case, 2)
    assert out[0] == out[1] == (40, (40, 47))


def _shared_disk_dir_case(rank, world, path):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.prefix_cache import PrefixCache, PrefixCacheConfig
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.tp import TPContext
    import torch.distributed as dist
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=1)
    tp = TPContext.create(device="cpu")
    greedy = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    cfg = PrefixCacheConfig(storage="tiered", vram_budget_mb=0, ram_budget_mb=0, disk_budget_mb=64, disk_dir=path, terminal_state="off")
    pc = PrefixCache(cfg, "fp")
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=512, tp=tp, prefix_cache=pc)
    pc.cfg.vram_budget_mb = 0
    g = torch.Generator().manual_seed(5)
    ps = [torch.randint(0, 1024, (130,), generator=g).tolist() for _ in range(3)]
    first = [eng.generate([p], greedy)[0] for p in ps]
    again = [eng.generate([p], greedy)[0] for p in ps]          # blocks come back from this rank's own files
    dist.barrier()
    pc2 = PrefixCache(cfg, "fp")
    LLMEngine(w, device="cpu", max_batch=2, max_context=512, tp=tp, prefix_cache=pc2)
    return first == again, pc.stats()["promoted"], pc.file_prefix, len(pc2.disk)


def test_ranks_sharing_a_disk_dir_keep_their_kv_shards_apart(tmp_path):
    out = run_ranks(_shared_disk_dir_case, 2, str(tmp_path))
    assert out[0][0] and out[1][0] and out[0][1] > 0 and out[1][1] > 0
    assert out[0][2] != out[1][2]                       # one file prefix per rank
    assert out[0][3] > 0 and out[1][3] > 0              # and a restart finds only its own files
    import os
    names = os.listdir(tmp_path)
    assert all(n.startswith(out[0][2] + "_") or n.startswith(out[1][2] + "_") for n in names)


def _prefix_agreement_case(rank, world):
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.prefix_cache import PrefixCache, PrefixCacheConfig
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.parallel.tp import TPContext
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=1)
    tp = TPContext.create(device="cpu")
    greedy = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    pc = PrefixCache(PrefixCacheConfig(storage="vram", terminal_state="off"), "fp")
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=512, tp=tp, prefix_cache=pc)
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, 1024, (200,), generator=g).tolist()
    first = eng.generate([prompt], greedy)[0]
    if rank == 1:                                      # this rank's cache loses the second block of the chain
        from llaminar_b200.engine.prefix_cache import chain_hashes
        hs = list(chain_hashes(prompt, pc.salt, pc.cfg.block_size))
        page = pc.device.pop(hs[1])
        eng.kv.allocator.release(page)
    before = eng.stats["prefix_hit_tokens"]
    again = eng.generate([prompt], greedy)[0]
    return first == again, eng.stats["prefix_hit_tokens"] - before, eng.stats.get("agreements", 0)


def test_ranks_agree_on_the_shortest_prefix_hit():
    """Rank 1 has lost a block that rank 0 still holds: both reuse only what both have (one 64-token block), so both
    prefill the same rows and stay in the same collectives; the tokens are unchanged."""
    out = run_ranks(_prefix_agreement_case, 2)
    assert out[0][0] and out[1][0]
    assert out[0][1] == out[1][1] == 64
    assert out[0][2] > 0 and out[0][2] == out[1][2]
