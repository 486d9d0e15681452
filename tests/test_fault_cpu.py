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
