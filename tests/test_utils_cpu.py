"""Perf-stats collector, environment-switch registry, collective-order checker, device inventory."""
import json

import pytest

from llaminar_b200.utils.perfstats import PerfStats
from tests.mp_utils import run_ranks


def test_perfstats_records_export_and_filter():
    p = PerfStats(enabled=True)
    p.set_phase("prefill")
    with p.timer("engine", "step", device="cpu", tags=("bs4",)):
        sum(range(1000))
    with p.timer("engine", "step", device="cpu", tags=("bs4",)):
        pass
    p.set_phase("decode")
    p.count("kv", "pages_allocated", 3)
    p.count("kv", "pages_allocated", 2)
    p.gauge("kv", "free_pages", 17)
    rows = p.rows()
    step = next(r for r in rows if r["name"] == "step")
    assert step["count"] == 2 and step["phase"] == "prefill" and step["tags"] == "bs4" and step["total_ms"] >= step["max_ms"] > 0
    pages = next(r for r in rows if r["name"] == "pages_allocated")
    assert pages["value"] == 5 and pages["phase"] == "decode"
    assert json.loads(p.to_json("kv")) and all(r["domain"] == "kv" for r in json.loads(p.to_json("kv")))
    csv = p.to_csv()
    assert csv.splitlines()[0].startswith("domain,name,phase,device,tags") and "free_pages" in csv
    assert "pages_allocated" in p.table()
    off = PerfStats(enabled=False)
    with off.timer("a", "b"):
        pass
    off.count("a", "c")
    assert off.rows() == []


def test_env_registry_types_and_unknown_names():
    from llaminar_b200.utils.env import DebugEnv
    env = DebugEnv({"LLAMINAR_PROFILING": "true", "LLAMINAR_TP_SPIN_LIMIT": "1000", "LLAMINAR_STAGE_DUMP_DIR": "/x"})
    assert env.profiling is True and env.tp_spin_limit == 1000 and env.stage_dump_dir == "/x" and env.pdl is True
    with pytest.raises(KeyError):
        env.get("LLAMINAR_NOT_A_SWITCH")
    with pytest.raises(ValueError):
        DebugEnv({"LLAMINAR_TP_SPIN_LIMIT": "many"}).tp_spin_limit
    assert "LLAMINAR_TP_FUSED" in env.describe()


def _order_check(rank, world, diverge):
    import torch
    from llaminar_b200.parallel.collective_check import CollectiveOrderChecker, CollectiveOrderMismatch
    chk = CollectiveOrderChecker(None, interval=1000)
    x = torch.zeros(4, 8)
    for i in range(5):
        chk.record("all_reduce", x)
    if diverge and rank == 1:
        chk.record("all_gather_vocab", x[:, :4])       # rank 1 issues a different collective
    else:
        chk.record("all_reduce", x)
    try:
        chk.verify()
        return "same"
    except CollectiveOrderMismatch as exc:
        return str(exc)


def test_collective_order_checker_names_the_divergence():
    assert run_ranks(_order_check, 2, False) == ["same", "same"]
    res = run_ranks(_order_check, 2, True)
    assert all("diverged" in r and "all_gather_vocab" in r for r in res)


def test_device_inventory_shape():
    from llaminar_b200.utils.devices import describe_devices as describe
    d = describe()
    assert "cpu" in d and "gpus" in d and isinstance(d["gpus"], list)


def test_tuning_table_keeps_only_clear_wins_and_validates_files(tmp_path):
    from llaminar_b200.ops import tuning
    t = tuning.TuningTable()
    assert t.ksplit("gemv", 0, 5120, 8192, 1) == 0                       # nothing measured: the kernel's heuristic decides
    assert t.record("gemv", 0, 5120, 8192, 1, {0: 20.0, 2: 19.8, 4: 17.0}) is True
    assert t.ksplit("gemv", 0, 5120, 8192, 1) == 4
    assert t.record("gemv", 0, 10240, 5120, 1, {0: 20.0, 2: 19.8}) is False    # 1 % is noise, not a win
    assert t.ksplit("gemv", 0, 10240, 5120, 1) == 0
    f = tmp_path / "tune.json"
    t.dump(f, {"device": "test"})
    back = tuning.TuningTable.load(f)
    assert back.entries == t.entries and back.ksplit("gemv", 0, 5120, 8192, 1) == 4
    bad = tmp_path / "bad.json"
    bad.write_text('{"entries": {"gemv:0:1x1:m1": {"ksplit": -3}}}')
    import pytest
    with pytest.raises(ValueError):
        tuning.TuningTable.load(bad)
    with pytest.raises(FileNotFoundError):
        tuning.TuningTable.load(tmp_path / "missing.json")
    from llaminar_b200.models.config import SHAPES
    shapes = dict((n, (a, b)) for n, a, b in tuning.projection_shapes(SHAPES["qwen3-32b"], tp=2))
    assert shapes["qkv"] == (5120, 5120) and shapes["down"] == (5120, 12800) and shapes["gate_up"] == (25600, 5120)


def test_perf_gate_flags_only_slowdowns_beyond_the_tolerance():
    from llaminar_b200.ops import perf_gate
    base = {"gemv": {"us": 40.0, "tolerance": 0.2}, "gemm_large": {"us": 500.0, "tolerance": 0.15}, "moe": {"us": 300.0}}
    bad, notes = perf_gate.compare(base, {"gemv": 47.0, "gemm_large": 580.0, "moe": 250.0, "extra": 1.0})
    assert len(bad) == 1 and bad[0].startswith("gemm_large") and "+16 %" in bad[0]
    assert any(n.startswith("moe") and "faster" in n for n in notes) and any(n.startswith("extra") for n in notes)
    bad, _ = perf_gate.compare(base, {"gemv": 40.0})
    assert sorted(b.split(":")[0] for b in bad) == ["gemm_large", "moe"]
    rec = {"mma_sync": {"us": 570.0, "tflops": 1.0}, "tcgen05": {"us": 480.0, "tflops": 1.0}}
    assert perf_gate.extract_us("attn_prefill", rec) == {"attn_prefill.mma_sync": 570.0, "attn_prefill.tcgen05": 480.0}
    assert perf_gate.extract_us("moe", {"us_three_launches": 315.0}) == {"moe": 315.0}
    import json
    doc = json.loads(perf_gate.BASELINE.read_text())
    assert {"gemv", "gemm_small", "gemm_large", "attn_decode", "moe"} <= set(doc["cases"])


def test_chat_view_wraps_scrolls_and_edits_without_a_terminal():
    from llaminar_b200.tui import ChatView, LineEditor
    v = ChatView(width=40, height=10)
    v.add("user", "hello there")
    v.append("assistant", "word " * 90)
    v.append("assistant", "tail")
    ls = v.lines()
    assert ls[0][1].startswith("you   | hello") and ls[1][1].startswith("model | word")
    assert all(len(t) <= 40 for _, t in ls) and len(v.entries) == 2 and "tail" in ls[-1][1]
    assert len(v.visible()) == v.pane_height == 7 and v.visible()[-1] == ls[-1]          # follows the newest text
    v.scroll_by(3)
    assert v.visible()[-1] == ls[-4]
    v.scroll_by(1000)
    assert v.visible()[0] == ls[0]                                                      # clamped at the top
    v.scroll_by(-1000)
    assert v.scroll == 0
    v.append("reasoning", "hmm")
    assert v.entries[-1] == ["reasoning", "hmm"] and v.lines()[-1][1].startswith("think |")
    assert len(v.status("m", 10, 100, 12.5, False)) == 39
    v.resize(100, 10)
    assert "generating" in v.status("m", 10, 100, 12.5, True) and "/reset" in v.status("m", 10, 100, 12.5, False)
    e = LineEditor()
    for ch in "helo":
        e.key(ch)
    e.key("LEFT"); e.key("l")
    assert (e.buf, e.cur) == ("hello", 4)
    e.key("HOME"); e.key("DELETE"); e.key("END"); e.key("BACKSPACE")
    assert e.buf == "ell"
    assert e.key("ENTER") == "ell" and e.buf == ""
    e.key("x"); e.key("KILL")
    assert e.buf == ""
    e.key("UP")
    assert e.buf == "ell"
    e.key("DOWN")
    assert e.buf == ""
    e.buf, e.cur = "a" * 50, 50
    text, col = e.window(10)
    assert len(text) <= 10 and col == 9


def test_chat_session_streams_answers_and_keeps_history():
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.tokenizer.bpe import BPETokenizer
    from llaminar_b200.tokenizer.chat_template import ChatTemplate
    from llaminar_b200.tui import ChatSession
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    eng = LLMEngine(w, device="cpu", max_batch=1, max_context=256)
    tok = BPETokenizer.from_metadata(w.metadata)
    tpl = ChatTemplate.resolve(None, tok.chat_template)
    s = ChatSession(eng, tok, tpl, 256, lambda: SamplingParams(temperature=0.0, max_tokens=6), "be brief")
    pieces = list(s.ask("hi"))
    assert all(k in ("reasoning", "content") for k, _ in pieces) and s.generated >= 1 and s.prompt_tokens > 0
    assert [m["role"] for m in s.history] == ["system", "user", "assistant"]
    assert s.history[-1]["content"] == "".join(p for k, p in pieces if k == "content")
    list(s.ask("again"))
    assert len(s.history) == 5 and s.context_used <= 256
    import pytest
    with pytest.raises(ValueError):
        list(s.ask("x " * 400))
    assert len(s.history) == 5                                   # the rejected turn left no trace
    s.reset()
    assert [m["role"] for m in s.history] == ["system"] and s.context_used == 0
    assert not eng.has_unfinished() and eng.kv.allocator.n_free == eng.kv.n_pages - 1


def test_full_screen_chat_runs_in_a_pseudo_terminal():
    """`chat --tui` under a pty: a question is typed, an answer is drawn, /exit leaves with status 0."""
    import os
    import pty
    import select
    import subprocess
    import sys
    import time
    master, slave = pty.openpty()
    import fcntl, struct, termios
    fcntl.ioctl(slave, termios.TIOCSWINSZ, struct.pack("HHHH", 24, 100, 0, 0))
    env = dict(os.environ, TERM="xterm", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = subprocess.Popen([sys.executable, "-m", "llaminar_b200", "chat", "--tui", "--synthetic", "tiny-qwen3", "--synthetic-recipe", "Q8_0",
                          "-d", "cpu", "-n", "6", "-c", "256"], stdin=slave, stdout=slave, stderr=subprocess.PIPE, env=env, close_fds=True)
    os.close(slave)
    seen = b""

    def pump(until: bytes, limit: float) -> bool:
        nonlocal seen
        t0 = time.time()
        while time.time() - t0 < limit:
            r, _, _ = select.select([master], [], [], 0.2)
            if r:
                try:
                    seen += os.read(master, 65536)
                except OSError:
                    return until in seen
            if until in seen:
                return True
            if p.poll() is not None:
                return until in seen
        return False

    try:
        assert pump(b"full-screen chat", 120), p.stderr.read().decode()[-2000:] if p.poll() is not None else seen[-500:]
        os.write(master, b"hello\r")
        assert pump(b"you   | hello", 60)
        assert pump(b"model |", 60)
        time.sleep(1.0)
        os.write(master, b"/exit\r")
        t0 = time.time()
        while p.poll() is None and time.time() - t0 < 60:
            pump(b"\x00never", 0.3)
        assert p.returncode == 0, p.stderr.read().decode()[-2000:]
    finally:
        if p.poll() is None:
            p.kill()
        os.close(master)
