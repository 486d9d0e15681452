"""OpenAI-compatible server, chat handler, templates, tool parsing: in-process against a tiny CPU engine."""
import http.client
import json

import pytest

from llaminar_b200.engine.engine import LLMEngine
from llaminar_b200.models.config import SHAPES
from llaminar_b200.models.synth import synthesize
from llaminar_b200.serve.chat_handler import ChatCompletionHandler, RequestError, parse_request
from llaminar_b200.serve.engine_loop import EngineLoop
from llaminar_b200.serve.server import Server
from llaminar_b200.serve.tool_parser import parse_tool_calls
from llaminar_b200.tokenizer.bpe import BPETokenizer
from llaminar_b200.tokenizer.chat_template import ChatTemplate, ThinkSplitter


@pytest.fixture(scope="module")
def server():
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    eng = LLMEngine(w, device="cpu", max_batch=4, max_context=512)
    tok = BPETokenizer.from_metadata(w.metadata)
    tpl = ChatTemplate.resolve(None, tok.chat_template)
    loop = EngineLoop(eng)
    chat = ChatCompletionHandler(loop, tok, tpl, "qwen3", 512, model_name="tiny", eos_ids=(tok.eos_id,) if tok.eos_id is not None else ())
    srv = Server(chat, "127.0.0.1", 0)
    srv.start_background()
    yield srv
    srv.stop()


def _post(srv, body, path="/v1/chat/completions", raw=None):
    c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=120)
    data = raw if raw is not None else json.dumps(body).encode()
    c.request("POST", path, body=data, headers={"Content-Type": "application/json"})
    r = c.getresponse()
    return r.status, r.read(), dict(r.getheaders())


def test_health_and_models(server):
    c = http.client.HTTPConnection("127.0.0.1", server.port, timeout=30)
    c.request("GET", "/health")
    r = c.getresponse()
    assert r.status == 200 and json.loads(r.read())["status"] == "ok"
    c.request("GET", "/v1/models")
    r = c.getresponse()
    assert r.status == 200 and json.loads(r.read())["data"][0]["id"] == "tiny"
    c.request("GET", "/nope")
    r = c.getresponse()
    assert r.status == 404
    r.read()


def test_completion_json_and_usage(server):
    st, body, _ = _post(server, {"messages": [{"role": "user", "content": "hi there"}], "max_tokens": 6, "temperature": 0})
    assert st == 200
    j = json.loads(body)
    assert j["object"] == "chat.completion" and j["choices"][0]["message"]["role"] == "assistant"
    assert j["choices"][0]["finish_reason"] in ("length", "stop")
    u = j["usage"]
    assert u["completion_tokens"] <= 6 and u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"]
    st2, body2, _ = _post(server, {"messages": [{"role": "user", "content": "hi there"}], "max_tokens": 6, "temperature": 0})
    assert json.loads(body2)["choices"][0]["message"] == j["choices"][0]["message"]       # greedy is deterministic


def test_streaming_sse(server):
    st, body, hdr = _post(server, {"messages": [{"role": "user", "content": "stream"}], "max_tokens": 5, "temperature": 0,
                                   "stream": True, "stream_options": {"include_usage": True}})
    assert st == 200 and hdr["Content-Type"].startswith("text/event-stream")
    events = [l[6:] for l in body.decode().split("\n") if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert chunks[0]["choices"][0]["delta"].get("role") == "assistant"
    assert any(c["choices"] and c["choices"][0].get("finish_reason") for c in chunks)
    assert any(c.get("usage") for c in chunks)


def test_errors(server):
    st, body, _ = _post(server, None, raw=b"{not json")
    assert st == 400 and json.loads(body)["error"]["type"] == "invalid_request_error"
    st, body, _ = _post(server, {"messages": []})
    assert st == 400
    st, body, _ = _post(server, {"messages": [{"role": "user", "content": "x " * 2000}]})
    assert st == 400 and "context" in json.loads(body)["error"]["message"]
    st, body, _ = _post(server, {"messages": [{"role": "user", "content": "x"}]}, path="/v1/other")
    assert st == 404


def test_parse_request_validation():
    with pytest.raises(RequestError):
        parse_request(b"[]")
    with pytest.raises(RequestError):
        parse_request(json.dumps({"messages": [{"role": "user", "content": "a"}], "temperature": "hot"}).encode())
    r = parse_request(json.dumps({"messages": [{"role": "user", "content": [{"type": "text", "text": "a"}, {"type": "text", "text": "b"}]}],
                                  "top_p": 0.5, "max_completion_tokens": 9}).encode())
    assert r.messages[0]["content"] == "ab" and r.sampling["top_p"] == 0.5 and r.max_tokens == 9


def test_think_splitter_handles_split_tags():
    s = ThinkSplitter()
    out = [s.push(p) for p in ["<th", "ink>plan", " more</thi", "nk>answer", " tail"]]
    out.append(s.flush())
    reasoning = "".join(o[0] for o in out)
    content = "".join(o[1] for o in out)
    assert reasoning == "plan more" and content == "answer tail"
    s2 = ThinkSplitter(starts_in_thinking=True)
    a = s2.push("deep</think>ok")
    b = s2.flush()
    assert a[0] + b[0] == "deep" and a[1] + b[1] == "ok"


def test_tool_call_parser():
    text = 'I will call.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>'
    p = parse_tool_calls(text)
    assert p.has_tool_calls and p.tool_calls[0]["function"]["name"] == "get_weather"
    assert json.loads(p.tool_calls[0]["function"]["arguments"]) == {"city": "Paris"}
    assert "tool_call" not in p.content
    assert not parse_tool_calls("plain text").has_tool_calls
    assert not parse_tool_calls("<tool_call>{broken</tool_call>").has_tool_calls


def test_chat_template_renders_tools_and_thinking():
    from llaminar_b200.models.synth import CHATML_TEMPLATE
    t = ChatTemplate(CHATML_TEMPLATE)
    s = t.render([{"role": "system", "content": "sys"}, {"role": "user", "content": "q"}])
    assert "<|im_start|>system\nsys<|im_end|>" in s and s.rstrip().endswith("<|im_start|>assistant")
    with pytest.raises(Exception):
        ChatTemplate("{{ raise_exception('bad') }}").render([])


def test_text_completion_endpoint(server):
    st, body, _ = _post(server, {"prompt": "once upon a time", "max_tokens": 5, "temperature": 0}, path="/v1/completions")
    assert st == 200
    j = json.loads(body)
    assert j["object"] == "text_completion" and j["usage"]["completion_tokens"] <= 5 and isinstance(j["choices"][0]["text"], str)
    st, body, _ = _post(server, {"prompt": "", "max_tokens": 5}, path="/v1/completions")
    assert st == 400 and json.loads(body)["error"]["param"] == "prompt"
    st, body, _ = _post(server, {"prompt": "x", "max_tokens": 0}, path="/v1/completions")
    assert st == 400


@pytest.mark.parametrize("shape,flags", [("tiny-qwen3", []), ("tiny-qwen35", ["--prefix-cache"])], ids=["dense", "hybrid-with-prefix-cache"])
def test_serve_process_end_to_end(tmp_path, shape, flags):
    """The `serve` command as a separate process: wait for /health, one chat completion, one streamed completion, a
    long prompt, then SIGTERM and a clean exit (the reference drives its server the same way from a shell script:
    tests/v2/e2e/server/test_server_e2e.sh).  Once for a dense model, once for a hybrid linear-attention model with the
    prefix cache on (state slots and snapshots behind the same API)."""
    import http.client
    import json
    import signal
    import socket
    import subprocess
    import sys
    import time
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    log = open(tmp_path / "serve.log", "w")
    proc = subprocess.Popen([sys.executable, "-m", "llaminar_b200", "serve", "--synthetic", shape, "--synthetic-recipe", "Q8_0",
                             "-d", "cpu", "--host", "127.0.0.1", "--port", str(port), "-c", "512"] + flags, stdout=log, stderr=subprocess.STDOUT)
    try:
        deadline = time.time() + 120
        ready = False
        while time.time() < deadline and proc.poll() is None:
            try:
                c = http.client.HTTPConnection("127.0.0.1", port, timeout=5)
                c.request("GET", "/health")
                if c.getresponse().status == 200:
                    ready = True
                    break
            except OSError:
                time.sleep(0.5)
        assert ready, (tmp_path / "serve.log").read_text()[-2000:]

        def post(body):
            c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
            c.request("POST", "/v1/chat/completions", body=json.dumps(body), headers={"Content-Type": "application/json"})
            r = c.getresponse()
            return r.status, r.read().decode()
        st, body = post({"messages": [{"role": "user", "content": "What is 2 + 2?"}], "max_tokens": 8, "temperature": 0})
        j = json.loads(body)
        assert st == 200 and j["choices"][0]["finish_reason"] in ("length", "stop") and j["usage"]["completion_tokens"] <= 8
        st, body = post({"messages": [{"role": "user", "content": "count"}], "max_tokens": 6, "temperature": 0, "stream": True})
        events = [ln[6:] for ln in body.splitlines() if ln.startswith("data: ")]
        assert st == 200 and events[-1] == "[DONE]" and all("chat.completion.chunk" in e for e in events[:-1])
        st, body = post({"messages": [{"role": "user", "content": "lorem ipsum " * 15}], "max_tokens": 4, "temperature": 0})
        assert st == 200 and json.loads(body)["usage"]["prompt_tokens"] > 100
        st, body = post({"messages": [{"role": "user", "content": "lorem ipsum " * 60}], "max_tokens": 4, "temperature": 0})
        assert st == 400 and json.loads(body)["error"]["type"] == "context_length_exceeded"
        st, body = post({"messages": "not a list"})
        assert st == 400
        proc.send_signal(signal.SIGTERM)
        assert proc.wait(timeout=60) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
        log.close()


def test_stop_sequences_cut_the_text_in_chat_stream_and_completions(server):
    from llaminar_b200.serve.chat_handler import StopMatcher
    m = StopMatcher(["END", "###"])
    out = [m.push(t) for t in ("abc E", "N", "x EN", "D tail")]
    assert "".join(out) == "abc ENx " and m.hit and m.flush() == ""          # held back "E", "EN" until they were settled
    m2 = StopMatcher(["END"])
    assert m2.push("no stop here E") == "no stop here " and m2.flush() == "E" and not m2.hit
    msgs = [{"role": "user", "content": "hi there"}]
    st, body, _ = _post(server, {"messages": msgs, "max_tokens": 10, "temperature": 0})
    full = json.loads(body)["choices"][0]["message"]["content"]
    assert len(full) > 12
    stop = full[len(full) // 2: len(full) // 2 + 5]
    want = full[:full.find(stop)]
    st, body, _ = _post(server, {"messages": msgs, "max_tokens": 10, "temperature": 0, "stop": stop})
    j = json.loads(body)
    assert st == 200 and j["choices"][0]["message"]["content"] == want and j["choices"][0]["finish_reason"] == "stop"
    st, body, _ = _post(server, {"messages": msgs, "max_tokens": 10, "temperature": 0, "stop": ["zzzz", stop], "stream": True})
    chunks = [json.loads(l[6:]) for l in body.decode().split("\n") if l.startswith("data: ") and l[6:] != "[DONE]"]
    streamed = "".join(c["choices"][0]["delta"].get("content") or "" for c in chunks if c["choices"])
    assert streamed == want
    st, body, _ = _post(server, {"messages": msgs, "stop": [1, 2]})
    assert st == 400 and json.loads(body)["error"]["param"] == "stop"
    st, body, _ = _post(server, {"prompt": "hi there", "max_tokens": 10, "temperature": 0}, path="/v1/completions")
    text = json.loads(body)["choices"][0]["text"]
    stop2 = text[len(text) // 2: len(text) // 2 + 5]
    st, body, _ = _post(server, {"prompt": "hi there", "max_tokens": 10, "temperature": 0, "stop": stop2}, path="/v1/completions")
    assert st == 200 and json.loads(body)["choices"][0]["text"] == text[:text.find(stop2)]
    # the engine is still healthy after the cancellations
    st, body, _ = _post(server, {"messages": msgs, "max_tokens": 4, "temperature": 0})
    assert st == 200


def test_metrics_endpoint_counts_requests_and_tokens(server):
    def scrape():
        c = http.client.HTTPConnection("127.0.0.1", server.port, timeout=30)
        c.request("GET", "/metrics")
        r = c.getresponse()
        text = r.read().decode()
        assert r.status == 200 and r.getheader("Content-Type").startswith("text/plain")
        return {ln.split()[0]: float(ln.split()[1]) for ln in text.splitlines() if ln and not ln.startswith("#")}, text
    before, text = scrape()
    assert "# TYPE llaminar_generated_tokens counter" in text and "# TYPE llaminar_requests_running gauge" in text
    st, body, _ = _post(server, {"messages": [{"role": "user", "content": "count me"}], "max_tokens": 5, "temperature": 0})
    used = json.loads(body)["usage"]
    after, _ = scrape()
    assert after["llaminar_requests_finished"] == before["llaminar_requests_finished"] + 1
    assert after["llaminar_generated_tokens"] - before["llaminar_generated_tokens"] == used["completion_tokens"]
    assert after["llaminar_prompt_tokens"] - before["llaminar_prompt_tokens"] == used["prompt_tokens"]
    assert after["llaminar_requests_running"] == 0 and after["llaminar_kv_pages_free"] > 0
    assert after["llaminar_ttft_seconds_count"] == before["llaminar_ttft_seconds_count"] + 1
    d_ttft = after["llaminar_ttft_seconds_sum"] - before["llaminar_ttft_seconds_sum"]
    d_req = after["llaminar_request_seconds_sum"] - before["llaminar_request_seconds_sum"]
    assert 0 < d_ttft <= d_req < 120


def test_n_choices_run_as_parallel_requests(server):
    msgs = [{"role": "user", "content": "pick something"}]
    st, body, _ = _post(server, {"messages": msgs, "max_tokens": 6, "temperature": 1.0, "top_k": 0, "top_p": 1.0, "seed": 3, "n": 3})
    j = json.loads(body)
    assert st == 200 and [c["index"] for c in j["choices"]] == [0, 1, 2]
    texts = [c["message"]["content"] for c in j["choices"]]
    assert len(set(texts)) > 1                                   # different seeds: the draws differ
    assert j["usage"]["completion_tokens"] <= 18 and j["usage"]["total_tokens"] == j["usage"]["prompt_tokens"] + j["usage"]["completion_tokens"]
    # choice 0 is what a single request with the same seed returns
    st, body, _ = _post(server, {"messages": msgs, "max_tokens": 6, "temperature": 1.0, "top_k": 0, "top_p": 1.0, "seed": 3})
    assert json.loads(body)["choices"][0]["message"]["content"] == texts[0]
    st, body, _ = _post(server, {"messages": msgs, "n": 2, "stream": True})
    assert st == 400 and json.loads(body)["error"]["param"] == "n"
    st, body, _ = _post(server, {"messages": msgs, "n": 0})
    assert st == 400


def test_logprobs_in_chat_completions(server):
    msgs = [{"role": "user", "content": "count to three"}]
    st, body, _ = _post(server, {"messages": msgs, "max_tokens": 5, "temperature": 0, "presence_penalty": 0,
                                 "logprobs": True, "top_logprobs": 2})
    j = json.loads(body)
    assert st == 200
    items = j["choices"][0]["logprobs"]["content"]
    assert 1 <= len(items) <= 5
    for it in items:
        assert it["logprob"] <= 0.0 and bytes(it["bytes"]).decode("utf-8", errors="replace") == it["token"]
        assert len(it["top_logprobs"]) == 2 and it["top_logprobs"][0]["logprob"] >= it["top_logprobs"][1]["logprob"]
        assert it["top_logprobs"][0]["token"] == it["token"]           # greedy, no penalties: the likeliest token is emitted
    st, body, _ = _post(server, {"messages": msgs, "max_tokens": 5, "temperature": 0})
    assert "logprobs" not in json.loads(body)["choices"][0]
    # streamed: the entries arrive with the chunks and add up to the same list
    st, body, _ = _post(server, {"messages": msgs, "max_tokens": 5, "temperature": 0, "presence_penalty": 0,
                                 "logprobs": True, "top_logprobs": 2, "stream": True})
    assert st == 200
    streamed = []
    for ln in body.decode().splitlines():
        if ln.startswith("data: {"):
            ch = json.loads(ln[6:])["choices"][0]
            streamed += (ch.get("logprobs") or {}).get("content", [])
    assert streamed == items
    for bad in ({"logprobs": 1}, {"top_logprobs": 2}, {"logprobs": True, "top_logprobs": 21}):
        st, body, _ = _post(server, dict({"messages": msgs}, **bad))
        assert st == 400 and json.loads(body)["error"]["param"] in ("logprobs", "top_logprobs")


def test_no_kv_page_leak_across_request_kinds(server):
    """Every way a request can end (length, stop sequence with cancellation, several choices, a client that goes away in
    mid-stream, a rejected request) gives its KV pages back: the free-page gauge returns to its idle value."""
    import time

    def free_pages():
        c = http.client.HTTPConnection("127.0.0.1", server.port, timeout=30)
        c.request("GET", "/metrics")
        text = c.getresponse().read().decode()
        vals = {ln.split()[0]: float(ln.split()[1]) for ln in text.splitlines() if ln and not ln.startswith("#")}
        return vals["llaminar_kv_pages_free"], vals["llaminar_requests_running"]

    def idle_free():
        for _ in range(100):
            free, running = free_pages()
            if running == 0:
                return free
            time.sleep(0.05)
        raise AssertionError("requests still running")

    base = idle_free()
    msgs = [{"role": "user", "content": "tell me a story about pages"}]
    _post(server, {"messages": msgs, "max_tokens": 40, "temperature": 0})
    _post(server, {"messages": msgs, "max_tokens": 40, "temperature": 1.0, "seed": 1, "n": 3})
    first = json.loads(_post(server, {"messages": msgs, "max_tokens": 12, "temperature": 0})[1])["choices"][0]["message"]["content"]
    if len(first) > 4:
        _post(server, {"messages": msgs, "max_tokens": 40, "temperature": 0, "stop": [first[2:4]]})
    # a streaming client that disconnects after the first chunk
    c = http.client.HTTPConnection("127.0.0.1", server.port, timeout=30)
    c.request("POST", "/v1/chat/completions", body=json.dumps({"messages": msgs, "max_tokens": 200, "stream": True}).encode(),
              headers={"Content-Type": "application/json"})
    r = c.getresponse()
    r.read(20)
    c.close()
    _post(server, {"messages": [{"role": "user", "content": "x " * 2000}], "max_tokens": 4})       # context overflow: 400
    assert idle_free() == base


def test_usage_reports_reasoning_tokens_for_thinking_templates(server):
    st, body, _ = _post(server, {"messages": [{"role": "user", "content": "think about it"}], "max_tokens": 8, "temperature": 0})
    u = json.loads(body)["usage"]
    if server.chat.template.expects_thinking:
        assert 0 <= u["completion_tokens_details"]["reasoning_tokens"] <= u["completion_tokens"]
    else:
        assert "completion_tokens_details" not in u


def test_tool_call_parser_reads_the_tagged_function_layout():
    text = ("Let me check.\n<tool_call>\n<function=get_weather>\n<parameter=city>\nParis\n</parameter>\n<parameter=days>\n3\n</parameter>\n"
            "<parameter=opts>\n{\"units\": \"C\"}\n</parameter>\n</function>\n</tool_call>")
    p = parse_tool_calls(text)
    assert p.has_tool_calls and p.content == "Let me check."
    fn = p.tool_calls[0]["function"]
    assert fn["name"] == "get_weather" and json.loads(fn["arguments"]) == {"city": "Paris", "days": 3, "opts": {"units": "C"}}
    # two calls in one block, a multi-line string value, and a block that is neither JSON nor tagged stays as text
    two = parse_tool_calls("<tool_call><function=a><parameter=x>line1\nline2</parameter></function><function=b></function></tool_call>")
    assert [c["function"]["name"] for c in two.tool_calls] == ["a", "b"]
    assert json.loads(two.tool_calls[0]["function"]["arguments"]) == {"x": "line1\nline2"}
    junk = parse_tool_calls("<tool_call>not a call</tool_call>")
    assert not junk.has_tool_calls and junk.content == "<tool_call>not a call</tool_call>"


def test_api_key_guards_the_v1_endpoints(server):
    srv = Server(server.chat, "127.0.0.1", 0, api_key="s3cret", owns_loop=False)
    srv.start_background()
    try:
        body = json.dumps({"messages": [{"role": "user", "content": "hi"}], "max_tokens": 2, "temperature": 0}).encode()

        def call(method, path, headers, data=None):
            c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=60)
            c.request(method, path, body=data, headers=headers)
            r = c.getresponse()
            return r.status, r.read()

        assert call("GET", "/health", {})[0] == 200                                    # probes stay open
        st, out = call("POST", "/v1/chat/completions", {"Content-Type": "application/json"}, body)
        assert st == 401 and json.loads(out)["error"]["code"] == "invalid_api_key"
        assert call("POST", "/v1/chat/completions", {"Authorization": "Bearer wrong"}, body)[0] == 401
        assert call("GET", "/v1/models", {})[0] == 401
        st, out = call("POST", "/v1/chat/completions", {"Authorization": "Bearer s3cret", "Content-Type": "application/json"}, body)
        assert st == 200 and json.loads(out)["object"] == "chat.completion"
        assert call("GET", "/v1/models", {"Authorization": "Bearer s3cret"})[0] == 200
    finally:
        srv.stop()
    assert _post(server, {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 2})[0] == 200     # the shared loop lives on


def test_text_completion_streams_the_same_text(server):
    req = {"prompt": "Once upon a time", "max_tokens": 8, "temperature": 0}
    st, body, _ = _post(server, req, path="/v1/completions")
    whole = json.loads(body)
    assert st == 200
    st, body, hdr = _post(server, dict(req, stream=True), path="/v1/completions")
    assert st == 200 and hdr["Content-Type"].startswith("text/event-stream")
    lines = [ln for ln in body.decode().splitlines() if ln.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(ln[6:]) for ln in lines[:-1]]
    assert all(c["object"] == "text_completion" for c in chunks)
    assert "".join(c["choices"][0]["text"] for c in chunks) == whole["choices"][0]["text"]
    assert chunks[-1]["choices"][0]["finish_reason"] == whole["choices"][0]["finish_reason"]
    assert chunks[-1]["usage"] == whole["usage"] and all(c["choices"][0]["finish_reason"] is None for c in chunks[:-1])
    st, body, _ = _post(server, {"prompt": "", "stream": True}, path="/v1/completions")
    assert st == 400                                              # setup errors arrive as JSON, not as a stream


def test_load_generator_against_the_in_process_server(server, tmp_path):
    from llaminar_b200.serve import loadgen
    s = loadgen.run(f"http://127.0.0.1:{server.port}", concurrency=3, requests=6, prompt_tokens=24, max_tokens=5)
    assert s["succeeded"] == 6 and s["failed"] == 0 and 6 <= s["output_tokens"] <= 30
    assert s["ttft_ms"]["p50"] > 0 and s["ttft_ms"]["p99"] >= s["ttft_ms"]["p50"] and s["output_tok_per_s"] > 0
    out = tmp_path / "lg.json"
    assert loadgen.main(["--url", f"http://127.0.0.1:{server.port}", "--concurrency", "2", "--requests", "2", "--prompt-tokens", "16",
                         "--max-tokens", "3", "--json", str(out)]) == 0
    assert json.loads(out.read_text())["succeeded"] == 2
    t = loadgen.run(f"http://127.0.0.1:{server.port}", concurrency=2, requests=3, prompt_tokens=16, max_tokens=4, endpoint="completions")
    assert t["succeeded"] == 3 and 3 <= t["output_tokens"] <= 12 and t["ttft_ms"]["p50"] > 0
    bad = loadgen.run("http://127.0.0.1:9", concurrency=1, requests=1, prompt_tokens=8, max_tokens=2, timeout=5)
    assert bad["failed"] == 1 and bad["errors"]
    assert loadgen.percentile([1.0, 2.0, 3.0, 4.0], 50) in (2.0, 3.0) and loadgen.percentile([], 99) == 0.0


def test_soak_under_kv_pressure_every_request_completes():
    """Streamed requests at a concurrency the KV cache cannot hold (prefix cache on): admission waits, sequences are
    preempted and resumed, and every request still gets its full answer; afterwards every page is either free or held
    by the prefix cache alone."""
    from llaminar_b200.engine.prefix_cache import PrefixCache, PrefixCacheConfig
    from llaminar_b200.serve import loadgen
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    pc = PrefixCache(PrefixCacheConfig(), "fp")
    eng = LLMEngine(w, device="cpu", max_batch=8, max_context=512, kv_pages=12, prefix_cache=pc)
    tok = BPETokenizer.from_metadata(w.metadata)
    loop = EngineLoop(eng)
    chat = ChatCompletionHandler(loop, tok, ChatTemplate.resolve(None, tok.chat_template), "qwen3", 512, model_name="tiny", eos_ids=())
    srv = Server(chat, "127.0.0.1", 0)
    srv.start_background()
    try:
        s = loadgen.run(f"http://127.0.0.1:{srv.port}", concurrency=8, requests=12, prompt_tokens=30, max_tokens=200, temperature=0.8)
        assert s["succeeded"] == 12 and s["failed"] == 0 and s["output_tokens"] == 12 * 200
        assert loop.errors == 0 and eng.stats["preemptions"] >= 1
        m = loop.metrics()
        assert m["requests_finished"] == 12 and m["requests_running"] == 0 and m["requests_waiting"] == 0
        assert eng.kv.allocator.n_free + len(pc.device) == eng.kv.n_pages - 1
        assert all(r <= 1 for r in eng.kv.allocator.refs)
    finally:
        srv.stop()


def test_prompt_that_cannot_fit_the_cache_gets_400_and_the_server_goes_on():
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=0)
    eng = LLMEngine(w, device="cpu", max_batch=2, max_context=512, kv_pages=3)            # room for 128 tokens in all
    tok = BPETokenizer.from_metadata(w.metadata)
    loop = EngineLoop(eng)
    chat = ChatCompletionHandler(loop, tok, ChatTemplate.resolve(None, tok.chat_template), "qwen3", 512, model_name="tiny", eos_ids=())
    srv = Server(chat, "127.0.0.1", 0)
    srv.start_background()
    try:
        long_msg = {"messages": [{"role": "user", "content": "word " * 60}], "max_tokens": 4}
        for stream in (False, True):
            st, body, _ = _post(srv, dict(long_msg, stream=stream))
            assert st == 400 and json.loads(body)["error"]["type"] == "context_length_exceeded", body[:200]
        st, body, _ = _post(srv, {"prompt": "word " * 150, "max_tokens": 4}, path="/v1/completions")
        assert st == 400
        st, body, _ = _post(srv, {"prompt": "hi", "max_tokens": 3, "temperature": 0}, path="/v1/completions")
        assert st == 200 and loop.errors == 0
    finally:
        srv.stop()


def test_the_official_openai_client_talks_to_the_server(server):
    """The `openai` Python client (which validates every response against its typed schema) against the in-process server:
    model list, chat completion, streamed chat completion with usage, `n` choices with log-probabilities, a stop sequence, a
    text completion, and the error shape for a bad request."""
    openai = pytest.importorskip("openai")
    client = openai.OpenAI(base_url=f"http://127.0.0.1:{server.port}/v1", api_key="unused", max_retries=0, timeout=120)
    assert [m.id for m in client.models.list().data] == ["tiny"]
    msgs = [{"role": "system", "content": "Be brief."}, {"role": "user", "content": "hello there"}]
    r = client.chat.completions.create(model="tiny", messages=msgs, max_tokens=6, temperature=0)
    assert r.object == "chat.completion" and r.choices[0].message.role == "assistant" and r.choices[0].finish_reason in ("length", "stop")
    assert r.usage.completion_tokens <= 6 and r.usage.total_tokens == r.usage.prompt_tokens + r.usage.completion_tokens
    chunks = list(client.chat.completions.create(model="tiny", messages=msgs, max_tokens=6, temperature=0, stream=True,
                                                 stream_options={"include_usage": True}))
    assert chunks and all(c.object == "chat.completion.chunk" for c in chunks)
    streamed = "".join(c.choices[0].delta.content or "" for c in chunks if c.choices)
    assert streamed == (r.choices[0].message.content or "")                     # greedy: the stream carries the same text
    assert any(c.choices and c.choices[0].finish_reason for c in chunks)
    r = client.chat.completions.create(model="tiny", messages=msgs, max_tokens=4, temperature=0.8, seed=3, n=2, logprobs=True, top_logprobs=2)
    assert len(r.choices) == 2 and [c.index for c in r.choices] == [0, 1]
    lp = r.choices[0].logprobs.content
    assert lp and all(len(t.top_logprobs) == 2 and t.logprob <= 0.0 for t in lp)
    full = client.chat.completions.create(model="tiny", messages=msgs, max_tokens=12, temperature=0).choices[0].message.content or ""
    if len(full) > 3:
        cut = client.chat.completions.create(model="tiny", messages=msgs, max_tokens=12, temperature=0, stop=[full[2:4]])
        assert cut.choices[0].finish_reason == "stop" and cut.choices[0].message.content == full[:2]
    t = client.completions.create(model="tiny", prompt="Once upon", max_tokens=5, temperature=0)
    assert t.object == "text_completion" and t.choices[0].finish_reason in ("length", "stop") and t.usage.completion_tokens <= 5
    with pytest.raises(openai.BadRequestError) as e:
        client.chat.completions.create(model="tiny", messages=[], max_tokens=1)
    assert e.value.status_code == 400
