"""OpenAI-compatible `/v1/chat/completions` request handling: validation, sampling merge, chat-template
encoding, context-window check, generation loop with stop tokens, reasoning / content split, thinking
budget with forced stop-thinking injection, tool-call extraction, `usage` accounting, SSE chunks.

Behaviour follows the reference handler (reference: src/v2/app/modes/ChatCompletionHandler.cpp:554 parse,
:753 setup, :867 non-streaming, :1165 streaming, :1137-1145 response schema; error objects are
`{"error": {"message", "type"}}` with 400 for invalid requests / context overflow and 500 for runtime failures).
"""
from __future__ import annotations

import json
import queue
import time
import uuid
from dataclasses import dataclass, field
from typing import Iterator

from ..engine.sampling import SamplingParams, merge_with_model_defaults
from ..tokenizer.bpe import StreamDecoder
from ..tokenizer.chat_template import ThinkSplitter
from .tool_parser import parse_tool_calls

SYSTEM_FINGERPRINT = "llaminar-b200"
STOP_THINKING_TEXT = "\n\nConsidering the limited time by the user, I have to give the solution based on the thinking directly now.\n</think>\n\n"
CACHE_FULL = "the prompt does not fit the KV cache of this server even when nothing else is running"
_SAMPLING_FIELDS = ("temperature", "top_p", "top_k", "seed", "presence_penalty", "frequency_penalty",
                    "dry_multiplier", "dry_base", "dry_allowed_length")


class RequestError(Exception):
    def __init__(self, message: str, status: int = 400, err_type: str = "invalid_request_error", param: str | None = None):
        super().__init__(message)
        self.status, self.err_type, self.param = status, err_type, param

    def body(self) -> dict:
        e = {"message": str(self), "type": self.err_type}
        if self.param:
            e["param"] = self.param
        return {"error": e}


@dataclass
class ChatRequest:
    messages: list[dict]
    max_tokens: int = -1
    stream: bool = False
    enable_thinking: bool = True
    model: str = ""
    sampling: dict = field(default_factory=dict)
    thinking_budget_tokens: int = -1
    tools: list | None = None
    tool_choice: object = None
    parallel_tool_calls: bool = True
    stop: list = field(default_factory=list)
    n: int = 1
    logprobs: bool = False
    top_logprobs: int = 0


def parse_stop(value) -> list[str]:
    """OpenAI ``stop``: a string or up to four strings (an extension of the reference's API, which stops on EOS only)."""
    if value is None:
        return []
    items = [value] if isinstance(value, str) else value
    if not isinstance(items, list) or len(items) > 4 or not all(isinstance(s, str) for s in items):
        raise RequestError("`stop` must be a string or an array of at most 4 strings", param="stop")
    return [s for s in items if s]


class StopMatcher:
    """Cuts generated text at the first stop sequence.  Text is released as soon as it can no longer be the beginning of
    a stop sequence, so streaming stays incremental and never shows a part of the sequence itself."""

    def __init__(self, stops: list[str]):
        self.stops = stops
        self.buf = ""
        self.hit = False

    def push(self, text: str) -> str:
        if self.hit or not self.stops:
            return "" if self.hit else text
        self.buf += text
        found = [i for i in (self.buf.find(s) for s in self.stops) if i >= 0]
        if found:
            out, self.buf, self.hit = self.buf[:min(found)], "", True
            return out
        hold = 0
        for k in range(min(max(len(s) for s in self.stops) - 1, len(self.buf)), 0, -1):
            if any(s.startswith(self.buf[-k:]) for s in self.stops):
                hold = k
                break
        out, self.buf = self.buf[:len(self.buf) - hold], self.buf[len(self.buf) - hold:]
        return out

    def flush(self) -> str:
        out, self.buf = ("" if self.hit else self.buf), ""
        return out


def parse_request(body_bytes: bytes) -> ChatRequest:
    try:
        body = json.loads(body_bytes)
    except (json.JSONDecodeError, UnicodeDecodeError) as exc:
        raise RequestError(f"Invalid JSON: {exc}") from exc
    if not isinstance(body, dict):
        raise RequestError("request body must be a JSON object")
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise RequestError('"messages" field is required and must be a non-empty array', param="messages")
    for m in msgs:
        if not isinstance(m, dict) or "role" not in m:
            raise RequestError('Each message must have a "role" field')
        role = m["role"]
        if role == "assistant" and "tool_calls" in m:
            continue
        if role == "tool":
            if "tool_call_id" not in m:
                raise RequestError('Tool messages must have a "tool_call_id" field')
            continue
        if "content" not in m:
            raise RequestError('Each message must have "role" and "content" fields')
    req = ChatRequest(messages=[])
    try:
        if "max_tokens" in body:
            req.max_tokens = int(body["max_tokens"])
        elif "max_completion_tokens" in body:
            req.max_tokens = int(body["max_completion_tokens"])
        req.stream = bool(body.get("stream", False))
        req.enable_thinking = bool(body.get("enable_thinking", True))
        req.model = str(body.get("model", ""))
        for k in _SAMPLING_FIELDS:
            if k in body and body[k] is not None:
                req.sampling[k] = int(body[k]) if k in ("top_k", "seed", "dry_allowed_length") else float(body[k])
        if "thinking_budget_tokens" in body:
            req.thinking_budget_tokens = int(body["thinking_budget_tokens"])
    except (TypeError, ValueError) as exc:
        raise RequestError(f"bad parameter value: {exc}") from exc
    if isinstance(body.get("tools"), list):
        req.tools = body["tools"]
    req.tool_choice = body.get("tool_choice")
    req.parallel_tool_calls = bool(body.get("parallel_tool_calls", True))
    req.stop = parse_stop(body.get("stop"))
    n = body.get("n", 1)
    if not isinstance(n, int) or isinstance(n, bool) or not 1 <= n <= 8:
        raise RequestError("`n` must be an integer between 1 and 8", param="n")
    if n > 1 and req.stream:
        raise RequestError("`n` > 1 is not supported together with `stream`", param="n")
    req.n = n
    lp, top = body.get("logprobs", False), body.get("top_logprobs")
    if not isinstance(lp, bool):
        raise RequestError("`logprobs` must be a boolean", param="logprobs")
    if top is not None:
        if not isinstance(top, int) or isinstance(top, bool) or not 0 <= top <= 20:
            raise RequestError("`top_logprobs` must be an integer between 0 and 20", param="top_logprobs")
        if not lp:
            raise RequestError("`top_logprobs` needs `logprobs` to be true", param="top_logprobs")
    req.logprobs, req.top_logprobs = lp, int(top or 0)
    for m in msgs:
        cm = {"role": str(m["role"]), "content": "" if m.get("content") is None else m.get("content")}
        if isinstance(cm["content"], list):        # OpenAI content parts: keep the text parts
            cm["content"] = "".join(p.get("text", "") for p in cm["content"] if isinstance(p, dict))
        if isinstance(m.get("tool_calls"), list):
            cm["tool_calls"] = m["tool_calls"]
        for k in ("tool_call_id", "name"):
            if k in m:
                cm[k] = m[k]
        req.messages.append(cm)
    return req


class ChatCompletionHandler:
    def __init__(self, loop, tokenizer, template, arch: str, max_context: int, model_name: str = "llaminar",
                 cli_sampling: SamplingParams | None = None, eos_ids: tuple[int, ...] = ()):
        self.loop, self.tok, self.template = loop, tokenizer, template
        self.arch, self.max_context, self.model_name = arch, max_context, model_name
        self.cli_sampling = cli_sampling
        self.eos_ids = tuple(eos_ids)

    # -- shared setup ---------------------------------------------------------------------------------------
    def _setup(self, req: ChatRequest):
        text = self.template.render(req.messages, tools=req.tools, add_generation_prompt=True,
                                    enable_thinking=req.enable_thinking)
        ids = self.tok.encode(text, add_special=True)
        if len(ids) + 1 >= self.max_context:
            raise RequestError(f"prompt of {len(ids)} tokens does not fit the context window of {self.max_context}",
                               err_type="context_length_exceeded")
        budget = self.max_context - len(ids) - 1
        max_tokens = budget if req.max_tokens < 0 else min(req.max_tokens, budget)
        if max_tokens < 1:
            raise RequestError("max_tokens must be at least 1")
        sp = merge_with_model_defaults(self.arch, req.sampling, self.cli_sampling)
        sp.max_tokens = max_tokens
        sp.stop_token_ids = tuple(self.eos_ids)
        if req.logprobs:
            sp.logprobs = req.top_logprobs
        starts_in_think = text.rstrip().endswith("<think>")
        return ids, sp, starts_in_think

    def _generate(self, req: ChatRequest) -> Iterator[tuple[str, object]]:
        """Yields ("delta", (reasoning, content)) ... then ("end", info dict).  When the request asks for log-probabilities
        the first event is ("logprobs", list): the live list that receives one entry per generated token (a streaming
        consumer sends the entries added since its previous chunk); ``info["logprobs"]`` is the same list."""
        ids, sp, starts_in_think = self._setup(req)
        ticket = self.loop.submit(ids, sp)
        dec = StreamDecoder(self.tok, skip_special=True)
        splitter = ThinkSplitter(starts_in_think) if self.template.expects_thinking else None
        budget_on = req.thinking_budget_tokens >= 0 and req.enable_thinking and splitter is not None
        stop_ids = self.tok.encode(STOP_THINKING_TEXT, parse_special=True) if budget_on else []
        injected = False
        thinking_tokens = 0
        n_completion = 0
        finish = "stop"
        stopper = StopMatcher(req.stop)
        token_logprobs: list = []
        if req.logprobs:
            yield "logprobs", token_logprobs              # the live list: a streaming consumer reads new entries from it
        if budget_on and req.thinking_budget_tokens == 0 and stop_ids:
            for t in stop_ids:
                self.loop.force_token(ticket, t)
            injected = True
        try:
            while True:
                try:
                    ev = ticket.events.get(timeout=600)
                except queue.Empty:
                    raise RequestError("generation timed out", 500, "server_error")
                if ev[0] == "error":
                    raise RequestError(ev[1], ev[2] if len(ev) > 2 else 500,
                                       "invalid_request_error" if (len(ev) > 2 and ev[2] == 400) else "server_error")
                if ev[0] == "done":
                    finish = ev[1] or "stop"
                    if finish == "cache_full":
                        raise RequestError(CACHE_FULL, err_type="context_length_exceeded")
                    break
                if stopper.hit:
                    continue                                  # tokens that were in flight when the stop sequence appeared
                for k, tid in enumerate(ev[1]):
                    n_completion += 1
                    if tid in self.eos_ids:
                        continue
                    if len(ev) > 2 and ev[2]:
                        token_logprobs.append(ev[2][k])
                    piece = dec.push(tid)
                    if splitter is None:
                        piece = stopper.push(piece)
                        if piece:
                            yield "delta", ("", piece)
                        if stopper.hit:
                            break
                        continue
                    was_thinking = splitter.in_think
                    r, c = splitter.push(piece)
                    c = stopper.push(c) if c else c
                    if was_thinking:
                        thinking_tokens += 1
                    if r or c:
                        yield "delta", (r, c)
                    if stopper.hit:
                        break
                    if budget_on and not injected and splitter.in_think and thinking_tokens >= req.thinking_budget_tokens:
                        for t in stop_ids:
                            self.loop.force_token(ticket, t)
                        injected = True
                if stopper.hit:
                    self.loop.cancel(ticket)                  # the engine frees the sequence; a "done" event follows
                    finish = "stop"
                    break
            if not stopper.hit:
                tail = dec.flush()
                if tail:
                    r, c = splitter.push(tail) if splitter else ("", tail)
                    c = stopper.push(c) if c else c
                    if r or c:
                        yield "delta", (r, c)
                if splitter and not stopper.hit:
                    r, c = splitter.flush()
                    c = stopper.push(c) if c else c
                    if r or c:
                        yield "delta", (r, c)
                rest = stopper.flush()
                if rest:
                    yield "delta", ("", rest)
        except GeneratorExit:
            self.loop.cancel(ticket)
            raise
        yield "end", {"prompt_tokens": len(ids), "completion_tokens": n_completion, "finish_reason": finish,
                      "prefix_hit_tokens": ticket.prefix_hit_tokens, "logprobs": token_logprobs,
                      "reasoning_tokens": thinking_tokens if splitter is not None else None}

    def _logprobs_object(self, entries: list) -> dict:
        """OpenAI `choices[i].logprobs`: one item per generated token with its text, bytes and log-probability under the
        model's distribution, and the `top_logprobs` likeliest alternatives (an extension of the reference's API)."""
        def item(tid: int, lp: float) -> dict:
            raw = self.tok.token_bytes(int(tid))
            return {"token": raw.decode("utf-8", errors="replace"), "logprob": max(float(lp), -9999.0), "bytes": list(raw)}
        return {"content": [dict(item(t, lp), top_logprobs=[item(a, b) for a, b in top]) for t, lp, top in entries]}

    def _usage(self, info: dict) -> dict:
        p, c = info["prompt_tokens"], info["completion_tokens"]
        u = {"prompt_tokens": p, "completion_tokens": c, "total_tokens": p + c, "context_window": self.max_context,
             "context_used": p + c}
        if info.get("prefix_hit_tokens"):
            u["prompt_tokens_details"] = {"cached_tokens": info["prefix_hit_tokens"]}
        if info.get("reasoning_tokens") is not None:
            u["completion_tokens_details"] = {"reasoning_tokens": info["reasoning_tokens"]}
        return u

    # -- non-streaming --------------------------------------------------------------------------------------
    def handle(self, req: ChatRequest) -> dict:
        if req.n > 1:
            return self._handle_many(req)
        return self._handle_one(req)

    def _handle_many(self, req: ChatRequest) -> dict:
        """OpenAI ``n``: the choices are independent requests that run side by side in the engine's batch (and share the
        prompt's prefix-cache blocks); choice i draws with seed + i when the request gives a seed."""
        import copy
        from concurrent.futures import ThreadPoolExecutor
        reqs = []
        for i in range(req.n):
            r = copy.copy(req)
            r.n = 1
            r.sampling = dict(req.sampling)
            if r.sampling.get("seed") is not None:
                r.sampling["seed"] = int(r.sampling["seed"]) + i
            reqs.append(r)
        with ThreadPoolExecutor(max_workers=req.n) as pool:
            outs = list(pool.map(self._handle_one, reqs))
        first = outs[0]
        first["choices"] = [dict(o["choices"][0], index=i) for i, o in enumerate(outs)]
        u = first["usage"]
        u["completion_tokens"] = sum(o["usage"]["completion_tokens"] for o in outs)
        u["total_tokens"] = u["prompt_tokens"] + u["completion_tokens"]
        return first

    def _handle_one(self, req: ChatRequest) -> dict:
        reasoning, content, info = [], [], None
        for kind, payload in self._generate(req):
            if kind == "delta":
                reasoning.append(payload[0])
                content.append(payload[1])
            elif kind == "end":
                info = payload
        text, think = "".join(content), "".join(reasoning)
        finish = "length" if info["finish_reason"] == "length" else "stop"
        message: dict = {"role": "assistant"}
        if req.tools:
            parsed = parse_tool_calls(text)
            if parsed.has_tool_calls:
                calls = parsed.tool_calls if req.parallel_tool_calls else parsed.tool_calls[:1]
                message["content"] = parsed.content or None
                message["tool_calls"] = calls
                finish = "tool_calls"
            else:
                message["content"] = text
        else:
            message["content"] = text
        if think:
            message["reasoning_content"] = think
        choice = {"index": 0, "message": message, "finish_reason": finish}
        if req.logprobs:
            choice["logprobs"] = self._logprobs_object(info["logprobs"])
        return {"id": "chatcmpl-" + uuid.uuid4().hex[:24], "object": "chat.completion", "created": int(time.time()),
                "model": req.model or self.model_name, "system_fingerprint": SYSTEM_FINGERPRINT,
                "choices": [choice], "usage": self._usage(info)}

    # -- raw text completion (no chat template) ---------------------------------------------------------------
    def complete(self, body_bytes: bytes):
        """`/v1/completions`: the prompt is tokenised as is (the reference's completion mode,
        src/v2/app/modes/CompletionMode.cpp).  Returns the OpenAI text_completion object, or with `"stream": true` an
        iterator of server-sent-event chunks of the same shape (setup errors are raised before the first chunk)."""
        try:
            body = json.loads(body_bytes)
        except Exception as exc:
            raise RequestError(f"request body is not valid JSON: {exc}") from exc
        if not isinstance(body, dict) or not isinstance(body.get("prompt"), str) or not body["prompt"]:
            raise RequestError("`prompt` must be a non-empty string", param="prompt")
        ids = self.tok.encode(body["prompt"], add_special=True)
        if len(ids) + 1 >= self.max_context:
            raise RequestError(f"prompt of {len(ids)} tokens does not fit the context window of {self.max_context}",
                               err_type="context_length_exceeded")
        given = {k: body[k] for k in ("temperature", "top_p", "top_k", "seed", "presence_penalty", "frequency_penalty") if k in body}
        for k, v in given.items():
            if not isinstance(v, (int, float)) or isinstance(v, bool):
                raise RequestError(f"`{k}` must be a number", param=k)
        sp = merge_with_model_defaults(self.arch, given, self.cli_sampling)
        budget = self.max_context - len(ids) - 1
        mt = body.get("max_tokens", 16)
        if not isinstance(mt, int) or isinstance(mt, bool) or mt < 1:
            raise RequestError("`max_tokens` must be a positive integer", param="max_tokens")
        sp.max_tokens = min(mt, budget)
        sp.stop_token_ids = tuple(self.eos_ids)
        stops = parse_stop(body.get("stop"))
        rid, created, model = "cmpl-" + uuid.uuid4().hex[:24], int(time.time()), body.get("model") or self.model_name
        pieces = self._complete_pieces(ids, sp, stops)

        def obj(text: str, finish, usage=None) -> dict:
            o = {"id": rid, "object": "text_completion", "created": created, "model": model,
                 "choices": [{"index": 0, "text": text, "finish_reason": finish}]}
            if usage is not None:
                o["usage"] = usage
            return o

        def usage_of(n: int) -> dict:
            return {"prompt_tokens": len(ids), "completion_tokens": n, "total_tokens": len(ids) + n}

        if body.get("stream"):
            first = next(pieces)                         # the request is in the engine (or has failed) before headers go out

            def sse():
                for kind, payload in _chain(first, pieces):
                    if kind == "text":
                        if payload:
                            yield b"data: " + json.dumps(obj(payload, None), ensure_ascii=False).encode() + b"\n\n"
                    else:
                        n, finish = payload
                        yield b"data: " + json.dumps(obj("", finish, usage_of(n)), ensure_ascii=False).encode() + b"\n\n"
                yield b"data: [DONE]\n\n"
            return sse()
        parts, n, finish = [], 0, "stop"
        for kind, payload in pieces:
            if kind == "text":
                parts.append(payload)
            else:
                n, finish = payload
        return obj("".join(parts), finish, usage_of(n))

    def _complete_pieces(self, ids: list[int], sp, stops: list[str]):
        """Yields ("text", piece) while the completion streams, then ("end", (tokens generated, finish reason))."""
        stopper = StopMatcher(stops)
        ticket = self.loop.submit(ids, sp)
        dec = StreamDecoder(self.tok, skip_special=True)
        n, finish = 0, "stop"
        try:
            while True:
                try:
                    ev = ticket.events.get(timeout=600)
                except queue.Empty:
                    raise RequestError("generation timed out", 500, "server_error")
                if ev[0] == "error":
                    raise RequestError(ev[1], ev[2] if len(ev) > 2 else 500,
                                       "invalid_request_error" if (len(ev) > 2 and ev[2] == 400) else "server_error")
                if ev[0] == "done":
                    finish = ev[1] or "stop"
                    if finish == "cache_full":
                        raise RequestError(CACHE_FULL, err_type="context_length_exceeded")
                    break
                if stopper.hit:
                    continue
                for tid in ev[1]:
                    n += 1
                    if tid not in self.eos_ids:
                        yield "text", stopper.push(dec.push(tid))
                    if stopper.hit:
                        self.loop.cancel(ticket)
                        finish = "stop"
                        break
                if stopper.hit:
                    break
            if not stopper.hit:
                yield "text", stopper.push(dec.flush())
                yield "text", stopper.flush()
        except GeneratorExit:
            self.loop.cancel(ticket)
            raise
        yield "end", (n, "length" if finish == "length" else "stop")

    # -- streaming (server-sent events) -------------------------------------------------------------------------
    def stream(self, req: ChatRequest) -> Iterator[bytes]:
        rid = "chatcmpl-" + uuid.uuid4().hex[:24]
        created = int(time.time())
        model = req.model or self.model_name

        live_lp: list | None = None
        sent_lp = 0

        def chunk(delta: dict, finish=None, usage=None) -> bytes:
            nonlocal sent_lp
            choice = {"index": 0, "delta": delta, "finish_reason": finish}
            if live_lp is not None and ("content" in delta or "reasoning_content" in delta) and "role" not in delta:
                # the entries of the tokens generated since the previous chunk travel with this one
                choice["logprobs"] = self._logprobs_object(live_lp[sent_lp:])
                sent_lp = len(live_lp)
            obj = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": model,
                   "system_fingerprint": SYSTEM_FINGERPRINT, "choices": [choice]}
            if usage is not None:
                obj["usage"] = usage
            return b"data: " + json.dumps(obj, ensure_ascii=False).encode() + b"\n\n"

        gen = self._generate(req)          # raises RequestError before the first byte if setup fails
        first = next(gen)
        if first[0] == "logprobs":
            live_lp = first[1]
            first = next(gen)
        yield chunk({"role": "assistant", "content": ""})
        content_all = []
        info = None
        for kind, payload in _chain(first, gen):
            if kind == "delta":
                r, c = payload
                if r:
                    yield chunk({"reasoning_content": r})
                if c:
                    content_all.append(c)
                    if not req.tools:
                        yield chunk({"content": c})
            else:
                info = payload
        finish = "length" if info["finish_reason"] == "length" else "stop"
        if live_lp is not None and sent_lp < len(live_lp) and not req.tools:
            yield chunk({"content": ""})               # tokens that produced no text of their own
        if req.tools:
            parsed = parse_tool_calls("".join(content_all))
            if parsed.has_tool_calls:
                if parsed.content:
                    yield chunk({"content": parsed.content})
                calls = parsed.tool_calls if req.parallel_tool_calls else parsed.tool_calls[:1]
                yield chunk({"tool_calls": [dict(c, index=i) for i, c in enumerate(calls)]})
                finish = "tool_calls"
            else:
                yield chunk({"content": "".join(content_all)})
        yield chunk({}, finish=finish, usage=self._usage(info))
        yield b"data: [DONE]\n\n"


def _chain(first, rest):
    yield first
    yield from rest

