"""Load generator for the OpenAI-compatible server: concurrent streamed chat requests, time to first token, inter-token
latency and aggregate throughput.

    python -m llaminar_b200.serve.loadgen --url http://127.0.0.1:8080 --concurrency 32 --requests 256 \\
        --prompt-tokens 512 --max-tokens 128 [--api-key KEY] [--json out.json]

Every worker thread keeps one request in flight; prompts are synthetic (a repeated word list of the requested length, with
a per-request prefix so that the prefix cache is not what gets measured unless `--shared-prefix` asks for it).  The
reference measures its server with shell scripts around curl (reference: tests/v2/e2e/server/test_server_e2e.sh); this
module is the equivalent a user can point at a running `serve`.
"""
from __future__ import annotations

import argparse
import http.client
import json
import statistics
import threading
import time
from urllib.parse import urlparse

WORDS = ("alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta", "theta", "iota", "kappa", "lambda", "mu")


def make_prompt(index: int, approx_tokens: int, shared_prefix: bool) -> str:
    body = " ".join(WORDS[(i + (0 if shared_prefix else index)) % len(WORDS)] for i in range(max(approx_tokens - 8, 1)))
    return f"request {index}: {body}" if not shared_prefix else f"{body} request {index}"


def percentile(xs: list[float], p: float) -> float:
    if not xs:
        return 0.0
    s = sorted(xs)
    return s[min(int(round(p / 100.0 * (len(s) - 1))), len(s) - 1)]


def one_request(url, payload: dict, api_key: str | None, timeout: float, path: str = "/v1/chat/completions") -> dict:
    """Streams one chat (or text) completion; returns timings (seconds) and token counts, or {"error": ...}."""
    u = urlparse(url)
    conn_cls = http.client.HTTPSConnection if u.scheme == "https" else http.client.HTTPConnection
    conn = conn_cls(u.hostname, u.port or (443 if u.scheme == "https" else 80), timeout=timeout)
    headers = {"Content-Type": "application/json"}
    if api_key:
        headers["Authorization"] = f"Bearer {api_key}"
    t0 = time.perf_counter()
    try:
        conn.request("POST", (u.path.rstrip("/") or "") + path, body=json.dumps(payload).encode(), headers=headers)
        resp = conn.getresponse()
        if resp.status != 200:
            return {"error": f"HTTP {resp.status}: {resp.read()[:200].decode(errors='replace')}"}
        stamps, usage = [], None
        for raw in resp:
            line = raw.strip()
            if not line.startswith(b"data: ") or line == b"data: [DONE]":
                continue
            obj = json.loads(line[6:])
            if "error" in obj:
                return {"error": obj["error"].get("message", "error")}
            choice = obj["choices"][0]
            delta = choice.get("delta", {})
            if delta.get("content") or delta.get("reasoning_content") or choice.get("text"):
                stamps.append(time.perf_counter())
            usage = obj.get("usage") or usage
        t1 = time.perf_counter()
        n = (usage or {}).get("completion_tokens", len(stamps))
        gaps = [b - a for a, b in zip(stamps, stamps[1:])]
        return {"ttft": (stamps[0] - t0) if stamps else (t1 - t0), "total": t1 - t0, "completion_tokens": n,
                "prompt_tokens": (usage or {}).get("prompt_tokens", 0), "itl": statistics.mean(gaps) if gaps else 0.0}
    except Exception as exc:                                  # connection refused, timeout, malformed chunk
        return {"error": f"{type(exc).__name__}: {exc}"}
    finally:
        conn.close()


def run(url: str, concurrency: int, requests: int, prompt_tokens: int, max_tokens: int, api_key: str | None = None,
        shared_prefix: bool = False, temperature: float = 0.0, timeout: float = 600.0, endpoint: str = "chat") -> dict:
    results: list[dict] = []
    lock = threading.Lock()
    counter = iter(range(requests))

    def worker():
        while True:
            with lock:
                i = next(counter, None)
            if i is None:
                return
            prompt = make_prompt(i, prompt_tokens, shared_prefix)
            payload = {"max_tokens": max_tokens, "temperature": temperature, "stream": True}
            if endpoint == "completions":                      # raw prompt, no chat template
                payload["prompt"] = prompt
                r = one_request(url, payload, api_key, timeout, "/v1/completions")
            else:
                payload["messages"] = [{"role": "user", "content": prompt}]
                r = one_request(url, payload, api_key, timeout)
            with lock:
                results.append(r)

    t0 = time.perf_counter()
    threads = [threading.Thread(target=worker, daemon=True) for _ in range(max(1, min(concurrency, requests)))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    ok = [r for r in results if "error" not in r]
    out_tok = sum(r["completion_tokens"] for r in ok)
    return {"requests": requests, "concurrency": concurrency, "succeeded": len(ok), "failed": len(results) - len(ok),
            "errors": sorted({r["error"] for r in results if "error" in r})[:5], "wall_s": wall,
            "output_tokens": out_tok, "output_tok_per_s": out_tok / wall if wall > 0 else 0.0,
            "prompt_tokens": sum(r["prompt_tokens"] for r in ok), "requests_per_s": len(ok) / wall if wall > 0 else 0.0,
            "ttft_ms": {"p50": 1e3 * percentile([r["ttft"] for r in ok], 50), "p90": 1e3 * percentile([r["ttft"] for r in ok], 90),
                        "p99": 1e3 * percentile([r["ttft"] for r in ok], 99)},
            "inter_token_ms": {"p50": 1e3 * percentile([r["itl"] for r in ok], 50), "p99": 1e3 * percentile([r["itl"] for r in ok], 99)},
            "latency_s": {"p50": percentile([r["total"] for r in ok], 50), "p99": percentile([r["total"] for r in ok], 99)}}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m llaminar_b200.serve.loadgen", description=__doc__.split("\n\n")[0])
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--prompt-tokens", type=int, default=512, help="approximate prompt length (one word is about one token)")
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--shared-prefix", action="store_true", help="all prompts share their beginning (measures the prefix cache)")
    ap.add_argument("--endpoint", choices=("chat", "completions"), default="chat", help="/v1/chat/completions or /v1/completions")
    ap.add_argument("--api-key", default=None)
    ap.add_argument("--json", default=None, help="also write the summary to this file")
    a = ap.parse_args(argv)
    summary = run(a.url, a.concurrency, a.requests, a.prompt_tokens, a.max_tokens, a.api_key, a.shared_prefix, a.temperature,
                  endpoint=a.endpoint)
    text = json.dumps(summary, indent=2)
    print(text)
    if a.json:
        with open(a.json, "w") as f:
            f.write(text + "\n")
    return 0 if summary["failed"] == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
