"""HTTP front end: `GET /health`, `POST /v1/chat/completions` (JSON or server-sent events), CORS, clean
shutdown on SIGINT/SIGTERM (reference: src/v2/app/modes/ServerMode.cpp:81-258).  Built on the standard
library's threading HTTP server; each connection thread talks to the engine loop through queues.
"""
from __future__ import annotations

import json
import signal
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from .chat_handler import ChatCompletionHandler, RequestError, parse_request

CORS = {"Access-Control-Allow-Origin": "*", "Access-Control-Allow-Methods": "GET, POST, OPTIONS",
        "Access-Control-Allow-Headers": "Content-Type, Authorization"}
MAX_BODY = 64 << 20


def make_handler(chat: ChatCompletionHandler, state: dict):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"
        server_version = "llaminar-b200"

        def log_message(self, fmt, *args):          # quiet by default; the app logger records requests
            if state.get("verbose"):
                super().log_message(fmt, *args)

        def _send_json(self, status: int, obj: dict) -> None:
            body = json.dumps(obj, ensure_ascii=False).encode()
            self.send_response(status)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            for k, v in CORS.items():
                self.send_header(k, v)
            self.end_headers()
            self.wfile.write(body)

        def _authorised(self) -> bool:
            """With a key configured, the /v1 endpoints want `Authorization: Bearer <key>` (the reference has no
            authentication; /health and /metrics stay open for probes)."""
            key = state.get("api_key")
            if not key:
                return True
            import hmac
            given = self.headers.get("Authorization") or ""
            if given.startswith("Bearer ") and hmac.compare_digest(given[7:].strip().encode(), key.encode()):
                return True
            n = int(self.headers.get("Content-Length") or 0)
            if 0 < n <= MAX_BODY:
                self.rfile.read(n)                      # keep the connection in step
            self._send_json(401, {"error": {"message": "missing or invalid API key", "type": "invalid_request_error",
                                            "code": "invalid_api_key"}})
            return False

        def _send_stream(self, it) -> None:
            """Server-sent events from an iterator of encoded chunks."""
            first = next(it)                         # setup errors surface here, before headers go out
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Connection", "close")
            for k, v in CORS.items():
                self.send_header(k, v)
            self.end_headers()
            try:
                self.wfile.write(first)
                self.wfile.flush()
                for b in it:
                    self.wfile.write(b)
                    self.wfile.flush()
            except (BrokenPipeError, ConnectionResetError):
                it.close()                           # client went away: cancels the generation
            except RequestError as exc:              # failure after the stream began: report in-band
                self.wfile.write(b"data: " + json.dumps(exc.body()).encode() + b"\n\n")
            self.close_connection = True

        def do_OPTIONS(self):
            self.send_response(204)
            for k, v in CORS.items():
                self.send_header(k, v)
            self.send_header("Content-Length", "0")
            self.end_headers()

        def do_GET(self):
            if self.path.rstrip("/") == "/health":
                self._send_json(200, {"status": "ok", "model": chat.model_name, "requests_served": state["served"],
                                      "engine_errors": chat.loop.errors})
            elif self.path.rstrip("/") == "/metrics":
                # Prometheus text exposition (the reference has no metrics endpoint; its counters live in log lines)
                lines = []
                for k, v in sorted(chat.loop.metrics().items()):
                    kind = "gauge" if k.startswith(("requests_running", "requests_waiting", "kv_")) else "counter"
                    lines += [f"# TYPE llaminar_{k} {kind}", f"llaminar_{k} {v}"]
                body = ("\n".join(lines) + "\n").encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4; charset=utf-8")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)
            elif self.path.rstrip("/") == "/v1/models":
                if not self._authorised():
                    return
                self._send_json(200, {"object": "list", "data": [{"id": chat.model_name, "object": "model", "owned_by": "local"}]})
            else:
                self._send_json(404, {"error": {"message": f"unknown path {self.path}", "type": "invalid_request_error"}})

        def do_POST(self):
            if self.path.startswith("/v1/") and not self._authorised():
                return
            if self.path.rstrip("/") == "/v1/completions":
                try:
                    n = int(self.headers.get("Content-Length") or 0)
                    if n <= 0 or n > MAX_BODY:
                        raise RequestError("missing or oversized request body")
                    result = chat.complete(self.rfile.read(n))
                    if isinstance(result, dict):
                        self._send_json(200, result)
                    else:
                        self._send_stream(result)
                    state["served"] += 1
                except RequestError as exc:
                    self._send_json(exc.status, exc.body())
                except Exception as exc:
                    self._send_json(500, {"error": {"message": f"{type(exc).__name__}: {exc}", "type": "server_error"}})
                return
            if self.path.rstrip("/") != "/v1/chat/completions":
                self._send_json(404, {"error": {"message": f"unknown path {self.path}", "type": "invalid_request_error"}})
                return
            try:
                n = int(self.headers.get("Content-Length") or 0)
                if n <= 0 or n > MAX_BODY:
                    raise RequestError("missing or oversized request body")
                req = parse_request(self.rfile.read(n))
                if req.stream:
                    self._send_stream(chat.stream(req))
                else:
                    self._send_json(200, chat.handle(req))
                state["served"] += 1
            except RequestError as exc:
                self._send_json(exc.status, exc.body())
            except Exception as exc:                 # never take the server down with a request
                self._send_json(500, {"error": {"message": f"{type(exc).__name__}: {exc}", "type": "server_error"}})

    return Handler


class Server:
    def __init__(self, chat: ChatCompletionHandler, host: str = "127.0.0.1", port: int = 8080, verbose: bool = False,
                 api_key: str | None = None, owns_loop: bool = True):
        self.state = {"served": 0, "verbose": verbose, "api_key": api_key}
        self.owns_loop = owns_loop                  # False: a second front end on an engine loop that someone else stops
        self.httpd = ThreadingHTTPServer((host, port), make_handler(chat, self.state))
        self.httpd.daemon_threads = True
        self.chat = chat

    @property
    def port(self) -> int:
        return self.httpd.server_address[1]

    def serve_forever(self, install_signals: bool = True) -> None:
        if install_signals and threading.current_thread() is threading.main_thread():
            for sig in (signal.SIGINT, signal.SIGTERM):
                signal.signal(sig, lambda *_: threading.Thread(target=self.httpd.shutdown, daemon=True).start())
        try:
            self.httpd.serve_forever(poll_interval=0.2)
        finally:
            self.httpd.server_close()
            if self.owns_loop:
                self.chat.loop.shutdown()

    def start_background(self) -> threading.Thread:
        t = threading.Thread(target=self.serve_forever, kwargs={"install_signals": False}, daemon=True)
        t.start()
        return t

    def stop(self) -> None:
        self.httpd.shutdown()
