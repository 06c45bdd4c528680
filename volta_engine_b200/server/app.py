"""The serving application: routes of the reference's HTTP surface on top of the native HTTP front end.

  POST /v1/chat/completions   OpenAI chat (SSE or complete)         GET /v1/models
  POST /v1/messages           Anthropic messages (event stream)     POST /v1/messages/count_tokens
  GET  /health  /metrics  /metrics/prometheus  /api/stats  /api/experts  /monitor

Reference: docs/server.md:10-74, src/server/server.cpp (routes, prometheus series :351-364),
src/server/chat.cpp:266-543 (prompt rendering, parser wiring, callbacks), src/server/monitor.cpp:32-115.
"""
from __future__ import annotations

import json
import threading
import time

from ..runtime.generator import Generator, Request
from .http import HttpRequest, HttpServer
from .monitor import MONITOR_HTML, prometheus_text, stats_payload
from .output_parser import OutputParser
from .protocol import (AnthropicResponder, ChatRequest, OpenAIResponder, ProtocolError, error_body, parse_anthropic,
                       parse_openai)


class VoltaServer:
    def __init__(self, generator: Generator, tokenizer, template, *, model_name: str = "volta", model_type: str = "dense",
                 host: str = "127.0.0.1", port: int = 0, api_key: str = "", defaults: dict | None = None,
                 max_context: int = 32768, default_max_tokens: int = 1024, request_timeout_s: int = 300, info: dict | None = None):
        self.gen, self.tok, self.template = generator, tokenizer, template
        self.model_name, self.model_type, self.api_key = model_name, model_type, api_key
        self.defaults = defaults or {}
        self.max_context, self.default_max_tokens = max_context, default_max_tokens
        self.info = info or {}
        self.http = HttpServer(host, port, request_timeout_s)
        self.port = self.http.port
        self.running = False
        self.thread = None
        self.t0 = time.time()
        self._active: dict[int, int] = {}     # connection id -> request id (for client-gone cancellation)
        self._lock = threading.Lock()

    # ------------------------------------------------------------------------------------------ lifecycle
    def start(self):
        self.running = True
        if self.gen.thread is None:
            self.gen.start()
        self.thread = threading.Thread(target=self._serve, name="volta-http-dispatch", daemon=True)
        self.thread.start()
        return self

    def stop(self):
        self.running = False
        if self.thread:
            self.thread.join(timeout=5)
        self.gen.stop()
        self.http.stop()

    def _serve(self):
        last_sweep = time.time()
        while self.running:
            req = self.http.next_request(200)
            if req is not None:
                try:
                    self._route(req)
                except Exception as ex:   # never let one request kill the dispatcher
                    self.http.respond(req.conn, 500, error_body("openai", f"internal error: {ex}", "server_error"))
            if time.time() - last_sweep > 1.0:      # client-gone detection -> cancel generation
                last_sweep = time.time()
                with self._lock:
                    gone = [(c, r) for c, r in self._active.items() if not self.http.alive(c)]
                for c, r in gone:
                    self.gen.cancel(r)
                    with self._lock:
                        self._active.pop(c, None)

    # ------------------------------------------------------------------------------------------ routing
    def _authorized(self, req: HttpRequest) -> bool:
        if not self.api_key:
            return True
        auth = req.headers.get("authorization", "")
        return auth == "Bearer " + self.api_key or req.headers.get("x-api-key", "") == self.api_key

    def _route(self, req: HttpRequest):
        p, m = req.path.rstrip("/") or "/", req.method
        if m == "OPTIONS":
            return self.http.respond(req.conn, 204, b"", headers="Access-Control-Allow-Headers: *\r\nAccess-Control-Allow-Methods: GET, POST, OPTIONS\r\n")
        if p == "/health":
            return self.http.respond(req.conn, 200, json.dumps({"status": "ok", "model": self.model_name}))
        if p in ("/monitor", "/"):
            return self.http.respond(req.conn, 200, MONITOR_HTML, "text/html; charset=utf-8")
        if p == "/api/stats":
            return self.http.respond(req.conn, 200, json.dumps(stats_payload(self)))
        if p == "/api/experts":
            return self.http.respond(req.conn, 200, json.dumps(self._experts()))
        if p == "/metrics":
            return self.http.respond(req.conn, 200, json.dumps(stats_payload(self, brief=True)))
        if p == "/metrics/prometheus":
            return self.http.respond(req.conn, 200, prometheus_text(self), "text/plain; version=0.0.4")
        if p.startswith("/v1/") and not self._authorized(req):
            proto = "anthropic" if p.startswith("/v1/messages") else "openai"
            return self.http.respond(req.conn, 401, error_body(proto, "invalid API key", "authentication_error"))
        if p == "/v1/models" and m == "GET":
            return self.http.respond(req.conn, 200, json.dumps({"object": "list", "data": [
                {"id": self.model_name, "object": "model", "created": int(self.t0), "owned_by": "volta"}]}))
        if p == "/v1/chat/completions" and m == "POST":
            return self._chat(req, "openai")
        if p == "/v1/messages" and m == "POST":
            return self._chat(req, "anthropic")
        if p == "/v1/messages/count_tokens" and m == "POST":
            return self._count_tokens(req)
        return self.http.respond(req.conn, 404, error_body("openai", f"no route for {m} {p}", "not_found_error"))

    def _experts(self) -> dict:
        heat = getattr(self.gen.engine.model, "expert_heat", None)
        if heat is None:
            return {"ranks": 0, "layers": 0, "experts": 0, "total": [], "recent": []}
        return heat()

    # ------------------------------------------------------------------------------------------ chat
    def render_prompt(self, cr: ChatRequest) -> str:
        extra = {}
        if cr.enable_thinking is not None:
            extra["enable_thinking"] = cr.enable_thinking
        elif "enable_thinking" in self.defaults:
            extra["enable_thinking"] = self.defaults["enable_thinking"]
        msgs = []
        for m in cr.messages:       # fold consecutive system messages into one leading system message
            if m["role"] == "system" and msgs and msgs[0]["role"] == "system" and len(msgs) == 1:
                msgs[0] = dict(msgs[0], content=msgs[0]["content"] + "\n\n" + m["content"])
            else:
                msgs.append(m)
        if self.template is None or self.model_type in ("deepseek_v4", "deepseek_v41", "deepseek41"):
            # these models ship no chat template: their prompt format is built in
            from ..loader import deepseek_encoding as ds
            return ds.encode(msgs, cr.tools or None, thinking=bool(extra.get("enable_thinking", True)),
                             reasoning_effort=str(getattr(cr, "reasoning_effort", "") or ""))
        return self.template.apply(msgs, tools=cr.tools, add_generation_prompt=True, **extra)

    def _parse(self, req: HttpRequest, proto: str) -> ChatRequest:
        try:
            body = json.loads(req.body.decode("utf-8") or "{}")
        except (json.JSONDecodeError, UnicodeDecodeError) as ex:
            raise ProtocolError(f"request body is not valid JSON: {ex}")
        if not isinstance(body, dict):
            raise ProtocolError("request body must be a JSON object")
        return parse_anthropic(body, self.defaults) if proto == "anthropic" else parse_openai(body, self.defaults)

    def _count_tokens(self, req: HttpRequest):
        try:
            body = json.loads(req.body.decode("utf-8") or "{}")
            body.setdefault("max_tokens", 1)
            cr = parse_anthropic(body, self.defaults)
            n = len(self.tok.encode(self.render_prompt(cr)))
        except ProtocolError as ex:
            return self.http.respond(req.conn, ex.status, error_body("anthropic", str(ex), ex.kind))
        except Exception as ex:
            return self.http.respond(req.conn, 400, error_body("anthropic", str(ex)))
        return self.http.respond(req.conn, 200, json.dumps({"input_tokens": n}))

    def _chat(self, req: HttpRequest, proto: str):
        conn = req.conn
        try:
            cr = self._parse(req, proto)
            mm_front = getattr(self.gen, "mm_frontend", None)
            if cr.n_images and mm_front is None:
                raise ProtocolError("this deployment has no vision tower loaded: image parts are not accepted")
            prompt_text = self.render_prompt(cr)
        except ProtocolError as ex:
            return self.http.respond(conn, ex.status, error_body(proto, str(ex), ex.kind))
        except Exception as ex:
            return self.http.respond(conn, 400, error_body(proto, f"chat template failed: {ex}"))
        ids = self.tok.encode(prompt_text)
        mm = cache_key = None
        if cr.images:
            # every image part left one placeholder token: it becomes the image's tokens, whose rows come from the tower
            from ..runtime.multimodal import MmPrompt
            try:
                ids, layout, feats = mm_front.prepare(ids, cr.images)
            except Exception as ex:
                return self.http.respond(conn, 400, error_body(proto, f"image input failed: {ex}"))
            mm, cache_key = MmPrompt.build(layout, feats), layout.cache_tokens(ids)
        max_new = cr.max_tokens or self.default_max_tokens
        if len(ids) + 1 > self.max_context:     # strict-context error instead of silent truncation
            return self.http.respond(conn, 400, error_body(
                proto, f"prompt has {len(ids)} tokens; the context window is {self.max_context}", "context_length_exceeded"))
        max_new = min(max_new, self.max_context - len(ids))
        in_reasoning = prompt_text.rstrip().endswith("<think>")
        parser = OutputParser(self.model_type, in_reasoning)
        send = (lambda s: self.http.stream_send(conn, s)) if cr.stream else (lambda s: None)
        if proto == "anthropic":
            responder = AnthropicResponder(cr, send, self.model_name, len(ids))
        else:
            responder = OpenAIResponder(cr, send, self.model_name)
        if cr.stream:
            self.http.stream_begin(conn, "text/event-stream")
        budget = cr.thinking_budget
        state = {"reasoning_tokens": 0}

        def on_text(text, tok_ids, logprobs):
            lp = None
            if logprobs:
                lp = [{"token": self.tok.decode([e["token"]]), "logprob": e["logprob"],
                       "top_logprobs": [{"token": self.tok.decode([i]), "logprob": v} for i, v in e["top"]]} for e in logprobs]
            events = parser.feed(text) if text else []
            for k, payload in events:
                responder.on_event(k, payload, lp)
                lp = None
            if budget and parser._lib.vh_parser_in_reasoning(parser._h):
                state["reasoning_tokens"] += len(tok_ids)

        def on_finish(reason, usage):
            for k, payload in parser.finish():
                responder.on_event(k, payload)
            body = responder.finish(reason, usage)
            with self._lock:
                self._active.pop(conn, None)
            if cr.stream:
                self.http.stream_end(conn)
            elif reason == "error":
                self.http.respond(conn, 500, error_body(proto, usage.get("error", "generation failed"), "server_error"))
            else:
                self.http.respond(conn, 200, json.dumps(body, ensure_ascii=False))

        sys_end = []
        prio = cr.priority
        low = [m.strip().lower() for m in str(getattr(self.gen.opt, "low_priority_models", "") or "").split(",") if m.strip()]
        if low and any(m in (cr.model or "").lower() for m in low):
            prio -= 100                 # requests that name one of these models queue behind the others
        steer_kw = {}
        scfg = getattr(self.gen, "steer_cfg", None)
        if scfg is not None and scfg.enabled:
            try:
                steer_kw = scfg.for_request(cr.steer)
            except (ValueError, OSError) as ex:
                return self.http.respond(conn, 400, error_body(proto, f"steering: {ex}"))
        elif cr.steer:
            return self.http.respond(conn, 400, error_body(proto, "steering is off on this server (launch option steer)"))
        r = Request(prompt=ids, mm=mm, cache_key=cache_key, max_tokens=max_new, params=cr.params, stop=cr.stop, priority=prio,
                    **steer_kw,
                    on_text=on_text, on_finish=on_finish, checkpoints=sys_end)
        rid = self.gen.submit(r)
        with self._lock:
            self._active[conn] = rid
