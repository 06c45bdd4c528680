"""HTTP load generator for the serving API: TTFT, inter-token gap percentiles, request and token throughput.

Drives ``/v1/chat/completions`` with streaming at a fixed concurrency. ``--selftest`` starts a built-in mock server
(no GPU, no model) that streams a fixed number of chunks with a known delay, so the measuring code itself can be
checked. Reference: tests/3_bench/bench_serve.py (``--selftest`` against a built-in mock server: lines 200-227).
"""
from __future__ import annotations

import argparse
import http.client
import json
import sys
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from urllib.parse import urlparse


def percentile(xs, q):
    if not xs:
        return 0.0
    s = sorted(xs)
    i = min(len(s) - 1, max(0, int(round(q * (len(s) - 1)))))
    return s[i]


def one_request(url: str, body: dict, api_key: str = "", timeout: float = 600.0) -> dict:
    """Stream one chat completion; -> {ok, ttft_s, gaps_s[], tokens, total_s, error}."""
    u = urlparse(url)
    conn = http.client.HTTPConnection(u.hostname, u.port or 80, timeout=timeout)
    headers = {"Content-Type": "application/json"}
    if api_key:
        headers["Authorization"] = "Bearer " + api_key
    t0 = time.perf_counter()
    res = {"ok": False, "ttft_s": 0.0, "gaps_s": [], "tokens": 0, "total_s": 0.0, "error": ""}
    try:
        conn.request("POST", "/v1/chat/completions", body=json.dumps(dict(body, stream=True)), headers=headers)
        r = conn.getresponse()
        if r.status != 200:
            res["error"] = f"http {r.status}: {r.read()[:200]!r}"
            return res
        last = None
        usage_tokens = None
        while True:
            line = r.readline()
            if not line:
                break
            line = line.strip()
            if not line.startswith(b"data: "):
                continue
            payload = line[6:]
            if payload == b"[DONE]":
                break
            ev = json.loads(payload)
            if ev.get("usage"):
                usage_tokens = ev["usage"].get("completion_tokens")
            ch = ev.get("choices") or []
            delta = ch[0].get("delta", {}) if ch else {}
            if delta.get("content") or delta.get("reasoning_content") or delta.get("tool_calls"):
                now = time.perf_counter()
                if last is None:
                    res["ttft_s"] = now - t0
                else:
                    res["gaps_s"].append(now - last)
                last = now
                res["tokens"] += 1
        if usage_tokens is not None:
            res["tokens"] = usage_tokens
        res["ok"] = last is not None
        if not res["ok"]:
            res["error"] = "no content received"
    except Exception as e:
        res["error"] = repr(e)
    finally:
        res["total_s"] = time.perf_counter() - t0
        conn.close()
    return res


def run_load(url: str, n_requests: int, concurrency: int, prompt: str, max_tokens: int, model: str = "volta",
             api_key: str = "") -> dict:
    body = {"model": model, "messages": [{"role": "user", "content": prompt}], "max_tokens": max_tokens,
            "temperature": 0.0, "stream_options": {"include_usage": True}}
    results, lock, nxt = [], threading.Lock(), [0]

    def worker():
        while True:
            with lock:
                if nxt[0] >= n_requests:
                    return
                nxt[0] += 1
            r = one_request(url, body, api_key)
            with lock:
                results.append(r)
    t0 = time.perf_counter()
    threads = [threading.Thread(target=worker, daemon=True) for _ in range(concurrency)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    ok = [r for r in results if r["ok"]]
    gaps = [g for r in ok for g in r["gaps_s"]]
    toks = sum(r["tokens"] for r in ok)
    return {"requests": n_requests, "ok": len(ok), "failed": len(results) - len(ok), "concurrency": concurrency,
            "wall_s": wall, "req_per_s": len(ok) / wall if wall > 0 else 0.0, "tok_per_s": toks / wall if wall > 0 else 0.0,
            "tokens": toks, "ttft_ms": {k: 1e3 * percentile([r["ttft_s"] for r in ok], q) for k, q in
                                        (("p50", 0.5), ("p90", 0.9), ("p99", 0.99))},
            "gap_ms": {k: 1e3 * percentile(gaps, q) for k, q in (("p50", 0.5), ("p90", 0.9), ("p99", 0.99), ("max", 1.0))},
            "errors": sorted({r["error"] for r in results if r["error"]})[:5]}


class _MockHandler(BaseHTTPRequestHandler):
    chunks, delay_s, first_delay_s = 8, 0.01, 0.05

    def log_message(self, *a):
        pass

    def do_POST(self):
        n = int(self.headers.get("Content-Length", 0))
        req = json.loads(self.rfile.read(n) or b"{}")
        self.send_response(200)
        self.send_header("Content-Type", "text/event-stream")
        self.end_headers()
        k = min(self.chunks, int(req.get("max_tokens", self.chunks)))
        time.sleep(self.first_delay_s)
        for i in range(k):
            ev = {"choices": [{"index": 0, "delta": {"content": f"t{i} "}}]}
            self.wfile.write(b"data: " + json.dumps(ev).encode() + b"\n\n")
            self.wfile.flush()
            time.sleep(self.delay_s)
        fin = {"choices": [{"index": 0, "delta": {}, "finish_reason": "length"}], "usage": {"completion_tokens": k}}
        self.wfile.write(b"data: " + json.dumps(fin).encode() + b"\n\ndata: [DONE]\n\n")
        self.wfile.flush()


def selftest() -> dict:
    srv = ThreadingHTTPServer(("127.0.0.1", 0), _MockHandler)
    th = threading.Thread(target=srv.serve_forever, daemon=True)
    th.start()
    try:
        url = f"http://127.0.0.1:{srv.server_address[1]}"
        rep = run_load(url, n_requests=6, concurrency=3, prompt="ping", max_tokens=8)
    finally:
        srv.shutdown()
        srv.server_close()
    ok = (rep["ok"] == 6 and rep["tokens"] == 48 and rep["ttft_ms"]["p50"] >= 45.0 and
          5.0 <= rep["gap_ms"]["p50"] <= 60.0)
    rep["selftest"] = "pass" if ok else "fail"
    return rep


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="bench_serve")
    p.add_argument("--url", default="http://127.0.0.1:8080")
    p.add_argument("--requests", type=int, default=16)
    p.add_argument("--concurrency", type=int, default=4)
    p.add_argument("--prompt", default="Write a short paragraph about the sea.")
    p.add_argument("--prompt-repeat", type=int, default=1, help="repeat the prompt text to lengthen the input")
    p.add_argument("--max-tokens", type=int, default=128)
    p.add_argument("--model", default="volta")
    p.add_argument("--api-key", default="")
    p.add_argument("--selftest", action="store_true")
    a = p.parse_args(argv)
    rep = selftest() if a.selftest else run_load(a.url, a.requests, a.concurrency, a.prompt * a.prompt_repeat,
                                                 a.max_tokens, a.model, a.api_key)
    print(json.dumps(rep, indent=1))
    return 0 if rep.get("selftest", "pass") == "pass" and rep["failed"] == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
