"""``volta_sessions``: turn recorded agent sessions (JSONL transcripts) into Anthropic Messages request bodies that can be
posted to the server (``/v1/messages`` or ``/v1/messages/count_tokens``) as calibration text.

Rules (reference: docs/QUANTIZATION.md:101, src/tools/volta_sessions.cpp): main-thread turns in order, consecutive entries
of one role joined into one message, thinking / tool calls / tool results kept as recorded, the conversation cut at a
message boundary once its text passes ``--max-chars``. ``--requests`` writes chat-completion bodies for a prompt list
instead; ``--conversations`` + ``--responses`` turn another server's replies into Anthropic bodies of the exchange
(reasoning as a thinking block).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def _blocks(content) -> list:
    if isinstance(content, str):
        return [{"type": "text", "text": content}] if content else []
    out = []
    for b in content or []:
        if isinstance(b, str):
            out.append({"type": "text", "text": b})
        elif isinstance(b, dict) and b.get("type") in ("text", "thinking", "tool_use", "tool_result", "image"):
            out.append(b)
    return out


def _chars(blocks: list) -> int:
    n = 0
    for b in blocks:
        if b["type"] == "text":
            n += len(b.get("text", ""))
        elif b["type"] == "thinking":
            n += len(b.get("thinking", ""))
        elif b["type"] == "tool_use":
            n += len(json.dumps(b.get("input", {})))
        elif b["type"] == "tool_result":
            c = b.get("content", "")
            n += len(c) if isinstance(c, str) else sum(len(x.get("text", "")) for x in c if isinstance(x, dict))
    return n


def session_to_body(lines, max_chars: int = 120000, model: str = "local", max_tokens: int = 1) -> dict | None:
    """One transcript (iterable of JSON lines) -> a Messages request body, or None when it has no usable turn."""
    system, msgs, total = None, [], 0
    for raw in lines:
        raw = raw.strip()
        if not raw:
            continue
        try:
            e = json.loads(raw)
        except ValueError:
            continue
        if e.get("isSidechain") or e.get("type") not in ("user", "assistant", "system"):
            continue                                           # side threads and bookkeeping entries are skipped
        m = e.get("message", e)
        role = m.get("role", e.get("type"))
        if role == "system":
            system = m.get("content") if isinstance(m.get("content"), str) else system
            continue
        blocks = _blocks(m.get("content"))
        if not blocks:
            continue
        if msgs and msgs[-1]["role"] == role:
            msgs[-1]["content"].extend(blocks)                 # consecutive entries of one role form one message
        else:
            if total > max_chars:
                break                                          # cut at a message boundary
            msgs.append({"role": role, "content": list(blocks)})
        total += _chars(blocks)
    while msgs and msgs[0]["role"] != "user":
        msgs.pop(0)
    if not msgs:
        return None
    body = {"model": model, "max_tokens": max_tokens, "messages": msgs}
    if system:
        body["system"] = system
    return body


def prompts_to_requests(prompts: list, model: str, max_tokens: int = 6000, temperature: float = 1.0, top_p: float = 0.95) -> list:
    return [{"model": model, "max_tokens": max_tokens, "temperature": temperature, "top_p": top_p,
             "messages": [{"role": "user", "content": p if isinstance(p, str) else p["prompt"]}]} for p in prompts]


def exchange_to_body(prompt: str, reply: dict, model: str = "local") -> dict:
    """A chat-completion reply of another server -> the Anthropic body of the exchange (reasoning as a thinking block; a
    reply cut inside its reasoning keeps the reasoning alone)."""
    msg = reply["choices"][0]["message"] if "choices" in reply else reply
    blocks = []
    if msg.get("reasoning_content"):
        blocks.append({"type": "thinking", "thinking": msg["reasoning_content"]})
    if msg.get("content"):
        blocks.append({"type": "text", "text": msg["content"]})
    return {"model": model, "max_tokens": 1, "messages": [{"role": "user", "content": [{"type": "text", "text": prompt}]},
                                                          {"role": "assistant", "content": blocks}]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="volta_sessions", description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-chars", type=int, default=120000)
    ap.add_argument("--model", default="local")
    ap.add_argument("--requests", help="prompt list (JSON) -> chat completion bodies")
    ap.add_argument("--conversations", help="prompt list (JSON) whose replies are under --responses")
    ap.add_argument("--responses", help="directory of reply_N.json files")
    ap.add_argument("--max-tokens", type=int, default=6000)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("sessions", nargs="*")
    a = ap.parse_args(argv)
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    n = 0
    if a.requests:
        for body in prompts_to_requests(json.loads(Path(a.requests).read_text()), a.model, a.max_tokens, a.temperature, a.top_p):
            (out / f"req_{n}.json").write_text(json.dumps(body))
            n += 1
    elif a.conversations:
        prompts = json.loads(Path(a.conversations).read_text())
        for i, p in enumerate(prompts):
            rp = Path(a.responses) / f"reply_{i}.json"
            if rp.exists():
                text = p if isinstance(p, str) else p["prompt"]
                (out / f"req_{n}.json").write_text(json.dumps(exchange_to_body(text, json.loads(rp.read_text()), a.model)))
                n += 1
    for path in a.sessions:
        with open(path) as f:
            body = session_to_body(f, a.max_chars, a.model)
        if body:
            (out / f"req_{n}.json").write_text(json.dumps(body))
            n += 1
    print(f"{n} request bodies written to {out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
