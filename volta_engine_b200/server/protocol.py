"""OpenAI ``/v1/chat/completions`` and Anthropic ``/v1/messages`` protocol objects: request normalisation
into one :class:`ChatRequest`, and responders that turn parser events into streamed or complete replies.

Reference surface: src/server/openai.cpp, src/server/anthropic.cpp and the shared request struct
inc/engine/server/chat.h:23-68 (tools normalisation, thinking budgets, logprobs, usage with cached tokens,
strict-context errors).
"""
from __future__ import annotations

import json
import time
import uuid
from dataclasses import dataclass, field

from ..runtime.sampling import SamplingParams
from .output_parser import REASONING, TEXT, TOOL_CALL


class ProtocolError(ValueError):
    def __init__(self, message: str, status: int = 400, kind: str = "invalid_request_error"):
        super().__init__(message)
        self.status, self.kind = status, kind


@dataclass
class ChatRequest:
    protocol: str
    messages: list
    tools: list | None = None
    stream: bool = False
    max_tokens: int = 0
    params: SamplingParams = field(default_factory=SamplingParams)
    stop: list = field(default_factory=list)
    enable_thinking: bool | None = None
    thinking_budget: int = 0
    model: str = ""
    include_usage: bool = True
    priority: int = 0
    n_images: int = 0
    images: list = field(default_factory=list)      # raw bytes of every image part, in prompt order
    steer: dict = field(default_factory=dict)       # request steering fields: steer_vector, steer_scale, steer_scope, think_penalty


# what an image part becomes in the rendered text: the tokenizer turns the middle piece into ONE placeholder token, which
# the multimodal front end expands to the image's token count
IMAGE_MARK = "<|vision_start|><|image_pad|><|vision_end|>"


def steer_fields(body: dict) -> dict:
    """The steering fields a request may carry (both protocols): ``steer_vector`` (a file name inside the server's
    steer_dir, or ``"off"``), ``steer_scale``, ``steer_scope``, ``think_penalty``, ``steer_probe`` (probe this prompt and
    clamp the declining direction when it leans that way)."""
    out = {}
    for k, conv in (("steer_vector", str), ("steer_scale", float), ("steer_scope", str), ("think_penalty", float), ("steer_probe", bool)):
        if body.get(k) is not None:
            try:
                out[k] = conv(body[k])
            except (TypeError, ValueError) as e:
                raise ProtocolError(f"{k}: {e}") from e
    return out


def _image_bytes(part: dict) -> bytes:
    """Bytes of an OpenAI ``image_url`` / ``input_image`` part or an Anthropic ``image`` part (base64 only: the server
    fetches nothing)."""
    import base64
    if part.get("type") == "image":
        src = part.get("source", {})
        if src.get("type") != "base64":
            raise ProtocolError("image sources must be base64")
        return base64.b64decode(src.get("data", ""))
    url = part.get("image_url", part.get("url", ""))
    if isinstance(url, dict):
        url = url.get("url", "")
    if not url.startswith("data:") or ";base64," not in url:
        raise ProtocolError("image_url must be a data: URL with base64 content")
    return base64.b64decode(url.split(";base64,", 1)[1])


def _text_of(content, images: list | None = None) -> str:
    """Flatten OpenAI / Anthropic content parts to text; image parts leave ``IMAGE_MARK`` and their bytes in ``images``."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    out = []
    for part in content:
        if isinstance(part, str):
            out.append(part)
        elif part.get("type") in ("text", "input_text", "output_text"):
            out.append(part.get("text", ""))
        elif part.get("type") in ("image_url", "input_image", "image") and images is not None:
            images.append(_image_bytes(part))
            out.append(IMAGE_MARK)
    return "".join(out)


def _sampling(body: dict, defaults: dict) -> SamplingParams:
    def num(key, dflt, lo=None, hi=None):
        v = body.get(key, dflt)
        if v is None:
            v = dflt
        if not isinstance(v, (int, float)) or isinstance(v, bool):
            raise ProtocolError(f"'{key}' must be a number")
        if (lo is not None and v < lo) or (hi is not None and v > hi):
            raise ProtocolError(f"'{key}' out of range")
        return v
    lp = body.get("top_logprobs", 0) or (1 if body.get("logprobs") else 0)
    return SamplingParams(
        temperature=float(num("temperature", defaults.get("temperature", 0.0), 0.0, 10.0)),
        top_p=float(num("top_p", defaults.get("top_p", 1.0), 0.0, 1.0)),
        top_k=int(num("top_k", defaults.get("top_k", 0), 0)),
        presence_penalty=float(num("presence_penalty", 0.0, -2.0, 2.0)),
        frequency_penalty=float(num("frequency_penalty", 0.0, -2.0, 2.0)),
        repetition_penalty=float(num("repetition_penalty", 1.0, 0.01, 10.0)),
        seed=body.get("seed"), logprobs=int(lp))


def parse_openai(body: dict, defaults: dict) -> ChatRequest:
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise ProtocolError("'messages' must be a non-empty array")
    out, n_img, images = [], 0, []
    for m in msgs:
        role = m.get("role")
        if role not in ("system", "developer", "user", "assistant", "tool"):
            raise ProtocolError(f"unknown role '{role}'")
        if role == "developer":
            role = "system"
        content = m.get("content")
        if isinstance(content, list):
            n_img += sum(1 for p in content if isinstance(p, dict) and p.get("type") in ("image_url", "input_image"))
        e = {"role": role, "content": _text_of(content, images)}
        if role == "assistant" and m.get("tool_calls"):
            calls = []
            for tc in m["tool_calls"]:
                fn = tc.get("function", {})
                args = fn.get("arguments", "{}")
                if isinstance(args, str):
                    try:
                        args = json.loads(args) if args.strip() else {}
                    except json.JSONDecodeError:
                        pass
                calls.append({"type": "function", "id": tc.get("id", ""), "function": {"name": fn.get("name", ""), "arguments": args}})
            e["tool_calls"] = calls
        if role == "assistant" and m.get("reasoning_content"):
            e["reasoning_content"] = m["reasoning_content"]
        if role == "tool":
            e["tool_call_id"] = m.get("tool_call_id", "")
        out.append(e)
    tools = body.get("tools") or None
    if tools is not None:
        for t in tools:
            if t.get("type") != "function" or "function" not in t:
                raise ProtocolError("only function tools are supported")
    stop = body.get("stop") or []
    if isinstance(stop, str):
        stop = [stop]
    kw = body.get("chat_template_kwargs") or {}
    think = kw.get("enable_thinking", body.get("enable_thinking"))
    mt = body.get("max_completion_tokens", body.get("max_tokens")) or 0
    so = body.get("stream_options") or {}
    return ChatRequest("openai", out, tools, bool(body.get("stream")), int(mt), _sampling(body, defaults), list(stop),
                       think, int(body.get("thinking_budget", 0) or 0), body.get("model", ""),
                       bool(so.get("include_usage", True)), int(body.get("priority", 0) or 0), n_img, images,
                       steer_fields(body))


def parse_anthropic(body: dict, defaults: dict) -> ChatRequest:
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise ProtocolError("'messages' must be a non-empty array")
    if "max_tokens" not in body:
        raise ProtocolError("'max_tokens' is required")
    out, n_img, images = [], 0, []
    sysm = body.get("system")
    if sysm:
        out.append({"role": "system", "content": _text_of(sysm)})
    for m in msgs:
        role = m.get("role")
        if role not in ("user", "assistant"):
            raise ProtocolError(f"unknown role '{role}'")
        content = m.get("content")
        if isinstance(content, str):
            out.append({"role": role, "content": content})
            continue
        text, calls, reasoning = [], [], []
        for part in content or []:
            t = part.get("type")
            if t == "text":
                text.append(part.get("text", ""))
            elif t == "image":
                n_img += 1
                images.append(_image_bytes(part))
                text.append(IMAGE_MARK)
            elif t == "thinking":
                reasoning.append(part.get("thinking", ""))
            elif t == "tool_use":
                calls.append({"type": "function", "id": part.get("id", ""),
                              "function": {"name": part.get("name", ""), "arguments": part.get("input", {})}})
            elif t == "tool_result":
                if text:
                    out.append({"role": role, "content": "".join(text)})
                    text = []
                out.append({"role": "tool", "content": _text_of(part.get("content")), "tool_call_id": part.get("tool_use_id", "")})
        if text or calls or reasoning:
            e = {"role": role, "content": "".join(text)}
            if calls:
                e["tool_calls"] = calls
            if reasoning:
                e["reasoning_content"] = "".join(reasoning)
            out.append(e)
    tools = None
    if body.get("tools"):
        tools = [{"type": "function", "function": {"name": t.get("name", ""), "description": t.get("description", ""),
                                                    "parameters": t.get("input_schema", {})}} for t in body["tools"]]
    th = body.get("thinking") or {}
    think = None
    if th.get("type") == "enabled":
        think = True
    elif th.get("type") == "disabled":
        think = False
    return ChatRequest("anthropic", out, tools, bool(body.get("stream")), int(body["max_tokens"]),
                       _sampling(body, defaults), list(body.get("stop_sequences") or []), think,
                       int(th.get("budget_tokens", 0) or 0), body.get("model", ""), True, 0, n_img, images,
                       steer_fields(body))


# ------------------------------------------------------------------------------------------------ responders
FINISH_OPENAI = {"stop": "stop", "stop_string": "stop", "length": "length", "loop": "stop", "cancelled": "stop",
                 "error": "stop"}
FINISH_ANTHROPIC = {"stop": "end_turn", "stop_string": "stop_sequence", "length": "max_tokens", "loop": "end_turn",
                    "cancelled": "end_turn", "error": "end_turn"}


class OpenAIResponder:
    """Builds ``chat.completion.chunk`` SSE lines, or one ``chat.completion`` object when not streaming."""

    def __init__(self, req: ChatRequest, send, model_name: str):
        self.req, self.send, self.model = req, send, model_name
        self.id = "chatcmpl-" + uuid.uuid4().hex[:24]
        self.created = int(time.time())
        self.text, self.reasoning, self.calls, self.logprobs = [], [], [], []
        self.first = True

    def _chunk(self, delta: dict, finish=None, usage=None, logprobs=None):
        obj = {"id": self.id, "object": "chat.completion.chunk", "created": self.created, "model": self.model,
               "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
        if logprobs:
            obj["choices"][0]["logprobs"] = {"content": logprobs}
        if usage is not None:
            obj["usage"] = usage
        self.send("data: " + json.dumps(obj, ensure_ascii=False) + "\n\n")

    def on_event(self, kind, payload, logprobs=None):
        if kind == TEXT:
            self.text.append(payload)
        elif kind == REASONING:
            self.reasoning.append(payload)
        else:
            self.calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function",
                               "function": {"name": payload["name"], "arguments": payload["arguments"]}})
        if logprobs:
            self.logprobs.extend(logprobs)
        if not self.req.stream:
            return
        delta = {"role": "assistant"} if self.first else {}
        self.first = False
        if kind == TEXT:
            delta["content"] = payload
        elif kind == REASONING:
            delta["reasoning_content"] = payload
        else:
            c = dict(self.calls[-1])
            c["index"] = len(self.calls) - 1
            delta["tool_calls"] = [c]
        self._chunk(delta, logprobs=logprobs)

    @staticmethod
    def usage(u: dict) -> dict:
        return {"prompt_tokens": u["prompt_tokens"], "completion_tokens": u["completion_tokens"],
                "total_tokens": u["total_tokens"], "prompt_tokens_details": {"cached_tokens": u.get("cached_tokens", 0)}}

    def finish(self, reason: str, usage: dict):
        fr = "tool_calls" if self.calls and reason in ("stop", "stop_string") else FINISH_OPENAI.get(reason, "stop")
        if self.req.stream:
            self._chunk({}, finish=fr)
            if self.req.include_usage:
                obj = {"id": self.id, "object": "chat.completion.chunk", "created": self.created, "model": self.model,
                       "choices": [], "usage": self.usage(usage)}
                self.send("data: " + json.dumps(obj) + "\n\n")
            self.send("data: [DONE]\n\n")
            return None
        msg = {"role": "assistant", "content": "".join(self.text) or (None if self.calls else "")}
        if self.reasoning:
            msg["reasoning_content"] = "".join(self.reasoning)
        if self.calls:
            msg["tool_calls"] = self.calls
        choice = {"index": 0, "message": msg, "finish_reason": fr}
        if self.logprobs:
            choice["logprobs"] = {"content": self.logprobs}
        return {"id": self.id, "object": "chat.completion", "created": self.created, "model": self.model,
                "choices": [choice], "usage": self.usage(usage)}


class AnthropicResponder:
    """Builds the Anthropic event stream (message_start, content_block_*, message_delta, message_stop)."""

    def __init__(self, req: ChatRequest, send, model_name: str, prompt_tokens: int = 0):
        self.req, self.send, self.model = req, send, model_name
        self.id = "msg_" + uuid.uuid4().hex[:24]
        self.blocks: list[dict] = []
        self.open_kind = None
        self.started = False
        self.prompt_tokens = prompt_tokens

    def _ev(self, name: str, obj: dict):
        obj = dict({"type": name}, **obj)
        self.send(f"event: {name}\ndata: " + json.dumps(obj, ensure_ascii=False) + "\n\n")

    def _start(self):
        if self.started or not self.req.stream:
            self.started = True
            return
        self.started = True
        self._ev("message_start", {"message": {"id": self.id, "type": "message", "role": "assistant", "model": self.model,
                                               "content": [], "stop_reason": None, "stop_sequence": None,
                                               "usage": {"input_tokens": self.prompt_tokens, "output_tokens": 0}}})

    def _close_block(self):
        if self.open_kind is not None and self.req.stream:
            self._ev("content_block_stop", {"index": len(self.blocks) - 1})
        self.open_kind = None

    def on_event(self, kind, payload, logprobs=None):
        self._start()
        if kind == TOOL_CALL:
            self._close_block()
            try:
                inp = json.loads(payload["arguments"] or "{}")
            except json.JSONDecodeError:
                inp = {"_raw": payload["arguments"]}
            blk = {"type": "tool_use", "id": "toolu_" + uuid.uuid4().hex[:24], "name": payload["name"], "input": inp}
            self.blocks.append(blk)
            if self.req.stream:
                i = len(self.blocks) - 1
                self._ev("content_block_start", {"index": i, "content_block": dict(blk, input={})})
                self._ev("content_block_delta", {"index": i, "delta": {"type": "input_json_delta", "partial_json": json.dumps(inp)}})
                self._ev("content_block_stop", {"index": i})
            return
        want = "thinking" if kind == REASONING else "text"
        if self.open_kind != want:
            self._close_block()
            self.blocks.append({"type": want, want: ""})
            self.open_kind = want
            if self.req.stream:
                self._ev("content_block_start", {"index": len(self.blocks) - 1, "content_block": {"type": want, want: ""}})
        self.blocks[-1][want] += payload
        if self.req.stream:
            d = {"type": "thinking_delta", "thinking": payload} if want == "thinking" else {"type": "text_delta", "text": payload}
            self._ev("content_block_delta", {"index": len(self.blocks) - 1, "delta": d})

    def finish(self, reason: str, usage: dict):
        self._start()
        self._close_block()
        sr = "tool_use" if any(b["type"] == "tool_use" for b in self.blocks) and reason in ("stop", "stop_string") \
            else FINISH_ANTHROPIC.get(reason, "end_turn")
        u = {"input_tokens": usage["prompt_tokens"], "output_tokens": usage["completion_tokens"],
             "cache_read_input_tokens": usage.get("cached_tokens", 0)}
        if self.req.stream:
            self._ev("message_delta", {"delta": {"stop_reason": sr, "stop_sequence": None}, "usage": u})
            self._ev("message_stop", {})
            return None
        return {"id": self.id, "type": "message", "role": "assistant", "model": self.model, "content": self.blocks,
                "stop_reason": sr, "stop_sequence": None, "usage": u}


def error_body(protocol: str, message: str, kind: str = "invalid_request_error") -> str:
    if protocol == "anthropic":
        return json.dumps({"type": "error", "error": {"type": kind, "message": message}})
    return json.dumps({"error": {"message": message, "type": kind, "param": None, "code": None}})
