"""Chat-template rendering through the native Jinja subset interpreter (csrc/host/jinja.cpp).

Reference surface: ``ChatTemplate::load`` + Jinja render of ``messages`` / ``tools`` /
``add_generation_prompt`` / ``enable_thinking`` (src/loader/chat_template.cpp, src/loader/jinja.cpp).
"""
from __future__ import annotations

import ctypes
import json
import os

from .. import _lib


class TemplateError(ValueError):
    pass


def render(template: str, context: dict) -> str:
    out = ctypes.c_char_p()
    lib = _lib.host()
    lib.vh_jinja_render.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_char_p)]
    lib.vh_jinja_render.restype = ctypes.c_int
    lib.vh_free.argtypes = [ctypes.c_void_p]
    rc = lib.vh_jinja_render(template.encode("utf-8"), json.dumps(context, ensure_ascii=False).encode("utf-8"),
                             ctypes.byref(out))
    text = ctypes.string_at(out).decode("utf-8")
    lib.vh_free(out)
    if rc != 0:
        raise TemplateError(text)
    return text


DEFAULT_CHATML = (
    "{%- for message in messages %}{{- '<|im_start|>' + message.role + '\\n' + message.content + '<|im_end|>\\n' }}"
    "{%- endfor %}{%- if add_generation_prompt %}{{- '<|im_start|>assistant\\n' }}{%- endif %}")


class ChatTemplate:
    def __init__(self, source: str, bos_token: str = "", eos_token: str = ""):
        self.source, self.bos_token, self.eos_token = source, bos_token, eos_token

    @classmethod
    def load(cls, model_dir: str) -> "ChatTemplate":
        src, bos, eos = None, "", ""
        for name in ("chat_template.jinja", "chat_template.json"):
            p = os.path.join(model_dir, name)
            if os.path.exists(p):
                with open(p) as f:
                    raw = f.read()
                src = json.loads(raw).get("chat_template") if name.endswith(".json") else raw
                break
        cfgp = os.path.join(model_dir, "tokenizer_config.json")
        if os.path.exists(cfgp):
            with open(cfgp) as f:
                cfg = json.load(f)
            if src is None:
                ct = cfg.get("chat_template")
                if isinstance(ct, list):
                    ct = next((c["template"] for c in ct if c.get("name") == "default"), ct[0]["template"])
                src = ct

            def tok(v):
                return v.get("content", "") if isinstance(v, dict) else (v or "")
            bos, eos = tok(cfg.get("bos_token")), tok(cfg.get("eos_token"))
        return cls(src or DEFAULT_CHATML, bos, eos)

    def apply(self, messages: list, tools: list | None = None, add_generation_prompt: bool = True, **extra) -> str:
        ctx = {"messages": messages, "add_generation_prompt": add_generation_prompt, "bos_token": self.bos_token,
               "eos_token": self.eos_token}
        if tools:
            ctx["tools"] = tools
        ctx.update(extra)
        return render(self.source, ctx)
