"""Binding of the native incremental output parser (csrc/host/output_parser.cpp)."""
from __future__ import annotations

import ctypes
import json

from .. import _lib

FAMILIES = {"qwen": 0, "hermes": 0, "glm": 1, "deepseek": 2, "gemma": 0, "dense": 0}
TEXT, REASONING, TOOL_CALL = 0, 1, 2


class OutputParser:
    def __init__(self, family: str = "qwen", in_reasoning: bool = False):
        lib = _lib.host()
        lib.vh_parser_new.restype = ctypes.c_void_p
        lib.vh_parser_feed.restype = ctypes.c_void_p
        lib.vh_parser_finish.restype = ctypes.c_void_p
        lib.vh_parser_feed.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
        lib.vh_parser_finish.argtypes = [ctypes.c_void_p]
        lib.vh_parser_free.argtypes = [ctypes.c_void_p]
        lib.vh_free.argtypes = [ctypes.c_void_p]
        self._lib = lib
        self._h = ctypes.c_void_p(lib.vh_parser_new(FAMILIES.get(family, 0), 1 if in_reasoning else 0))

    def _events(self, p):
        s = ctypes.string_at(p).decode("utf-8")
        self._lib.vh_free(p)
        out = []
        for e in json.loads(s):
            if e["kind"] == TOOL_CALL:
                out.append((TOOL_CALL, json.loads(e["payload"])))
            else:
                out.append((e["kind"], e["payload"]))
        return out

    def feed(self, text: str):
        """-> list of (kind, payload): TEXT / REASONING strings, TOOL_CALL {"name", "arguments" (JSON string)}."""
        raw = text.encode("utf-8")
        return self._events(self._lib.vh_parser_feed(self._h, raw, len(raw)))

    def finish(self):
        return self._events(self._lib.vh_parser_finish(self._h))

    def __del__(self):
        try:
            if self._h:
                self._lib.vh_parser_free(self._h)
        except Exception:
            pass
