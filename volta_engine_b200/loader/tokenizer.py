"""Python face of the native tokenizer (csrc/host/tokenizer.cpp): byte-level BPE families and the SentencePiece-style
BPE with byte fallback (Gemma).

Reference surface: ``Tokenizer::load / encode / decode`` over ``tokenizer.json`` or ``vocab.json`` +
``merges.txt`` (inc/engine/loader/tokenizer.h:11-88).
"""
from __future__ import annotations

import ctypes
import json
import os

from .. import _lib

MODES = {"qwen": 0, "gpt2": 1, "llama3": 2, "deepseek": 3, "glm": 0, "spm": 4, "gemma": 4}


class Tokenizer:
    def __init__(self, handle, mode: str):
        if not handle:
            raise ValueError("tokenizer files could not be loaded")
        self._h = ctypes.c_void_p(handle)
        self.mode = mode
        self.vocab_size = _lib.hcall("tok_vocab_size", "p", self._h)
        self.eos_ids: list[int] = []
        self.bos_id: int | None = None

    @classmethod
    def load(cls, model_dir: str, mode: str | None = None) -> "Tokenizer":
        """Loads ``tokenizer.json`` (preferred) or ``vocab.json`` + ``merges.txt`` from a model directory."""
        lib = _lib.host()
        lib.vh_tok_load_json.restype = ctypes.c_void_p
        lib.vh_tok_load_vocab_merges.restype = ctypes.c_void_p
        cfg = {}
        p = os.path.join(model_dir, "tokenizer_config.json")
        if os.path.exists(p):
            with open(p) as f:
                cfg = json.load(f)
        if mode is None:
            mt = ""
            cp = os.path.join(model_dir, "config.json")
            if os.path.exists(cp):
                with open(cp) as f:
                    mt = json.load(f).get("model_type", "")
            mode = "deepseek" if "deepseek" in mt else "llama3" if "llama" in mt else "spm" if "gemma" in mt else "qwen"
        tj = os.path.join(model_dir, "tokenizer.json")
        if mode == "qwen" and os.path.exists(tj):
            # SentencePiece-style vocabularies announce themselves: byte fallback pieces and no byte-level pre-tokenizer
            with open(tj) as f:
                head = json.load(f)
            if head.get("model", {}).get("byte_fallback"):
                mode = "spm"
        if os.path.exists(tj):
            h = lib.vh_tok_load_json(tj.encode(), MODES[mode])
        else:
            h = lib.vh_tok_load_vocab_merges(os.path.join(model_dir, "vocab.json").encode(),
                                             os.path.join(model_dir, "merges.txt").encode(), MODES[mode])
        t = cls(h, mode)
        for key in ("eos_token",):
            tok = cfg.get(key)
            if isinstance(tok, dict):
                tok = tok.get("content")
            if tok:
                i = t.piece_id(tok)
                if i >= 0:
                    t.eos_ids.append(i)
        bos = cfg.get("bos_token")
        if isinstance(bos, dict):
            bos = bos.get("content")
        if bos:
            i = t.piece_id(bos)
            t.bos_id = i if i >= 0 else None
        gp = os.path.join(model_dir, "generation_config.json")
        if os.path.exists(gp):
            with open(gp) as f:
                e = json.load(f).get("eos_token_id")
            for i in ([e] if isinstance(e, int) else (e or [])):
                if i not in t.eos_ids:
                    t.eos_ids.append(i)
        return t

    def piece_id(self, piece: str) -> int:
        return _lib.hcall("tok_piece_id", "ps", self._h, piece.encode())

    def add_special(self, piece: str, idx: int) -> None:
        _lib.hcall("tok_add_special", "psi", self._h, piece.encode(), idx)
        self.vocab_size = _lib.hcall("tok_vocab_size", "p", self._h)

    def encode(self, text: str, allow_special: bool = True) -> list[int]:
        raw = text.encode("utf-8")
        cap = len(raw) + 16
        buf = (ctypes.c_int * cap)()
        n = _lib.hcall("tok_encode", "psiipi", self._h, raw, len(raw), 1 if allow_special else 0, buf, cap)
        if n > cap:
            buf = (ctypes.c_int * n)()
            n = _lib.hcall("tok_encode", "psiipi", self._h, raw, len(raw), 1 if allow_special else 0, buf, n)
        return list(buf[:n])

    def decode_bytes(self, ids, skip_special: bool = False) -> bytes:
        n = len(ids)
        arr = (ctypes.c_int * n)(*ids)
        cap = 16 * n + 64
        out = ctypes.create_string_buffer(cap)
        w = _lib.hcall("tok_decode", "ppiipi", self._h, arr, n, 1 if skip_special else 0, out, cap)
        if w > cap:
            out = ctypes.create_string_buffer(w)
            w = _lib.hcall("tok_decode", "ppiipi", self._h, arr, n, 1 if skip_special else 0, out, w)
        return out.raw[:w]

    def decode(self, ids, skip_special: bool = False) -> str:
        return self.decode_bytes(ids, skip_special).decode("utf-8", errors="replace")

    def is_special(self, idx: int) -> bool:
        return bool(_lib.hcall("tok_is_special", "pi", self._h, idx))
