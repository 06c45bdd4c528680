"""GGUF v3 container: reader over an mmap (single file or ``-0000N-of-0000M`` split set), writer, and the
llama.cpp -> checkpoint tensor-name mapping with the converter's transforms undone at load.

Layout: magic ``GGUF``, u32 version, u64 tensor count, u64 kv count; kv entries (string key, u32 type, value);
tensor infos (name, u32 n_dims, u64 dims innermost first, u32 ggml type, u64 offset); data section aligned to
``general.alignment`` (32 by default), every tensor aligned likewise.
Reference: inc/engine/loader/gguf.h:17-38 (``gguf_open``), src/loader/gguf_arch.h:21-66 (per-architecture
adapters: name maps and inverse transforms).
"""
from __future__ import annotations

import mmap
import re
import struct
from pathlib import Path

import torch

from ..quant import gguf as gq

GGML_F32, GGML_F16, GGML_BF16 = 0, 1, 30
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
T_STRING, T_ARRAY = 8, 9
_PLAIN = {GGML_F32: (torch.float32, 4), GGML_F16: (torch.float16, 2), GGML_BF16: (torch.bfloat16, 2)}


class GGUFTensor:
    __slots__ = ("name", "shape", "ggml_type", "offset", "nbytes", "file")

    def __init__(self, name, shape, ggml_type, offset, nbytes, file):
        self.name, self.shape, self.ggml_type, self.offset, self.nbytes, self.file = name, shape, ggml_type, offset, nbytes, file


def tensor_nbytes(ggml_type: int, shape) -> int:
    n = 1
    for d in shape:
        n *= d
    if ggml_type in _PLAIN:
        return n * _PLAIN[ggml_type][1]
    K = shape[-1]
    return (n // K) * gq.row_bytes(ggml_type, K)


class _Reader:
    def __init__(self, mm):
        self.mm, self.p = mm, 0

    def take(self, fmt):
        v = struct.unpack_from(fmt, self.mm, self.p)
        self.p += struct.calcsize(fmt)
        return v[0]

    def string(self):
        n = self.take("<Q")
        s = self.mm[self.p:self.p + n].decode("utf-8", errors="replace")
        self.p += n
        return s

    def value(self, t):
        if t in _SCALAR:
            return self.take(_SCALAR[t])
        if t == T_STRING:
            return self.string()
        if t == T_ARRAY:
            et, n = self.take("<I"), self.take("<Q")
            if et in _SCALAR and et != 7:
                fmt = _SCALAR[et][1]
                sz = struct.calcsize(fmt)
                out = list(struct.unpack_from("<%d%s" % (n, fmt), self.mm, self.p))
                self.p += n * sz
                return out
            return [self.value(et) for _ in range(n)]
        raise ValueError(f"unknown GGUF value type {t}")


class GGUFFile:
    """Metadata and tensors of one GGUF model (all parts of a split set merged)."""

    def __init__(self, path):
        p = Path(path)
        if p.is_dir():
            parts = sorted(p.glob("*.gguf"))
            parts = [q for q in parts if "mmproj" not in q.name.lower()]
        else:
            m = re.match(r"(.*)-(\d{5})-of-(\d{5})\.gguf$", p.name)
            parts = sorted(p.parent.glob(m.group(1) + "-*-of-" + m.group(3) + ".gguf")) if m else [p]
        if not parts:
            raise FileNotFoundError(f"no .gguf under {p}")
        self.metadata: dict = {}
        self.tensors: dict[str, GGUFTensor] = {}
        self._files = []
        for fp in parts:
            self._open(fp)

    def _open(self, fp: Path):
        f = open(fp, "rb")
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        self._files.append((f, mm))
        r = _Reader(mm)
        if mm[:4] != b"GGUF":
            raise ValueError(f"{fp}: not a GGUF file")
        r.p = 4
        version = r.take("<I")
        if version not in (2, 3):
            raise ValueError(f"{fp}: GGUF version {version} is not supported")
        n_tensors, n_kv = r.take("<Q"), r.take("<Q")
        for _ in range(n_kv):
            key = r.string()
            t = r.take("<I")
            val = r.value(t)
            self.metadata.setdefault(key, val)
        infos = []
        for _ in range(n_tensors):
            name = r.string()
            nd = r.take("<I")
            dims = [r.take("<Q") for _ in range(nd)]
            gt = r.take("<I")
            off = r.take("<Q")
            infos.append((name, tuple(reversed(dims)), gt, off))
        align = int(self.metadata.get("general.alignment", 32))
        data0 = (r.p + align - 1) // align * align
        for name, shape, gt, off in infos:
            self.tensors[name] = GGUFTensor(name, shape, gt, data0 + off, tensor_nbytes(gt, shape), len(self._files) - 1)

    @property
    def arch(self) -> str:
        return self.metadata.get("general.architecture", "")

    def raw(self, name: str) -> torch.Tensor:
        t = self.tensors[name]
        mm = self._files[t.file][1]
        return torch.frombuffer(mm, dtype=torch.uint8, count=t.nbytes, offset=t.offset)

    def load(self, name: str) -> torch.Tensor:
        """Plain types come back typed and shaped; block types as uint8 [rows, row_bytes]."""
        t = self.tensors[name]
        raw = self.raw(name)
        if t.ggml_type in _PLAIN:
            return raw.view(_PLAIN[t.ggml_type][0]).reshape(t.shape)
        rows = 1
        for d in t.shape[:-1]:
            rows *= d
        return raw.reshape(rows, -1)

    def dequantize(self, name: str) -> torch.Tensor:
        t = self.tensors[name]
        if t.ggml_type in _PLAIN:
            return self.load(name).float()
        return gq.dequantize(self.load(name), t.ggml_type, t.shape[-1]).reshape(t.shape)


def _w_string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _w_value(v) -> bytes:
    if isinstance(v, bool):
        return struct.pack("<I?", 7, v)
    if isinstance(v, int):
        return struct.pack("<Iq", 11, v) if v < 0 or v >= 1 << 32 else struct.pack("<II", 4, v)
    if isinstance(v, float):
        return struct.pack("<If", 6, v)
    if isinstance(v, str):
        return struct.pack("<I", T_STRING) + _w_string(v)
    if isinstance(v, (list, tuple)):
        if all(isinstance(e, str) for e in v):
            return struct.pack("<IIQ", T_ARRAY, T_STRING, len(v)) + b"".join(_w_string(e) for e in v)
        if all(isinstance(e, int) for e in v):
            if all(-(1 << 31) <= e < (1 << 31) for e in v):
                return struct.pack("<IIQ", T_ARRAY, 5, len(v)) + struct.pack("<%di" % len(v), *v)
            return struct.pack("<IIQ", T_ARRAY, 11, len(v)) + struct.pack("<%dq" % len(v), *v)
        return struct.pack("<IIQ", T_ARRAY, 6, len(v)) + struct.pack("<%df" % len(v), *[float(e) for e in v])
    raise TypeError(f"unsupported GGUF metadata value {type(v)}")


def write_gguf(path, metadata: dict, tensors: dict, align: int = 32):
    """``tensors``: name -> (tensor, ggml_type, logical_shape). Plain types pass typed tensors; block types pass
    the packed uint8 rows."""
    head = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(metadata)))
    for k, v in metadata.items():
        head += _w_string(k) + _w_value(v)
    blobs, off = [], 0
    for name, (t, gt, shape) in tensors.items():
        raw = t.detach().cpu().contiguous().view(torch.uint8).reshape(-1).numpy().tobytes()
        head += _w_string(name) + struct.pack("<I", len(shape))
        for d in reversed(shape):
            head += struct.pack("<Q", d)
        head += struct.pack("<IQ", gt, off)
        blobs.append((off, raw))
        off = (off + len(raw) + align - 1) // align * align
    pad = (-len(head)) % align
    with open(path, "wb") as f:
        f.write(head + b"\0" * pad)
        pos = 0
        for o, raw in blobs:
            f.write(b"\0" * (o - pos))
            f.write(raw)
            pos = o + len(raw)


# ---------------------------------------------------------------------------------------------- name mapping
_LAYER_MAP = {
    "attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm",
    "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
    "attn_output": "self_attn.o_proj", "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm",
    "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj",
    "ffn_gate_inp": "mlp.gate", "ffn_gate_exps": "mlp.experts.gate_proj", "ffn_up_exps": "mlp.experts.up_proj",
    "ffn_down_exps": "mlp.experts.down_proj", "ffn_gate_shexp": "mlp.shared_expert.gate_proj",
    "ffn_up_shexp": "mlp.shared_expert.up_proj", "ffn_down_shexp": "mlp.shared_expert.down_proj",
    "ffn_gate_inp_shexp": "mlp.shared_expert_gate", "exp_probs_b": "mlp.gate.e_score_correction_bias",
    "attn_q_a": "self_attn.q_a_proj", "attn_q_b": "self_attn.q_b_proj", "attn_q_a_norm": "self_attn.q_a_layernorm",
    "attn_kv_a_mqa": "self_attn.kv_a_proj_with_mqa", "attn_kv_b": "self_attn.kv_b_proj",
    "attn_kv_a_norm": "self_attn.kv_a_layernorm", "post_attention_norm": "post_attention_layernorm",
    "post_ffw_norm": "post_feedforward_layernorm", "attn_gate": "self_attn.gate_proj",
}
_TOP_MAP = {"token_embd": "model.embed_tokens", "output_norm": "model.norm", "output": "lm_head"}
# architectures whose converter stores RMSNorm weights as (1 + w): loading subtracts the one again
_NORM_PLUS_ONE = {"gemma4", "gemma3", "gemma2", "qwen35", "qwen4exp"}
# architectures whose converter permutes q/k rows from half-split to interleaved rotary order
_ROPE_PERMUTED = {"llama"}


def hf_name(gguf_name: str) -> str | None:
    """llama.cpp tensor name -> checkpoint name (``None`` for tensors without a counterpart, e.g. rope tables)."""
    m = re.match(r"blk\.(\d+)\.([a-z0-9_]+)\.(weight|bias)$", gguf_name)
    if m:
        inner = _LAYER_MAP.get(m.group(2))
        return f"model.layers.{m.group(1)}.{inner}.{m.group(3)}" if inner else None
    m = re.match(r"([a-z_]+)\.(weight|bias)$", gguf_name)
    if m and m.group(1) in _TOP_MAP:
        return f"{_TOP_MAP[m.group(1)]}.{m.group(2)}"
    return None


def unpermute_rope_rows(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Inverse of the converter's q/k permutation (interleaved pairs back to the half-split rotary layout)."""
    rows = w.shape[0]
    hd = rows // n_heads
    return w.reshape(n_heads, hd // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def name_index(g: GGUFFile) -> dict[str, str]:
    """checkpoint name -> GGUF tensor name for every mappable tensor."""
    out = {}
    for n in g.tensors:
        h = hf_name(n)
        if h:
            out[h] = n
    return out
