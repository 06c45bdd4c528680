"""Vision tower (ViT with window-free bidirectional attention, 2-D rotary embedding and a 2x2 patch merger) that turns
the patches of ``loader.image.prepare_image`` into image tokens of the language model's width.

GPU: patch embedding, projections and MLPs run on the tcgen05 GEMM (``LinearBF16``), LayerNorm / bias+GELU / 2-D rope
on csrc/cuda/vision.cu, attention on the paged attention kernel with every row allowed to see all patches
(``key_end`` = last patch). CPU: the same arithmetic in PyTorch (oracle).
Reference: inc/engine/modules/vision.h, src/models/qwen3_vision.cpp (tower layout: patch embed -> blocks -> merger).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .._lib import call, ptr
from ..ops import kernels as K
from ..ops.linear import LinearBF16


@dataclass
class VisionConfig:
    depth: int = 2
    hidden: int = 128
    heads: int = 2
    mlp: int = 256
    patch: int = 16
    temporal: int = 2
    merge: int = 2
    out_hidden: int = 256
    rope_theta: float = 10000.0
    eps: float = 1e-6

    @classmethod
    def from_hf(cls, v: dict) -> "VisionConfig":
        """``vision_config`` of a Qwen3-VL-style ``config.json``."""
        return cls(depth=int(v.get("depth", 27)), hidden=int(v.get("hidden_size", 1152)), heads=int(v.get("num_heads", 16)),
                   mlp=int(v.get("intermediate_size", 4304)), patch=int(v.get("patch_size", 16)),
                   temporal=int(v.get("temporal_patch_size", 2)), merge=int(v.get("spatial_merge_size", 2)),
                   out_hidden=int(v.get("out_hidden_size", v.get("hidden_size", 1152))), eps=float(v.get("layer_norm_eps", 1e-6)))

    @property
    def patch_dim(self) -> int:
        return 3 * self.temporal * self.patch * self.patch

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


def _ln(x, w, b, eps):
    if x.is_cuda:
        y = torch.empty_like(x)
        call("layernorm", "plppplii" + "f", ptr(x), x.stride(0), ptr(w), ptr(b), ptr(y), y.stride(0), x.shape[0], x.shape[1], float(eps))
        return y
    return F.layer_norm(x.float(), (x.shape[1],), w, b, eps).to(x.dtype)


def _bias_act(x, bias, act):
    """act: 0 none, 1 gelu (erf)."""
    if x.is_cuda:
        call("bias_act", "plplii", ptr(x), x.stride(0), ptr(bias), x.shape[0], x.shape[1], act)
        return x
    v = x.float() + (bias if bias is not None else 0.0)
    if act == 1:
        v = F.gelu(v)
    return v.to(x.dtype)


def rope2d(x, prow, pcol, heads, hd, theta):
    """In-place 2-D rotary embedding of [rows, heads*hd]."""
    if x.is_cuda:
        call("rope2d", "plppiiif", ptr(x), x.stride(0), ptr(prow), ptr(pcol), x.shape[0], heads, hd, float(theta))
        return x
    half, quarter = hd // 2, hd // 4
    j = torch.arange(quarter, dtype=torch.float32)
    inv = torch.exp2(-math.log2(theta) * (2.0 * j / half))
    ang = torch.cat([prow.float()[:, None] * inv[None], pcol.float()[:, None] * inv[None]], 1)    # [rows, half]
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    v = x.float().reshape(x.shape[0], heads, hd)
    a, b = v[..., :half], v[..., half:]
    out = torch.cat([a * cs - b * sn, b * cs + a * sn], -1).reshape(x.shape[0], heads * hd)
    x.copy_(out.to(x.dtype))
    return x


class VisionTower:
    def __init__(self, cfg: VisionConfig, device):
        self.cfg, self.device = cfg, torch.device(device)
        self.blocks = []
        self.patch_embed = self.patch_bias = None
        self.merger = None

    def init_random(self, seed: int = 0, std: float = 0.02):
        c, dev = self.cfg, self.device
        g = torch.Generator().manual_seed(seed)
        rnd = lambda n, k: LinearBF16((torch.randn(n, k, generator=g) * std).to(torch.bfloat16).to(dev))
        vec = lambda n, v=0.0: torch.full((n,), v, dtype=torch.float32, device=dev) + (torch.randn(n, generator=g) * std).to(dev)
        self.patch_embed, self.patch_bias = rnd(c.hidden, c.patch_dim), vec(c.hidden)
        for _ in range(c.depth):
            self.blocks.append({"ln1_w": vec(c.hidden, 1.0), "ln1_b": vec(c.hidden), "qkv": rnd(3 * c.hidden, c.hidden),
                                "qkv_b": vec(3 * c.hidden), "proj": rnd(c.hidden, c.hidden), "proj_b": vec(c.hidden),
                                "ln2_w": vec(c.hidden, 1.0), "ln2_b": vec(c.hidden), "fc1": rnd(c.mlp, c.hidden),
                                "fc1_b": vec(c.mlp), "fc2": rnd(c.hidden, c.mlp), "fc2_b": vec(c.hidden)})
        m = c.merge * c.merge
        self.merger = {"ln_w": vec(c.hidden, 1.0), "ln_b": vec(c.hidden), "fc1": rnd(c.hidden * m, c.hidden * m),
                       "fc1_b": vec(c.hidden * m), "fc2": rnd(c.out_hidden, c.hidden * m), "fc2_b": vec(c.out_hidden)}
        return self

    # ---- checkpoint tensors ("model.visual.*" of the Qwen3-VL layout; the merger's Qwen2-VL names are read too)
    def load(self, src, prefix: str = "model.visual.") -> "VisionTower":
        """``src``: a tensor source with ``has(name)`` / ``tensor(name, device, dtype)`` (models.factory.TensorSource).
        Reference: src/models/qwen3_vision.cpp (tensor names), inc/engine/modules/vision.h."""
        c, dev, bf, f32 = self.cfg, self.device, torch.bfloat16, torch.float32

        def name(*cands):
            for n in cands:
                if src.has(prefix + n):
                    return prefix + n
            raise KeyError(f"vision tower: none of {[prefix + n for n in cands]} in the checkpoint")

        def lin(*cands):
            return LinearBF16(src.tensor(name(*(n + ".weight" for n in cands)), dev, bf).reshape(-1, src.tensor(
                name(*(n + ".weight" for n in cands)), dev, bf).shape[-1]).contiguous())

        def vec(*cands):
            return src.tensor(name(*cands), dev, f32).contiguous()
        pe = src.tensor(name("patch_embed.proj.weight"), dev, bf)               # conv [hidden, 3, t, p, p] = a linear over the patch
        self.patch_embed = LinearBF16(pe.reshape(c.hidden, -1).contiguous())
        self.patch_bias = vec("patch_embed.proj.bias") if src.has(prefix + "patch_embed.proj.bias") else torch.zeros(c.hidden, device=dev)
        self.blocks = []
        for i in range(c.depth):
            b = f"blocks.{i}."
            self.blocks.append({"ln1_w": vec(b + "norm1.weight"), "ln1_b": vec(b + "norm1.bias"), "qkv": lin(b + "attn.qkv"),
                                "qkv_b": vec(b + "attn.qkv.bias"), "proj": lin(b + "attn.proj"), "proj_b": vec(b + "attn.proj.bias"),
                                "ln2_w": vec(b + "norm2.weight"), "ln2_b": vec(b + "norm2.bias"),
                                "fc1": lin(b + "mlp.linear_fc1", b + "mlp.fc1"), "fc1_b": vec(b + "mlp.linear_fc1.bias", b + "mlp.fc1.bias"),
                                "fc2": lin(b + "mlp.linear_fc2", b + "mlp.fc2"), "fc2_b": vec(b + "mlp.linear_fc2.bias", b + "mlp.fc2.bias")})
        self.merger = {"ln_w": vec("merger.norm.weight", "merger.ln_q.weight"), "ln_b": vec("merger.norm.bias", "merger.ln_q.bias"),
                       "fc1": lin("merger.linear_fc1", "merger.mlp.0"), "fc1_b": vec("merger.linear_fc1.bias", "merger.mlp.0.bias"),
                       "fc2": lin("merger.linear_fc2", "merger.mlp.2"), "fc2_b": vec("merger.linear_fc2.bias", "merger.mlp.2.bias")}
        return self

    def load_mmproj(self, gguf) -> "VisionTower":
        """The tower from a llama.cpp vision projector file (``*mmproj*.gguf``, architecture ``clip``): ``v.patch_embd.weight``
        (+ ``.weight.1``: the second temporal slice), ``v.blk.N.{ln1,ln2}``, ``attn_qkv`` (or ``attn_q / attn_k / attn_v``),
        ``attn_out``, ``ffn_up`` / ``ffn_down``, ``v.post_ln`` (the merger's norm) and ``mm.0`` / ``mm.2`` (the merger's two
        linears). ``gguf``: a loader.gguf_file.GGUFFile."""
        c, dev, bf, f32 = self.cfg, self.device, torch.bfloat16, torch.float32
        names = set(gguf.tensors)

        def t(name, dt):
            return gguf.dequantize(name).to(dt).to(dev).contiguous()

        def lin(name):
            w = t(name + ".weight", bf)
            return LinearBF16(w.reshape(w.shape[0], -1).contiguous())

        def vec(name, n):
            return t(name, f32) if name in names else torch.zeros(n, dtype=f32, device=dev)
        pe = t("v.patch_embd.weight", bf).reshape(c.hidden, 3, 1, c.patch, c.patch)
        if "v.patch_embd.weight.1" in names:                       # the converter splits the temporal axis of the conv kernel
            pe = torch.cat([pe, t("v.patch_embd.weight.1", bf).reshape(c.hidden, 3, 1, c.patch, c.patch)], 2)
        else:
            pe = pe.expand(-1, -1, c.temporal, -1, -1) / c.temporal
        self.patch_embed = LinearBF16(pe.reshape(c.hidden, -1).contiguous())
        self.patch_bias = vec("v.patch_embd.bias", c.hidden)
        self.blocks = []
        for i in range(c.depth):
            b = f"v.blk.{i}."
            if b + "attn_qkv.weight" in names:
                qkv, qkv_b = lin(b + "attn_qkv"), vec(b + "attn_qkv.bias", 3 * c.hidden)
            else:
                qkv = LinearBF16(torch.cat([t(b + f"attn_{n}.weight", bf) for n in "qkv"], 0).contiguous())
                qkv_b = torch.cat([vec(b + f"attn_{n}.bias", c.hidden) for n in "qkv"], 0).contiguous()
            self.blocks.append({"ln1_w": vec(b + "ln1.weight", c.hidden), "ln1_b": vec(b + "ln1.bias", c.hidden), "qkv": qkv, "qkv_b": qkv_b,
                                "proj": lin(b + "attn_out"), "proj_b": vec(b + "attn_out.bias", c.hidden),
                                "ln2_w": vec(b + "ln2.weight", c.hidden), "ln2_b": vec(b + "ln2.bias", c.hidden),
                                "fc1": lin(b + "ffn_up"), "fc1_b": vec(b + "ffn_up.bias", c.mlp),
                                "fc2": lin(b + "ffn_down"), "fc2_b": vec(b + "ffn_down.bias", c.hidden)})
        m = c.merge * c.merge
        self.merger = {"ln_w": vec("v.post_ln.weight", c.hidden), "ln_b": vec("v.post_ln.bias", c.hidden),
                       "fc1": lin("mm.0"), "fc1_b": vec("mm.0.bias", c.hidden * m), "fc2": lin("mm.2"), "fc2_b": vec("mm.2.bias", c.out_hidden)}
        return self

    def state_tensors(self, prefix: str = "model.visual.") -> dict:
        """The tower's tensors under their checkpoint names (what ``load`` reads back)."""
        c = self.cfg
        out = {prefix + "patch_embed.proj.weight": self.patch_embed.weight.reshape(c.hidden, 3, c.temporal, c.patch, c.patch).cpu(),
               prefix + "patch_embed.proj.bias": self.patch_bias.cpu()}
        for i, b in enumerate(self.blocks):
            q = f"{prefix}blocks.{i}."
            for ours, theirs in (("ln1", "norm1"), ("ln2", "norm2")):
                out[q + theirs + ".weight"], out[q + theirs + ".bias"] = b[ours + "_w"].cpu(), b[ours + "_b"].cpu()
            for ours, theirs in (("qkv", "attn.qkv"), ("proj", "attn.proj"), ("fc1", "mlp.linear_fc1"), ("fc2", "mlp.linear_fc2")):
                out[q + theirs + ".weight"], out[q + theirs + ".bias"] = b[ours].weight.cpu(), b[ours + "_b"].cpu()
        m = self.merger
        out[prefix + "merger.norm.weight"], out[prefix + "merger.norm.bias"] = m["ln_w"].cpu(), m["ln_b"].cpu()
        for ours, theirs in (("fc1", "merger.linear_fc1"), ("fc2", "merger.linear_fc2")):
            out[prefix + theirs + ".weight"], out[prefix + theirs + ".bias"] = m[ours].weight.cpu(), m[ours + "_b"].cpu()
        return out

    def patch_positions(self, grid_h: int, grid_w: int):
        """(row, col) of every patch in merge-block order (the order ``prepare_image`` emits)."""
        ms = self.cfg.merge
        r = torch.arange(grid_h).reshape(grid_h // ms, ms, 1, 1).expand(grid_h // ms, ms, grid_w // ms, ms)
        c = torch.arange(grid_w).reshape(1, 1, grid_w // ms, ms).expand(grid_h // ms, ms, grid_w // ms, ms)
        r, c = r.permute(0, 2, 1, 3).reshape(-1), c.permute(0, 2, 1, 3).reshape(-1)
        return r.int().to(self.device), c.int().to(self.device)

    def _attention(self, q, k, v):
        """Bidirectional attention over one image: q, k, v [n, heads*hd]."""
        c = self.cfg
        n, hd = q.shape[0], c.head_dim
        if not q.is_cuda or hd not in (64, 128, 256):
            qh, kh, vh = (t.float().reshape(n, c.heads, hd).transpose(0, 1) for t in (q, k, v))
            p = torch.softmax(qh @ kh.transpose(1, 2) / math.sqrt(hd), -1)
            return (p @ vh).transpose(0, 1).reshape(n, c.heads * hd).to(q.dtype)
        pages = (n + 63) // 64 + 1
        kpool = torch.zeros(pages, c.heads, 64, hd, dtype=torch.bfloat16, device=q.device)
        vpool = torch.zeros_like(kpool)
        idx = torch.arange(n, device=q.device)
        kpool[1 + idx // 64, :, idx % 64] = k.reshape(n, c.heads, hd)
        vpool[1 + idx // 64, :, idx % 64] = v.reshape(n, c.heads, hd)
        table = torch.arange(1, pages, dtype=torch.int32, device=q.device)[None].contiguous()
        pos = idx.int()
        slot = torch.zeros(n, dtype=torch.int32, device=q.device)
        key_end = torch.full((n,), n - 1, dtype=torch.int32, device=q.device)
        tiles = K.make_prefill_tiles([0] * n, 1, q.device)
        qkv = torch.cat([q, k, v], 1).contiguous()
        return K.attention(qkv, pos, slot, table, kpool, vpool, c.heads, c.heads, hd, 1.0 / math.sqrt(hd), key_end=key_end,
                           tiles=tiles)

    def forward(self, patches: torch.Tensor, grid_h: int, grid_w: int) -> torch.Tensor:
        """patches [grid_h*grid_w, patch_dim] -> image tokens [grid_h*grid_w / merge^2, out_hidden] (bf16)."""
        c = self.cfg
        x = patches.to(self.device).to(torch.bfloat16)
        prow, pcol = self.patch_positions(grid_h, grid_w)
        h = _bias_act(self.patch_embed.forward(x), self.patch_bias, 0)
        for b in self.blocks:
            y = _ln(h, b["ln1_w"], b["ln1_b"], c.eps)
            qkv = _bias_act(b["qkv"].forward(y), b["qkv_b"], 0)
            q, k, v = (qkv[:, i * c.hidden:(i + 1) * c.hidden].contiguous() for i in range(3))
            rope2d(q, prow, pcol, c.heads, c.head_dim, c.rope_theta)
            rope2d(k, prow, pcol, c.heads, c.head_dim, c.rope_theta)
            a = self._attention(q, k, v)
            h = h + _bias_act(b["proj"].forward(a), b["proj_b"], 0)
            y = _ln(h, b["ln2_w"], b["ln2_b"], c.eps)
            y = _bias_act(b["fc1"].forward(y), b["fc1_b"], 1)
            h = h + _bias_act(b["fc2"].forward(y), b["fc2_b"], 0)
        m = self.merger
        y = _ln(h, m["ln_w"], m["ln_b"], c.eps).reshape(-1, c.hidden * c.merge * c.merge)
        y = _bias_act(m["fc1"].forward(y), m["fc1_b"], 1)
        return _bias_act(m["fc2"].forward(y), m["fc2_b"], 0)
