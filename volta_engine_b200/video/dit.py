"""MiniMax-H3-style video / audio diffusion transformer: the denoiser and its multi-GPU forms.

What is here (reference: inc/engine/video/h3_dit.h, src/video/h3_dit.cu, h3_dit_group.cpp, docs/video.md:120-160):

  * ``ConvRotLinear``: the checkpoint's INT8 "ConvRot" matrices: int8 rows with one fp32 scale per row and a Hadamard
    rotation over groups of 256 input channels folded into the stored matrix; the forward rotates the activation
    groups instead of un-rotating the matrix (the same product), dequantises the rows to bf16 and runs the tensor-core
    GEMM (``ops.kernels.gemm_bf16`` on the GPU).
  * ``H3Block``: AdaLN-indexed RMSNorm (a [1025, 8] timestep table interpolated at t = 1 - sigma, one [6 x modalities x
    H, 8] linear per block, rows pick their modality's shift / scale / gate), fused qkv, per-head RMSNorm of q and k, 3-D
    rotary embedding from (t, h, w) positions, non-causal attention over the whole packed sequence, gated residuals
    around the out projection and the gated-SiLU MLP; fp32 residual stream.
  * ``H3DiT``: patch embedders for video (96) and audio (32) latents and text states (5120), the block stack, the
    AdaLN final layer and the two output heads; ``forward`` takes one packed request.
  * multi-GPU: ``sp_group`` runs every block sequence parallel (each rank owns a contiguous slice of the rows with the
    full weights, attention over the local keys first and then over every peer's slice,
    ``parallel.sequence_parallel.context_parallel_attention``); ``tp_rank / tp_ranks`` shard heads and MLP width with
    fp32 all-reduces of the two partial projections per block.
  * ``denoise``: flow-matching Euler steps over a shifted sigma schedule (``sigma' = s sigma / (1 + (s - 1) sigma)``).

Not here: the text tower, the video / audio VAEs, the job service and the mux (the other files of this package); LoRA
adapters are ``video/lora.py`` (``add_lora`` / ``set_lora_scale`` / ``clear_loras`` below). The bf16 GEMM removes the reference's power-of-two row scaling of the
gated activation (an fp16 range device).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..parallel.sequence_parallel import attention_finish, attention_partial, context_parallel_attention

VIDEO, TEXT, AUDIO = 0, 1, 2
MODALITIES = 3


@dataclass
class H3Config:
    hidden: int = 5376
    layers: int = 50
    heads: int = 56
    head_dim: int = 128
    ffn: int = 14336
    latents: int = 96             # video patch width: 24 channels x (1 x 2 x 2)
    audio_latents: int = 32
    text_dim: int = 5120
    adaln_grid: int = 1025
    adaln_dim: int = 8
    rope_freqs: int = 16          # frequencies per axis: 3 x 2 x 16 = 96 rotated dims of every head
    eps: float = 1e-5
    qk_eps: float = 1e-5

    @classmethod
    def tiny(cls, **kw):
        c = cls(hidden=256, layers=2, heads=4, head_dim=64, ffn=512, latents=24, audio_latents=8, text_dim=64, adaln_grid=17,
                rope_freqs=8)
        for k, v in kw.items():
            setattr(c, k, v)
        return c


# ------------------------------------------------------------------------------------------------ ConvRot INT8
def hadamard_groups(x: torch.Tensor, group: int = 256) -> torch.Tensor:
    """Orthonormal Walsh-Hadamard transform over consecutive groups of ``group`` channels (last dim)."""
    shape = x.shape
    y = x.reshape(-1, shape[-1] // group, group).float()
    h = 1
    while h < group:
        y = y.reshape(y.shape[0], y.shape[1], group // (2 * h), 2, h)
        a, b = y[..., 0, :], y[..., 1, :]
        y = torch.stack((a + b, a - b), dim=-2).reshape(y.shape[0], y.shape[1], group)
        h *= 2
    return (y * group ** -0.5).reshape(shape)


class ConvRotLinear:
    """y = x W^T with W stored as int8 rows of (W H_256) and one scale per row."""

    def __init__(self, q: torch.Tensor, scale: torch.Tensor, group: int = 256):
        self.q, self.scale, self.group = q.contiguous(), scale.float().contiguous(), group
        self.out_features, self.in_features = q.shape
        assert self.in_features % group == 0, "the rotation works on whole groups of input channels"

    @classmethod
    def from_dense(cls, w: torch.Tensor, group: int = 256):
        rot = hadamard_groups(w.float(), group)                     # rows of W H (H symmetric and orthonormal)
        scale = rot.abs().amax(dim=1).clamp(min=1e-12) / 127.0
        q = torch.round(rot / scale[:, None]).clamp(-127, 127).to(torch.int8)
        return cls(q, scale, group)

    def to(self, device):
        return ConvRotLinear(self.q.to(device), self.scale.to(device), self.group)

    def shard(self, rows: torch.Tensor | None = None, cols: tuple | None = None):
        """A tensor-parallel piece: ``rows`` (output features; their scales travel with them) and / or a column range
        that keeps whole rotation groups."""
        q, s = self.q, self.scale
        if rows is not None:
            q, s = q[rows], s[rows]
        if cols is not None:
            assert cols[0] % self.group == 0 and cols[1] % self.group == 0, "column shards keep whole rotation groups"
            q = q[:, cols[0]:cols[1]]
        return ConvRotLinear(q, s, self.group)

    def dequant(self) -> torch.Tensor:
        """The effective dense weight [out, in] (fp32)."""
        return hadamard_groups(self.q.float() * self.scale[:, None], self.group)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xr = hadamard_groups(x, self.group)
        if x.is_cuda:
            w = (self.q.float() * self.scale[:, None]).to(torch.bfloat16)
            return K.gemm_bf16(w, xr.to(torch.bfloat16).contiguous(), out_f32=True)
        return xr @ (self.q.float() * self.scale[:, None]).t()

    def nbytes(self) -> int:
        return self.q.numel() + self.scale.numel() * 4


# ------------------------------------------------------------------------------------------------ pieces
def rms(x: torch.Tensor, w: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + eps)
    return y * w.float() if w is not None else y


def rope3d(x: torch.Tensor, pos: torch.Tensor, freqs: int, theta: float = 10000.0) -> torch.Tensor:
    """x [rows, heads, hd]; pos [rows, 3] (t, h, w). Axis a rotates dims [2 a freqs, 2 (a + 1) freqs) as NeoX pairs; the rest
    of the head is left alone."""
    inv = theta ** (-torch.arange(freqs, device=x.device, dtype=torch.float32) / freqs)
    out = x.float().clone()
    for a in range(3):
        ang = pos[:, a].float()[:, None] * inv[None]                 # [rows, freqs]
        cs, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]
        lo = 2 * a * freqs
        u, v = x[..., lo:lo + freqs].float(), x[..., lo + freqs:lo + 2 * freqs].float()
        out[..., lo:lo + freqs] = u * cs - v * sn
        out[..., lo + freqs:lo + 2 * freqs] = v * cs + u * sn
    return out


def timestep_embedding(table: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
    """Linear interpolation of the [grid, dim] table at t in [0, 1] (t = 1 - sigma): -> [len(t), dim]."""
    grid = table.shape[0]
    p = t.float().clamp(0, 1) * (grid - 1)
    lo = p.floor().long().clamp(max=grid - 2)
    fr = (p - lo.float())[:, None]
    return table[lo] + fr * (table[lo + 1] - table[lo])


@dataclass
class H3Request:
    """One packed request; row order [text | audio | video] (any order works: rows carry their own tags)."""
    video: torch.Tensor           # [n_img, latents] fp32
    audio: torch.Tensor           # [n_audio, audio_latents]
    prompt: torch.Tensor          # [text_len, text_dim]
    pos: torch.Tensor             # [rows, 3] (t, h, w)
    tags: torch.Tensor            # [rows] modality of every row
    t: torch.Tensor               # [rows] timestep of every row (t = 1 - sigma; text rows: 1)


class H3Block:
    def __init__(self, cfg: H3Config, w: dict, tp_rank: int = 0, tp_ranks: int = 1, group=None):
        self.cfg, self.tp_rank, self.tp_ranks, self.group = cfg, tp_rank, tp_ranks, group
        self.heads = cfg.heads // tp_ranks
        self.qkv, self.out, self.fc1, self.fc2 = w["qkv"], w["out"], w["fc1"], w["fc2"]
        self.aw, self.ab = w["adaln_w"], w["adaln_b"]                 # [6 * MODALITIES * H, adaln_dim], [6 * MODALITIES * H]
        self.n1, self.n2, self.qn, self.kn = w["norm1"], w["norm2"], w["q_norm"], w["k_norm"]
        self.sp_group = None
        self.layer, self.adapters = 0, None          # block index and the model's list of active LoRA adapters

    def _lora(self, slot: int, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        if self.adapters:
            from .lora import apply_lora
            apply_lora(self.adapters, self.layer, slot, x, y)
        return y

    def _mod(self, temb_rows: torch.Tensor, tags: torch.Tensor):
        """Per row (shift1, scale1, gate1, shift2, scale2, gate2), each [rows, H], from its timestep and modality."""
        H = self.cfg.hidden
        ada = temb_rows @ self.aw.t() + self.ab                          # [rows, 6 * MODALITIES * H]
        ada = ada.reshape(-1, MODALITIES, 6, H)
        pick = ada[torch.arange(ada.shape[0], device=ada.device), tags.long()]      # [rows, 6, H]
        return [pick[:, i] for i in range(6)]

    def _sum(self, y: torch.Tensor) -> torch.Tensor:
        if self.tp_ranks > 1:
            y = y.float().contiguous()
            dist.all_reduce(y, group=self.group)
        return y

    def forward(self, x: torch.Tensor, temb_rows, tags, pos) -> torch.Tensor:
        cfg = self.cfg
        hd, nh = cfg.head_dim, self.heads
        sh1, sc1, g1, sh2, sc2, g2 = self._mod(temb_rows, tags)
        h = rms(x, self.n1, cfg.eps) * (1 + sc1) + sh1
        qkv = self._lora(0, h, self.qkv.forward(h).float())
        rows = x.shape[0]
        q = rms(qkv[:, : nh * hd].reshape(rows, nh, hd), self.qn, cfg.qk_eps)
        k = rms(qkv[:, nh * hd:2 * nh * hd].reshape(rows, nh, hd), self.kn, cfg.qk_eps)
        v = qkv[:, 2 * nh * hd:].reshape(rows, nh, hd)
        q, k = rope3d(q, pos, cfg.rope_freqs), rope3d(k, pos, cfg.rope_freqs)
        if self.sp_group is not None:
            att = context_parallel_attention(q, k, v, hd ** -0.5, causal=False, group=self.sp_group[0])
        elif x.is_cuda and hd in (64, 128):
            # one GPU: the engine's paged attention kernel over the packed rows (head_dim 128: the tcgen05 prefill kernel)
            from .common import full_attention
            att = full_attention(q.reshape(rows, nh * hd), k.reshape(rows, nh * hd), v.reshape(rows, nh * hd), nh, hd).float()
        else:
            att = attention_finish(attention_partial(q, k, v, None, hd ** -0.5))
        att = att.reshape(rows, nh * hd)
        x = x + g1 * self._sum(self._lora(1, att, self.out.forward(att)))      # (a tensor-parallel delta is partial like the base product)
        h = rms(x, self.n2, cfg.eps) * (1 + sc2) + sh2
        a = self._lora(2, h, self.fc1.forward(h).float())
        f = a.shape[1] // 2
        z = torch.nn.functional.silu(a[:, :f]) * a[:, f:]
        return x + g2 * self._sum(self._lora(3, z, self.fc2.forward(z)))


class H3DiT:
    def __init__(self, cfg: H3Config, device="cpu", tp_rank: int = 0, tp_ranks: int = 1, tp_group=None):
        self.cfg, self.device = cfg, torch.device(device)
        self.tp_rank, self.tp_ranks, self.tp_group = tp_rank, tp_ranks, tp_group
        self.blocks: list[H3Block] = []
        self.sp = None
        self.adapters: list = []                     # active LoRA adapters (video/lora.py), shared with the blocks

    def init_random(self, seed: int = 0, std: float = 0.02):
        """Random weights of the full architecture; a tensor-parallel instance keeps its shard (every rank draws the same
        matrices)."""
        cfg, dev = self.cfg, self.device
        g = torch.Generator().manual_seed(seed)
        rnd = lambda *s, sc=std: torch.randn(*s, generator=g) * sc
        H, hd, nh, F = cfg.hidden, cfg.head_dim, cfg.heads, cfg.ffn
        r, n = self.tp_rank, self.tp_ranks
        hl, fl = nh // n, F // n
        assert n == 1 or (nh % n == 0 and F % n == 0 and (hl * hd) % 256 == 0 and fl % 256 == 0), \
            "tensor-parallel shards keep whole 256-channel rotation groups"
        self.embed_v, self.embed_a, self.embed_t = rnd(H, cfg.latents).to(dev), rnd(H, cfg.audio_latents).to(dev), rnd(H, cfg.text_dim).to(dev)
        self.table = rnd(cfg.adaln_grid, cfg.adaln_dim, sc=1.0).to(dev)
        ar = torch.arange
        for _ in range(cfg.layers):
            qkv = ConvRotLinear.from_dense(rnd(3 * nh * hd, H))
            out = ConvRotLinear.from_dense(rnd(H, nh * hd))
            fc1 = ConvRotLinear.from_dense(rnd(2 * F, H))
            fc2 = ConvRotLinear.from_dense(rnd(H, F))
            if n > 1:
                hrows = ar(r * hl * hd, (r + 1) * hl * hd)
                qkv = qkv.shard(rows=torch.cat([hrows, nh * hd + hrows, 2 * nh * hd + hrows]))
                out = out.shard(cols=(r * hl * hd, (r + 1) * hl * hd))
                frows = ar(r * fl, (r + 1) * fl)
                fc1 = fc1.shard(rows=torch.cat([frows, F + frows]))
                fc2 = fc2.shard(cols=(r * fl, (r + 1) * fl))
            w = {"qkv": qkv.to(dev), "out": out.to(dev), "fc1": fc1.to(dev), "fc2": fc2.to(dev),
                 "adaln_w": rnd(6 * MODALITIES * H, cfg.adaln_dim, sc=0.1).to(dev), "adaln_b": torch.zeros(6 * MODALITIES * H, device=dev),
                 "norm1": torch.ones(H, device=dev), "norm2": torch.ones(H, device=dev),
                 "q_norm": torch.ones(hd, device=dev), "k_norm": torch.ones(hd, device=dev)}
            w["adaln_b"].view(MODALITIES, 6, H)[:, (2, 5)] = 1.0          # gates start open
            self.blocks.append(H3Block(cfg, w, r, n, self.tp_group))
            self.blocks[-1].layer, self.blocks[-1].adapters = len(self.blocks) - 1, self.adapters
        self.final_w, self.final_b = rnd(2 * H, cfg.adaln_dim, sc=0.1).to(dev), torch.zeros(2 * H, device=dev)
        self.head_v, self.head_a = rnd(cfg.latents, H).to(dev), rnd(cfg.audio_latents, H).to(dev)
        return self

    def add_lora(self, path, scale: float = 1.0) -> int:
        """Stage an adapter file beside the base weights (this rank's shard of it); returns its id."""
        from .lora import load_adapter
        self.adapters.append(load_adapter(path, self.cfg, scale, self.tp_rank, self.tp_ranks, self.device))
        return len(self.adapters) - 1

    def set_lora_scale(self, idx: int, scale: float) -> None:
        if 0 <= idx < len(self.adapters):
            self.adapters[idx].scale = float(scale)

    def clear_loras(self) -> None:
        del self.adapters[:]                          # in place: the blocks hold the same list

    def set_sp(self, group, rank: int, ranks: int):
        """Sequence parallelism: this instance owns a contiguous 1 / ranks of the rows of every packed sequence."""
        self.sp = (group, rank, ranks)
        for b in self.blocks:
            b.sp_group = self.sp

    def embed(self, req: H3Request) -> torch.Tensor:
        H = self.cfg.hidden
        x = torch.zeros(req.tags.shape[0], H, dtype=torch.float32, device=self.device)
        x[req.tags == VIDEO] = req.video.float() @ self.embed_v.t()
        x[req.tags == AUDIO] = req.audio.float() @ self.embed_a.t()
        x[req.tags == TEXT] = req.prompt.float() @ self.embed_t.t()
        return x

    def forward(self, req: H3Request):
        """-> (video_out [n_img, latents], audio_out [n_audio, audio_latents]): the predicted velocity of every latent row.
        Sequence parallel: every rank passes the whole request and gets the whole outputs back (rows are gathered)."""
        cfg = self.cfg
        x = self.embed(req)
        temb = timestep_embedding(self.table, req.t.to(self.device))
        tags, pos = req.tags.to(self.device), req.pos.to(self.device)
        rows = x.shape[0]
        sl = slice(0, rows)
        if self.sp is not None:
            _, r, n = self.sp
            per = rows // n
            assert per * n == rows, "packed rows must divide by the sequence-parallel ranks (pad with rows of their own)"
            sl = slice(r * per, (r + 1) * per)
        x, temb_l, tags_l, pos_l = x[sl], temb[sl], tags[sl], pos[sl]
        for b in self.blocks:
            x = b.forward(x, temb_l, tags_l, pos_l)
        fin = temb_l @ self.final_w.t() + self.final_b
        H = cfg.hidden
        x = rms(x, None, cfg.eps) * (1 + fin[:, H:]) + fin[:, :H]
        if self.sp is not None:
            full = torch.empty(rows, H, dtype=x.dtype, device=x.device)
            dist.all_gather_into_tensor(full, x.contiguous(), group=self.sp[0])
            x = full
        return x[tags == VIDEO] @ self.head_v.t(), x[tags == AUDIO] @ self.head_a.t()

    def weight_bytes(self) -> int:
        return sum(b.qkv.nbytes() + b.out.nbytes() + b.fc1.nbytes() + b.fc2.nbytes() for b in self.blocks)


# ------------------------------------------------------------------------------------------------ sampler
def sigma_schedule(steps: int, shift: float = 6.0) -> torch.Tensor:
    """steps + 1 noise levels from 1 to 0, warped by the flow shift: sigma' = s sigma / (1 + (s - 1) sigma)."""
    s = torch.linspace(1.0, 0.0, steps + 1)
    return shift * s / (1 + (shift - 1) * s)


def make_request(video, audio, prompt, grid: tuple, sigma_v: float, sigma_a: float) -> H3Request:
    """Pack latents and text states: positions (t, h, w) of the video rows from the latent grid (frames, height, width),
    audio rows along t, text rows at the origin; timesteps t = 1 - sigma per modality (text rows: 1)."""
    F_, Hh, Ww = grid
    assert video.shape[0] == F_ * Hh * Ww
    dev = video.device
    tt, hh, ww = torch.meshgrid(torch.arange(F_), torch.arange(Hh), torch.arange(Ww), indexing="ij")
    pv = torch.stack([tt, hh, ww], -1).reshape(-1, 3).float().to(dev)
    pa = torch.stack([torch.arange(audio.shape[0]).float(), torch.zeros(audio.shape[0]), torch.zeros(audio.shape[0])], -1).to(dev)
    pt = torch.zeros(prompt.shape[0], 3, device=dev)
    tags = torch.cat([torch.full((prompt.shape[0],), TEXT), torch.full((audio.shape[0],), AUDIO), torch.full((video.shape[0],), VIDEO)]).to(dev)
    t = torch.cat([torch.ones(prompt.shape[0]), torch.full((audio.shape[0],), 1 - sigma_a), torch.full((video.shape[0],), 1 - sigma_v)]).to(dev)
    return H3Request(video, audio, prompt, torch.cat([pt, pa, pv]), tags, t)


def denoise(model: H3DiT, prompt: torch.Tensor, grid: tuple, audio_rows: int, steps: int, seed: int = 0,
            video_shift: float = 6.0, audio_shift: float = 3.0, pad_to: int = 1):
    """Flow-matching sampler: latents start as noise and follow x <- x + (sigma_next - sigma) v(x, sigma) along each
    modality's schedule. Returns (video latents [frames * h * w, latents], audio latents)."""
    cfg, dev = model.cfg, model.device
    g = torch.Generator().manual_seed(seed)
    n_img = grid[0] * grid[1] * grid[2]
    total = prompt.shape[0] + audio_rows + n_img
    assert total % pad_to == 0, "pad the prompt so the packed rows divide by the sequence-parallel ranks"
    xv = torch.randn(n_img, cfg.latents, generator=g).to(dev)
    xa = torch.randn(audio_rows, cfg.audio_latents, generator=g).to(dev)
    sv, sa = sigma_schedule(steps, video_shift), sigma_schedule(steps, audio_shift)
    for i in range(steps):
        req = make_request(xv, xa, prompt.to(dev), grid, float(sv[i]), float(sa[i]))
        vv, va = model.forward(req)
        xv = xv + float(sv[i + 1] - sv[i]) * vv.to(xv.dtype)
        xa = xa + float(sa[i + 1] - sa[i]) * va.to(xa.dtype)
    return xv, xa


def frames_rgb8(latents: torch.Tensor, grid: tuple, proj: torch.Tensor | None = None) -> torch.Tensor:
    """A quick look at latents without the VAE decoder (``video.vae.VideoDecoder`` is the real one): unpatchify the [frames * h * w, 24 x 2 x 2] latents to
    [frames, 2 h, 2 w, 24] and project 24 channels to RGB with ``proj`` [3, 24] (default: the first three channels);
    returns uint8 [frames, 2 h, 2 w, 3]."""
    F_, Hh, Ww = grid
    c = latents.shape[1] // 4
    x = latents.float().reshape(F_, Hh, Ww, c, 2, 2).permute(0, 1, 4, 2, 5, 3).reshape(F_, 2 * Hh, 2 * Ww, c)
    rgb = x @ proj.t().float() if proj is not None else x[..., :3]
    return ((rgb.clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8)
