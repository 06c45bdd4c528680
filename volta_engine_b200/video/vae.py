"""Video VAE of the MiniMax-H3 pipeline: a ViT decoder run on overlapping tiles, and a causal 3-D convolution encoder
whose convolutions are im2col + GEMM with the taps that fall into the causal padding skipped.

Decoder (reference: src/video/h3_vae.cu; docs/video.md:197-203): a latent frame block [T, h, w, 24] becomes one token per
latent pixel; ViT blocks (LayerNorm, bidirectional attention with heads of 64, GELU MLP) run over the tokens of a tile;
a linear head turns every token into its 4 x 16 x 16 x 3 output patch (temporal 4x, spatial 16x). A picture is decoded in
temporal chunks of 7 latent frames and spatial tiles of 16 latent pixels (256 px) that overlap by 4 (64 px); overlaps are
blended with linear ramps and the result is streamed to RGB8.

Encoder (reference: src/video/h3_vae_enc.cu): stride-2 stages of causal 3-D convolutions (time is padded in front only,
so frame t never sees frame t + 1), SiLU, a residual convolution per stage; 16x spatial and 4x temporal reduction to 24
latent channels. The first frame of a clip stands alone (1 + 4k frames -> 1 + k latent frames), as in causal video VAEs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .common import full_attention, layer_norm


@dataclass
class VaeConfig:
    latent: int = 24
    dim: int = 2048
    blocks: int = 36
    heads: int = 32
    head_dim: int = 64
    mlp: int = 8192
    t_up: int = 4                 # output frames per latent frame
    s_up: int = 16                # output pixels per latent pixel (each axis)
    tile: int = 16                # latent pixels per tile edge (256 px)
    overlap: int = 4              # latent pixels shared by neighbouring tiles (64 px)
    chunk: int = 7                # latent frames per temporal chunk
    enc_width: int = 128          # channels of the encoder's first stage (doubling per stage up to 4x)
    eps: float = 1e-6

    @classmethod
    def tiny(cls, **kw):
        c = cls(latent=4, dim=64, blocks=2, heads=2, head_dim=32, mlp=128, t_up=4, s_up=4, tile=4, overlap=2, chunk=3, enc_width=8)
        for k, v in kw.items():
            setattr(c, k, v)
        return c


# ------------------------------------------------------------------------------------------------ decoder
class VideoDecoder:
    def __init__(self, cfg: VaeConfig, device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        self.w = None

    def init_random(self, seed: int = 0, std: float = 0.02):
        c, g = self.cfg, torch.Generator().manual_seed(seed)

        def rnd(*shape, s=std):
            return (torch.randn(*shape, generator=g) * s).to(self.device)
        patch = c.t_up * c.s_up * c.s_up * 3
        self.w = {"in": rnd(c.dim, c.latent), "in_b": torch.zeros(c.dim, device=self.device),
                  "pos_t": rnd(64, c.dim), "pos_h": rnd(256, c.dim), "pos_w": rnd(256, c.dim),
                  "blocks": [{"ln1": torch.ones(c.dim, device=self.device), "ln1_b": torch.zeros(c.dim, device=self.device),
                              "qkv": rnd(3 * c.heads * c.head_dim, c.dim), "proj": rnd(c.dim, c.heads * c.head_dim),
                              "ln2": torch.ones(c.dim, device=self.device), "ln2_b": torch.zeros(c.dim, device=self.device),
                              "fc1": rnd(c.mlp, c.dim), "fc2": rnd(c.dim, c.mlp)} for _ in range(c.blocks)],
                  "ln_f": torch.ones(c.dim, device=self.device), "ln_f_b": torch.zeros(c.dim, device=self.device),
                  "head": rnd(patch, c.dim, s=0.1), "head_b": torch.zeros(patch, device=self.device)}
        return self

    def decode_tile(self, lat: torch.Tensor, t0: int = 0, h0: int = 0, w0: int = 0) -> torch.Tensor:
        """lat [T, h, w, latent] (one tile of one temporal chunk; (t0, h0, w0) = its place in the clip, for the position
        embeddings) -> pixels [T * t_up, h * s_up, w * s_up, 3] in [-1, 1]."""
        c, W = self.cfg, self.w
        T, h, w, _ = lat.shape
        dt = torch.bfloat16 if lat.is_cuda else torch.float32
        tt, hh, ww = torch.meshgrid(torch.arange(T) + t0, torch.arange(h) + h0, torch.arange(w) + w0, indexing="ij")
        x = lat.reshape(-1, c.latent).float() @ W["in"].t() + W["in_b"]
        x = x + W["pos_t"][tt.reshape(-1) % 64] + W["pos_h"][hh.reshape(-1) % 256] + W["pos_w"][ww.reshape(-1) % 256]
        for b in W["blocks"]:
            y = layer_norm(x, b["ln1"], b["ln1_b"], c.eps).to(dt)
            qkv = y @ b["qkv"].t().to(dt)
            n = c.heads * c.head_dim
            a = full_attention(qkv[:, :n].contiguous(), qkv[:, n:2 * n].contiguous(), qkv[:, 2 * n:].contiguous(), c.heads, c.head_dim)
            x = x + (a.to(dt) @ b["proj"].t().to(dt)).float()
            y = layer_norm(x, b["ln2"], b["ln2_b"], c.eps).to(dt)
            x = x + (F.gelu(y @ b["fc1"].t().to(dt), approximate="tanh") @ b["fc2"].t().to(dt)).float()
        y = layer_norm(x, W["ln_f"], W["ln_f_b"], c.eps)
        px = (y @ W["head"].t() + W["head_b"]).reshape(T, h, w, c.t_up, c.s_up, c.s_up, 3)
        return torch.tanh(px.permute(0, 3, 1, 4, 2, 5, 6).reshape(T * c.t_up, h * c.s_up, w * c.s_up, 3))

    @staticmethod
    def tile_starts(size: int, tile: int, overlap: int) -> list[int]:
        """First latent pixel of every tile along one axis: steps of tile - overlap, the last tile flush with the edge."""
        if size <= tile:
            return [0]
        step = tile - overlap
        starts = list(range(0, size - tile, step)) + [size - tile]
        return sorted(set(starts))

    def decode(self, latents: torch.Tensor, on_tile=None) -> torch.Tensor:
        """latents [F, H, W, latent] -> uint8 frames [F * t_up, H * s_up, W * s_up, 3]. Tiles are blended where they
        overlap with weights that ramp linearly from the tile's edge (tiles at the picture's edge keep full weight
        there). ``on_tile(done, total)`` reports progress."""
        c = self.cfg
        Fr, H, Wd, _ = latents.shape
        out = torch.zeros(Fr * c.t_up, H * c.s_up, Wd * c.s_up, 3)
        hs, ws = self.tile_starts(H, c.tile, c.overlap), self.tile_starts(Wd, c.tile, c.overlap)
        chunks = list(range(0, Fr, c.chunk))
        total, done = len(chunks) * len(hs) * len(ws), 0
        for f0 in chunks:
            f1 = min(Fr, f0 + c.chunk)
            acc = torch.zeros((f1 - f0) * c.t_up, H * c.s_up, Wd * c.s_up, 3)
            wsum = torch.zeros(H * c.s_up, Wd * c.s_up, 1)
            for h0 in hs:
                for w0 in ws:
                    h1, w1 = min(H, h0 + c.tile), min(Wd, w0 + c.tile)
                    px = self.decode_tile(latents[f0:f1, h0:h1, w0:w1].to(self.device), f0, h0, w0).float().cpu()
                    wy = self._ramp(h1 - h0, h0 > 0, h1 < H, c.overlap, c.s_up)
                    wx = self._ramp(w1 - w0, w0 > 0, w1 < Wd, c.overlap, c.s_up)
                    wt = (wy[:, None] * wx[None, :])[..., None]
                    ys, xs = slice(h0 * c.s_up, h1 * c.s_up), slice(w0 * c.s_up, w1 * c.s_up)
                    acc[:, ys, xs] += px * wt
                    wsum[ys, xs] += wt
                    done += 1
                    if on_tile is not None:
                        on_tile(done, total)
            out[f0 * c.t_up:f1 * c.t_up] = acc / wsum.clamp(min=1e-6)
        return ((out.clamp(-1, 1) + 1) * 127.5).round().to(torch.uint8)

    @staticmethod
    def _ramp(n_lat: int, ramp_lo: bool, ramp_hi: bool, overlap: int, up: int) -> torch.Tensor:
        n, r = n_lat * up, overlap * up
        w = torch.ones(n)
        if r > 0:
            ramp = (torch.arange(r).float() + 0.5) / r
            if ramp_lo:
                w[:r] = ramp
            if ramp_hi:
                w[n - r:] = torch.minimum(w[n - r:], ramp.flip(0))
        return w


# ------------------------------------------------------------------------------------------------ encoder
def causal_conv3d(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None, stride=(1, 1, 1)) -> torch.Tensor:
    """x [C, T, H, W], w [O, C, kt, kh, kw]: time is padded by kt - 1 zero frames in FRONT (causal), height and width by
    (k - 1) / 2 on both sides. Computed as im2col + GEMM per output frame; for the first output frames the taps that would
    read the front padding are left out of the GEMM instead of being multiplied by zeros."""
    O, C, kt, kh, kw = w.shape
    st, sh, sw = stride
    _, T, H, W = x.shape
    xp = F.pad(x, (kw // 2, kw // 2, kh // 2, kh // 2))
    Ho, Wo = (H + 2 * (kh // 2) - kh) // sh + 1, (W + 2 * (kw // 2) - kw) // sw + 1
    To = (T - 1) // st + 1
    out = torch.empty(O, To, Ho, Wo, dtype=x.dtype, device=x.device)
    for to in range(To):
        t_last = to * st                                  # newest input frame this output frame sees
        taps = [(k, t_last - (kt - 1) + k) for k in range(kt) if t_last - (kt - 1) + k >= 0]      # valid taps only
        cols = torch.cat([F.unfold(xp[:, t][None], (kh, kw), stride=(sh, sw)) for _, t in taps], 1)[0]   # [taps*C*kh*kw, Ho*Wo]
        wk = torch.cat([w[:, :, k].reshape(O, C * kh * kw) for k, _ in taps], 1)
        y = wk.to(cols.dtype) @ cols
        if b is not None:
            y = y + b[:, None].to(y.dtype)
        out[:, to] = y.reshape(O, Ho, Wo)
    return out


class VideoEncoder:
    """conv_in -> four stride-2 spatial stages (the first two also halve time) -> conv_out to the latent channels."""

    def __init__(self, cfg: VaeConfig, device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        self.w = None

    def init_random(self, seed: int = 0, std: float = 0.05):
        c, g = self.cfg, torch.Generator().manual_seed(seed)

        def conv(o, i, k=3):
            return ((torch.randn(o, i, k, k, k, generator=g) * std / math.sqrt(i)).to(self.device), torch.zeros(o, device=self.device))
        stages, ch = [], c.enc_width
        n_stage = int(round(math.log2(c.s_up)))
        n_time = int(round(math.log2(c.t_up)))
        prev = ch
        for s in range(n_stage):
            nxt = min(ch * (2 ** s), ch * 4)
            stages.append({"down": conv(nxt, prev), "res": conv(nxt, nxt), "stride": (2 if s < n_time else 1, 2, 2)})
            prev = nxt
        self.w = {"in": conv(ch, 3), "stages": stages, "out": conv(c.latent, prev, 1)}
        return self

    def encode(self, frames: torch.Tensor) -> torch.Tensor:
        """frames [T, H, W, 3] uint8 or float in [-1, 1], T = 1 + t_up * k -> latents [1 + k, H / s_up, W / s_up, latent].
        The first frame is encoded by itself (repeated to fill one temporal block), the rest in blocks of t_up."""
        c = self.cfg
        x = frames.float()
        if frames.dtype == torch.uint8:
            x = x / 127.5 - 1
        T = x.shape[0]
        assert (T - 1) % c.t_up == 0, "a clip holds 1 + t_up * k frames"
        x = torch.cat([x[:1].expand(c.t_up, -1, -1, -1), x[1:]], 0)          # the lone first frame fills a block of its own
        x = x.permute(3, 0, 1, 2).contiguous().to(self.device)              # [3, T', H, W]
        W = self.w
        x = F.silu(causal_conv3d(x, *W["in"]))
        for s in W["stages"]:
            x = F.silu(causal_conv3d(x, *s["down"], stride=s["stride"]))
            x = x + F.silu(causal_conv3d(x, *s["res"]))
        z = causal_conv3d(x, *W["out"])
        # strided causal convolutions keep output frame j = input frames <= j * stride: take the last frame of every block
        k = z.shape[1]
        want = 1 + (T - 1) // c.t_up
        return z[:, k - want:].permute(1, 2, 3, 0).contiguous()
