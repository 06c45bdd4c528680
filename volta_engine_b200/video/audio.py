"""Audio VAE of the MiniMax-H3 pipeline: a DAC-style convolutional encoder and a BigVGAN-style decoder (snake activations
between alias-free 2x up / down resamplers, transposed-convolution upsampling, residual dilated convolutions), 1-D
convolutions throughout. Latents: 32 channels; output: stereo PCM at 32 kHz.
Reference: src/video/h3_audio.cu (conv1d / snake / resample kernels and the two stacks); docs/video.md:204.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class AudioConfig:
    latent: int = 32
    channels: int = 2
    width: int = 1536                         # decoder channels at the latent rate (halved per upsampling stage)
    rates: tuple = (8, 5, 4, 2, 2)            # upsampling factors: 640 samples per latent frame
    dilations: tuple = (1, 3, 5)
    sample_rate: int = 32000

    @classmethod
    def tiny(cls, **kw):
        c = cls(latent=4, channels=2, width=16, rates=(4, 2), dilations=(1, 3), sample_rate=8000)
        for k, v in kw.items():
            setattr(c, k, v)
        return c

    @property
    def hop(self) -> int:
        return math.prod(self.rates)


def snake(x: torch.Tensor, log_alpha: torch.Tensor, log_beta: torch.Tensor | None = None) -> torch.Tensor:
    """x + sin^2(alpha x) / beta per channel (alpha, beta stored as logarithms; beta = alpha when not given). x [C, T]."""
    a = log_alpha.exp()[:, None]
    b = a if log_beta is None else log_beta.exp()[:, None]
    return x + torch.sin(a * x) ** 2 / (b + 1e-9)


def kaiser_sinc(cutoff: float, half_width: float, taps: int) -> torch.Tensor:
    """Low-pass filter: a sinc at ``cutoff`` (cycles per sample) under a Kaiser window whose shape follows from the
    transition width; normalised to unit sum."""
    delta = 2.285 * (taps // 2 - 1) * math.pi * 4 * half_width + 7.95
    beta = 0.1102 * (delta - 8.7) if delta > 50 else (0.5842 * (delta - 21) ** 0.4 + 0.07886 * (delta - 21) if delta >= 21 else 0.0)
    win = torch.kaiser_window(taps, periodic=False, beta=beta)
    t = torch.arange(taps).float() - (taps - 1) / 2
    f = 2 * cutoff * win * torch.sinc(2 * cutoff * t)
    return f / f.sum()


def upsample2(x: torch.Tensor, taps: int = 12) -> torch.Tensor:
    """[C, T] -> [C, 2 T]: zero stuffing + low-pass at a quarter of the new rate (alias-free)."""
    f = kaiser_sinc(0.25, 0.3, taps).to(x)
    C = x.shape[0]
    pad = taps // 2 - 1
    xp = F.pad(x[None], (pad + 1, pad + 1), mode="replicate")
    y = F.conv_transpose1d(xp, (2 * f)[None, None].expand(C, 1, taps), stride=2, groups=C)[0]
    cut = (y.shape[1] - 2 * x.shape[1]) // 2
    return y[:, cut:cut + 2 * x.shape[1]]


def downsample2(x: torch.Tensor, taps: int = 12) -> torch.Tensor:
    """[C, 2 T] -> [C, T]: low-pass at a quarter of the rate, then every second sample."""
    f = kaiser_sinc(0.25, 0.3, taps).to(x)
    C = x.shape[0]
    xp = F.pad(x[None], (taps // 2 - 1, taps // 2), mode="replicate")
    return F.conv1d(xp, f[None, None].expand(C, 1, taps), stride=2, groups=C)[0]


def act1d(x: torch.Tensor, log_alpha: torch.Tensor) -> torch.Tensor:
    """The anti-aliased activation: the snake runs at twice the rate so that the harmonics it creates can be filtered."""
    return downsample2(snake(upsample2(x), log_alpha))


def conv1d(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None, stride: int = 1, dilation: int = 1) -> torch.Tensor:
    k = w.shape[-1]
    pad = dilation * (k - 1) // 2
    return F.conv1d(x[None], w, b, stride=stride, padding=pad, dilation=dilation)[0]


class AudioDecoder:
    def __init__(self, cfg: AudioConfig, device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        self.w = None

    def init_random(self, seed: int = 0, std: float = 0.05):
        c, g = self.cfg, torch.Generator().manual_seed(seed)

        def conv(o, i, k):
            return (torch.randn(o, i, k, generator=g) * std / math.sqrt(i * k)).to(self.device), torch.zeros(o, device=self.device)
        ch = c.width
        stages = []
        for r in c.rates:
            nxt = max(c.channels * 2, ch // 2)
            up = (torch.randn(ch, nxt, 2 * r, generator=g) * std / math.sqrt(ch)).to(self.device)     # transposed conv: [in, out, k]
            res = [{"a1": torch.zeros(nxt, device=self.device), "c1": conv(nxt, nxt, 3), "a2": torch.zeros(nxt, device=self.device),
                    "c2": conv(nxt, nxt, 3), "d": d} for d in c.dilations]
            stages.append({"up": up, "rate": r, "res": res})
            ch = nxt
        self.w = {"pre": conv(c.width, c.latent, 7), "stages": stages, "post_a": torch.zeros(ch, device=self.device),
                  "post": conv(c.channels, ch, 7)}
        return self

    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        """latents [frames, latent] -> PCM float [channels, frames * hop] in [-1, 1]."""
        W = self.w
        x = conv1d(latents.t().float().to(self.device), *W["pre"])
        for s in W["stages"]:
            r = s["rate"]
            x = F.conv_transpose1d(x[None], s["up"], stride=r, padding=r // 2 + r % 2, output_padding=r % 2)[0]
            for b in s["res"]:
                y = conv1d(act1d(x, b["a1"]), *b["c1"], dilation=b["d"])
                x = x + conv1d(act1d(y, b["a2"]), *b["c2"])
        return torch.tanh(conv1d(act1d(x, W["post_a"]), *W["post"]))


class AudioEncoder:
    """Strided convolutions mirroring the decoder's rates, residual units with snake activations: PCM -> latent frames."""

    def __init__(self, cfg: AudioConfig, device="cpu"):
        self.cfg, self.device = cfg, torch.device(device)
        self.w = None

    def init_random(self, seed: int = 0, std: float = 0.05):
        c, g = self.cfg, torch.Generator().manual_seed(seed)

        def conv(o, i, k):
            return (torch.randn(o, i, k, generator=g) * std / math.sqrt(i * k)).to(self.device), torch.zeros(o, device=self.device)
        ch = max(8, c.width // (2 ** len(c.rates)))
        stages, prev = [], ch
        for r in reversed(c.rates):
            nxt = min(c.width, prev * 2)
            stages.append({"a": torch.zeros(prev, device=self.device), "res": conv(prev, prev, 7), "down": conv(nxt, prev, 2 * r), "rate": r})
            prev = nxt
        self.w = {"in": conv(ch, c.channels, 7), "stages": stages, "out_a": torch.zeros(prev, device=self.device),
                  "out": conv(c.latent, prev, 3)}
        return self

    def encode(self, pcm: torch.Tensor) -> torch.Tensor:
        """pcm [channels, samples] (samples a multiple of the hop) -> latents [samples / hop, latent]."""
        c, W = self.cfg, self.w
        assert pcm.shape[1] % c.hop == 0
        x = conv1d(pcm.float().to(self.device), *W["in"])
        for s in W["stages"]:
            x = x + conv1d(snake(x, s["a"]), *s["res"])
            r = s["rate"]
            w, b = s["down"]
            x = F.conv1d(F.pad(x[None], (r // 2, r - r // 2)), w, b, stride=r)[0]            # kernel 2 r, stride r: T -> T / r
        return conv1d(snake(x, W["out_a"]), *W["out"]).t().contiguous()


def write_wav(path, pcm: torch.Tensor, sample_rate: int) -> None:
    """16-bit PCM WAV of [channels, samples] in [-1, 1]."""
    import struct
    ch, n = pcm.shape
    data = (pcm.clamp(-1, 1).t().contiguous() * 32767).round().to(torch.int16).numpy().tobytes()
    with open(path, "wb") as f:
        f.write(b"RIFF" + struct.pack("<I", 36 + len(data)) + b"WAVEfmt " + struct.pack("<IHHIIHH", 16, 1, ch, sample_rate,
                                                                                         sample_rate * ch * 2, ch * 2, 16))
        f.write(b"data" + struct.pack("<I", len(data)) + data)
