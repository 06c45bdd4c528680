"""One video job from prompt to files: the stages of the MiniMax-H3 pipeline on this engine's components.

  plan      picture size and frame count -> latent grid (16x spatial, 4x temporal, transformer patch 1 x 2 x 2), audio rows,
            the two sigma schedules (flow shift per modality), the noise seed
  refs      first / last keyframes -> video VAE encoder -> latent frames that the sampler holds fixed (they are written
            back into the video latents before every step and after the last one)
  text      prompt -> token ids -> text tower -> condition rows [n, 5120]
  denoise   flow-matching Euler steps of the diffusion transformer over [text | audio | video] rows (``video.dit``)
  decode    video latents -> tiled ViT decoder -> RGB8 frames; audio latents -> BigVGAN-style decoder -> stereo PCM
  mux       an MP4 through the ``ffmpeg`` binary when there is one; otherwise the frames (binary PPM), a WAV file and a
            manifest in the job's directory

Reference: src/video/h3_pipeline.cu, h3_engine.cpp, h3_stage_*.cpp (H3Run stages: plan_shape, encode_references,
encode_prompt, plan_denoise, denoise, decode, mux); docs/video.md:15-28,110-118.
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import time
from dataclasses import dataclass, field

import torch

from . import dit as D
from .audio import AudioConfig, AudioDecoder, write_wav
from .vae import VaeConfig, VideoDecoder, VideoEncoder

FPS = 24


@dataclass
class H3Job:
    prompt: str = ""
    width: int = 1280
    height: int = 736
    frames: int = 121
    steps: int = 4
    seed: int = 0
    video_shift: float = 0.0      # 0 = the default (12)
    audio_shift: float = 0.0      # 0 = the default (3)
    images: list = field(default_factory=list)      # [(uint8 [H, W, 3] tensor, frame_index)]: keyframes (first / last)
    loras: list = field(default_factory=list)       # [(file, scale)]

    def validate(self, vae: VaeConfig, max_rows: int = 0) -> None:
        px = vae.s_up * 2                            # a transformer patch covers 2 x 2 latent pixels
        if self.width % px or self.height % px or self.width <= 0 or self.height <= 0:
            raise ValueError(f"width and height must be positive multiples of {px}")
        if self.frames < 1 or (self.frames - 1) % vae.t_up:
            raise ValueError(f"frames must be 1 + {vae.t_up} k")
        if not 1 <= self.steps <= 50:
            raise ValueError("steps must be 1..50")
        for s in (self.video_shift, self.audio_shift):
            if s and not 0.5 <= s <= 40:
                raise ValueError("a flow shift is 0 (default) or 0.5..40")
        if len(self.loras) > 6:
            raise ValueError("at most six adapters per job")
        for _, idx in self.images:
            if idx not in (0, -1, self.frames - 1):
                raise ValueError("keyframes are the first or the last frame")
        if max_rows and self.rows(vae) > max_rows:
            raise ValueError(f"the job packs {self.rows(vae)} rows, the limit is {max_rows}")

    def grid(self, vae: VaeConfig) -> tuple:
        return (1 + (self.frames - 1) // vae.t_up, self.height // vae.s_up // 2, self.width // vae.s_up // 2)

    def audio_rows(self, audio: AudioConfig) -> int:
        return max(1, round(self.frames / FPS * audio.sample_rate / audio.hop))

    def rows(self, vae: VaeConfig) -> int:
        g = self.grid(vae)
        return g[0] * g[1] * g[2]


def patchify(lat: torch.Tensor) -> torch.Tensor:
    """[F, H, W, C] latent frames -> transformer rows [F * H/2 * W/2, C * 4] (channel-major 2 x 2 patches)."""
    F_, H, W, C = lat.shape
    return lat.reshape(F_, H // 2, 2, W // 2, 2, C).permute(0, 1, 3, 5, 2, 4).reshape(F_ * (H // 2) * (W // 2), C * 4)


def unpatchify(rows: torch.Tensor, grid: tuple) -> torch.Tensor:
    F_, h, w = grid
    C = rows.shape[1] // 4
    return rows.reshape(F_, h, w, C, 2, 2).permute(0, 1, 4, 2, 5, 3).reshape(F_, 2 * h, 2 * w, C)


class H3Pipeline:
    """Owns the components and runs jobs one at a time. ``tokenize`` maps a prompt to token ids of the text tower."""

    def __init__(self, dit: D.H3DiT, text, vae_cfg: VaeConfig, audio_cfg: AudioConfig, tokenize, device="cpu", seed: int = 0):
        self.dit, self.text, self.tokenize, self.device = dit, text, tokenize, torch.device(device)
        self.vae_cfg, self.audio_cfg = vae_cfg, audio_cfg
        assert dit.cfg.latents == vae_cfg.latent * 4 and dit.cfg.audio_latents == audio_cfg.latent
        self.decoder = VideoDecoder(vae_cfg, device).init_random(seed + 1)
        self.encoder = VideoEncoder(vae_cfg, device).init_random(seed + 2)
        self.audio = AudioDecoder(audio_cfg, device).init_random(seed + 3)
        self.ffmpeg = shutil.which("ffmpeg")
        self.catalog = None                          # video.lora.AdapterCatalog of the configured directories, when there are any
        self.captioner = None                        # video.text.H3Captioner when the text tower was built with all its layers
        self._staged: list = []                      # paths of the adapters the denoiser currently holds

    @classmethod
    def tiny(cls, device="cpu", seed: int = 0, captioner: bool = False):
        from .text import H3TextTower
        vae, aud = VaeConfig.tiny(), AudioConfig.tiny()
        cfg = D.H3Config.tiny(latents=vae.latent * 4, audio_latents=aud.latent, text_dim=64)
        dit = D.H3DiT(cfg, device).init_random(seed)
        text = H3TextTower.tiny(device, hidden=64, captioner=captioner).init_random(seed + 7)
        tok = lambda s: [1 + (b % 500) for b in s.encode()][:256] or [1]
        p = cls(dit, text, vae, aud, tok, device, seed)
        if captioner:
            p.attach_captioner(lambda ids: bytes(32 + (i % 90) for i in ids).decode(), eos_ids=(0,), max_new=24)
        return p

    def attach_captioner(self, detokenize, frontend=None, image_token_id=None, eos_ids=(), max_new: int = 400):
        """Captions through the text tower (it must have been built with all its layers); ``frontend`` turns picture bytes
        into embedding rows (without one a caption is written from the prompt box alone)."""
        from .text import H3Captioner
        tok = self.tokenize
        if frontend is not None and image_token_id is not None:
            def tok(s, base=self.tokenize, pad=image_token_id):        # the placeholder becomes the image token id
                out = []
                for i, part in enumerate(s.split("<|image_pad|>")):
                    out += ([pad] if i else []) + (base(part) if part else [])
                return out
        self.captioner = H3Captioner(self.text, tok, detokenize, frontend, image_token_id, eos_ids, max_new)
        return self.captioner

    # ---- stages --------------------------------------------------------------------------------------------------
    def stage_adapters(self, job: H3Job) -> None:
        """The job's LoRA adapters, resolved through the catalogue (a bare file name) or as paths. The set staged by the
        previous job is kept when it names the same files (only the scales are updated); otherwise it is replaced."""
        want = []
        for file, scale in job.loras:
            info = self.catalog.find(file) if self.catalog is not None else None
            path = info.path if info is not None else file
            if not os.path.isfile(path):
                raise ValueError(f"adapter {file!r} is not in the configured directories")
            want.append((path, float(scale)))
        if [p for p, _ in want] == self._staged:
            for i, (_, sc) in enumerate(want):
                self.dit.set_lora_scale(i, sc)
            return
        self.dit.clear_loras()
        self._staged = []
        for path, sc in want:
            self.dit.add_lora(path, sc)
            self._staged.append(path)

    def encode_references(self, job: H3Job, grid: tuple) -> dict:
        """{latent frame index: rows of that frame} for the keyframes of the job."""
        per = grid[1] * grid[2]
        cond = {}
        for img, idx in job.images:
            assert tuple(img.shape) == (job.height, job.width, 3), "keyframes are given at the job's size"
            lat = self.encoder.encode(img[None])                   # one frame -> one latent frame [1, H/16, W/16, C]
            f = 0 if idx == 0 else grid[0] - 1
            cond[f] = patchify(lat.float().cpu())[:per]
        return cond

    def encode_prompt(self, job: H3Job) -> torch.Tensor:
        return self.text.encode(self.tokenize(job.prompt)).float()

    def denoise(self, job: H3Job, prompt: torch.Tensor, grid: tuple, cond: dict, progress=None):
        cfg, dev = self.dit.cfg, self.device
        g = torch.Generator().manual_seed(job.seed)
        n_img, per = grid[0] * grid[1] * grid[2], grid[1] * grid[2]
        a_rows = job.audio_rows(self.audio_cfg)
        xv = torch.randn(n_img, cfg.latents, generator=g).to(dev)
        xa = torch.randn(a_rows, cfg.audio_latents, generator=g).to(dev)
        sv = D.sigma_schedule(job.steps, job.video_shift or 12.0)
        sa = D.sigma_schedule(job.steps, job.audio_shift or 3.0)

        def hold(x):
            for f, rows in cond.items():                            # the condition rows are reset to their clean latents
                x[f * per:(f + 1) * per] = rows.to(x)
            return x
        for i in range(job.steps):
            xv = hold(xv)
            req = D.make_request(xv, xa, prompt.to(dev), grid, float(sv[i]), float(sa[i]))
            if cond:                                                # clean rows carry timestep 1 (sigma 0)
                off = prompt.shape[0] + a_rows
                for f in cond:
                    req.t[off + f * per: off + (f + 1) * per] = 1.0
            vv, va = self.dit.forward(req)
            xv = xv + float(sv[i + 1] - sv[i]) * vv.to(xv.dtype)
            xa = xa + float(sa[i + 1] - sa[i]) * va.to(xa.dtype)
            if progress is not None:
                progress("denoise", i + 1, job.steps)
        return hold(xv), xa

    def decode(self, xv: torch.Tensor, xa: torch.Tensor, grid: tuple, frames: int, progress=None):
        lat = unpatchify(xv.float().cpu(), grid)
        rgb = self.decoder.decode(lat, on_tile=(lambda d, t: progress("decode", d, t)) if progress else None)
        rgb = rgb[self.vae_cfg.t_up - 1:][:frames]                  # the first latent frame stands for one picture
        pcm = self.audio.decode(xa.float().cpu()).cpu()
        return rgb, pcm

    def mux(self, rgb: torch.Tensor, pcm: torch.Tensor, out_dir: str, job: H3Job) -> dict:
        os.makedirs(out_dir, exist_ok=True)
        wav = os.path.join(out_dir, "audio.wav")
        write_wav(wav, pcm, self.audio_cfg.sample_rate)
        n, H, W, _ = rgb.shape
        raw = os.path.join(out_dir, "frames.rgb")
        with open(raw, "wb") as f:
            f.write(rgb.contiguous().numpy().tobytes())
        out = {"frames": n, "width": W, "height": H, "fps": FPS, "audio": wav, "raw": raw, "video": None}
        if self.ffmpeg:
            mp4 = os.path.join(out_dir, "video.mp4")
            cmd = [self.ffmpeg, "-y", "-loglevel", "error", "-f", "rawvideo", "-pix_fmt", "rgb24", "-s", f"{W}x{H}", "-r", str(FPS),
                   "-i", raw, "-i", wav, "-c:v", "libx264", "-pix_fmt", "yuv420p", "-c:a", "aac", "-shortest", mp4]
            if subprocess.run(cmd).returncode == 0:
                out["video"] = mp4
        else:                                                       # headless: the first frame as a PPM thumbnail
            with open(os.path.join(out_dir, "thumb.ppm"), "wb") as f:
                f.write(f"P6 {W} {H} 255\n".encode() + rgb[0].contiguous().numpy().tobytes())
            out["thumb"] = os.path.join(out_dir, "thumb.ppm")
        with open(os.path.join(out_dir, "job.json"), "w") as f:
            json.dump({"prompt": job.prompt, "width": job.width, "height": job.height, "frames": job.frames, "steps": job.steps,
                       "seed": job.seed, "result": out}, f)
        return out

    def run(self, job: H3Job, out_dir: str, progress=None, cancelled=None) -> dict:
        """All stages; ``progress(stage, done, total)`` is called as they advance, ``cancelled()`` is polled between stages
        and steps (a job stops at the next boundary)."""
        t0 = time.time()
        job.validate(self.vae_cfg)
        grid = job.grid(self.vae_cfg)

        def check():
            if cancelled is not None and cancelled():
                raise InterruptedError("cancelled")

        def prog(stage, d, t):
            check()
            if progress is not None:
                progress(stage, d, t)
        prog("plan", 1, 1)
        self.stage_adapters(job)
        cond = self.encode_references(job, grid)
        prog("references", 1, 1)
        prompt = self.encode_prompt(job)
        prog("text", 1, 1)
        xv, xa = self.denoise(job, prompt, grid, cond, prog)
        rgb, pcm = self.decode(xv, xa, grid, job.frames, prog)
        out = self.mux(rgb, pcm, out_dir, job)
        out["seconds"] = round(time.time() - t0, 3)
        return out
