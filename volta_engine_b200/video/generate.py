"""Command-line tool for one video job (or a few, with ``--repeat``):

    h3_generate --root <MiniMax-H3 directory> --prompt "..." [--size 1280x736] [--frames 121] [--steps 4] [--seed 0]
                [--image first.rgb [--image last.rgb]] [--video-shift S] [--audio-shift S] [--out DIR] [--repeat N]
                [--lora FILE[:scale]]...
    h3_generate --root <directory> --caption IMAGE [--prompt GUIDANCE]      a detailed video prompt for a picture

``--root`` is a directory with a ``model_index.json`` of class MiniMaxH3Pipeline (the synthetic form: see
``server.cli.build_video_service``). Keyframes are raw RGB8 files of the job's size. Prints one JSON line per job.
Reference: src/video/h3_generate_main.cpp, docs/video.md:50-76.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def main(argv=None) -> int:
    from ..server.cli import build_video_service
    from .pipeline import H3Job
    ap = argparse.ArgumentParser(prog="h3_generate")
    ap.add_argument("--root", required=True)
    ap.add_argument("--prompt", default="")
    ap.add_argument("--size", default="1280x736")
    ap.add_argument("--frames", type=int, default=121)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--image", action="append", default=[])
    ap.add_argument("--video-shift", type=float, default=0.0)
    ap.add_argument("--audio-shift", type=float, default=0.0)
    ap.add_argument("--out", default="h3_out")
    ap.add_argument("--repeat", type=int, default=1)
    ap.add_argument("--device", default=None)
    ap.add_argument("--caption", default="", help="picture file (PNG / JPEG): write a video prompt for it instead of a video")
    ap.add_argument("--lora", action="append", default=[], help="adapter file, optionally FILE:scale; repeatable")
    a = ap.parse_args(argv)
    w, h = (int(v) for v in a.size.lower().split("x"))
    svc = build_video_service(a.root, a.out, device=a.device, captioner=bool(a.caption))
    try:
        if a.caption:
            print(json.dumps({"caption": svc.p.captioner.caption(open(a.caption, "rb").read(), a.prompt, seed=a.seed)}))
            return 0
        imgs = []
        for i, path in enumerate(a.image[:2]):
            raw = open(path, "rb").read()
            if len(raw) != w * h * 3:
                print(f"h3_generate: {path} is not raw RGB8 of {w}x{h}", file=sys.stderr)
                return 2
            imgs.append((torch.frombuffer(bytearray(raw), dtype=torch.uint8).reshape(h, w, 3), 0 if i == 0 else a.frames - 1))
        loras = []
        for spec in a.lora:
            path, _, sc = spec.rpartition(":")
            if path and sc.replace(".", "", 1).replace("-", "", 1).isdigit():
                loras.append((path, float(sc)))
            else:
                loras.append((spec, 1.0))
        for r in range(a.repeat):
            job = H3Job(prompt=a.prompt, width=w, height=h, frames=a.frames, steps=a.steps, seed=a.seed + r,
                        video_shift=a.video_shift, audio_shift=a.audio_shift, images=imgs, loras=loras)
            out = svc.p.run(job, os.path.join(a.out, f"job{r}"), progress=lambda s, d, t: None)
            print(json.dumps(out))
    except ValueError as e:
        print(f"h3_generate: {e}", file=sys.stderr)
        return 2
    finally:
        svc.stop()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
