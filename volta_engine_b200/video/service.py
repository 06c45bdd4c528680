"""Video service: a job queue with one worker thread that owns the pipeline, and the HTTP routes over it.

Routes (reference: docs/video.md:93-104, src/server/video/*):
  GET  /api/info                         model shape, limits, queue length
  GET  /api/jobs        POST /api/jobs   list / submit ({prompt, width, height, frames, steps, seed, video_shift, audio_shift,
                                         loras: [{file, scale}], images: [{data (base64 raw RGB8 of the job's size), frame_index}]})
  GET  /api/jobs/<id>   DELETE /api/jobs/<id>
  POST /api/jobs/<id>/cancel
  GET  /api/jobs/<id>/video              the MP4 when ffmpeg muxed one, else the raw RGB8 frames (Range supported)
  GET  /api/jobs/<id>/thumb
  POST /api/caption     GET /api/caption/<id>   with a captioner: {image: base64 PNG / JPEG, prompt} -> a detailed video
                                         prompt; runs between jobs, ahead of the queued ones
  GET  /health
``handle(method, path, body, headers)`` returns (status, content type, bytes, extra headers) so any HTTP front end can
mount it; ``serve`` runs it on the engine's epoll server.
"""
from __future__ import annotations

import base64
import json
import os
import queue
import threading
import time
import uuid

import torch

from .pipeline import H3Job, H3Pipeline


class VideoService:
    def __init__(self, pipeline: H3Pipeline, out_dir: str, max_rows: int = 0, max_queue: int = 64):
        self.p, self.out_dir, self.max_rows, self.max_queue = pipeline, out_dir, max_rows, max_queue
        os.makedirs(out_dir, exist_ok=True)
        self.jobs: dict[str, dict] = {}
        self.q: queue.Queue = queue.Queue()
        self.captions: dict[str, dict] = {}           # caption requests: they run between jobs, ahead of the queued ones
        self.cq: queue.Queue = queue.Queue()
        self.lock = threading.Lock()
        self.stop_flag = False
        self.worker = threading.Thread(target=self._work, name="video-worker", daemon=True)
        self.worker.start()

    # ---- queue ---------------------------------------------------------------------------------------------------
    def submit(self, body: dict) -> dict:
        imgs = []
        w, h = int(body.get("width", 1280)), int(body.get("height", 736))
        for im in body.get("images", []):
            raw = base64.b64decode(im["data"])
            if len(raw) != w * h * 3:
                raise ValueError("an image is raw RGB8 of the job's width x height")
            imgs.append((torch.frombuffer(bytearray(raw), dtype=torch.uint8).reshape(h, w, 3), int(im.get("frame_index", 0))))
        job = H3Job(prompt=str(body.get("prompt", "")), width=w, height=h, frames=int(body.get("frames", 121)),
                    steps=int(body.get("steps", 4)), seed=int(body.get("seed", 0)), video_shift=float(body.get("video_shift", 0) or 0),
                    audio_shift=float(body.get("audio_shift", 0) or 0), images=imgs,
                    loras=[(l["file"], float(l.get("scale", 1.0))) for l in body.get("loras", [])])
        job.validate(self.p.vae_cfg, self.max_rows)
        with self.lock:
            if sum(1 for j in self.jobs.values() if j["status"] in ("queued", "running")) >= self.max_queue:
                raise OverflowError("the queue is full")
            jid = uuid.uuid4().hex[:12]
            self.jobs[jid] = {"id": jid, "status": "queued", "stage": "", "done": 0, "total": 0, "submitted": time.time(),
                              "params": {k: v for k, v in body.items() if k != "images"}, "result": None, "error": None,
                              "_job": job, "_cancel": False}
        self.q.put(jid)
        return self.public(jid)

    def public(self, jid: str) -> dict:
        j = self.jobs[jid]
        return {k: v for k, v in j.items() if not k.startswith("_")}

    def cancel(self, jid: str) -> dict:
        with self.lock:
            j = self.jobs[jid]
            if j["status"] in ("queued", "running"):
                j["_cancel"] = True
                if j["status"] == "queued":
                    j["status"] = "cancelled"
        return self.public(jid)

    def delete(self, jid: str) -> None:
        self.cancel(jid)
        with self.lock:
            j = self.jobs.get(jid)
            if j is not None and j["status"] != "running":
                del self.jobs[jid]

    def submit_caption(self, body: dict) -> dict:
        """{image: base64 of an encoded picture (PNG / JPEG), prompt: optional text of the prompt box} -> the request's
        record; the text arrives in it once the worker has run it."""
        cap = getattr(self.p, "captioner", None)
        if cap is None:
            raise ValueError("the captioner is not configured (video.captioner)")
        img = base64.b64decode(body["image"]) if body.get("image") else None
        if img is None and not str(body.get("prompt", "")).strip():
            raise ValueError("a caption needs a picture or a prompt")
        cid = uuid.uuid4().hex[:12]
        self.captions[cid] = {"id": cid, "status": "queued", "text": None, "error": None, "submitted": time.time(),
                              "_image": img, "_idea": str(body.get("prompt", "")), "_greedy": bool(body.get("greedy", False)),
                              "_seed": int(body.get("seed", 0))}
        self.cq.put(cid)
        return {k: v for k, v in self.captions[cid].items() if not k.startswith("_")}

    def _caption(self, cid: str) -> None:
        c = self.captions[cid]
        c["status"] = "running"
        try:
            c["text"] = self.p.captioner.caption(c["_image"], c["_idea"], greedy=c["_greedy"], seed=c["_seed"])
            c["status"] = "done"
        except Exception as e:                      # a failed caption must not take the worker down
            c["status"], c["error"] = "failed", f"{type(e).__name__}: {e}"
        c["_image"] = None
        c["finished"] = time.time()

    def _work(self):
        while not self.stop_flag:
            try:
                self._caption(self.cq.get_nowait())
                continue
            except queue.Empty:
                pass
            try:
                jid = self.q.get(timeout=0.05)
            except queue.Empty:
                continue
            j = self.jobs.get(jid)
            if j is None or j["status"] != "queued":
                continue
            j["status"], j["started"] = "running", time.time()

            def progress(stage, d, t, j=j):
                j["stage"], j["done"], j["total"] = stage, d, t
            try:
                j["result"] = self.p.run(j["_job"], os.path.join(self.out_dir, jid), progress, lambda j=j: j["_cancel"])
                j["status"] = "done"
            except InterruptedError:
                j["status"] = "cancelled"
            except Exception as e:                  # a failed job must not take the worker down
                j["status"], j["error"] = "failed", f"{type(e).__name__}: {e}"
            j["finished"] = time.time()

    def wait(self, jid: str, timeout: float = 60.0) -> dict:
        t0 = time.time()
        while time.time() - t0 < timeout and self.jobs[jid]["status"] in ("queued", "running"):
            time.sleep(0.02)
        return self.public(jid)

    def stop(self):
        self.stop_flag = True
        self.worker.join(timeout=5)

    # ---- HTTP ----------------------------------------------------------------------------------------------------
    def info(self) -> dict:
        c = self.p.dit.cfg
        return {"model": "minimax_h3", "hidden": c.hidden, "layers": c.layers, "heads": c.heads, "max_rows": self.max_rows,
                "queued": sum(1 for j in self.jobs.values() if j["status"] == "queued"),
                "running": sum(1 for j in self.jobs.values() if j["status"] == "running"), "ffmpeg": bool(self.p.ffmpeg),
                "captioner": getattr(self.p, "captioner", None) is not None, "adapters": [{"file": a.file, "label": a.label, "format": a.format, "task": a.task, "turbo": a.turbo, "mb": a.mb}
                             for a in (self.p.catalog.all() if self.p.catalog is not None else [])]}

    def handle(self, method: str, path: str, body: bytes = b"", headers: dict | None = None):
        def js(status, obj):
            return status, "application/json", json.dumps(obj).encode(), {}
        path = path.split("?")[0].rstrip("/") or "/"
        parts = [p for p in path.split("/") if p]
        try:
            if path == "/health":
                return js(200, {"status": "ok"})
            if path == "/api/info" and method == "GET":
                return js(200, self.info())
            if path == "/api/jobs" and method == "GET":
                return js(200, {"jobs": [self.public(i) for i in sorted(self.jobs, key=lambda i: self.jobs[i]["submitted"])]})
            if path == "/api/jobs" and method == "POST":
                return js(200, self.submit(json.loads(body or b"{}")))
            if path == "/api/caption" and method == "POST":
                return js(200, self.submit_caption(json.loads(body or b"{}")))
            if len(parts) == 3 and parts[:2] == ["api", "caption"] and method == "GET":
                if parts[2] not in self.captions:
                    return js(404, {"error": "no such caption"})
                return js(200, {k: v for k, v in self.captions[parts[2]].items() if not k.startswith("_")})
            if len(parts) >= 3 and parts[:2] == ["api", "jobs"]:
                jid = parts[2]
                if jid not in self.jobs:
                    return js(404, {"error": "no such job"})
                if len(parts) == 3 and method == "GET":
                    return js(200, self.public(jid))
                if len(parts) == 3 and method == "DELETE":
                    self.delete(jid)
                    return js(200, {"deleted": jid})
                if len(parts) == 4 and parts[3] == "cancel" and method == "POST":
                    return js(200, self.cancel(jid))
                if len(parts) == 4 and parts[3] in ("video", "thumb") and method == "GET":
                    res = self.jobs[jid]["result"]
                    if not res:
                        return js(409, {"error": "the job has no result yet"})
                    if parts[3] == "thumb":
                        f, ctype = res.get("thumb") or res["raw"], "image/x-portable-pixmap"
                    else:
                        f, ctype = (res["video"], "video/mp4") if res.get("video") else (res["raw"], "application/octet-stream")
                    return self._file(f, ctype, (headers or {}).get("range"))
            return js(404, {"error": "no such route"})
        except (ValueError, KeyError, json.JSONDecodeError) as e:
            return js(400, {"error": str(e)})
        except OverflowError as e:
            return js(429, {"error": str(e)})

    @staticmethod
    def _file(path: str, ctype: str, rng: str | None):
        size = os.path.getsize(path)
        lo, hi, status = 0, size - 1, 200
        if rng and rng.startswith("bytes="):
            a, _, b = rng[6:].partition("-")
            lo = int(a) if a else max(0, size - int(b))
            hi = min(size - 1, int(b)) if (a and b) else size - 1
            if lo > hi or lo >= size:
                return 416, "application/json", b'{"error": "range"}', {"Content-Range": f"bytes */{size}"}
            status = 206
        with open(path, "rb") as f:
            f.seek(lo)
            data = f.read(hi - lo + 1)
        extra = {"Accept-Ranges": "bytes"}
        if status == 206:
            extra["Content-Range"] = f"bytes {lo}-{hi}/{size}"
        return status, ctype, data, extra


def serve(service: VideoService, host: str = "127.0.0.1", port: int = 0, stop=None):
    """Run the routes on the engine's HTTP server until ``stop()`` says so; returns the server (its port is chosen when 0)."""
    from ..server.http import HttpServer
    srv = HttpServer(host, port)

    def loop():
        while not (stop and stop()):
            req = srv.next_request(200)
            if req is None:
                continue
            status, ctype, data, extra = service.handle(req.method, req.path, req.body, getattr(req, "headers", {}))
            srv.respond(req.conn, status, data, ctype, "".join(f"{k}: {v}\r\n" for k, v in extra.items()))
    t = threading.Thread(target=loop, name="video-http", daemon=True)
    t.start()
    return srv
