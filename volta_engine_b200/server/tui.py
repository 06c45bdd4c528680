"""``volta_top``: terminal dashboard over ``/api/stats`` (same JSON contract as the web monitor).

``render_frame`` is a pure function from the stats document to a text frame, so frames are unit-testable;
``run_tui`` polls a server and repaints with ANSI escapes. Reference: src/server/tui/* (``volta_top``, ``--tui``).
"""
from __future__ import annotations

import json
import sys
import time
import urllib.request

_BARS = " ▁▂▃▄▅▆▇█"


def spark(values, width: int) -> str:
    vals = list(values)[-width:]
    if not vals:
        return ""
    hi = max(max(vals), 1e-9)
    return "".join(_BARS[min(8, int(v / hi * 8 + 0.5))] for v in vals)


def _bar(frac: float, width: int) -> str:
    n = max(0, min(width, int(frac * width + 0.5)))
    return "█" * n + "░" * (width - n)


def _fmt_bytes(n) -> str:
    n = float(n or 0)
    for unit in ("B", "KiB", "MiB", "GiB", "TiB"):
        if n < 1024 or unit == "TiB":
            return f"{n:.1f} {unit}" if unit != "B" else f"{int(n)} B"
        n /= 1024


def render_frame(s: dict, width: int = 100) -> str:
    sv, t, a = s.get("server", {}), s.get("totals", {}), s.get("averages", {})
    lat, sp = s.get("latency", {}), s.get("speculation", {})
    L = []
    up = int(sv.get("uptime_s", 0))
    L.append(f"volta_top  {sv.get('model', '?')} [{sv.get('model_type', '?')}]  tp={sv.get('tp', 1)}  "
             f"kv={sv.get('kv_format', 'bf16')}  up {up // 3600:02d}:{up % 3600 // 60:02d}:{up % 60:02d}  "
             f"queued {sv.get('queued', 0)}")
    L.append("─" * width)
    L.append(f"requests {t.get('requests', 0)}  done {t.get('completed', 0)}  out {t.get('tokens_out', 0)} tok  "
             f"prefilled {t.get('tokens_prefilled', 0)} tok  cached {t.get('cached_tokens', 0)} tok")
    L.append(f"avg  ttft {a.get('ttft_ms', 0):.0f} ms   prefill {a.get('prefill_tok_s', 0):.0f} tok/s   "
             f"decode {a.get('decode_tok_s', 0):.1f} tok/s")
    gap = lat.get("gap_ms") or [0] * 5
    L.append("gap  p50 {:.1f}  p90 {:.1f}  p99 {:.1f}  p99.9 {:.1f}  max {:.1f} ms  ({} samples)".format(
        *(list(gap) + [0] * 5)[:5], lat.get("gap_samples", 0)))
    if sv.get("speculation"):
        L.append(f"spec [{sv.get('speculator')}] rounds {sp.get('rounds', 0)}  accept {100 * sp.get('accept_rate', 0):.1f}%  "
                 f"tok/round {sp.get('tokens_per_round', 0):.2f}")
    h = s.get("history", {})
    if h.get("decode"):
        L.append("decode  " + spark(h["decode"], width - 10))
        L.append("prefill " + spark(h.get("prefill", []), width - 10))
    pc = s.get("prefix_cache")
    if pc:
        frac = pc.get("bytes", 0) / max(1, pc.get("budget_bytes", 1))
        L.append(f"prefix cache {_bar(frac, 20)} {_fmt_bytes(pc.get('bytes'))} / {_fmt_bytes(pc.get('budget_bytes'))}  "
                 f"hits {pc.get('hits', 0)}/{pc.get('lookups', 0)}  entries {pc.get('entries', 0)}  evicted {pc.get('evictions', 0)}")
    L.append("─" * width)
    L.append(f"{'slot':>4} {'phase':<9} {'req':>6} {'pos':>8} {'prompt':>8} {'cached':>8} {'gen':>6} {'max':>6} {'age s':>7} {'tok/s':>7}")
    for v in s.get("slots", []):
        L.append(f"{v.get('slot', 0):>4} {v.get('phase', 'idle'):<9} {v.get('req_id', 0):>6} {v.get('pos', 0):>8} "
                 f"{v.get('prompt_tokens', 0):>8} {v.get('cached_tokens', 0):>8} {v.get('generated', 0):>6} "
                 f"{v.get('max_tokens', 0):>6} {v.get('age_s', 0):>7.1f} {v.get('decode_tok_s', 0):>7.1f}")
    for g in s.get("gpus", []):
        mem = g.get("mem_used", 0) / max(1, g.get("mem_total", 1))
        thr = ",".join(g.get("throttle", [])) or "-"
        L.append(f"gpu{g.get('index', 0)} {g.get('name', '')[:18]:<18} {g.get('power_w', 0):>5.0f}/{g.get('power_limit_w', 0):.0f} W "
                 f"{g.get('temp_c', 0):>3.0f}C  sm {g.get('sm_mhz', 0):>4} MHz  util {g.get('util_gpu', 0):>3}%  "
                 f"mem {_bar(mem, 12)} {_fmt_bytes(g.get('mem_used'))}  throttle {thr}")
    ho = s.get("host")
    if ho:
        L.append(f"host cpu {ho.get('cpu_pct', 0):.0f}%  load {ho.get('load1', 0):.2f}  mem {_fmt_bytes(ho.get('mem_used'))}"
                 f" / {_fmt_bytes(ho.get('mem_total'))}  rss {_fmt_bytes(ho.get('rss'))}")
    rec = s.get("recent", [])[:8]
    if rec:
        L.append("─" * width)
        L.append(f"{'req':>6} {'prompt':>8} {'cached':>8} {'gen':>6} {'queue':>7} {'ttft':>7} {'total':>8} {'tok/s':>7} reason")
        for r in rec:
            L.append(f"{r.get('req_id', 0):>6} {r.get('prompt_tokens', 0):>8} {r.get('cached_tokens', 0):>8} {r.get('generated', 0):>6} "
                     f"{r.get('queue_ms', 0):>7.0f} {r.get('ttft_ms', 0):>7.0f} {r.get('total_ms', 0):>8.0f} "
                     f"{r.get('decode_tok_s', 0):>7.1f} {r.get('reason', '')}")
    return "\n".join(ln[:width] for ln in L) + "\n"


def fetch(url: str, api_key: str = "", timeout: float = 3.0) -> dict:
    req = urllib.request.Request(url.rstrip("/") + "/api/stats")
    if api_key:
        req.add_header("Authorization", "Bearer " + api_key)
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def run_tui(url: str, stop=None, interval: float = 1.0, out=sys.stdout, frames: int = 0) -> int:
    n = 0
    while not (stop is not None and stop.is_set()):
        try:
            frame = render_frame(fetch(url))
        except Exception as e:                      # server not up yet / gone: keep the screen, show the error
            frame = f"volta_top: {url}: {e}\n"
        out.write("\x1b[H\x1b[2J" + frame)
        out.flush()
        n += 1
        if frames and n >= frames:
            break
        if stop is not None:
            stop.wait(interval)
        else:
            time.sleep(interval)
    return n


def main(argv=None) -> int:
    import argparse
    p = argparse.ArgumentParser(prog="volta_top")
    p.add_argument("url", nargs="?", default="http://127.0.0.1:8080")
    p.add_argument("--interval", type=float, default=1.0)
    p.add_argument("--once", action="store_true")
    a = p.parse_args(argv)
    try:
        run_tui(a.url, interval=a.interval, frames=1 if a.once else 0)
    except KeyboardInterrupt:
        pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
