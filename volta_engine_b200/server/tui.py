"""``volta_top``: terminal dashboard over ``/api/stats`` (same JSON contract as the web monitor).

``render_frame`` is a pure function from the stats document to a text frame, so frames are unit-testable;
``run_tui`` polls a server and repaints with ANSI escapes. Views (``--view`` or, on a terminal, the keys 1-4; q quits):
overview (totals, latency, slots, GPUs, recent requests), experts (``/api/experts``: routing heat per layer, hottest
experts), speculation (rounds, acceptance per draft position), memory (GPU memory, arena, prefix cache, host).
Reference: src/server/tui/* (``volta_top``, ``--tui``).
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


VIEWS = ("overview", "experts", "speculation", "memory")


def render_experts(e: dict, width: int = 100, top: int = 8) -> str:
    """``/api/experts``: per layer a bar of the routed share of its hottest experts and their ids."""
    layers, experts, tot = int(e.get("layers", 0)), int(e.get("experts", 0)), e.get("total", [])
    L = [f"experts  {layers} layers x {experts} experts  ({e.get('ranks', 1)} ranks)", "─" * width]
    if not layers or not experts or len(tot) < layers * experts:
        return "\n".join(L + ["no routing histogram (dense model, or expert_stats = false)"]) + "\n"
    L.append(f"{'layer':>5} {'routes':>10} {'top share':<24} hottest experts")
    for li in range(layers):
        row = tot[li * experts:(li + 1) * experts]
        total = sum(row)
        if total <= 0:
            continue
        order = sorted(range(experts), key=lambda i: (-row[i], i))[:top]
        share = sum(row[i] for i in order) / total
        L.append(f"{li:>5} {int(total):>10} {_bar(share, 16)} {100 * share:>5.1f}%  " + " ".join(f"{i}:{100 * row[i] / total:.0f}%" for i in order))
    return "\n".join(ln[:width] for ln in L) + "\n"


def render_speculation(s: dict, width: int = 100) -> str:
    sv, sp = s.get("server", {}), s.get("speculation", {})
    L = [f"speculation  [{sv.get('speculator', 'none')}]", "─" * width]
    if not sv.get("speculation"):
        return "\n".join(L + ["off"]) + "\n"
    L.append(f"rounds {sp.get('rounds', 0)}  proposed {sp.get('proposed', 0)}  accepted {sp.get('accepted', 0)}  "
             f"accept {100 * sp.get('accept_rate', 0):.1f}%  tok/round {sp.get('tokens_per_round', 0):.2f}  "
             f"tree rounds {sp.get('tree_rounds', 0)} ({sp.get('tree_nodes', 0)} nodes)")
    steps = sp.get("steps", [])
    if steps:
        L.append(f"{'draft':>5} {'attempts':>9} {'hits':>8}  rate")
        for i, st in enumerate(steps):
            att, hit = st.get("attempts", 0), st.get("hits", 0)
            L.append(f"{i + 1:>5} {att:>9} {hit:>8}  {_bar(hit / max(1, att), 24)} {100 * hit / max(1, att):.1f}%")
    return "\n".join(ln[:width] for ln in L) + "\n"


def render_memory(s: dict, width: int = 100) -> str:
    L = ["memory", "─" * width]
    for g in s.get("gpus", []):
        mem = g.get("mem_used", 0) / max(1, g.get("mem_total", 1))
        L.append(f"gpu{g.get('index', 0)} {_bar(mem, 30)} {_fmt_bytes(g.get('mem_used'))} / {_fmt_bytes(g.get('mem_total'))}"
                 + (f"  arena {_fmt_bytes(g.get('arena_bytes'))}" if g.get("arena_bytes") else ""))
    pc = s.get("prefix_cache")
    if pc:
        L.append(f"prefix cache  ram {_fmt_bytes(pc.get('bytes'))} / {_fmt_bytes(pc.get('budget_bytes'))}  disk {_fmt_bytes(pc.get('disk_bytes', 0))}  "
                 f"entries {pc.get('entries', 0)}  hits {pc.get('hits', 0)}/{pc.get('lookups', 0)}")
    ho = s.get("host")
    if ho:
        L.append(f"host  mem {_fmt_bytes(ho.get('mem_used'))} / {_fmt_bytes(ho.get('mem_total'))}  rss {_fmt_bytes(ho.get('rss'))}  "
                 f"cpu {ho.get('cpu_pct', 0):.0f}%  load {ho.get('load1', 0):.2f}")
    kv = s.get("server", {})
    L.append(f"kv pool {kv.get('kv_pool_tokens', 0)} tokens  format {kv.get('kv_format', 'bf16')}  slots {len(s.get('slots', []))}")
    return "\n".join(ln[:width] for ln in L) + "\n"


def render_view(view: str, stats: dict, experts: dict | None = None, width: int = 100) -> str:
    if view == "experts":
        return render_experts(experts or {}, width)
    if view == "speculation":
        return render_speculation(stats, width)
    if view == "memory":
        return render_memory(stats, width)
    return render_frame(stats, width)


def fetch(url: str, api_key: str = "", timeout: float = 3.0, path: str = "/api/stats") -> dict:
    req = urllib.request.Request(url.rstrip("/") + path)
    if api_key:
        req.add_header("Authorization", "Bearer " + api_key)
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def _poll_key(timeout: float):
    """One key from a terminal within ``timeout`` seconds (None when stdin is not a terminal or nothing was pressed)."""
    try:
        import select
        import termios
        import tty
        if not sys.stdin.isatty():
            time.sleep(timeout)
            return None
        fd = sys.stdin.fileno()
        old = termios.tcgetattr(fd)
        try:
            tty.setcbreak(fd)
            if select.select([sys.stdin], [], [], timeout)[0]:
                return sys.stdin.read(1)
        finally:
            termios.tcsetattr(fd, termios.TCSADRAIN, old)
    except Exception:
        time.sleep(timeout)
    return None


def run_tui(url: str, stop=None, interval: float = 1.0, out=sys.stdout, frames: int = 0, view: str = "overview", keys: bool = False) -> int:
    n = 0
    while not (stop is not None and stop.is_set()):
        try:
            stats = fetch(url)
            frame = render_view(view, stats, fetch(url, path="/api/experts") if view == "experts" else None)
        except Exception as e:                      # server not up yet / gone: keep the screen, show the error
            frame = f"volta_top: {url}: {e}\n"
        out.write("\x1b[H\x1b[2J" + frame + ("[1] overview [2] experts [3] speculation [4] memory [q] quit\n" if keys else ""))
        out.flush()
        n += 1
        if frames and n >= frames:
            break
        if keys:
            k = _poll_key(interval)
            if k == "q":
                break
            if k in ("1", "2", "3", "4"):
                view = VIEWS[int(k) - 1]
        elif stop is not None:
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
    p.add_argument("--view", choices=VIEWS, default="overview")
    a = p.parse_args(argv)
    try:
        run_tui(a.url, interval=a.interval, frames=1 if a.once else 0, view=a.view, keys=not a.once and sys.stdin.isatty())
    except KeyboardInterrupt:
        pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
