"""/api/stats payload, Prometheus text and the self-contained /monitor page.

Schema of /api/stats follows the reference contract consumed by its monitor page and TUI
(src/server/monitor.cpp:32-94): server, totals, averages, latency, speculation, slots, recent, history,
prefix_cache, gpus, host. Prometheus series mirror src/server/server.cpp:351-364.
"""
from __future__ import annotations

import time

from .system_stats import gpu_stats, host_stats


def stats_payload(srv, brief: bool = False) -> dict:
    g = srv.gen
    snap = g.metrics.snapshot()
    comm = g.engine.comm
    out = {
        "server": {"model": srv.model_name, "model_type": srv.model_type, "uptime_s": time.time() - srv.t0,
                   "slots": g.max_slots, "max_context": srv.max_context, "tp": comm.size, "queued": g.queued(),
                   "speculation": g.speculator != "none", "speculator": g.speculator,
                   "kv_format": srv.info.get("kv_format", "bf16")},
        "totals": snap["totals"], "averages": snap["averages"], "latency": snap["latency"],
        "speculation": snap["speculation"],
    }
    if g.cache is not None:
        c = g.cache.summary()
        out["prefix_cache"] = {"lookups": c["lookups"], "hits": c["hits"], "hit_tokens": c["hit_tokens"],
                               "inserts": c["inserts"], "evictions": c["evictions"], "entries": c["entries"],
                               "bytes": c["bytes"], "budget_bytes": c["budget_bytes"],
                               "disk": {"hits": c["disk_hits"], "entries": c["disk_entries"], "bytes": c["disk_bytes"]}}
    if brief:
        return out
    out["slots"] = g.slot_views()
    out["recent"] = snap["recent"]
    out["history"] = snap["history"]
    out["gpus"] = gpu_stats()
    arena = getattr(g.engine, "arena", None)
    if arena is not None and out["gpus"]:
        idx = arena.device.index or 0
        for row in out["gpus"]:
            if row.get("index") == idx:
                row["arena_bytes"] = arena.capacity
    out["host"] = host_stats()
    return out


def prometheus_text(srv) -> str:
    s = stats_payload(srv, brief=True)
    t, a, sp = s["totals"], s["averages"], s["speculation"]
    pc = s.get("prefix_cache", {})
    active = sum(1 for v in srv.gen.slots if v.phase != "idle")
    rows = [
        ("volta_uptime_seconds", "gauge", s["server"]["uptime_s"]),
        ("volta_active_slots", "gauge", active),
        ("volta_requests_total", "counter", t["requests"]),
        ("volta_avg_ttft_ms", "gauge", a["ttft_ms"]),
        ("volta_avg_prefill_tok_s", "gauge", a["prefill_tok_s"]),
        ("volta_avg_decode_tok_s", "gauge", a["decode_tok_s"]),
        ("volta_spec_accept_rate", "gauge", sp["accept_rate"]),
        ("volta_prefix_cache_lookups_total", "counter", pc.get("lookups", 0)),
        ("volta_prefix_cache_hits_total", "counter", pc.get("hits", 0)),
        ("volta_prefix_cache_hit_tokens_total", "counter", pc.get("hit_tokens", 0)),
        ("volta_prefix_cache_evictions_total", "counter", pc.get("evictions", 0)),
        ("volta_prefix_cache_entries", "gauge", pc.get("entries", 0)),
        ("volta_prefix_cache_bytes", "gauge", pc.get("bytes", 0)),
    ]
    lines = []
    for name, kind, val in rows:
        lines.append(f"# TYPE {name} {kind}")
        lines.append(f"{name} {float(val):.6g}")
    return "\n".join(lines) + "\n"


MONITOR_HTML = """<!doctype html><html><head><meta charset="utf-8"><title>volta monitor</title>
<style>body{font:13px/1.4 system-ui,sans-serif;background:#111;color:#ddd;margin:16px}h1{font-size:16px}
table{border-collapse:collapse;margin:8px 0}td,th{border:1px solid #333;padding:3px 8px;text-align:right}
th{background:#1c1c1c}.l{text-align:left}.k{color:#8ac}canvas{background:#181818;border:1px solid #333}</style></head>
<body><h1>volta engine <span id="model" class="k"></span></h1><div id="top"></div>
<canvas id="chart" width="900" height="140"></canvas>
<h1>slots</h1><table id="slots"></table><h1>recent requests</h1><table id="recent"></table>
<h1>GPUs</h1><table id="gpus"></table>
<script>
function row(cells,th){return '<tr>'+cells.map(c=>(th?'<th>':'<td>')+c+(th?'</th>':'</td>')).join('')+'</tr>'}
function f(x,d){return (x==null)?'-':Number(x).toFixed(d==null?1:d)}
async function tick(){try{const s=await (await fetch('/api/stats')).json();
document.getElementById('model').textContent=s.server.model+' ('+s.server.model_type+', tp'+s.server.tp+')';
document.getElementById('top').innerHTML='uptime '+f(s.server.uptime_s,0)+'s &middot; requests '+s.totals.requests+
' &middot; completed '+s.totals.completed+' &middot; queued '+s.server.queued+' &middot; out tokens '+s.totals.tokens_out+
' &middot; ttft '+f(s.averages.ttft_ms)+' ms &middot; decode '+f(s.averages.decode_tok_s)+' tok/s &middot; prefill '+
f(s.averages.prefill_tok_s,0)+' tok/s &middot; gap p50/p99 '+f(s.latency.gap_ms[0])+'/'+f(s.latency.gap_ms[2])+
' ms &middot; spec accept '+f(100*s.speculation.accept_rate)+'%'+(s.prefix_cache?' &middot; cache hits '+
s.prefix_cache.hits+'/'+s.prefix_cache.lookups:'');
document.getElementById('slots').innerHTML=row(['slot','phase','req','pos','prompt','cached','generated','tok/s'],1)+
s.slots.map(x=>row([x.slot,x.phase,x.req_id,x.pos,x.prompt_tokens,x.cached_tokens,x.generated,f(x.decode_tok_s)])).join('');
document.getElementById('recent').innerHTML=row(['req','prompt','cached','gen','queue ms','ttft ms','prefill ms','total ms','tok/s','reason'],1)+
s.recent.slice().reverse().map(x=>row([x.req_id,x.prompt_tokens,x.cached_tokens,x.generated,f(x.queue_ms),f(x.ttft_ms),
f(x.prefill_ms),f(x.total_ms),f(x.decode_tok_s),x.reason])).join('');
document.getElementById('gpus').innerHTML=row(['gpu','name','W','limit','temp','util','SM MHz','mem used GB','throttle'],1)+
s.gpus.map(g=>row([g.index,g.name,f(g.power_w,0),f(g.power_limit_w,0),g.temp_c,g.util_gpu,g.sm_mhz,f(g.mem_used/1e9),
g.throttle.join(' ')])).join('');
const c=document.getElementById('chart').getContext('2d');c.clearRect(0,0,900,140);const d=s.history.decode;
const m=Math.max(1,...d);c.strokeStyle='#6c6';c.beginPath();d.forEach((v,i)=>{const x=i*900/Math.max(1,d.length-1),y=135-v/m*130;
i?c.lineTo(x,y):c.moveTo(x,y)});c.stroke();c.fillStyle='#888';c.fillText('decode tok/s (max '+f(m)+')',6,12)}catch(e){}}
setInterval(tick,1000);tick();
</script></body></html>
"""
