"""Read-only GPU and host telemetry for /api/stats (reference: src/server/system_stats.cpp:14-47 loads NVML
with dlopen). Only queries are issued; no clock, power or mode setting is ever changed."""
from __future__ import annotations

import os
import time

_nvml = None
_nvml_failed = False


def _init():
    global _nvml, _nvml_failed
    if _nvml is not None or _nvml_failed:
        return _nvml
    try:
        import pynvml
        pynvml.nvmlInit()
        _nvml = pynvml
    except Exception:
        _nvml_failed = True
    return _nvml


def gpu_stats(indices=None) -> list[dict]:
    nv = _init()
    if nv is None:
        return []
    out = []
    try:
        n = nv.nvmlDeviceGetCount()
    except Exception:
        return []
    for i in (indices if indices is not None else range(n)):
        try:
            h = nv.nvmlDeviceGetHandleByIndex(i)
            mem = nv.nvmlDeviceGetMemoryInfo(h)
            util = nv.nvmlDeviceGetUtilizationRates(h)
            name = nv.nvmlDeviceGetName(h)
            reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                else nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
            throttle = [nm for bit, nm in ((0x8, "hw_slowdown"), (0x40, "hw_thermal"), (0x20, "sw_thermal"), (0x4, "sw_power_cap"))
                        if reasons & bit]
            out.append({"index": i, "name": name if isinstance(name, str) else name.decode(),
                        "power_w": nv.nvmlDeviceGetPowerUsage(h) / 1000.0,
                        "power_limit_w": nv.nvmlDeviceGetEnforcedPowerLimit(h) / 1000.0,
                        "energy_kj": nv.nvmlDeviceGetTotalEnergyConsumption(h) / 1e6,
                        "temp_c": nv.nvmlDeviceGetTemperature(h, nv.NVML_TEMPERATURE_GPU),
                        "util_gpu": util.gpu, "util_mem": util.memory,
                        "sm_mhz": nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
                        "mem_mhz": nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_MEM),
                        "mem_used": mem.used, "mem_total": mem.total, "arena_bytes": 0, "throttle": throttle})
        except Exception:
            continue
    return out


_last_cpu = None


def host_stats() -> dict:
    global _last_cpu
    out = {"cpu_pct": 0.0, "mem_used": 0, "mem_total": 0, "rss": 0, "load1": 0.0}
    try:
        with open("/proc/stat") as f:
            parts = [int(x) for x in f.readline().split()[1:8]]
        idle, total = parts[3] + parts[4], sum(parts)
        if _last_cpu is not None and total > _last_cpu[1]:
            out["cpu_pct"] = 100.0 * (1.0 - (idle - _last_cpu[0]) / (total - _last_cpu[1]))
        _last_cpu = (idle, total)
        mem = {}
        with open("/proc/meminfo") as f:
            for ln in f:
                k, v = ln.split(":")
                mem[k] = int(v.split()[0]) * 1024
        out["mem_total"] = mem.get("MemTotal", 0)
        out["mem_used"] = out["mem_total"] - mem.get("MemAvailable", 0)
        with open("/proc/self/statm") as f:
            out["rss"] = int(f.read().split()[1]) * os.sysconf("SC_PAGE_SIZE")
        out["load1"] = os.getloadavg()[0]
    except Exception:
        pass
    return out
