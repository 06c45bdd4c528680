"""Four-level logger with printf-style calls: errors and warnings to stderr, the rest to stdout; level from the
``log_level`` option / ``ENGINE_LOG_LEVEL``. Reference: inc/engine/core/log.h, src/core/log.cpp."""
from __future__ import annotations

import os
import sys
import threading
import time

LEVELS = {"error": 0, "warn": 1, "info": 2, "debug": 3}
_level = LEVELS.get(os.environ.get("ENGINE_LOG_LEVEL", "info").lower(), 2)
_lock = threading.Lock()
_t0 = time.time()


def set_level(name: str):
    global _level
    if name.lower() not in LEVELS:
        raise ValueError(f"log level must be one of {sorted(LEVELS)}")
    _level = LEVELS[name.lower()]


def get_level() -> str:
    return next(k for k, v in LEVELS.items() if v == _level)


def _emit(lvl: str, fmt: str, args, stream):
    if LEVELS[lvl] > _level:
        return
    msg = fmt % args if args else fmt
    with _lock:
        stream.write(f"[{time.time() - _t0:9.3f}] {lvl.upper():5s} {msg}\n")
        stream.flush()


def error(fmt, *a): _emit("error", fmt, a, sys.stderr)
def warn(fmt, *a): _emit("warn", fmt, a, sys.stderr)
def info(fmt, *a): _emit("info", fmt, a, sys.stdout)
def debug(fmt, *a): _emit("debug", fmt, a, sys.stdout)
