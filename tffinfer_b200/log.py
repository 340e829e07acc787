"""A small leveled logger to stderr.

The reference logs through glog behind ``Logger::info / warning / error / fatal`` (printf-style, a file
sink, stderr only for FATAL: src/log/Logger.cpp:32-45).  Here: four levels, one line a message on stderr,
the threshold from ``TFFINFER_LOG`` (``error``, ``warning`` (default), ``info``, ``debug``) or
:func:`set_level`, no dependency.  Counters of the engine are not log lines: ``Engine.stats()`` has them.
"""
from __future__ import annotations

import os
import sys
import time

LEVELS = {"debug": 10, "info": 20, "warning": 30, "error": 40, "off": 100}
_level = LEVELS.get(os.environ.get("TFFINFER_LOG", "warning").lower(), 30)
_t0 = time.time()


def set_level(name: str) -> None:
    global _level
    if name.lower() not in LEVELS:
        raise ValueError(f"log level must be one of {sorted(LEVELS)}, got '{name}'")
    _level = LEVELS[name.lower()]


def get_level() -> str:
    return next(k for k, v in LEVELS.items() if v == _level)


def enabled(name: str) -> bool:
    return LEVELS[name] >= _level


def _emit(name: str, msg: str, args) -> None:
    if LEVELS[name] < _level:
        return
    if args:
        msg = msg % args
    print(f"[tffinfer_b200 {name.upper()} +{time.time() - _t0:.3f}s] {msg}", file=sys.stderr, flush=True)


def debug(msg: str, *args) -> None:
    _emit("debug", msg, args)


def info(msg: str, *args) -> None:
    _emit("info", msg, args)


def warning(msg: str, *args) -> None:
    _emit("warning", msg, args)


def error(msg: str, *args) -> None:
    _emit("error", msg, args)
