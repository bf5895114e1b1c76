"""Levelled logging and timing helpers.

``HETU_INTERNAL_LOG_LEVEL`` (TRACE | DEBUG | INFO | WARN | ERROR | FATAL, default WARN) selects the level, as
in the reference (hetu/common/logging.cc:14); messages carry time, rank, level and call site.  ``TIK`` / ``TOK``
/ ``COST_MSEC`` mirror hetu/common/timing.h, ``ht_assert`` mirrors HT_ASSERT (raises with a formatted message).
"""
from __future__ import annotations

import inspect
import os
import sys
import time

LEVELS = {"TRACE": 0, "DEBUG": 1, "INFO": 2, "WARN": 3, "ERROR": 4, "FATAL": 5}
_level = LEVELS.get(os.environ.get("HETU_INTERNAL_LOG_LEVEL", "WARN").upper(), 3)
_timers: dict = {}


def set_level(name: str) -> None:
    global _level
    _level = LEVELS[name.upper()]


def get_level() -> str:
    return next(k for k, v in LEVELS.items() if v == _level)


def log(level: str, *parts) -> None:
    lv = LEVELS[level]
    if lv < _level:
        return
    fr = inspect.stack()[2] if len(inspect.stack()) > 2 else inspect.stack()[-1]
    rank = os.environ.get("RANK", "0")
    stamp = time.strftime("%H:%M:%S")
    sys.stderr.write(f"[{stamp}][rank {rank}][{level}] {os.path.basename(fr.filename)}:{fr.lineno} "
                     + " ".join(str(p) for p in parts) + "\n")
    if level == "FATAL":
        raise RuntimeError(" ".join(str(p) for p in parts))


def trace(*p): log("TRACE", *p)
def debug(*p): log("DEBUG", *p)
def info(*p): log("INFO", *p)
def warn(*p): log("WARN", *p)
def error(*p): log("ERROR", *p)
def fatal(*p): log("FATAL", *p)


def ht_assert(cond, *msg) -> None:
    if not cond:
        raise AssertionError("HT_ASSERT failed: " + " ".join(str(m) for m in msg))


def TIK(name: str = "default") -> None:
    _timers[name] = time.perf_counter()


def TOK(name: str = "default") -> float:
    """Milliseconds since the matching TIK."""
    _timers[name + "/cost"] = (time.perf_counter() - _timers[name]) * 1e3
    return _timers[name + "/cost"]


def COST_MSEC(name: str = "default") -> float:
    return _timers.get(name + "/cost", 0.0)
