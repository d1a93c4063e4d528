"""Leveled logging with a pluggable sink.

Levels follow ``ov::log::Level`` (NO, ERR, WARNING, INFO, DEBUG, TRACE; src/inference/include/openvino/runtime/
properties.hpp:667-722); the level comes from the ``LOG_LEVEL`` core property or the ``OVB_LOG_LEVEL`` environment
variable. ``set_log_callback`` replaces the sink (default: stderr), as ``ov::util::set_log_callback`` does
(src/core/include/openvino/core/log.hpp).
"""
from __future__ import annotations

import os
import sys
import threading
from typing import Callable, Optional

LEVELS = {"NO": -1, "LOG_NONE": -1, "ERR": 0, "LOG_ERROR": 0, "WARNING": 1, "LOG_WARNING": 1, "INFO": 2, "LOG_INFO": 2, "DEBUG": 3, "LOG_DEBUG": 3,
          "TRACE": 4, "LOG_TRACE": 4}
_NAMES = {0: "ERR", 1: "WARNING", 2: "INFO", 3: "DEBUG", 4: "TRACE"}
_lock = threading.Lock()
_level = LEVELS.get(os.environ.get("OVB_LOG_LEVEL", "WARNING").upper(), 1)
_callback: Optional[Callable[[str], None]] = None


def set_level(level) -> None:
    """``level``: a name ("INFO"), an ``ov::log::Level`` style value, or an integer -1..4."""
    global _level
    if isinstance(level, int):
        _level = max(-1, min(4, level))
        return
    name = str(getattr(level, "name", level)).upper().split(".")[-1]
    if name not in LEVELS:
        raise ValueError("unknown log level %r" % (level,))
    _level = LEVELS[name]


def get_level() -> str:
    return "NO" if _level < 0 else _NAMES[_level]


def set_log_callback(callback: Callable[[str], None]) -> None:
    global _callback
    with _lock:
        _callback = callback


def reset_log_callback() -> None:
    global _callback
    with _lock:
        _callback = None


def _emit(level: int, component: str, msg: str) -> None:
    if level > _level:
        return
    line = "[%s] %s: %s" % (_NAMES[level], component, msg)
    with _lock:
        cb = _callback
    if cb is not None:
        cb(line)
    else:
        print(line, file=sys.stderr)


def err(component: str, msg: str) -> None: _emit(0, component, msg)
def warn(component: str, msg: str) -> None: _emit(1, component, msg)
def info(component: str, msg: str) -> None: _emit(2, component, msg)
def debug(component: str, msg: str) -> None: _emit(3, component, msg)
def trace(component: str, msg: str) -> None: _emit(4, component, msg)
