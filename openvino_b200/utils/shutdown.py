"""Ordered release of process-wide resources: ``openvino_b200.shutdown()``.

Libraries that own device contexts, worker threads or mapped peer memory register a callback; ``shutdown()`` runs the
callbacks in reverse registration order (what was created last goes first), once, and is also hooked to interpreter
exit so that worker threads and peer-memory mappings are gone before the CUDA context is torn down. Role in the
reference: ``ov::shutdown()`` and the registry of unload callbacks, src/common/shutdown/shutdown.cpp and
src/inference/include/openvino/runtime/core.hpp:970.
"""
from __future__ import annotations

import atexit
import threading
from typing import Callable, List, Tuple

_lock = threading.Lock()
_callbacks: List[Tuple[int, str, Callable[[], None]]] = []
_next_id = 0
_done = False


def register_shutdown_callback(fn: Callable[[], None], name: str = "") -> int:
    """Run ``fn`` at ``shutdown()`` (or interpreter exit). Returns a handle for ``unregister_shutdown_callback``."""
    global _next_id
    with _lock:
        _next_id += 1
        _callbacks.append((_next_id, name or getattr(fn, "__qualname__", "callback"), fn))
        return _next_id


def unregister_shutdown_callback(handle: int) -> bool:
    with _lock:
        for i, (h, _, _) in enumerate(_callbacks):
            if h == handle:
                del _callbacks[i]
                return True
    return False


def shutdown() -> List[str]:
    """Run the registered callbacks, last registered first; a failing callback does not stop the others. Returns the
    names of the callbacks that ran. Later calls (and the exit hook after an explicit call) find nothing left to do;
    callbacks registered after a shutdown run at the next one."""
    global _done
    with _lock:
        todo = list(reversed(_callbacks))
        _callbacks.clear()
        _done = True
    ran = []
    for _, name, fn in todo:
        try:
            fn()
        except Exception as e:   # noqa: BLE001 - keep releasing the rest
            from . import log
            log.warn("shutdown", "%s failed: %s: %s" % (name, type(e).__name__, e))
        ran.append(name)
    return ran


atexit.register(shutdown)
