"""Conditional compilation, the analysing stage: which kernel variants did this process use?

``OVB_CC_COLLECT=<file>`` in the environment (or ``enable(path)``) writes the statistics when the process shuts down:
one line per GEMM variant that was launched, ``gemm,<token tile>,<weight format>,<fp16>``. Statistics of several runs
are merged by concatenating the files. ``python -m openvino_b200.build --cc-stats=<file> [--cc-out=<dir>]`` then compiles
a kernel library that holds only those variants (``build.build_selective``); ``OVB_CUDA_LIB=<dir>/libovb_cuda.so`` loads it.
Role in the reference: the collector of src/common/conditional_compilation (SELECTIVE_BUILD=COLLECT, ITT counters
written to a csv that the selective build reads)."""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Tuple

_path: Optional[str] = None
_TILES = (16, 32, 64, 128, 256)


def used_gemm_variants() -> List[Tuple[int, int, int]]:
    """(token tile, weight format, fp16) of every GEMM variant launched so far (empty when the library is not loaded)."""
    from ..ops import cuda as K
    if K._lib is None:
        return []
    fn = K._lib.ovb_cc_used_gemm
    fn.restype = C.c_uint
    out = []
    for wmode in range(8):
        for f16 in (0, 1):
            mask = int(fn(C.c_int(wmode), C.c_int(f16)))
            out += [(bt, wmode, f16) for i, bt in enumerate(_TILES) if mask >> i & 1]
    return out


def is_selective_build() -> bool:
    from ..ops import cuda as K
    return bool(K.lib().ovb_cc_is_selective())


def write_stats(path: str) -> int:
    rows = used_gemm_variants()
    with open(path, "a") as f:
        for bt, wmode, f16 in rows:
            f.write("gemm,%d,%d,%d\n" % (bt, wmode, f16))
    return len(rows)


def enable(path: str) -> None:
    """Write the statistics to ``path`` at shutdown (appending, so that several runs accumulate)."""
    global _path
    first = _path is None
    _path = path
    if first:
        from .shutdown import register_shutdown_callback
        register_shutdown_callback(lambda: write_stats(_path), "conditional-compilation statistics")


if os.environ.get("OVB_CC_COLLECT"):
    enable(os.environ["OVB_CC_COLLECT"])
