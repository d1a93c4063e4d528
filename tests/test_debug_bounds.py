"""The bounds-checking debug build of the kernels: indices read from device memory are checked, reported, and skipped."""
import os
import subprocess
import sys

import pytest

from openvino_b200 import build

HERE = os.path.dirname(os.path.abspath(__file__))


def test_debug_library_exports_the_same_entry_points():
    lib = build.LIB / "libovb_cuda_dbg.so"
    if not lib.exists():
        build.build_cuda_debug()
    import ctypes
    dbg, rel = ctypes.CDLL(str(lib)), ctypes.CDLL(str(build.build_cuda()))
    assert dbg.ovb_debug_bounds_enabled() == 1 and rel.ovb_debug_bounds_enabled() == 0
    for name in ("ovb_gemm", "ovb_paged_attention", "ovb_rope_kv_write", "ovb_embedding", "ovb_debug_set_limits"):
        assert hasattr(dbg, name) and hasattr(rel, name)
    # the checks cost the debug build a few registers at most: no spills in its attention kernels either
    rep = (build.OBJ / "dbg" / "attention.ptxas.txt").read_text()
    assert "bytes spill stores" in rep and all(" 0 bytes spill stores" in l for l in rep.splitlines() if "spill stores" in l)


@pytest.mark.gpu
def test_out_of_range_indices_are_reported_not_dereferenced():
    lib = build.LIB / "libovb_cuda_dbg.so"
    assert lib.exists(), "build the debug kernel library first: python -m openvino_b200.build --debug-bounds"
    r = subprocess.run([sys.executable, os.path.join(HERE, "debug_bounds_worker.py")], capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, OVB_CUDA_LIB=str(lib)))
    assert r.returncode == 0 and "DEBUG_BOUNDS_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])
