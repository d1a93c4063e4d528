"""Host-side checks of the sampling kernels' arithmetic (no GPU needed)."""
import ctypes as C

import numpy as np
import pytest


@pytest.fixture(scope="module")
def lib():
    from openvino_b200 import build
    path = build.build_cuda()
    l = C.CDLL(str(path))
    l.ovb_gumbel_uniform.restype = C.c_float
    l.ovb_gumbel_uniform.argtypes = [C.c_uint64]
    return l


def test_gumbel_uniform_is_strictly_inside_the_unit_interval(lib):
    hi = lib.ovb_gumbel_uniform(2 ** 64 - 1)
    lo = lib.ovb_gumbel_uniform(0)
    assert 0.0 < lo < 1e-6 and hi < 1.0 and np.float32(hi) == np.float32(1.0 - 2.0 ** -24)
    # the noise -log(-log(u)) is finite at both ends in fp32
    for u in (lo, hi):
        g = -np.log(-np.log(np.float32(u), dtype=np.float32), dtype=np.float32)
        assert np.isfinite(g)
    # the mapping is monotone in the top 23 bits and ignores the rest
    a = lib.ovb_gumbel_uniform(5 << 41)
    assert a == lib.ovb_gumbel_uniform((5 << 41) | ((1 << 41) - 1)) and a < lib.ovb_gumbel_uniform(6 << 41)
