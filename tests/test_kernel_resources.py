"""Resource usage of the hot kernels as ptxas reports it at build time (no GPU needed).

A by-reference lambda that stops being inlined, or a locally indexed array, moves a kernel's working set into a stack
frame; the GEMM then loses a third of its speed without any functional symptom. The build keeps ptxas' report, this
test reads it."""
import pytest

from openvino_b200 import build


@pytest.fixture(scope="module")
def gemm():
    build.build_cuda()
    res = build.kernel_resources("gemm_sm100")
    if not res:
        build.build_cuda(force=True)
        res = build.kernel_resources("gemm_sm100")
    assert res, "no ptxas report for gemm_sm100.cu"
    return res


def test_gemm_variants_have_no_stack_working_set(gemm):
    assert len(gemm) >= 25                     # 5 token-tile sizes x 5 weight formats
    for name, r in gemm.items():
        assert r["stack"] <= 64, (name, r)     # a few words for the bounded-wait helper are fine; hundreds of bytes are not
        assert r["spill_stores"] <= 16 and r["spill_loads"] <= 32, (name, r)


def test_decode_variants_fit_two_ctas_per_sm(gemm):
    # decode-sized quantised tiles run two CTAs of 352 threads per SM: at most 65536 / 704 = 93 registers per thread
    small = [r for n, r in gemm.items() if r["registers"] <= 93]
    assert len(small) >= 9                     # u4 / u8 / fp8 at 16, 32 and 64 tokens


def test_gemm_uses_no_static_shared_memory(gemm):
    # the kernel opts in to the whole dynamic shared-memory limit of the SM: one static __shared__ word makes the opt-in fail
    assert all(r["static_smem"] == 0 for r in gemm.values()), {n: r["static_smem"] for n, r in gemm.items() if r["static_smem"]}
