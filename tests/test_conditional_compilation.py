"""Conditional compilation: statistics of an analysing run drive a selective build of the kernel library."""
import re

import pytest

from openvino_b200 import build


def test_selective_build_instantiates_only_the_recorded_gemm_variants(tmp_path):
    stats = tmp_path / "stats.csv"
    stats.write_text("gemm,64,1,0\ngemm,256,1,0\ngemm,64,1,0\n")            # two u4 variants (a repeated line is harmless)
    out = build.build_selective(stats, tmp_path / "sel", stems={"gemm_sm100"}, link=False)
    header = (out / "cc_selected.h").read_text()
    assert "bt == 64 && wmode == 1" in header and "bt == 256 && wmode == 1" in header
    report = (out / "gemm_sm100.ptxas.txt").read_text()
    kernels = set(re.findall(r"Compiling entry function '(\S*gemm_ws_kernel\S*)'", report))
    assert len(kernels) == 2, kernels
    full = build.kernel_resources("gemm_sm100")
    if full:
        assert len([k for k in full if "gemm_ws_kernel" in k]) >= 25
        assert (out / "gemm_sm100.o").stat().st_size < 0.35 * (build.OBJ / "gemm_sm100.o").stat().st_size


@pytest.mark.gpu
def test_analysing_run_records_launched_variants():
    import torch
    from openvino_b200.ops import cuda as K
    from openvino_b200.utils import cc
    x = torch.randn(40, 256, device="cuda", dtype=torch.bfloat16)
    w = K.PackedWeight.from_dense((torch.randn(128, 256, device="cuda") * 0.1).to(torch.bfloat16))
    K.gemm(x, w)
    torch.cuda.synchronize()
    used = cc.used_gemm_variants()
    assert (64, 0, 0) in used and not cc.is_selective_build()      # 40 tokens -> the 64-token tile, bf16 weights
