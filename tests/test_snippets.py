"""Snippets: tokenisation into Subgraph nodes, lowering to the linear IR (stages, loop fusion, register reuse), the host
executor against the untokenised model, and the generated kernels on a GPU against fp32 PyTorch."""
import numpy as np
import pytest
import torch

import openvino_b200 as ov
from openvino_b200 import opset as ops
from openvino_b200.snippets import body_of, classify, tokenize
from openvino_b200.snippets.emit_cuda import generate_source, vec_width


def _types(m):
    return [n.get_type_name() for n in m.get_ops()]


def _mlp_tail_model(dtype="f32"):
    x = ops.parameter([-1, 6, 32], dtype, "x")
    bias = ops.constant(np.linspace(-1, 1, 32).astype(np.float32 if dtype == "f32" else np.float16))
    scale = ops.parameter([-1, 6, 1], dtype, "s")
    h = ops.gelu(ops.add(x, bias), "TANH")
    h = ops.multiply(h, scale)
    h = ops.clamp(h, -2.0, 2.0)
    y = ops.add(ops.softmax(h, 2), x)
    return ov.Model([y], [x, scale], "tail")


def test_tokenizer_forms_one_subgraph_and_host_matches():
    m = _mlp_tail_model()
    rng = np.random.default_rng(0)
    x, s = rng.standard_normal((3, 6, 32)).astype(np.float32), rng.random((3, 6, 1)).astype(np.float32) + 0.5
    ref = ov.compile_model(m.clone(), "CPU")([x, s])[0]
    assert tokenize(m) == 1
    assert sorted(_types(m)) == sorted(["Parameter", "Parameter", "Constant", "Subgraph", "Result"])
    sub = next(n for n in m.get_ops() if n.get_type_name() == "Subgraph")
    assert "fused_names_0" in sub.get_rt_info() and list(sub.get_output_partial_shape(0))[1].get_length() == 6
    got = ov.compile_model(m, "CPU")([x, s])[0]
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-6)
    # lowering: softmax gives two reductions -> three passes; the per-row scale is a col-domain value
    lir = body_of(sub).linear_ir(("full", "row", "col"))
    assert len(lir.loops) == 3 and [len(lp.reduces) for lp in lir.loops] == [1, 1, 0] and len(lir.loops[2].stores) == 1
    assert any(e.kind == "param" and e.domain == "col" for e in lir.exprs)
    assert max(lir.loops[2].regs.values()) <= 2                 # registers are reused along the chain
    src = generate_source(lir)
    assert "block_max" in src and "block_sum" in src and src.count("for (long long c =") == 3 and vec_width(lir) == 4
    # the clamped value and the exponentials are held in registers between the passes of the second kernel form,
    # and the division by the row sum became a multiplication by its reciprocal
    assert len(lir.kept) == 2 and "run_kept" in src and "snippet_vec_k4" in src
    assert [len(lp.readback) for lp in lir.loops_kept] == [0, 1, 1]
    assert any(e.op == "Reciprocal" and e.domain == "col" for e in lir.exprs) and not any(e.op == "Divide" for e in lir.exprs)


def test_independent_reductions_share_a_loop_and_col_outputs():
    # mean and mean of squares of the same row: one pass; the variance leaves the snippet as a [rows, 1] value
    x = ops.parameter([4, 16], "f32", "x")
    mean = ops.reduce_mean(x, np.array([1], np.int64), True)
    sq = ops.reduce_mean(ops.multiply(x, x), np.array([1], np.int64), True)
    var = ops.subtract(sq, ops.multiply(mean, mean))
    y = ops.divide(ops.subtract(x, mean), ops.sqrt(ops.add(var, np.float32(1e-5))))
    m = ov.Model([y, var], [x], "norm")
    xv = np.random.default_rng(1).standard_normal((4, 16)).astype(np.float32)
    ref = ov.compile_model(m.clone(), "CPU")([xv])
    ref = [ref[0], ref[1]]
    assert tokenize(m) == 1
    sub = next(n for n in m.get_ops() if n.get_type_name() == "Subgraph")
    lir = body_of(sub).linear_ir(("full",))
    assert len(lir.loops) == 2 and len(lir.loops[0].reduces) == 2
    assert sorted(s.domain for s in lir.stores) == ["col", "full"]
    got = ov.compile_model(m, "CPU")([xv])
    np.testing.assert_allclose(got[0], ref[0], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(got[1], ref[1], rtol=1e-4, atol=1e-6)
    assert got[1].shape == (4, 1)


def test_groups_do_not_close_cycles_and_small_groups_stay():
    x = ops.parameter([2, 8], "f32", "x")
    a = ops.relu(ops.add(x, np.float32(1)))                       # group 1
    mm = ops.matmul(a, np.eye(8, dtype=np.float32), False, False)  # not element-wise, reads group 1
    b = ops.multiply(ops.add(a, mm), np.float32(2))               # reads group 1 and, through MatMul, group 1 again: must start a new group
    single = ops.sigmoid(ops.matmul(b, np.eye(8, dtype=np.float32), False, False))        # one operation: stays as it is
    m = ov.Model([single], [x], "c")
    xv = np.random.default_rng(2).standard_normal((2, 8)).astype(np.float32)
    ref = ov.compile_model(m.clone(), "CPU")([xv])[0]
    assert tokenize(m) == 2
    t = _types(m)
    assert t.count("Subgraph") == 2 and t.count("Sigmoid") == 1 and t.count("MatMul") == 2
    np.testing.assert_allclose(ov.compile_model(m, "CPU")([xv])[0], ref, rtol=1e-5, atol=1e-6)
    # inputs that do not fit [rows, cols] forms are reported by classify
    assert classify([[2, 3, 8], [2, 1, 8]], [2, 3, 8]) is None
    assert classify([[2, 3, 8], [8], [2, 3, 1], []], [2, 3, 8]) == (("full", "row", "col", "scalar"), 6, 8)


def test_select_and_comparisons_in_half_precision():
    x = ops.parameter([5, 24], "f16", "x")
    y = ops.parameter([5, 24], "f16", "y")
    z = ops.select(ops.greater(x, y), ops.multiply(x, np.float16(2)), ops.negative(y))
    m = ov.Model([ops.convert(z, "f32")], [x, y], "sel")
    rng = np.random.default_rng(3)
    xv, yv = rng.standard_normal((5, 24)).astype(np.float16), rng.standard_normal((5, 24)).astype(np.float16)
    ref = ov.compile_model(m.clone(), "CPU")([xv, yv])[0]
    assert tokenize(m) == 1
    np.testing.assert_allclose(ov.compile_model(m, "CPU")([xv, yv])[0], ref, rtol=1e-3, atol=1e-3)
    sub = next(n for n in m.get_ops() if n.get_type_name() == "Subgraph")
    assert vec_width(body_of(sub).linear_ir(("full", "full"))) == 4          # an fp32 output is involved


@pytest.mark.gpu
def test_generated_kernels_on_gpu(tmp_path, monkeypatch):
    monkeypatch.setenv("OVB_SNIPPETS_CACHE", str(tmp_path))
    core = ov.Core()
    rng = np.random.default_rng(4)
    for dtype, tol in (("f32", 1e-5), ("f16", 2e-3)):
        m = _mlp_tail_model(dtype)
        npdt = np.float32 if dtype == "f32" else np.float16
        cm = core.compile_model(m, "CUDA", {"SNIPPETS_MODE": "ENABLE", "INFERENCE_PRECISION_HINT": dtype})
        assert any(n.get_type_name() == "Subgraph" for n in cm.get_runtime_model().get_ops())
        for B in (3, 1, 7):                                   # dynamic batch: one kernel, three launches
            x, s = rng.standard_normal((B, 6, 32)).astype(npdt), (rng.random((B, 6, 1)) + 0.5).astype(npdt)
            xt, st = torch.from_numpy(x).float(), torch.from_numpy(s).float()
            bias = torch.linspace(-1, 1, 32)
            h = torch.nn.functional.gelu(xt + bias, approximate="tanh") * st
            ref = torch.softmax(h.clamp(-2, 2), -1) + xt
            got = np.asarray(cm([x, s])[0], dtype=np.float32)
            np.testing.assert_allclose(got, ref.numpy(), rtol=tol, atol=tol)
    assert len(list(tmp_path.glob("snippet_*.so"))) == 2
    # element-wise only, odd extents (scalar instance) and aligned extents (vector instance), bf16
    for shape in ((3, 5, 7), (4, 64)):
        x = ops.parameter(list(shape), "bf16", "x")
        y = ops.parameter([shape[-1]], "bf16", "y")
        z = ops.swish(ops.add(ops.multiply(x, y), ops.convert(np.float32(0.25), "bf16")))
        m2 = ov.Model([ops.maximum(z, ops.negative(x))], [x, y], "ew")
        cm2 = core.compile_model(m2, "CUDA", {"SNIPPETS_MODE": "ENABLE", "INFERENCE_PRECISION_HINT": "bf16"})
        xt, yt = torch.randn(shape).bfloat16(), torch.randn(shape[-1]).bfloat16()
        got = cm2([ov.Tensor(xt), ov.Tensor(yt)])[0]
        v = xt.float() * yt.float() + 0.25
        ref = torch.maximum(v * torch.sigmoid(v), -xt.float())
        got_t = torch.from_numpy(np.asarray(got).astype(np.uint16).astype(np.int32) << 16).view(torch.float32) if np.asarray(got).dtype == np.uint16 else torch.as_tensor(np.asarray(got, dtype=np.float32))
        torch.testing.assert_close(got_t.reshape(shape), ref, rtol=2e-2, atol=2e-2)
