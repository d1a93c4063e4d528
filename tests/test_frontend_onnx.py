"""ONNX frontend: models are written with a minimal protobuf encoder here and compared with eager PyTorch."""
import struct

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import openvino_b200 as ov
from openvino_b200.frontend import onnx as fe


# ---- a tiny ONNX writer (wire format only)
def _vi(v):
    out = b""
    v &= (1 << 64) - 1
    while True:
        b = v & 0x7F
        v >>= 7
        out += bytes([b | (0x80 if v else 0)])
        if not v:
            return out


def _ld(field, payload):
    return _vi(field << 3 | 2) + _vi(len(payload)) + payload


def _int(field, v):
    return _vi(field << 3) + _vi(v)


def tensor(name, arr):
    arr = np.ascontiguousarray(arr)
    dt = {np.dtype("float32"): 1, np.dtype("int64"): 7, np.dtype("int32"): 6, np.dtype("bool"): 9, np.dtype("float16"): 10}[arr.dtype]
    return b"".join(_int(1, d) for d in arr.shape) + _int(2, dt) + _ld(8, name.encode()) + _ld(9, arr.tobytes())


def attr(name, v):
    b = _ld(1, name.encode())
    if isinstance(v, float):
        return b + _vi(2 << 3 | 5) + struct.pack("<f", v) + _int(20, 1)
    if isinstance(v, int):
        return b + _int(3, v) + _int(20, 2)
    if isinstance(v, bytes):
        return b + _ld(4, v) + _int(20, 3)
    if isinstance(v, np.ndarray):
        return b + _ld(5, tensor("", v)) + _int(20, 4)
    if isinstance(v, list) and all(isinstance(x, int) for x in v):
        return b + b"".join(_int(8, x) for x in v) + _int(20, 7)
    if isinstance(v, list) and all(isinstance(x, float) for x in v):
        return b + _ld(7, struct.pack("<%df" % len(v), *v)) + _int(20, 6)
    raise TypeError(v)


def node(op, inputs, outputs, name="", **attrs):
    return (b"".join(_ld(1, i.encode()) for i in inputs) + b"".join(_ld(2, o.encode()) for o in outputs) + _ld(3, name.encode()) +
            _ld(4, op.encode()) + b"".join(_ld(5, attr(k, v)) for k, v in attrs.items()))


def value_info(name, elem, dims):
    shape = b"".join(_ld(1, _int(1, d) if d >= 0 else _ld(2, b"N")) for d in dims)
    return _ld(1, name.encode()) + _ld(2, _ld(1, _int(1, elem) + _ld(2, shape)))


def model(nodes, inits, inputs, outputs):
    g = b"".join(_ld(1, n) for n in nodes) + _ld(2, b"g") + b"".join(_ld(5, tensor(k, v)) for k, v in inits.items())
    g += b"".join(_ld(11, value_info(*i)) for i in inputs) + b"".join(_ld(12, value_info(*o)) for o in outputs)
    return _int(1, 8) + _ld(8, _ld(1, b"") + _int(2, 17)) + _ld(7, g)


def test_convnet(tmp_path):
    rng = np.random.default_rng(0)
    w1, b1 = rng.standard_normal((6, 3, 3, 3)).astype(np.float32), rng.standard_normal(6).astype(np.float32)
    g, be, mu, var = (rng.uniform(0.5, 1.5, 6).astype(np.float32) for _ in range(4))
    fc_w, fc_b = rng.standard_normal((5, 6)).astype(np.float32), rng.standard_normal(5).astype(np.float32)
    nodes = [node("Conv", ["x", "w1", "b1"], ["c"], "conv", kernel_shape=[3, 3], pads=[1, 1, 1, 1], strides=[2, 2]),
             node("BatchNormalization", ["c", "g", "be", "mu", "var"], ["bn"], "bn", epsilon=1e-5),
             node("Relu", ["bn"], ["r"], "relu"),
             node("MaxPool", ["r"], ["p"], "pool", kernel_shape=[2, 2], strides=[2, 2]),
             node("GlobalAveragePool", ["p"], ["gap"], "gap"),
             node("Flatten", ["gap"], ["fl"], "flat", axis=1),
             node("Gemm", ["fl", "fc_w", "fc_b"], ["logits"], "fc", transB=1),
             node("Softmax", ["logits"], ["prob"], "sm", axis=-1)]
    data = model(nodes, {"w1": w1, "b1": b1, "g": g, "be": be, "mu": mu, "var": var, "fc_w": fc_w, "fc_b": fc_b},
                 [("x", 1, [-1, 3, 16, 16])], [("prob", 1, [-1, 5])])
    path = tmp_path / "net.onnx"
    path.write_bytes(data)
    m = ov.Core().read_model(str(path))
    assert m.input("x").get_partial_shape().to_string() == "[?,3,16,16]" and m.output("prob").get_partial_shape().to_string() == "[?,5]"
    x = rng.standard_normal((2, 3, 16, 16)).astype(np.float32)
    t = torch.tensor
    ref = F.conv2d(t(x), t(w1), t(b1), 2, 1)
    ref = F.relu(F.batch_norm(ref, t(mu), t(var), t(g), t(be), False, 0.0, 1e-5))
    ref = F.max_pool2d(ref, 2, 2).mean((2, 3))
    ref = torch.softmax(ref @ t(fc_w).t() + t(fc_b), -1).numpy()
    np.testing.assert_allclose(ov.compile_model(m, "CPU")(x)[0], ref, rtol=1e-4, atol=1e-5)


def test_transformer_style_ops():
    rng = np.random.default_rng(1)
    w = rng.standard_normal((8, 8)).astype(np.float32)
    nodes = [node("MatMul", ["x", "w"], ["h"]),
             node("Constant", [], ["shape"], value=np.array([0, -1, 2, 4], dtype=np.int64)),
             node("Reshape", ["h", "shape"], ["r"]),
             node("Transpose", ["r"], ["tr"], perm=[0, 2, 1, 3]),
             node("LayerNormalization", ["tr", "gamma", "beta"], ["ln"], axis=-1, epsilon=1e-5),
             node("Constant", [], ["two"], value=np.array(2.0, dtype=np.float32)),
             node("Pow", ["ln", "two"], ["sq"]),
             node("ReduceMean", ["sq"], ["mean"], axes=[-1], keepdims=1),
             node("Sqrt", ["mean"], ["rt"]),
             node("Div", ["ln", "rt"], ["nrm"]),
             node("Erf", ["nrm"], ["erf"]),
             node("Concat", ["nrm", "erf"], ["cat"], axis=-1),
             node("Slice", ["cat", "st", "en", "ax"], ["sl"]),
             node("Split", ["sl"], ["s0", "s1"], axis=1),
             node("Where", ["cond", "s0", "s1"], ["out"])]
    inits = {"w": w, "gamma": np.ones(4, np.float32) * 1.5, "beta": np.zeros(4, np.float32), "st": np.array([1], np.int64),
             "en": np.array([7], np.int64), "ax": np.array([3], np.int64), "cond": np.array([True, False, True, True, False, True])}
    data = model(nodes, inits, [("x", 1, [2, 5, 8])], [("out", 1, [2, 1, 5, 6])])
    m = ov.convert_model(fe.convert(data))
    x = rng.standard_normal((2, 5, 8)).astype(np.float32)
    h = torch.tensor(x @ w).reshape(2, 5, 2, 4).permute(0, 2, 1, 3)
    ln = F.layer_norm(h, [4]) * 1.5
    nrm = ln / (ln ** 2).mean(-1, keepdim=True).sqrt()
    cat = torch.cat([nrm, torch.erf(nrm)], -1)[..., 1:7]
    s0, s1 = cat[:, :1], cat[:, 1:]
    ref = torch.where(torch.tensor(inits["cond"]), s0, s1).numpy()
    np.testing.assert_allclose(ov.compile_model(m, "CPU")(x)[0], ref, rtol=1e-4, atol=1e-5)


def test_unknown_operator_is_reported():
    data = model([node("NoSuchOp", ["x"], ["y"])], {}, [("x", 1, [1])], [("y", 1, [1])])
    with pytest.raises(fe.OnnxError, match="NoSuchOp"):
        fe.convert(data)
    assert {"Conv", "Gemm", "LayerNormalization", "Resize"} <= set(fe.supported_ops())
