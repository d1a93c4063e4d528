"""TensorFlow frontend: frozen GraphDefs are written with a minimal protobuf encoder and compared with PyTorch math."""
import struct

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import openvino_b200 as ov
from openvino_b200.frontend import tensorflow as fe


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


DT = {np.dtype("float32"): 1, np.dtype("int32"): 3, np.dtype("int64"): 9}


def shape_proto(dims):
    return b"".join(_ld(2, _int(1, d)) for d in dims)


def tensor_proto(arr):
    arr = np.ascontiguousarray(arr)
    return _int(1, DT[arr.dtype]) + _ld(2, shape_proto(arr.shape)) + _ld(4, arr.tobytes())


def attr(v):
    if isinstance(v, bool):
        return _int(5, int(v))
    if isinstance(v, int):
        return _int(3, v)
    if isinstance(v, float):
        return _vi(4 << 3 | 5) + struct.pack("<f", v)
    if isinstance(v, bytes):
        return _ld(2, v)
    if isinstance(v, np.ndarray):
        return _ld(8, tensor_proto(v))
    if isinstance(v, tuple) and v[0] == "type":
        return _int(6, v[1])
    if isinstance(v, tuple) and v[0] == "shape":
        return _ld(7, shape_proto(v[1]))
    if isinstance(v, list):
        return _ld(1, b"".join(_int(3, x) for x in v))
    raise TypeError(v)


def node(name, op, inputs=(), **attrs):
    body = _ld(1, name.encode()) + _ld(2, op.encode()) + b"".join(_ld(3, i.encode()) for i in inputs)
    for k, v in attrs.items():
        body += _ld(5, _ld(1, k.encode()) + _ld(2, attr(v)))
    return _ld(1, body)


def const(name, arr):
    return node(name, "Const", value=np.asarray(arr), dtype=("type", DT[np.asarray(arr).dtype]))


def test_nhwc_convnet(tmp_path):
    rng = np.random.default_rng(0)
    w = rng.standard_normal((3, 3, 3, 8)).astype(np.float32) * 0.2          # HWIO
    b = rng.standard_normal(8).astype(np.float32)
    dw = rng.standard_normal((3, 3, 8, 1)).astype(np.float32) * 0.2         # depthwise HWIM
    g, be, mu, var = (rng.uniform(0.5, 1.5, 8).astype(np.float32) for _ in range(4))
    fc = rng.standard_normal((8, 5)).astype(np.float32)
    graph = b"".join([
        node("x", "Placeholder", dtype=("type", 1), shape=("shape", [2, 16, 16, 3])),
        const("w", w), const("b", b), const("dw", dw), const("g", g), const("be", be), const("mu", mu), const("var", var), const("fc", fc),
        const("axes", np.array([1, 2], np.int32)),
        node("conv", "Conv2D", ["x", "w"], strides=[1, 2, 2, 1], padding=b"SAME", data_format=b"NHWC"),
        node("bias", "BiasAdd", ["conv", "b"], data_format=b"NHWC"),
        node("relu6", "Relu6", ["bias"]),
        node("dwc", "DepthwiseConv2dNative", ["relu6", "dw"], strides=[1, 1, 1, 1], padding=b"VALID"),
        node("bn", "FusedBatchNormV3", ["dwc", "g", "be", "mu", "var"], epsilon=1e-3, is_training=False),
        node("pool", "MaxPool", ["bn:0"], ksize=[1, 2, 2, 1], strides=[1, 2, 2, 1], padding=b"VALID"),
        node("gap", "Mean", ["pool", "axes"], keep_dims=False),
        node("logits", "MatMul", ["gap", "fc"], transpose_a=False, transpose_b=False),
        node("prob", "Softmax", ["logits", "^x"]),
    ])
    path = tmp_path / "frozen.pb"
    path.write_bytes(graph)
    m = ov.Core().read_model(str(path))
    assert m.input("x").get_partial_shape().to_string() == "[2,16,16,3]" and m.output("prob").get_partial_shape().to_string() == "[2,5]"
    x = rng.standard_normal((2, 16, 16, 3)).astype(np.float32)
    t = torch.tensor
    xt = t(x).permute(0, 3, 1, 2)
    # TF "SAME" with stride 2 on 16 -> 8 outputs: total padding 1, all of it at the end
    y = F.conv2d(F.pad(xt, (0, 1, 0, 1)), t(w).permute(3, 2, 0, 1), t(b), 2)
    y = torch.clamp(y, 0, 6)
    y = F.conv2d(y, t(dw).permute(2, 3, 0, 1), None, 1, 0, 1, groups=8)
    y = F.batch_norm(y, t(mu), t(var), t(g), t(be), False, 0.0, 1e-3)
    y = F.max_pool2d(y, 2, 2).mean((2, 3))
    ref = torch.softmax(y @ t(fc), -1).numpy()
    np.testing.assert_allclose(ov.compile_model(m, "CPU")(x)[0], ref, rtol=1e-4, atol=1e-5)


def test_shape_ops_and_errors():
    graph = b"".join([
        node("x", "Placeholder", dtype=("type", 1), shape=("shape", [2, 3, 4])),
        const("perm", np.array([0, 2, 1], np.int32)), const("shp", np.array([2, 12], np.int32)), const("ax", np.array(1, np.int32)),
        const("begin", np.array([0, 2], np.int32)), const("end", np.array([0, 10], np.int32)), const("st", np.array([1, 2], np.int32)),
        node("tr", "Transpose", ["x", "perm"]),
        node("rs", "Reshape", ["tr", "shp"]),
        node("sl", "StridedSlice", ["rs", "begin", "end", "st"], begin_mask=1, end_mask=1, shrink_axis_mask=0, new_axis_mask=0, ellipsis_mask=0),
        node("sq", "Square", ["sl"]),
        node("cat", "ConcatV2", ["sl", "sq", "ax"], N=2),
        node("out", "Rsqrt", ["cat"]),
    ])
    m = fe.convert(graph)
    x = np.random.default_rng(1).uniform(0.5, 2.0, (2, 3, 4)).astype(np.float32)
    sl = x.transpose(0, 2, 1).reshape(2, 12)[:, 2:10:2]
    ref = 1.0 / np.sqrt(np.concatenate([sl, sl * sl], 1))
    np.testing.assert_allclose(ov.compile_model(m, "CPU")(x)[0], ref, rtol=1e-5)
    with pytest.raises(fe.TensorFlowError, match="NoSuchOp"):
        fe.convert(node("x", "Placeholder", dtype=("type", 1), shape=("shape", [1])) + node("y", "NoSuchOp", ["x"]))
