"""Paddle frontend: a program and its combined parameter file are written with a minimal protobuf encoder and compared
with PyTorch."""
import struct

import numpy as np
import torch

import openvino_b200 as ov


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


FP32, INT64 = 5, 3


def tensor_desc(dtype, dims):
    return _int(1, dtype) + b"".join(_int(2, d) for d in dims)


def var(name, dims, dtype=FP32, persistable=False):
    vtype = _int(1, 7) + _ld(3, _ld(1, tensor_desc(dtype, dims)))               # LOD_TENSOR with a LoDTensorDesc
    return _ld(1, name.encode()) + _ld(2, vtype) + (_int(3, 1) if persistable else b"")


def attr(name, v):
    b = _ld(1, name.encode())
    if isinstance(v, bool):
        return b + _int(2, 6) + _int(10, int(v))
    if isinstance(v, int):
        return b + _int(2, 0) + _int(3, v)
    if isinstance(v, float):
        return b + _int(2, 1) + _vi(4 << 3 | 5) + struct.pack("<f", v)
    if isinstance(v, str):
        return b + _int(2, 2) + _ld(5, v.encode())
    if isinstance(v, list):
        return b + _int(2, 3) + b"".join(_int(6, x) for x in v)
    raise TypeError(v)


def op(type_, inputs, outputs, **attrs):
    b = b""
    for k, args in inputs.items():
        b += _ld(1, _ld(1, k.encode()) + b"".join(_ld(2, a.encode()) for a in args))
    for k, args in outputs.items():
        b += _ld(2, _ld(1, k.encode()) + b"".join(_ld(2, a.encode()) for a in args))
    b += _ld(3, type_.encode())
    for k, v in attrs.items():
        b += _ld(4, attr(k, v))
    return b


def program(vars_, ops_):
    block = _int(1, 0) + _int(2, (1 << 64) - 1) + b"".join(_ld(3, v) for v in vars_) + b"".join(_ld(4, o) for o in ops_)
    return _ld(1, block)


def params_file(tensors):
    out = b""
    for name in sorted(tensors):
        arr = np.ascontiguousarray(tensors[name])
        desc = tensor_desc({np.dtype("float32"): FP32, np.dtype("int64"): INT64}[arr.dtype], arr.shape)
        out += struct.pack("<I", 0) + struct.pack("<Q", 0) + struct.pack("<I", 0) + struct.pack("<i", len(desc)) + desc + arr.tobytes()
    return out


def test_cnn_program_with_combined_parameters(tmp_path):
    rng = np.random.default_rng(0)
    w = {"conv_w": rng.standard_normal((8, 3, 3, 3)).astype(np.float32) * 0.3, "bn_scale": rng.uniform(0.5, 1.5, 8).astype(np.float32),
         "bn_bias": rng.standard_normal(8).astype(np.float32), "bn_mean": rng.standard_normal(8).astype(np.float32) * 0.1,
         "bn_var": rng.uniform(0.5, 1.5, 8).astype(np.float32), "fc_w": rng.standard_normal((8, 5)).astype(np.float32),
         "fc_b": rng.standard_normal(5).astype(np.float32)}
    vars_ = [var("feed", []), var("fetch", []), var("image", [-1, 3, 10, 10]), var("c", [-1, 8, 5, 5]), var("b", [-1, 8, 5, 5]), var("r", [-1, 8, 5, 5]),
             var("p", [-1, 8, 1, 1]), var("f", [-1, 8]), var("m", [-1, 5]), var("a", [-1, 5]), var("prob", [-1, 5])]
    vars_ += [var(k, list(v.shape), persistable=True) for k, v in w.items()]
    ops_ = [op("feed", {"X": ["feed"]}, {"Out": ["image"]}, col=0),
            op("conv2d", {"Input": ["image"], "Filter": ["conv_w"]}, {"Output": ["c"]}, strides=[2, 2], paddings=[1, 1], dilations=[1, 1], groups=1,
               padding_algorithm="EXPLICIT"),
            op("batch_norm", {"X": ["c"], "Scale": ["bn_scale"], "Bias": ["bn_bias"], "Mean": ["bn_mean"], "Variance": ["bn_var"]}, {"Y": ["b"]}, epsilon=1e-5),
            op("relu", {"X": ["b"]}, {"Out": ["r"]}),
            op("pool2d", {"X": ["r"]}, {"Out": ["p"]}, pooling_type="avg", global_pooling=True, ksize=[1, 1]),
            op("flatten_contiguous_range", {"X": ["p"]}, {"Out": ["f"]}, start_axis=1, stop_axis=3),
            op("matmul_v2", {"X": ["f"], "Y": ["fc_w"]}, {"Out": ["m"]}, trans_x=False, trans_y=False),
            op("elementwise_add", {"X": ["m"], "Y": ["fc_b"]}, {"Out": ["a"]}, axis=-1),
            op("softmax", {"X": ["a"]}, {"Out": ["prob"]}, axis=-1),
            op("fetch", {"X": ["prob"]}, {"Out": ["fetch"]}, col=0)]
    (tmp_path / "net.pdmodel").write_bytes(program(vars_, ops_))
    (tmp_path / "net.pdiparams").write_bytes(params_file(w))
    m = ov.Core().read_model(str(tmp_path / "net.pdmodel"))
    assert [p.get_friendly_name() for p in m.get_parameters()] == ["image"] and m.input(0).get_partial_shape().is_dynamic
    x = rng.standard_normal((2, 3, 10, 10)).astype(np.float32)
    got = ov.compile_model(m, "CPU")([x])[0]
    t = torch.nn.functional.conv2d(torch.from_numpy(x), torch.from_numpy(w["conv_w"]), None, 2, 1)
    t = torch.nn.functional.batch_norm(t, torch.from_numpy(w["bn_mean"]), torch.from_numpy(w["bn_var"]), torch.from_numpy(w["bn_scale"]),
                                       torch.from_numpy(w["bn_bias"]), False, 0.0, 1e-5)
    t = torch.relu(t).mean((2, 3))
    want = torch.softmax(t @ torch.from_numpy(w["fc_w"]) + torch.from_numpy(w["fc_b"]), -1).numpy()
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)


def test_unsupported_operator_is_named(tmp_path):
    vars_ = [var("x", [1, 4]), var("y", [1, 4])]
    ops_ = [op("feed", {"X": ["feed"]}, {"Out": ["x"]}, col=0), op("strange_op", {"X": ["x"]}, {"Out": ["y"]}), op("fetch", {"X": ["y"]}, {"Out": ["fetch"]}, col=0)]
    (tmp_path / "bad.pdmodel").write_bytes(program(vars_, ops_))
    try:
        ov.Core().read_model(str(tmp_path / "bad.pdmodel"))
    except RuntimeError as e:
        assert "strange_op" in str(e)
    else:
        raise AssertionError("expected an error")
