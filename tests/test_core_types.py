"""Element types, dimensions, shapes and host tensors."""
import numpy as np
import pytest

import openvino_b200 as ov
from openvino_b200 import Dimension, PartialShape, Shape, Tensor, Type


def test_type_properties():
    assert Type.f32.bitwidth == 32 and Type.f32.is_real() and Type.f32.size == 4
    assert Type.u4.bitwidth == 4 and not Type.u4.is_real() and not Type.u4.is_signed()
    assert Type.i4.is_signed()
    assert Type("FP16") is Type.f16 or Type("f16") is Type.f16
    assert Type(np.float32) is Type.f32
    assert Type.bf16.to_dtype() == np.uint16
    assert Type.dynamic.is_dynamic()
    assert Type.f32 == "f32"
    for name in ("f8e4m3", "f8e5m2", "nf4", "u1", "u2", "u3", "u6", "i4", "f4e2m1", "f8e8m0", "string", "boolean"):
        assert getattr(Type, name).name == name


def test_dimension():
    d = Dimension(3)
    assert d.is_static and d.get_length() == 3 and d == 3
    assert Dimension().is_dynamic and Dimension(-1).is_dynamic
    r = Dimension(2, 8)
    assert r.get_min_length() == 2 and r.get_max_length() == 8 and r.to_string() == "2..8"
    assert Dimension("?").is_dynamic and Dimension("1..").to_string() == "1.." and Dimension("..5").to_string() == "..5"
    assert r.compatible(4) and not r.compatible(9)
    assert Dimension(4).refines(r) and r.relaxes(Dimension(4))
    with pytest.raises(RuntimeError):
        Dimension().get_length()


def test_partial_shape():
    s = PartialShape([1, -1, (2, 8), 3])
    assert s.to_string() == "[1,?,2..8,3]"
    assert s.rank.get_length() == 4 and s.is_dynamic
    assert PartialShape("[1,?,2..8,3]") == s
    assert PartialShape("1,3,224,224").get_shape() == [1, 3, 224, 224]
    assert PartialShape.dynamic().rank.is_dynamic and PartialShape("...").rank.is_dynamic
    assert s.compatible([1, 5, 4, 3]) and not s.compatible([1, 5, 9, 3])
    assert PartialShape([1, 5, 4, 3]).refines(s)
    assert PartialShape.dynamic(3).to_string() == "[?,?,?]"
    with pytest.raises(RuntimeError):
        s.get_shape()


def test_tensor_from_numpy_copy_and_share():
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    t = Tensor(a)
    a[0, 0] = 100
    assert t.data[0, 0] == 0 and t.shape == [2, 3] and t.element_type == Type.f32 and t.byte_size == 24
    s = Tensor(a, shared_memory=True)
    a[0, 1] = 7
    assert s.data[0, 1] == 7
    s.data[1, 1] = -1
    assert a[1, 1] == -1


def test_tensor_type_shape_ctor_and_set_shape():
    t = Tensor(Type.i32, [2, 2])
    assert t.data.dtype == np.int32 and t.data.shape == (2, 2) and (t.data == 0).all()
    t.shape = [3, 1]
    assert t.data.shape == (3, 1) and t.size == 3
    p = Tensor(Type.u4, [3, 5])
    assert p.byte_size == 8 and p.data.dtype == np.uint8 and p.data.size == 8


def test_tensor_packed_and_bf16_conversion():
    vals = np.array([0, 1, 7, 15, 8, 3], dtype=np.float32)
    u4 = Tensor(vals).astype(Type.u4)
    assert u4.element_type == Type.u4 and u4.byte_size == 3
    # low nibble first
    assert u4.data[0] == (1 << 4 | 0) and u4.data[1] == (15 << 4 | 7)
    assert (u4.to_float32() == vals).all()
    i4 = Tensor(np.array([-8, -1, 0, 7], dtype=np.float32)).astype(Type.i4)
    assert (i4.to_float32() == [-8, -1, 0, 7]).all()
    b = Tensor(np.array([1.0, -2.5, 3.140625], dtype=np.float32)).astype(Type.bf16)
    assert b.data.dtype == np.uint16 and np.allclose(b.to_float32(), [1.0, -2.5, 3.140625])
    f8 = Tensor(np.array([0.5, 448.0, -1.75], dtype=np.float32)).astype(Type.f8e4m3)
    assert np.allclose(f8.to_float32(), [0.5, 448.0, -1.75])


def test_tensor_reinterpret_and_roi():
    raw = np.array([0x21, 0x43], dtype=np.uint8)
    t = Tensor(raw, [4], Type.u4)
    assert (t.to_float32() == [1, 2, 3, 4]).all()
    base = Tensor(np.arange(24, dtype=np.int32).reshape(2, 3, 4))
    roi = Tensor(base, begin=[0, 1, 1], end=[2, 3, 3])
    assert roi.shape == [2, 2, 2] and roi.data[0, 0, 0] == 5 and not roi.is_continuous()


def test_string_tensor():
    t = Tensor(np.array(["ab", "c"]))
    assert t.element_type == Type.string and t.shape == [2] and list(t.str_data) == ["ab", "c"]


def test_tensor_copy_to():
    a, b = Tensor(np.ones((2, 2), np.float32)), Tensor(Type.f32, [1])
    a.copy_to(b)
    assert b.shape == [2, 2] and (b.data == 1).all()
    with pytest.raises(RuntimeError):
        Tensor(np.ones(2, np.int32)).copy_to(b)


def test_version():
    assert "b200" in ov.get_version()


def test_import_order_with_torch_does_not_matter():
    """The native core hides its C++ runtime symbols: importing it before PyTorch must not crash PyTorch."""
    import subprocess
    import sys
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for code in ("import openvino_b200, torch; print(torch.zeros(2).sum().item())", "import torch, openvino_b200; print(torch.zeros(2).sum().item())"):
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=root, timeout=300)
        assert r.returncode == 0 and "0.0" in r.stdout, (r.returncode, r.stderr[-500:])
