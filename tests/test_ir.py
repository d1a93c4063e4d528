"""IR v11 writer / reader: layout of the xml, weights deduplication, determinism, round trips."""
import os
import re

import numpy as np
import pytest

import openvino_b200 as ov
from openvino_b200 import Model, PartialShape, Tensor, Type
from openvino_b200 import opset as ops
from openvino_b200 import _ovcore as _c


def small_model(dynamic=False):
    x = ops.parameter([-1 if dynamic else 1, 3, 8, 8], "f32", "data")
    x.output(0).set_names({"data", "input:0"})
    w = np.arange(4 * 3 * 3 * 3, dtype=np.float32).reshape(4, 3, 3, 3) / 100
    c = ops.convolution(x, ops.constant(w, name="w"), [1, 1], [1, 1], [1, 1], [1, 1], name="conv")
    b = ops.add(c, ops.constant(np.ones((1, 4, 1, 1), np.float32), name="b"), name="bias")
    r = ops.relu(b, name="act")
    r.output(0).set_names({"out"})
    res = ops.result(r, name="res")
    return Model([res], [x], "net")


def test_xml_layout_matches_ir_v11_conventions():
    xml, weights = _c.serialize(small_model()._m)
    text = xml.decode()
    assert text.startswith('<?xml version="1.0"?>\n<net name="net" version="11">\n\t<layers>\n')
    assert '<layer id="0" name="data" type="Parameter" version="opset1">' in text
    assert '<data shape="1,3,8,8" element_type="f32" />' in text
    assert 'type="Const" version="opset1"' in text and 'type="ReLU"' in text
    assert '<data element_type="f32" shape="4, 3, 3, 3" offset="0" size="432" />' in text
    assert 'names="data,input:0"' in text or 'names="input:0,data"' in text
    assert '<edge from-layer="0" from-port="0" to-layer="2" to-port="0" />' in text
    assert text.rstrip().endswith("</net>")
    # port ids continue from inputs to outputs
    conv = text[text.index('name="conv"'):]
    conv = conv[:conv.index("</layer>")]
    assert re.findall(r'<port id="(\d)"', conv) == ["0", "1", "2"]
    assert len(weights) == 432 + 16


def test_round_trip_is_bit_exact_and_deterministic():
    m = small_model()
    xml1, bin1 = _c.serialize(m._m)
    xml1b, bin1b = _c.serialize(m._m)
    assert xml1 == xml1b and bin1 == bin1b
    m2 = Model._wrap(_c.deserialize(xml1.decode(), bin1))
    xml2, bin2 = _c.serialize(m2._m)
    assert xml1 == xml2 and bin1 == bin2
    # a structurally identical model built again serialises identically
    xml3, bin3 = _c.serialize(small_model()._m)
    assert xml3 == xml1 and bin3 == bin1


def test_read_back_preserves_structure(tmp_path):
    m = small_model(dynamic=True)
    path = str(tmp_path / "m.xml")
    ov.serialize(m, path)
    assert os.path.exists(str(tmp_path / "m.bin"))
    r = ov.Core().read_model(path)
    assert r.get_friendly_name() == "net"
    assert r.input(0).get_partial_shape().to_string() == "[?,3,8,8]"
    assert r.input("data") == r.input(0) and r.input("input:0") == r.input(0)
    assert r.output("out") == r.output(0)
    assert [n.get_type_name() for n in r.get_ops()] == [n.get_type_name() for n in m.get_ops()]
    assert [n.get_friendly_name() for n in r.get_ops()] == [n.get_friendly_name() for n in m.get_ops()]
    x = np.random.default_rng(0).standard_normal((2, 3, 8, 8)).astype(np.float32)
    a = ov.compile_model(m, "CPU")(x)[0]
    b = ov.compile_model(r, "CPU")(x)[0]
    np.testing.assert_array_equal(a, b)


def test_identical_constants_are_stored_once():
    x = ops.parameter([4], "f32")
    c1 = ops.constant(np.arange(4, dtype=np.float32))
    c2 = ops.constant(np.arange(4, dtype=np.float32))
    m = Model([ops.add(ops.add(x, c1), c2)], [x], "dedup")
    xml, weights = _c.serialize(m._m)
    assert len(weights) == 16
    assert xml.decode().count('offset="0" size="16"') == 2


def test_rt_info_round_trip():
    m = small_model()
    m.set_rt_info("1.2.3", ["MO_version"])
    m.set_rt_info("value", ["conversion_parameters", "framework"])
    m.set_rt_info({"a": "1", "b": "x"}, ["nncf", "quantization"])
    node = [n for n in m.get_ops() if n.get_friendly_name() == "conv"][0]
    node.rt_info["fused_names_0"] = "conv,bias"
    xml, weights = _c.serialize(m._m)
    text = xml.decode()
    assert "<rt_info>" in text and '<MO_version value="1.2.3" />' in text
    r = Model._wrap(_c.deserialize(text, weights))
    assert r.get_rt_info(["MO_version"]).value == "1.2.3"
    assert r.get_rt_info(["conversion_parameters", "framework"]).astype(str) == "value"
    assert r.has_rt_info(["nncf", "quantization", "b"]) and not r.has_rt_info(["nncf", "nope"])
    xml2, _ = _c.serialize(r._m)
    assert xml2 == xml


def test_low_precision_constants_round_trip():
    x = ops.parameter([2, 8], "f32")
    q = Tensor(np.arange(16, dtype=np.float32).reshape(2, 8) % 16).astype(Type.u4)
    w = ops.constant(q)
    assert w.get_output_element_type(0) == Type.u4 and w.get_output_shape(0) == [2, 8]
    deq = ops.multiply(ops.subtract(ops.convert(w, "f32"), np.float32(8)), np.float32(0.5))
    m = Model([ops.matmul(x, deq, False, True)], [x], "q")
    xml, weights = _c.serialize(m._m)
    assert 'element_type="u4"' in xml.decode() and 'precision="U4"' in xml.decode()
    r = Model._wrap(_c.deserialize(xml.decode(), weights))
    inp = np.ones((2, 8), np.float32)
    np.testing.assert_array_equal(ov.compile_model(m, "CPU")(inp)[0], ov.compile_model(r, "CPU")(inp)[0])
    bf = ops.constant(Tensor(np.array([1.5, -2.0], np.float32)).astype(Type.bf16))
    m2 = Model([ops.convert(bf, "f32")], [], "bf")
    xml, weights = _c.serialize(m2._m)
    r2 = Model._wrap(_c.deserialize(xml.decode(), weights))
    np.testing.assert_array_equal(ov.compile_model(r2, "CPU")()[0], [1.5, -2.0])


def test_sub_graph_ops_round_trip():
    x = ops.parameter([3], "f32", "x")
    acc_p, x_p = ops.parameter([3], "f32"), ops.parameter([3], "f32")
    new_acc = ops.add(acc_p, x_p)
    body = Model([ops.constant(np.array(True)), new_acc], [acc_p, x_p], "body")
    lb = ops.loop(np.array(3, dtype=np.int64), np.array(True))
    lb.set_function(body)
    lb.set_special_body_ports(-1, 0)
    lb.set_merged_input(acc_p, np.zeros(3, np.float32), new_acc)
    lb.set_invariant_input(x_p, x)
    lb.get_iter_value(new_acc, -1)
    m = Model([lb.build()], [x], "looped")
    xml, weights = _c.serialize(m._m)
    text = xml.decode()
    assert "<port_map>" in text and "<back_edges>" in text and "<body>" in text
    r = Model._wrap(_c.deserialize(text, weights))
    v = np.array([1, 2, 3], np.float32)
    np.testing.assert_array_equal(ov.compile_model(r, "CPU")(v)[0], 3 * v)
    assert _c.serialize(r._m)[0] == xml


def test_save_model_compresses_to_fp16(tmp_path):
    m = small_model()
    ov.save_model(m, str(tmp_path / "c.xml"))
    ov.save_model(m, str(tmp_path / "f.xml"), compress_to_fp16=False)
    assert os.path.getsize(tmp_path / "c.bin") < os.path.getsize(tmp_path / "f.bin")
    text = open(tmp_path / "c.xml").read()
    assert 'element_type="f16"' in text and "decompression" in text
    r = ov.Core().read_model(str(tmp_path / "c.xml"))
    x = np.random.default_rng(1).standard_normal((1, 3, 8, 8)).astype(np.float32)
    np.testing.assert_allclose(ov.compile_model(r, "CPU")(x)[0], ov.compile_model(m, "CPU")(x)[0], rtol=1e-2, atol=1e-2)


def test_read_errors():
    core = ov.Core()
    with pytest.raises(RuntimeError):
        core.read_model("/nonexistent/model.xml")
    with pytest.raises(RuntimeError):
        core.read_model('<?xml version="1.0"?><net name="x" version="11"><layers><layer id="0" name="a"')
    # an operation that no opset knows is kept as a framework node; no device runs it
    text = ('<?xml version="1.0"?><net name="x" version="11"><layers>'
            '<layer id="0" name="p" type="Parameter" version="opset1"><data shape="2" element_type="f32"/><output><port id="0" precision="FP32"><dim>2</dim></port></output></layer>'
            '<layer id="1" name="a" type="NoSuchOp" version="custom"><input><port id="0" precision="FP32"><dim>2</dim></port></input>'
            '<output><port id="1" precision="FP32"><dim>2</dim></port></output></layer>'
            '<layer id="2" name="r" type="Result" version="opset1"><input><port id="0" precision="FP32"><dim>2</dim></port></input></layer></layers>'
            '<edges><edge from-layer="0" from-port="0" to-layer="1" to-port="0"/><edge from-layer="1" from-port="1" to-layer="2" to-port="0"/></edges></net>')
    m = core.read_model(text)
    assert [n.get_type_name() for n in m.get_ops()] == ["Parameter", "NoSuchOp", "Result"]
    assert "a" not in core.query_model(m, "CPU")
    with pytest.raises(RuntimeError):
        core.compile_model(m, "CPU")(np.zeros(2, np.float32))


def test_read_from_memory_with_tensor_weights():
    xml, weights = _c.serialize(small_model()._m)
    w = Tensor(np.frombuffer(weights, dtype=np.uint8))
    r = ov.Core().read_model(xml.decode(), w)
    assert r.get_output_partial_shape(0) == [1, 4, 8, 8]
    r2 = ov.Core().read_model(bytes(xml), bytes(weights))
    assert len(r2.get_ops()) == len(r.get_ops())


# ---------------------------------------------------------------------------------------------- reference goldens
_GOLDEN_DIR = "/root/reference/src/core/tests/models/ir"
# files in that folder that the reference's own serializer wrote (IR v11, pugixml layout): they must come back byte for byte
_WRITTEN_BY_SERIALIZER = ("dynamic_variable", "string_parameter", "const_string")


def _goldens():
    import glob
    return sorted(glob.glob(os.path.join(_GOLDEN_DIR, "*.xml")))


@pytest.mark.skipif(not os.path.isdir(_GOLDEN_DIR), reason="reference tree not present")
def test_every_reference_golden_loads_and_reserialises_to_a_fixed_point(tmp_path):
    core = ov.Core()
    files = _goldens()
    assert len(files) >= 20
    for x in files:
        m = core.read_model(x)
        a_xml, a_bin = str(tmp_path / "a.xml"), str(tmp_path / "a.bin")
        ov.serialize(m, a_xml, a_bin)
        m2 = core.read_model(a_xml)
        b_xml, b_bin = str(tmp_path / "b.xml"), str(tmp_path / "b.bin")
        ov.serialize(m2, b_xml, b_bin)
        assert open(a_xml, "rb").read() == open(b_xml, "rb").read(), x
        assert open(a_bin, "rb").read() == open(b_bin, "rb").read(), x
        assert len(m2.get_ops()) == len(m.get_ops())


@pytest.mark.skipif(not os.path.isdir(_GOLDEN_DIR), reason="reference tree not present")
@pytest.mark.parametrize("name", _WRITTEN_BY_SERIALIZER)
def test_goldens_written_by_the_reference_serializer_come_back_byte_for_byte(tmp_path, name):
    core = ov.Core()
    src = os.path.join(_GOLDEN_DIR, name + ".xml")
    m = core.read_model(src)
    out_xml, out_bin = str(tmp_path / "o.xml"), str(tmp_path / "o.bin")
    ov.serialize(m, out_xml, out_bin)
    assert open(out_xml, "rb").read() == open(src, "rb").read()
    src_bin = src[:-4] + ".bin"
    if os.path.exists(src_bin):
        assert open(out_bin, "rb").read() == open(src_bin, "rb").read()


def test_string_constant_uses_the_packed_layout_of_the_reference(tmp_path):
    # count, begin offsets, last end, characters (src/core/src/runtime/string_aligned_buffer.cpp:19)
    import struct
    c = ops.constant(np.array([["abc", ""], ["de", "f"]], dtype=object))
    m = ov.Model([ops.result(c)], [], "strings")
    ov.serialize(m, str(tmp_path / "s.xml"), str(tmp_path / "s.bin"))
    raw = open(tmp_path / "s.bin", "rb").read()
    assert struct.unpack("<6i", raw[:24]) == (4, 0, 3, 3, 5, 6) and raw[24:] == b"abcdef"
    back = ov.Core().read_model(str(tmp_path / "s.xml"))
    const = [n for n in back.get_ops() if n.get_type_name() == "Constant"][0]
    assert [s.decode() if isinstance(s, bytes) else s for s in const.get_data().reshape(-1).tolist()] == ["abc", "", "de", "f"]
