"""ovc command line: file in, IR out, with input shapes and fp16 compression."""
import os

import numpy as np

import openvino_b200 as ov
from openvino_b200 import opset as ops
from openvino_b200.tools import ovc


def test_convert_reshape_and_compress(tmp_path, capsys):
    x = ops.parameter([-1, 8], "f32", "x")
    w = np.random.default_rng(0).standard_normal((4, 8)).astype(np.float32)
    y = ops.relu(ops.matmul(x, w, False, True))
    y.output(0).set_names({"y"})
    src = str(tmp_path / "src.xml")
    ov.serialize(ov.Model([ops.result(y)], [x], "m"), src)
    out = str(tmp_path / "out" / "converted.xml")
    os.makedirs(os.path.dirname(out))
    assert ovc.main([src, "--output_model", out, "--input", "x[3,8]", "--verbose"]) == 0
    assert "[ SUCCESS ] XML file" in capsys.readouterr().out
    m = ov.Core().read_model(out)
    assert m.input("x").get_partial_shape().to_string() == "[3,8]"
    # fp16 compression is the default: the weight constant is stored as f16 behind a Convert
    assert any(n.get_type_name() == "Constant" and n.get_output_element_type(0).name == "f16" for n in m.get_ops())
    data = np.random.default_rng(1).standard_normal((3, 8)).astype(np.float32)
    np.testing.assert_allclose(ov.compile_model(m, "CPU")(data)[0], np.maximum(data @ w.T, 0), rtol=2e-3, atol=2e-3)
    out32 = str(tmp_path / "full.xml")
    assert ovc.main([src, "--output_model", out32, "--compress_to_fp16", "False"]) == 0
    assert os.path.getsize(out32[:-4] + ".bin") > os.path.getsize(out[:-4] + ".bin")
    assert ovc.parse_input("a[1,3,?,224],b[2]") == {"a": [1, 3, -1, 224], "b": [2]} and ovc.parse_input("[1,-1]") == [[1, -1]]
    assert ovc.main([str(tmp_path / "missing.onnx")]) == 1


def test_compile_tool_writes_a_blob_that_imports_back(tmp_path, capsys):
    import numpy as np
    import openvino_b200 as ov
    from openvino_b200 import opset as ops
    from openvino_b200.tools import compile_tool
    x = ops.parameter([-1, 8], "f32", "x")
    w = ops.constant(np.random.default_rng(0).standard_normal((4, 8)).astype(np.float32))
    m = ov.Model([ops.relu(ops.matmul(x, w, False, True))], [x], "fc")
    src, blob = str(tmp_path / "fc.xml"), str(tmp_path / "fc.blob")
    ov.serialize(m, src)
    assert compile_tool.main(["-m", src, "-d", "CPU", "-o", blob, "--shape", "x[3,8]", "-p", "PERFORMANCE_HINT=LATENCY", "--check"]) == 0
    assert "check ok" in capsys.readouterr().out
    back = ov.Core().import_model(open(blob, "rb").read(), "CPU")
    xin = np.ones((3, 8), np.float32)
    np.testing.assert_allclose(back([xin])[0], np.maximum(xin @ np.asarray(w.get_data()).T, 0), rtol=1e-5)
