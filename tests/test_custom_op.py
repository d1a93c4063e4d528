"""Operations defined in Python: inference, evaluation on the CPU device, IR round trip, cloning."""
import numpy as np

import openvino_b200 as ov
from openvino_b200 import opset as ops


class ScaledClamp(ov.Op):
    class_type_info = ov.DiscreteTypeInfo("ScaledClamp", "extension")

    def __init__(self, x, scale=1.0, limit=1.0):
        super().__init__([x], {"scale": float(scale), "limit": float(limit)})

    def validate_and_infer_types(self):
        self.set_output_type(0, self.get_input_element_type(0), self.get_input_partial_shape(0))

    def evaluate(self, outputs, inputs):
        a = self.get_attributes()
        y = np.clip(inputs[0].data * a["scale"], -a["limit"], a["limit"])
        outputs[0].shape = list(y.shape)
        outputs[0].data[...] = y
        return True


def test_python_op_infers_runs_and_round_trips(tmp_path):
    x = ops.parameter([-1, 4], "f32", "x")
    node = ScaledClamp(ops.relu(x), scale=3.0, limit=2.0)
    assert node.get_type_name() == "ScaledClamp" and node.get_output_partial_shape(0).to_string() == "[?,4]"
    m = ov.Model([ops.result(ops.add(node, np.float32(1.0)))], [x], "custom")
    data = np.array([[-1, 0.2, 0.5, 1.0], [2.0, 0.1, 0.9, 0.4]], np.float32)
    want = np.clip(np.maximum(data, 0) * 3.0, -2.0, 2.0) + 1.0
    np.testing.assert_allclose(ov.compile_model(m, "CPU")(data)[0], want, rtol=1e-6)
    # the operation survives serialisation with its attributes, and clones
    xml = str(tmp_path / "custom.xml")
    ov.serialize(m, xml)
    m2 = ov.Core().read_model(xml)
    n2 = [n for n in m2.get_ops() if n.get_type_name() == "ScaledClamp"][0]
    assert abs(n2.get_attributes()["scale"] - 3.0) < 1e-6
    np.testing.assert_allclose(ov.compile_model(m2.clone(), "CPU")(data)[0], want, rtol=1e-6)


def test_functional_registration():
    ov.register_op("RowSum", lambda n: [(n.get_input_element_type(0), [n.get_input_partial_shape(0)[0]])],
                   lambda n, ins: [ins[0].sum(axis=1)])
    x = ops.parameter([3, 5], "f32", "x")
    from openvino_b200._graph import make_op
    y = make_op("RowSum", [x], version="extension")
    assert list(y.get_output_shape(0)) == [3]
    m = ov.Model([ops.result(y)], [x], "rs")
    a = np.arange(15, dtype=np.float32).reshape(3, 5)
    np.testing.assert_allclose(ov.compile_model(m, "CPU")(a)[0], a.sum(1))
