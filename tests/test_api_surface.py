"""Public API surface beyond the core classes: versioned opset modules, small container types, extension objects,
PyTorch decoders and module extensions, plugin registration from a file, packing helpers."""
import importlib

import numpy as np
import pytest
import torch

import openvino_b200 as ov
from openvino_b200 import opset as ops


def test_versioned_opset_modules():
    o1, o8, o15 = (importlib.import_module("openvino_b200.opset%d" % n) for n in (1, 8, 15))
    x = o1.parameter([2, 3], "f32", "x")
    assert o1.softmax(x, 1).get_version() == "opset1" and o8.softmax(x, 1).get_version() == "opset8"
    assert not hasattr(o1, "gelu") and hasattr(o8, "gelu") and not hasattr(o8, "stft") and hasattr(o15, "stft")
    for n in range(1, 18):
        m = importlib.import_module("openvino_b200.opset%d" % n)
        assert callable(m.parameter) and callable(m.add) and callable(m.constant)
    assert ov.opset13 is importlib.import_module("openvino_b200.opset13")


def test_container_types_any_and_batch_helpers(tmp_path):
    assert list(ov.Coordinate([1, 2])) == [1, 2] and ov.AxisSet([3, 1]).to_vector() == [1, 3] and list(ov.Strides((2, 2))) == [2, 2]
    assert ov.OVAny("YES").astype(bool) is True and ov.OVAny("CPU,CUDA").aslist() == ["CPU", "CUDA"] and ov.OVAny(3) == 3 and ov.Any is ov.OVAny
    x = ops.parameter([1, 3, 8, 8], "f32", "x")
    m = ov.Model([ops.relu(x)], [x], "b")
    assert ov.get_batch(m).get_length() == 1
    ov.set_batch(m, 4)
    assert list(m.get_parameters()[0].get_output_shape(0)) == [4, 3, 8, 8] and list(m.get_output_shape(0)) == [4, 3, 8, 8]
    (tmp_path / "blob.bin").write_bytes(bytes(range(7)))
    t = ov.tensor_from_file(str(tmp_path / "blob.bin"))
    assert t.data.tolist() == list(range(7)) and str(t.element_type) == "u8"
    from openvino_b200.helpers import pack_data, unpack_data
    v = np.array([-8, -1, 0, 7, 3], np.int8)
    np.testing.assert_array_equal(unpack_data(pack_data(v, "i4"), "i4", [5]), v)
    bits = np.array([1, 0, 1, 1, 0, 0, 1, 0, 1], np.uint8)
    np.testing.assert_array_equal(unpack_data(pack_data(bits, "u1"), "u1", [9]), bits)
    assert ov.passes.Version.IR_V11 == "IR_V11" and ov.properties.intel_gpu.hint.queue_throttle == "GPU_QUEUE_THROTTLE"
    assert ov.properties.intel_npu.use_npuw == "NPU_USE_NPUW" and ov.properties.intel_cpu.denormals_optimization == "CPU_DENORMALS_OPTIMIZATION"


def test_core_extensions_and_plugins_file(tmp_path):
    class Twice(ov.Op):
        class_type_info = ov.DiscreteTypeInfo("TwiceOp", "extension")

        def __init__(self, x=None):
            super().__init__(self, [x] if x is not None else None)

        def validate_and_infer_types(self):
            self.set_output_type(0, self.get_input_element_type(0), self.get_input_partial_shape(0))

        def evaluate(self, outputs, inputs):
            outputs[0].data[...] = inputs[0].data * 2
            return True
    core = ov.Core()
    core.add_extension(ov.OpExtension(Twice))
    core.add_extension([Twice])
    with pytest.raises(RuntimeError):
        core.add_extension("libcustom_ops.so")
    # a plugins file: another name for the CPU device class, with a property
    (tmp_path / "plugins.xml").write_text('<ie><plugins><plugin name="MYCPU" location="openvino_b200.runtime.core:CpuPlugin">'
                                          '<properties><property key="NUM_STREAMS" value="2"/></properties></plugin></plugins></ie>')
    core.register_plugins(str(tmp_path / "plugins.xml"))
    assert "MYCPU" in core.available_devices or "MYCPU" in core.get_available_devices()
    x = ops.parameter([2], "f32", "x")
    cm = core.compile_model(ov.Model([ops.relu(x)], [x], "p"), "MYCPU")
    np.testing.assert_array_equal(cm([np.array([-1, 2], np.float32)])[0], [0, 2])
    with pytest.raises(RuntimeError):
        cm.get_context()                                       # the host device has no device memory context


def test_pytorch_decoders_and_module_extension():
    from openvino_b200.frontend import DecoderTransformationExtension, FrontEndManager
    from openvino_b200.frontend.pytorch import ModuleExtension, TorchFXPythonDecoder, TorchScriptPythonDecoder

    class Inner(torch.nn.Module):
        def forward(self, x):
            return torch.sin(x)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.inner = Inner()
            self.lin = torch.nn.Linear(4, 3)

        def forward(self, x):
            return self.inner(self.lin(x)) + 1
    net = Net().eval()
    x = torch.randn(2, 4)
    fe = FrontEndManager().load_by_framework("pytorch")
    dec = TorchScriptPythonDecoder(net, example_input=(x,))
    assert fe.supported(dec)
    m = fe.convert(fe.load(dec))
    np.testing.assert_allclose(ov.compile_model(m, "CPU")([x.numpy()])[0], net(x).detach().numpy(), rtol=1e-5, atol=1e-6)
    ep = torch.export.export(net, (x,))
    m2 = fe.convert(fe.load(TorchFXPythonDecoder.from_exported_program(ep)))
    np.testing.assert_allclose(ov.compile_model(m2, "CPU")([x.numpy()])[0], net(x).detach().numpy(), rtol=1e-5, atol=1e-6)
    # the inner module is swapped for a cosine while converting; the module itself is left as it was
    seen = []
    fe2 = FrontEndManager().load_by_framework("pytorch")
    fe2.add_extension(ModuleExtension(Inner, convert=lambda module, target, x: torch.cos(x)))
    fe2.add_extension(DecoderTransformationExtension(lambda model: seen.append(len(model.get_ops()))))
    m3 = fe2.convert(fe2.load(net, {"example_input": (x,)}))
    ref = torch.cos(net.lin(x)).detach().numpy() + 1
    np.testing.assert_allclose(ov.compile_model(m3, "CPU")([x.numpy()])[0], ref, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(net(x).detach().numpy(), torch.sin(net.lin(x)).detach().numpy() + 1, rtol=1e-6)
    assert seen and seen[0] > 3
