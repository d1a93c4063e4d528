"""TFLite frontend: flatbuffers written by tests/fb_writer.py against numpy / PyTorch references."""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import openvino_b200 as ov   # noqa: E402
from fb_writer import Tab, Vec, build   # noqa: E402

F32, I32, U8, I8, F16 = 0, 2, 3, 9, 1


class TfliteBuilder:
    """Collects tensors / buffers / operators and writes the Model table."""

    def __init__(self):
        self.buffers = [Tab([None])]              # buffer 0: the empty buffer
        self.tensors, self.ops, self.codes = [], [], []

    def tensor(self, name, shape, ttype=F32, data=None, quant=None):
        b = 0
        if data is not None:
            self.buffers.append(Tab([Vec(np.uint8, np.frombuffer(np.ascontiguousarray(data).tobytes(), np.uint8))]))
            b = len(self.buffers) - 1
        q = None
        if quant is not None:
            scale, zp, axis = quant
            q = Tab([None, None, Vec(np.float32, scale), Vec(np.int64, zp), None, None, ("i", axis)])
        self.tensors.append(Tab([Vec(np.int32, shape), ("b", ttype), ("I", b), name, q]))
        return len(self.tensors) - 1

    def op(self, code, inputs, outputs, opt_type=0, options=None):
        if code not in self.codes:
            self.codes.append(code)
        self.ops.append(Tab([("I", self.codes.index(code)), Vec(np.int32, inputs), Vec(np.int32, outputs),
                             ("B", opt_type) if options is not None else None, options]))

    def finish(self, inputs, outputs) -> bytes:
        sub = Tab([Vec("tables", self.tensors), Vec(np.int32, inputs), Vec(np.int32, outputs), Vec("tables", self.ops), "main"])
        codes = [Tab([("b", c if c < 127 else 127), None, ("i", 1), ("i", c)]) for c in self.codes]
        return build(Tab([("I", 3), Vec("tables", codes), Vec("tables", [sub]), "written by a test", Vec("tables", self.buffers)]))


def test_cnn_float_model(tmp_path):
    rng = np.random.default_rng(0)
    w_conv = rng.standard_normal((8, 3, 3, 3)).astype(np.float32) * 0.3       # [O, kh, kw, I]
    b_conv = rng.standard_normal(8).astype(np.float32)
    w_dw = rng.standard_normal((1, 3, 3, 8)).astype(np.float32) * 0.3         # depth multiplier 1
    w_fc = rng.standard_normal((5, 8)).astype(np.float32)
    b_fc = rng.standard_normal(5).astype(np.float32)
    b = TfliteBuilder()
    x = b.tensor("input", [1, 12, 12, 3])
    t_wc, t_bc = b.tensor("conv/w", list(w_conv.shape), data=w_conv), b.tensor("conv/b", [8], data=b_conv)
    c1 = b.tensor("conv", [1, 6, 6, 8])
    b.op(3, [x, t_wc, t_bc], [c1], 1, Tab([("b", 0), ("i", 2), ("i", 2), ("b", 1)]))                  # CONV_2D, SAME, stride 2, fused RELU
    t_wd = b.tensor("dw/w", list(w_dw.shape), data=w_dw)
    d1 = b.tensor("dw", [1, 4, 4, 8])
    b.op(4, [c1, t_wd, -1], [d1], 2, Tab([("b", 1), ("i", 1), ("i", 1), ("i", 1), ("b", 3)]))            # DEPTHWISE, VALID, RELU6
    p1 = b.tensor("pool", [1, 2, 2, 8])
    b.op(17, [d1], [p1], 5, Tab([("b", 1), ("i", 2), ("i", 2), ("i", 2), ("i", 2), ("b", 0)]))           # MAX_POOL 2x2
    axes = b.tensor("axes", [2], I32, np.array([1, 2], np.int32))
    m1 = b.tensor("mean", [1, 8])
    b.op(40, [p1, axes], [m1], 27, Tab([("b", 0)]))                                                      # MEAN over H, W
    t_wf, t_bf = b.tensor("fc/w", [5, 8], data=w_fc), b.tensor("fc/b", [5], data=b_fc)
    f1 = b.tensor("fc", [1, 5])
    b.op(9, [m1, t_wf, t_bf], [f1], 8, Tab([("b", 0)]))                                                  # FULLY_CONNECTED
    s1 = b.tensor("prob", [1, 5])
    b.op(25, [f1], [s1], 9, Tab([("f", 1.0)]))                                                           # SOFTMAX
    path = tmp_path / "cnn.tflite"
    path.write_bytes(b.finish([x], [s1]))

    m = ov.Core().read_model(str(path))
    assert [p.get_friendly_name() for p in m.get_parameters()] == ["input"] and list(m.output(0).get_shape()) == [1, 5]
    xin = rng.standard_normal((1, 12, 12, 3)).astype(np.float32)
    got = ov.compile_model(m, "CPU")([xin])[0]

    t = torch.from_numpy(xin).permute(0, 3, 1, 2)
    t = torch.nn.functional.pad(t, [0, 1, 0, 1])                                                        # SAME with stride 2: the extra cell goes after
    t = torch.relu(torch.nn.functional.conv2d(t, torch.from_numpy(w_conv).permute(0, 3, 1, 2), torch.from_numpy(b_conv), stride=2))
    t = torch.nn.functional.conv2d(t, torch.from_numpy(w_dw).permute(3, 0, 1, 2), None, groups=8).clamp(0, 6)
    t = torch.nn.functional.max_pool2d(t, 2).mean((2, 3))
    want = torch.softmax(t @ torch.from_numpy(w_fc).t() + torch.from_numpy(b_fc), -1).numpy()
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)


def test_quantised_and_fp16_constants_are_dequantised():
    rng = np.random.default_rng(1)
    wq = rng.integers(-127, 127, (4, 6), dtype=np.int8)
    scale = rng.uniform(0.01, 0.05, 4).astype(np.float32)                     # per output channel (axis 0)
    bias16 = rng.standard_normal(4).astype(np.float16)
    b = TfliteBuilder()
    x = b.tensor("x", [2, 6])
    w = b.tensor("w", [4, 6], I8, wq, quant=(scale, np.zeros(4, np.int64), 0))
    bh = b.tensor("bias_f16", [4], F16, bias16)
    bf = b.tensor("bias", [4])
    b.op(6, [bh], [bf])                                                        # DEQUANTIZE fp16 -> fp32
    y = b.tensor("y", [2, 4])
    b.op(9, [x, w, bf], [y], 8, Tab([("b", 4)]))                               # FULLY_CONNECTED + fused TANH
    z = b.tensor("z", [2, 4])
    two = b.tensor("two", [1], data=np.array([2.0], np.float32))
    b.op(18, [y, two], [z], 21, Tab([("b", 0)]))                               # MUL
    m = ov.convert_model(b.finish([x], [z]))
    xin = rng.standard_normal((2, 6)).astype(np.float32)
    got = ov.compile_model(m, "CPU")([xin])[0]
    want = np.tanh(xin @ (wq.astype(np.float32) * scale[:, None]).T + bias16.astype(np.float32)) * 2
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-5)


def test_unsupported_operator_is_named():
    b = TfliteBuilder()
    x = b.tensor("x", [1, 4])
    y = b.tensor("y", [1, 4])
    b.op(44, [x], [y])                                                         # UNIDIRECTIONAL_SEQUENCE_LSTM: a code without a translator
    try:
        ov.convert_model(b.finish([x], [y]))
    except RuntimeError as e:
        assert "44" in str(e)
    else:
        raise AssertionError("expected an error")
