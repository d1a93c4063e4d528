"""PyTorch frontend: convert -> (save -> read) -> compile on CPU -> equal to eager PyTorch."""
import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import openvino_b200 as ov
from openvino_b200.frontend import pytorch as ptfe
from openvino_b200.models.torch_zoo import ResNet18, bert_tiny


def check(module, inputs, rtol=1e-4, atol=1e-4, **kw):
    module.eval()
    with torch.no_grad():
        want = module(*inputs)
    want = [want] if isinstance(want, torch.Tensor) else list(want)
    m = ov.convert_model(module, example_input=tuple(inputs), **kw)
    got = ov.compile_model(m, "CPU")([t.numpy() for t in inputs])
    assert len(got) == len(want)
    for i, w in enumerate(want):
        np.testing.assert_allclose(got[i], w.numpy(), rtol=rtol, atol=atol)
    return m


def test_resnet18_slice_convert_save_read_infer(tmp_path):
    """The plumbing benchmark configuration at reduced width: convert_model -> save_model -> read_model -> CPU."""
    torch.manual_seed(0)
    net = ResNet18(num_classes=10, width=8).eval()
    x = torch.randn(2, 3, 64, 64)
    m = check(net, [x], rtol=1e-3, atol=1e-3)
    types = [n.get_type_name() for n in m.get_ops()]
    assert types.count("Convolution") == 20 and types.count("BatchNormInference") == 20 and "MaxPool" in types
    ov.save_model(m, str(tmp_path / "resnet.xml"), compress_to_fp16=False)
    r = ov.Core().read_model(str(tmp_path / "resnet.xml"))
    cm = ov.Core().compile_model(r, "CPU")
    with torch.no_grad():
        want = net(x).numpy()
    np.testing.assert_allclose(cm(x.numpy())[0], want, rtol=1e-3, atol=1e-3)
    # the compiled graph has batch norms folded away
    rt_types = [n.get_type_name() for n in cm.runtime_model.get_ops()]
    assert "BatchNormInference" not in rt_types


def test_bert_encoder():
    torch.manual_seed(0)
    net = bert_tiny().eval()
    ids = torch.randint(0, 100, (2, 12))
    mask = torch.ones(2, 12, dtype=torch.int64)
    mask[1, 8:] = 0
    typ = torch.zeros(2, 12, dtype=torch.int64)
    m = check(net, [ids, mask, typ], rtol=1e-3, atol=1e-3)
    assert [p.get_any_name() for p in m.inputs] == ["input_ids", "attention_mask", "token_type_ids"]
    assert "ScaledDotProductAttention" in [n.get_type_name() for n in m.get_ops()]


class Misc(nn.Module):
    def forward(self, x, idx):
        a = x[:, 1:3] * 2
        b = torch.cat([a, x[:, -2:]], 1).permute(1, 0)
        c = torch.where(b > 0, b, torch.zeros_like(b)).sum(0, keepdim=True)
        d = x.index_select(1, idx).clamp(-0.5, 0.5)
        e = torch.stack([d, d.abs()], 0).mean(0)
        f = F.pad(e, (1, 2), value=3.0)
        g, gi = f.max(1)
        return c, f.softmax(-1), g, gi, x.unsqueeze(1).expand(-1, 2, -1).reshape(x.shape[0], -1), torch.arange(4) + 1


def test_misc_ops():
    torch.manual_seed(1)
    check(Misc(), [torch.randn(3, 6), torch.tensor([0, 5, 2])])


class DynamicBatch(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc = nn.Linear(8, 4)

    def forward(self, x):
        b = x.shape[0]
        return self.fc(x).view(b, 2, 2).transpose(1, 2).reshape(b, -1)


def test_dynamic_batch_stays_symbolic():
    net = DynamicBatch().eval()
    m = ov.convert_model(net, example_input=(torch.randn(3, 8),), input=[[-1, 8]])
    assert m.input(0).get_partial_shape().to_string() == "[?,8]"
    cm = ov.compile_model(m, "CPU")
    for b in (1, 5):
        x = torch.randn(b, 8)
        with torch.no_grad():
            np.testing.assert_allclose(cm(x.numpy())[0], net(x).numpy(), rtol=1e-5, atol=1e-5)


def test_unsupported_op_is_reported():
    class Odd(nn.Module):
        def forward(self, x):
            return torch.linalg.svdvals(x)
    with pytest.raises(ptfe.ConversionError, match="no translator"):
        ov.convert_model(Odd(), example_input=(torch.randn(3, 3),))
    assert "aten.conv2d.default" in ptfe.supported_ops()


def test_weights_are_shared_not_copied():
    net = nn.Linear(4, 4, bias=False).eval()
    m = ov.convert_model(net, example_input=(torch.zeros(1, 4),))
    const = [n for n in m.get_ops() if n.get_type_name() == "Constant"][0]
    with torch.no_grad():
        net.weight.fill_(2.0)
    assert (const.get_data() == 2.0).all()
    out = ov.compile_model(m, "CPU")(np.ones((1, 4), np.float32))[0]
    assert (out == 8.0).all()


def test_output_selection():
    net = ResNet18(num_classes=4, width=4).eval()
    m = ov.convert_model(net, example_input=(torch.randn(1, 3, 32, 32),))
    first_relu = [n for n in m.get_ops() if n.get_type_name() == "Relu"][0]
    cut = ov.convert_model(m, output=[first_relu.get_friendly_name()])
    assert cut.get_output_partial_shape(0) == [1, 4, 16, 16] and len(cut.get_ops()) < len(m.get_ops())
