"""TorchScript decoder and the torch.compile backend (CPU device)."""
import numpy as np
import pytest
import torch

import openvino_b200 as ov


class _Cnn(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.c = torch.nn.Conv2d(3, 8, 3, padding=1)
        self.bn = torch.nn.BatchNorm2d(8)
        self.fc = torch.nn.Linear(8, 5)

    def forward(self, x):
        y = torch.relu(self.bn(self.c(x)))
        y = torch.nn.functional.max_pool2d(y, 2)
        y = y.mean((2, 3))
        return torch.softmax(self.fc(y), -1) * 2 + y.size(0)


def test_traced_module_converts_through_the_torchscript_decoder():
    torch.manual_seed(0)
    net = _Cnn().eval()
    x = torch.randn(2, 3, 8, 8)
    traced = torch.jit.trace(net, (x,))
    m = ov.convert_model(traced, example_input=(x,))
    types = {n.get_type_name() for n in m.get_ops()}
    assert "Convolution" in types and "MaxPool" in types
    out = ov.compile_model(m, "CPU")([x.numpy()])[0]
    assert np.abs(out - net(x).detach().numpy()).max() < 1e-5


def test_scripted_module_with_static_branch_lists_and_two_outputs():
    class S(torch.nn.Module):
        def forward(self, x, y):
            z = x @ y.transpose(0, 1)
            if z.shape[0] > 1:
                z = z + 1
            parts = torch.chunk(z, 2, dim=1)
            return parts[0] - parts[1], z.reshape(-1, 2)
    s = torch.jit.script(S())
    a, b = torch.randn(4, 6), torch.randn(8, 6)
    m = ov.convert_model(s, example_input=(a, b))
    got = ov.compile_model(m, "CPU")([a.numpy(), b.numpy()])
    want = s(a, b)
    for i in range(2):
        assert np.abs(got[i] - want[i].numpy()).max() < 1e-5


def test_script_function_and_dynamic_batch():
    @torch.jit.script
    def f(x: torch.Tensor):
        return torch.tanh(x) * x.size(0)
    m = ov.convert_model(f, input=[[-1, 4]])
    assert m.input(0).get_partial_shape().is_dynamic
    c = ov.compile_model(m, "CPU")
    for n in (2, 5):
        x = torch.randn(n, 4)
        assert np.abs(c([x.numpy()])[0] - f(x).numpy()).max() < 1e-5


class _Mlp(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1, self.fc2, self.ln = torch.nn.Linear(16, 32), torch.nn.Linear(32, 4), torch.nn.LayerNorm(32)

    def forward(self, x):
        h = torch.nn.functional.gelu(self.ln(self.fc1(x)))
        return torch.softmax(self.fc2(h), -1), h.sum()


def test_torch_compile_backend_runs_partitions_on_the_device():
    import openvino_b200.torch  # noqa: F401 - registers the backend
    torch.manual_seed(0)
    net = _Mlp().eval()
    c = torch.compile(net, backend="openvino_b200", options={"device": "CPU"})
    for n in (5, 9):                    # a new batch size recompiles
        x = torch.randn(n, 16)
        with torch.no_grad():
            a, b = c(x)
            ra, rb = net(x)
        assert (a - ra).abs().max() < 1e-5 and (b - rb).abs() < 1e-4
    torch._dynamo.reset()


def test_backend_partitions_around_an_operator_without_a_translator():
    from openvino_b200.frontend import torchdynamo

    def f(x, w):
        h = torch.relu(x @ w)
        h = torch.special.bessel_j0(h)          # no translator: stays in eager mode between two compiled partitions
        return torch.tanh(h) + 1

    x, w = torch.randn(3, 8), torch.randn(8, 8)
    gm = torch.fx.symbolic_trace(f)
    run = torchdynamo.compile_fx(gm, [x, w], {"device": "CPU"})
    assert run._ovb_partitions == 2
    assert (run(x, w) - f(x, w)).abs().max() < 1e-5
    parts = [m.partition for _, m in run._ovb_graph.named_children() if hasattr(m, "partition")]
    assert parts and all(not p.fallback and p.cache for p in parts)
