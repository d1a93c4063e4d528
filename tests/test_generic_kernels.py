"""The graph executor's generic primitives (csrc/cuda/generic.cu) against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def G():
    from openvino_b200.ops import cuda as K
    from openvino_b200.ops import generic
    if not K.available():
        raise RuntimeError("libovb_cuda.so is missing: run python -m openvino_b200.build")
    return generic


def _close(y, ref, dtype):
    tol = {torch.float32: 2e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dtype]
    ref = ref.float()
    assert y.shape == ref.shape, (y.shape, ref.shape)
    err = (y.float() - ref).abs().max().item()
    scale = max(ref.abs().max().item(), 1.0)
    assert err <= tol * scale, (err, scale)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_unary(G, dtype):
    torch.manual_seed(0)
    F = torch.nn.functional
    x = (torch.randn(5, 77, 33, device="cuda") * 2).to(dtype)
    xf = x.float()
    refs = {"relu": torch.relu(xf), "sigmoid": torch.sigmoid(xf), "tanh": torch.tanh(xf), "gelu_erf": F.gelu(xf), "gelu_tanh": F.gelu(xf, approximate="tanh"),
            "exp": torch.exp(xf), "abs": xf.abs(), "neg": -xf, "hswish": F.hardswish(xf), "hsigmoid": F.hardsigmoid(xf), "mish": F.mish(xf),
            "softplus": F.softplus(xf), "erf": torch.erf(xf), "floor": xf.floor(), "ceil": xf.ceil(), "sign": xf.sign(), "sin": xf.sin(), "cos": xf.cos(),
            "softsign": F.softsign(xf), "round_even": xf.round()}
    for name, ref in refs.items():
        _close(G.unary(name, x), ref, dtype)
    _close(G.unary("swish", x, 1.5), xf * torch.sigmoid(1.5 * xf), dtype)
    _close(G.unary("clamp", x, -0.5, 1.25), xf.clamp(-0.5, 1.25), dtype)
    _close(G.unary("elu", x, 0.7), F.elu(xf, 0.7), dtype)
    _close(G.unary("scale_shift", x, 0.25, 3.0), xf * 0.25 + 3.0, dtype)
    pos = x.abs() + 0.5
    _close(G.unary("log", pos), pos.float().log(), dtype)
    _close(G.unary("sqrt", pos), pos.float().sqrt(), dtype)
    _close(G.unary("rsqrt", pos), pos.float().rsqrt(), dtype)
    # a non-contiguous view and a length that is not a multiple of the vector width
    v = x[:, ::2, 1:]
    _close(G.unary("relu", v), torch.relu(v.float()), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_binary_broadcast(G, dtype):
    torch.manual_seed(1)
    a = torch.randn(4, 3, 17, 9, device="cuda").to(dtype)
    cases = [torch.randn(4, 3, 17, 9, device="cuda"), torch.randn(9, device="cuda"), torch.randn(1, 3, 1, 1, device="cuda"),
             torch.randn(4, 1, 17, 1, device="cuda"), torch.randn(1, device="cuda"), torch.randn(2, 1, 4, 3, 17, 9, device="cuda")]
    for b in cases:
        b = b.to(dtype)
        af, bf = a.float(), b.float()
        _close(G.binary("add", a, b), af + bf, dtype)
        _close(G.binary("sub", b, a), bf - af, dtype)
        _close(G.binary("mul", a, b), af * bf, dtype)
        _close(G.binary("max", a, b), torch.maximum(af, bf), dtype)
        _close(G.binary("min", a, b), torch.minimum(af, bf), dtype)
        _close(G.binary("sqdiff", a, b), (af - bf) ** 2, dtype)
        _close(G.binary("prelu", a, b), torch.where(af >= 0, af, af * bf), dtype)
    d = a.abs() + 0.5
    _close(G.binary("div", a, d), a.float() / d.float(), dtype)
    _close(G.binary("pow", d, torch.full((1,), 1.5, device="cuda", dtype=dtype)), d.float() ** 1.5, dtype)
    # a transposed operand
    t = torch.randn(9, 17, device="cuda").to(dtype).t()
    _close(G.binary("add", a, t), a.float() + t.float(), dtype)


def test_copies_transpose_concat(G):
    torch.manual_seed(2)
    for dtype in (torch.float32, torch.bfloat16):
        x = torch.randn(3, 5, 70, 45, device="cuda").to(dtype)
        for perm in ([0, 1, 3, 2], [0, 2, 1, 3], [3, 2, 1, 0], [1, 0, 2, 3], [0, 3, 1, 2]):
            assert torch.equal(G.contiguous(x.permute(perm)), x.permute(perm).contiguous())
        assert torch.equal(G.contiguous(x[:, 1:4, ::3, 2:40]), x[:, 1:4, ::3, 2:40].contiguous())
        assert torch.equal(G.contiguous(x[:, :1].expand(3, 4, 70, 45)), x[:, :1].expand(3, 4, 70, 45).contiguous())
        parts = [x, x[:, :2], x[:, 1:2]]
        assert torch.equal(G.concat(parts, 1), torch.cat(parts, 1))
        parts = [x[..., :7], x.permute(0, 1, 2, 3)[..., 10:11], x]
        assert torch.equal(G.concat(parts, -1), torch.cat(parts, -1))
    i8 = torch.randint(0, 255, (4, 6, 10), device="cuda", dtype=torch.uint8)
    out = torch.empty(4, 10, 6, device="cuda", dtype=torch.uint8)
    G.strided_copy(i8.permute(0, 2, 1), out)
    assert torch.equal(out, i8.permute(0, 2, 1).contiguous())


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_softmax(G, dtype):
    torch.manual_seed(3)
    for shape, axis in (((6, 7, 130), -1), ((6, 7, 130), 1), ((4, 5000), 1), ((3, 9000), -1), ((2, 3, 4, 5), 0), ((64, 1), 1)):
        x = (torch.randn(*shape, device="cuda") * 3).to(dtype)
        _close(G.softmax(x, axis), torch.softmax(x.float(), axis), dtype)
        _close(G.softmax(x, axis, log=True), torch.log_softmax(x.float(), axis), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reduce(G, dtype):
    torch.manual_seed(4)
    x = torch.randn(4, 6, 50, 9, device="cuda").to(dtype)
    xf = x.float()
    for axes in ([3], [2, 3], [1], [0, 1], [0, 2], [1, 3], [0, 1, 2, 3]):
        for keep in (False, True):
            _close(G.reduce("sum", x, axes, keep), xf.sum(axes, keepdim=keep), dtype)
            _close(G.reduce("mean", x, axes, keep), xf.mean(axes, keepdim=keep), dtype)
            _close(G.reduce("max", x, axes, keep), xf.amax(axes, keepdim=keep), dtype)
            _close(G.reduce("min", x, axes, keep), xf.amin(axes, keepdim=keep), dtype)
            _close(G.reduce("l1", x, axes, keep), xf.abs().sum(axes, keepdim=keep), dtype)
            _close(G.reduce("l2", x, axes, keep), (xf * xf).sum(axes, keepdim=keep).sqrt(), dtype)
    small = (torch.rand(3, 4, 5, device="cuda") + 0.5).to(dtype)
    _close(G.reduce("prod", small, [1, 2], False), small.float().prod(2).prod(1), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pool2d(G, dtype):
    torch.manual_seed(5)
    F = torch.nn.functional
    x = torch.randn(2, 5, 23, 19, device="cuda").to(dtype)
    xf = x.float()
    for k, s, p in (([3, 3], [2, 2], [1, 1]), ([2, 2], [2, 2], [0, 0]), ([5, 3], [1, 2], [2, 1]), ([3, 3], [1, 1], [0, 0])):
        ref = F.max_pool2d(xf, k, s, p)
        _close(G.pool2d(x, k, s, p, p, [1, 1], ref.shape[2:], True, False), ref, dtype)
        for excl in (True, False):
            ref = F.avg_pool2d(xf, k, s, p, count_include_pad=not excl)
            _close(G.pool2d(x, k, s, p, p, [1, 1], ref.shape[2:], False, excl), ref, dtype)
    # ceil rounding and dilation
    ref = F.max_pool2d(xf, [3, 3], [2, 2], [1, 1], dilation=[2, 2], ceil_mode=True)
    _close(G.pool2d(x, [3, 3], [2, 2], [1, 1], [1, 1], [2, 2], ref.shape[2:], True, False), ref, dtype)
    ref = F.avg_pool2d(xf, [3, 3], [2, 2], [1, 1], ceil_mode=True, count_include_pad=True)
    _close(G.pool2d(x, [3, 3], [2, 2], [1, 1], [1, 1], [1, 1], ref.shape[2:], False, False), ref, dtype)
    # asymmetric padding (only an end pad): reference through an explicit pad
    ref = F.avg_pool2d(F.pad(xf, [0, 1, 0, 1]), [2, 2], [2, 2], count_include_pad=True)
    _close(G.pool2d(x, [2, 2], [2, 2], [0, 0], [1, 1], [1, 1], ref.shape[2:], False, False), ref, dtype)
