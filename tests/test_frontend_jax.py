"""JAX frontend on jaxprs built from small stand-in classes (the ``jax`` package is not needed to decode a jaxpr: only
its structure is used). The stand-ins carry exactly the attributes the decoder reads."""
from types import SimpleNamespace as NS

import numpy as np
import torch

import openvino_b200 as ov
from openvino_b200.frontend import jax as fe


def var(shape, dtype="float32"):
    return NS(aval=NS(shape=tuple(shape), dtype=np.dtype(dtype)))


def lit(value, dtype="float32"):
    return NS(val=np.asarray(value, dtype=dtype), aval=NS(shape=(), dtype=np.dtype(dtype)))


def eqn(prim, invars, outvars, **params):
    return NS(primitive=NS(name=prim), invars=list(invars), outvars=list(outvars), params=params)


def closed(invars, constvars, consts, eqns, outvars):
    return NS(jaxpr=NS(invars=invars, constvars=constvars, eqns=eqns, outvars=outvars), consts=consts)


def test_mlp_with_layer_norm_and_inlined_call():
    rng = np.random.default_rng(0)
    w1, b1 = rng.standard_normal((16, 32)).astype(np.float32), rng.standard_normal(32).astype(np.float32)
    x, cw1, cb1 = var([4, 16]), var([16, 32]), var([32])
    h0, bb, h1 = var([4, 32]), var([4, 32]), var([4, 32])
    # inner jaxpr (what pjit wraps): gelu-like x * logistic(1.702 x)
    ix, it, isg, io = var([4, 32]), var([4, 32]), var([4, 32]), var([4, 32])
    inner = closed([ix], [], [], [eqn("mul", [ix, lit(1.702)], [it]), eqn("logistic", [it], [isg]), eqn("mul", [ix, isg], [io])], [io])
    act = var([4, 32])
    mean, cent, sq, varr, inv, normed = var([4]), var([4, 32]), var([4, 32]), var([4]), var([4]), var([4, 32])
    meanb, invb = var([4, 32]), var([4, 32])
    out = var([4])
    eqns = [
        eqn("dot_general", [x, cw1], [h0], dimension_numbers=(((1,), (0,)), ((), ())), precision=None, preferred_element_type=None),
        eqn("broadcast_in_dim", [cb1], [bb], shape=(4, 32), broadcast_dimensions=(1,)),
        eqn("add", [h0, bb], [h1]),
        eqn("pjit", [h1], [act], jaxpr=inner, name="quick_gelu"),
        eqn("reduce_sum", [act], [mean], axes=(1,)),
        eqn("broadcast_in_dim", [mean], [meanb], shape=(4, 32), broadcast_dimensions=(0,)),
        eqn("sub", [act, NS(val=np.float32(0.0), aval=NS(shape=(), dtype=np.dtype("float32")))], [cent]),
        eqn("integer_pow", [cent], [sq], y=2),
        eqn("reduce_max", [sq], [varr], axes=(1,)),
        eqn("rsqrt", [varr], [inv]),
        eqn("broadcast_in_dim", [inv], [invb], shape=(4, 32), broadcast_dimensions=(0,)),
        eqn("mul", [cent, invb], [normed]),
        eqn("argmax", [normed], [out], axes=(1,), index_dtype=np.dtype("int32")),
    ]
    m = fe.convert(closed([x], [cw1, cb1], [w1, b1], eqns, [normed, out, meanb]))
    xin = rng.standard_normal((4, 16)).astype(np.float32)
    res = ov.compile_model(m, "CPU")([xin])
    h = torch.from_numpy(xin) @ torch.from_numpy(w1) + torch.from_numpy(b1)
    a = h * torch.sigmoid(1.702 * h)
    want = a * torch.rsqrt((a * a).amax(1, keepdim=True))
    np.testing.assert_allclose(res[0], want.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_array_equal(res[1], want.argmax(1).numpy())
    np.testing.assert_allclose(res[2], a.sum(1, keepdim=True).expand(4, 32).numpy(), rtol=1e-4, atol=1e-4)


def test_nhwc_convolution_dimension_numbers():
    rng = np.random.default_rng(1)
    w = rng.standard_normal((3, 3, 4, 6)).astype(np.float32) * 0.2             # HWIO
    x, cw, y, r = var([2, 8, 8, 4]), var([3, 3, 4, 6]), var([2, 4, 4, 6]), var([2, 4, 4, 6])
    dn = NS(lhs_spec=(0, 3, 1, 2), rhs_spec=(3, 2, 0, 1), out_spec=(0, 3, 1, 2))
    eqns = [eqn("conv_general_dilated", [x, cw], [y], dimension_numbers=dn, window_strides=(2, 2), padding=((1, 1), (1, 1)), lhs_dilation=(1, 1),
                rhs_dilation=(1, 1), feature_group_count=1, batch_group_count=1),
            eqn("max", [y, lit(0.0)], [r])]
    m = fe.convert(closed([x], [cw], [w], eqns, [r]))
    xin = rng.standard_normal((2, 8, 8, 4)).astype(np.float32)
    got = ov.compile_model(m, "CPU")([xin])[0]
    ref = torch.nn.functional.conv2d(torch.from_numpy(xin).permute(0, 3, 1, 2), torch.from_numpy(w).permute(3, 2, 0, 1), None, 2, 1)
    np.testing.assert_allclose(got, torch.relu(ref).permute(0, 2, 3, 1).numpy(), rtol=1e-4, atol=1e-5)


def test_unsupported_primitive_is_named():
    x, y = var([2]), var([2])
    try:
        fe.convert(closed([x], [], [], [eqn("strange_primitive", [x], [y])], [y]))
    except RuntimeError as e:
        assert "strange_primitive" in str(e)
    else:
        raise AssertionError("expected an error")
