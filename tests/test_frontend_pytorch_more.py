"""Second part of the ATen translator table (frontend/pytorch_more.py) and the decomposition fallback of
``from_exported_program``: operations without a translator are rewritten by their ATen decompositions first."""
import warnings

import numpy as np
import pytest
import torch

import openvino_b200 as ov

F = torch.nn.functional

GROUPS = {
    "decomposed": {
        "addcmul": lambda x, y: torch.addcmul(x, x, y, value=0.5),
        "var": lambda x, y: torch.var(x, dim=-1, keepdim=True),
        "std": lambda x, y: torch.std(x, dim=-1),
        "logsumexp": lambda x, y: torch.logsumexp(x, dim=-1),
        "glu": lambda x, y: F.glu(x, -1),
        "outer": lambda x, y: torch.outer(x[0], y[0]),
        "normalize": lambda x, y: F.normalize(x, dim=-1),
        "cosine_similarity": lambda x, y: torch.cosine_similarity(x, y, dim=-1),
        "lerp": lambda x, y: torch.lerp(x, y, 0.3),
        "nan_to_num": lambda x, y: torch.nan_to_num(x / (y - y), nan=1.0, posinf=2.0, neginf=-2.0),
        "roll": lambda x, y: torch.roll(x, 1, 1),
    },
    "elementwise": {
        "selu": lambda x, y: F.selu(x), "relu6": lambda x, y: F.relu6(x * 4), "log1p": lambda x, y: torch.log1p(x.abs()),
        "expm1": lambda x, y: torch.expm1(x), "trunc": lambda x, y: torch.trunc(x * 3), "frac": lambda x, y: torch.frac(x * 3),
        "atan2": lambda x, y: torch.atan2(x, y), "hypot": lambda x, y: torch.hypot(x, y), "cumprod": lambda x, y: torch.cumprod(x, 1),
        "round": lambda x, y: torch.round(x * 10, decimals=1), "log2": lambda x, y: torch.log2(x.abs() + 1), "erfc": lambda x, y: torch.erfc(x),
    },
    "indexing": {
        "flip": lambda x, y: torch.flip(x, [1]), "narrow": lambda x, y: torch.narrow(x, 1, 1, 3), "diagonal": lambda x, y: torch.diagonal(x[:4, :4], 1),
        "sort": lambda x, y: torch.sort(x, -1, descending=True)[0], "argsort": lambda x, y: torch.argsort(x, -1),
        "movedim": lambda x, y: torch.movedim(x.reshape(4, 2, 3), 0, 2), "tile": lambda x, y: torch.tile(x, (2, 1)),
        "one_hot": lambda x, y: F.one_hot(torch.argmax(x, -1), 6), "repeat_interleave": lambda x, y: torch.repeat_interleave(x, 2, dim=1),
        "index_add": lambda x, y: torch.index_add(x, 0, torch.tensor([0, 2, 0]), y[:3]),
        "searchsorted": lambda x, y: torch.searchsorted(torch.sort(x, -1)[0], y),
    },
    "linear_algebra_and_layout": {
        "vector_norm_1": lambda x, y: torch.linalg.vector_norm(x, 1, dim=1), "vector_norm_inf": lambda x, y: torch.linalg.vector_norm(x, float("inf"), dim=0),
        "cross": lambda x, y: torch.cross(x[:, :3], y[:, :3], dim=-1), "dot": lambda x, y: torch.dot(x[0], y[0]), "mv": lambda x, y: torch.mv(x, y[0]),
        "reflection_pad": lambda x, y: F.pad(x.reshape(1, 1, 4, 6), (1, 2, 1, 1), mode="reflect"),
        "replication_pad": lambda x, y: F.pad(x.reshape(1, 1, 4, 6), (2, 1, 0, 1), mode="replicate"),
        "pixel_unshuffle": lambda x, y: F.pixel_unshuffle(x.reshape(1, 1, 4, 6), 2),
        "grid_sample": lambda x, y: F.grid_sample(x.reshape(1, 1, 4, 6), torch.tanh(y.reshape(1, 3, 4, 2)), align_corners=False),
        "prelu": lambda x, y: F.prelu(x.reshape(1, 4, 6), y[:, 0].abs()),
    },
}


@pytest.mark.parametrize("group", sorted(GROUPS))
def test_aten_operations(group):
    fns = GROUPS[group]

    class M(torch.nn.Module):
        def forward(self, a, b):
            return tuple(f(a, b) for f in fns.values())
    torch.manual_seed(0)
    x, y = torch.randn(4, 6), torch.randn(4, 6)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        om = ov.convert_model(M().eval(), example_input=(x, y))
    got = ov.compile_model(om, "CPU")([x.numpy(), y.numpy()])
    ref = M()(x, y)
    for k, (name, r) in enumerate(zip(fns, ref)):
        g = np.asarray(got[k])
        assert g.shape == tuple(r.shape), name
        np.testing.assert_allclose(g.astype(np.float64), r.numpy().astype(np.float64), rtol=1e-4, atol=1e-5, err_msg=name)


def test_an_operation_without_translator_or_decomposition_is_named():
    class M(torch.nn.Module):
        def forward(self, a):
            return torch.linalg.svd(a)[1]
    with pytest.raises(Exception, match="svd"):
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            ov.convert_model(M().eval(), example_input=(torch.randn(4, 4),))
