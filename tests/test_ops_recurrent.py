"""Recurrent-state operations (selective SSM, gated delta rule, paged forms, paged causal conv, KV reorder, AUGRU) against
PyTorch restatements of their specifications."""
import numpy as np
import pytest
import torch

import openvino_b200 as ov
from openvino_b200 import opset as ops


def run(outputs, params, feeds):
    m = ov.Model(outputs, params, "t")
    xml, weights = ov._ovcore.serialize(m._m)
    back = ov.Model._wrap(ov._ovcore.deserialize(xml.decode(), np.frombuffer(weights, dtype=np.uint8)))
    res = ov.compile_model(back, "CPU")(feeds)
    return [res[i] for i in range(len(outputs))]


def torch_ssm(A, dt, B, x, C, state):
    b, L, H, P = x.shape
    G = B.shape[2]
    B = B.repeat_interleave(H // G, dim=2)
    C = C.repeat_interleave(H // G, dim=2)
    dA = torch.exp(A * dt).reshape(b, L, H, 1, 1)
    dBx = (dt.reshape(b, L, H, 1) * B).reshape(b, L, H, 1, -1) * x.reshape(b, L, H, P, 1)
    out = torch.zeros(b, L, H, P)
    for t in range(L):
        state = state * dA[:, t] + dBx[:, t]
        out[:, t] = (state * C[:, t].reshape(b, H, 1, -1)).sum(-1)
    return out, state


def torch_gdn(q, k, v, state, g, beta, norm=False, eps=1e-6):
    # q, k: [b, L, Hq, Dk]; v: [b, L, Hv, Dv]; state: [b, Hv, Dk, Dv]
    if norm:
        q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + eps)
        k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + eps)
    groups = v.shape[2] // q.shape[2]
    q = q.repeat_interleave(groups, dim=2) / q.shape[-1] ** 0.5
    k = k.repeat_interleave(groups, dim=2)
    out = torch.zeros_like(v)
    for i in range(q.shape[1]):
        state = state * g[:, i].exp()[..., None, None]
        mem = (state * k[:, i].unsqueeze(-1)).sum(-2)
        delta = (v[:, i] - mem) * beta[:, i].unsqueeze(-1)
        state = state + k[:, i].unsqueeze(-1) * delta.unsqueeze(-2)
        out[:, i] = (state * q[:, i].unsqueeze(-1)).sum(-2)
    return out, state


def P(shape, name, dt="f32"):
    return ops.parameter(list(shape), dt, name)


def test_selective_ssm_and_gated_delta_net_dense():
    torch.manual_seed(0)
    b, L, H, Pd, G, S = 2, 5, 4, 3, 2, 6
    A = -torch.rand(H)
    dt, B, x, C, st = torch.rand(b, L, H), torch.randn(b, L, G, S), torch.randn(b, L, H, Pd), torch.randn(b, L, G, S), torch.randn(b, H, Pd, S)
    ps = [P(t.shape, "i%d" % i) for i, t in enumerate((A, dt, B, x, C, st))]
    n = ops.selective_ssm(*ps)
    assert list(n.get_output_shape(0)) == [b, L, H, Pd] and list(n.get_output_shape(1)) == [b, H, Pd, S]
    y, s2 = run([n.output(0), n.output(1)], ps, [t.numpy() for t in (A, dt, B, x, C, st)])
    ry, rs = torch_ssm(A, dt, B, x, C, st)
    np.testing.assert_allclose(y, ry.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(s2, rs.numpy(), rtol=1e-4, atol=1e-5)

    Hq, Hv, Dk, Dv = 2, 4, 8, 5
    q, k, v = torch.randn(b, L, Hq, Dk), torch.randn(b, L, Hq, Dk), torch.randn(b, L, Hv, Dv)
    st, g, beta = torch.randn(b, Hv, Dk, Dv) * 0.1, -torch.rand(b, L, Hv), torch.rand(b, L, Hv)
    for norm in (False, True):
        ps = [P(t.shape, "g%d" % i) for i, t in enumerate((q, k, v, st, g, beta))]
        n = ops.gated_delta_net(*ps, fuse_qk_l2norm=norm)
        y, s2 = run([n.output(0), n.output(1)], ps, [t.numpy() for t in (q, k, v, st, g, beta)])
        ry, rs = torch_gdn(q, k, v, st, g, beta, norm)
        np.testing.assert_allclose(y, ry.numpy(), rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(s2, rs.numpy(), rtol=1e-4, atol=1e-5)


def test_paged_forms_follow_the_dense_ones_and_cache_snapshots():
    torch.manual_seed(1)
    # two sequences in one token batch: 5 new tokens after 3 processed (interval 4), and 2 new tokens without caching
    lens, past, interval = [5, 2], [3, 0], [4, 0]
    begins = np.array([0, 5, 7], np.int32)
    # sequence 0: (3 % 4 + 5) / 4 -> 2 writes: read slot 0 = block 2, write blocks 2 (in place, after 1 token) and 4 (after 5); sequence 1: read 1, write 1
    blocks = np.array([2, 2, 4, 1, 1], np.int32)
    bbeg = np.array([0, 3, 5], np.int32)
    T, Hq, Hv, Dk, Dv = 7, 2, 4, 6, 3
    q, k, v = torch.randn(T, Hq, Dk), torch.randn(T, Hq, Dk), torch.randn(T, Hv, Dv)
    g, beta = -torch.rand(T, Hv), torch.rand(T, Hv)
    table = torch.randn(5, Hv, Dv, Dk) * 0.1
    tab_np = table.numpy().copy()
    ps = [P(q.shape, "q"), P(k.shape, "k"), P(v.shape, "v"), P(table.shape, "tab"), P(g.shape, "g"), P(beta.shape, "b"),
          P([3], "sb", "i32"), P([5], "bi", "i32"), P([3], "bb", "i32"), P([2], "pt", "i32"), P([2], "ci", "i32")]
    n = ops.paged_gated_delta_net(*ps, use_qk_l2norm=True)
    feeds = [q.numpy(), k.numpy(), v.numpy(), tab_np, g.numpy(), beta.numpy(), begins, blocks, bbeg, np.array(past, np.int32), np.array(interval, np.int32)]
    y = run([n.output(0)], ps, feeds)[0]
    # dense restatement per sequence; the paged state is [Dv, Dk]
    ref0, s_mid = torch_gdn(q[None, 0:1], k[None, 0:1], v[None, 0:1], table[2].transpose(-1, -2)[None], g[None, 0:1], beta[None, 0:1], True)
    ref0b, s_end = torch_gdn(q[None, 1:5], k[None, 1:5], v[None, 1:5], s_mid, g[None, 1:5], beta[None, 1:5], True)
    ref1, s1 = torch_gdn(q[None, 5:7], k[None, 5:7], v[None, 5:7], table[1].transpose(-1, -2)[None], g[None, 5:7], beta[None, 5:7], True)
    np.testing.assert_allclose(y[0:1], ref0[0].numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(y[1:5], ref0b[0].numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(y[5:7], ref1[0].numpy(), rtol=1e-4, atol=1e-5)
    # the host device updates the caller's table in place
    np.testing.assert_allclose(tab_np[2], s_mid[0].transpose(-1, -2).numpy(), rtol=1e-4, atol=1e-5)      # snapshot at the interval boundary
    np.testing.assert_allclose(tab_np[4], s_end[0].transpose(-1, -2).numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(tab_np[1], s1[0].transpose(-1, -2).numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_array_equal(tab_np[0], table.numpy()[0])

    # selective SSM, paged: one sequence, decode step after 6 tokens with interval 3 (6 % 3 == 0: read block 0, write block 3)
    H, Pd, G, S = 4, 3, 2, 5
    A = -torch.rand(H)
    dt, B, x, C = torch.rand(1, H), torch.randn(1, G, S), torch.randn(1, H, Pd), torch.randn(1, G, S)
    tab = torch.randn(4, H, Pd, S)
    tab_np = tab.numpy().copy()
    ps = [P([H], "A"), P(dt.shape, "dt"), P(B.shape, "B"), P(x.shape, "x"), P(C.shape, "C"), P(tab.shape, "t"),
          P([2], "sb", "i64"), P([2], "bi", "i64"), P([2], "bb", "i64"), P([1], "pt", "i64"), P([1], "ci", "i64")]
    n = ops.paged_selective_ssm(*ps)
    y = run([n.output(0)], ps, [A.numpy(), dt.numpy(), B.numpy(), x.numpy(), C.numpy(), tab_np, np.array([0, 1]), np.array([0, 3]), np.array([0, 2]), np.array([6]), np.array([3])])[0]
    ry, rs = torch_ssm(A, dt[None], B[None], x[None], C[None], tab[0][None])
    np.testing.assert_allclose(y, ry[0].numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(tab_np[3], rs[0].numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_array_equal(tab_np[0], tab.numpy()[0])


def test_paged_causal_conv1d_matches_conv1d():
    torch.manual_seed(2)
    Hd, Kk, T = 6, 4, 5
    x = torch.randn(T, Hd)
    w = torch.randn(Hd, 2, Kk)                       # 3 groups of 2 channels
    bias = torch.randn(Hd)
    table = torch.zeros(2, Hd, Kk)
    ps = [P(x.shape, "x"), P(table.shape, "t"), P(w.shape, "w"), P(bias.shape, "b"), P([2], "sb", "i32"), P([2], "bi", "i32"), P([2], "bb", "i32"), P([1], "pt", "i32"), P([1], "ci", "i32")]
    n = ops.paged_causal_conv1d(*ps)
    tab_np = table.numpy().copy()
    y = run([n.output(0)], ps, [x.numpy(), tab_np, w.numpy(), bias.numpy(), np.array([0, T], np.int32), np.array([1, 1], np.int32), np.array([0, 2], np.int32),
                                np.array([0], np.int32), np.array([0], np.int32)])[0]
    # a zero state is left padding of Kk - 1 zeros (the oldest slot is shifted out before the first product)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(x.t()[None], (Kk - 1, 0)), w, bias, groups=3)[0].t()
    np.testing.assert_allclose(y, ref.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(tab_np[1], x[-Kk:].t().numpy(), rtol=1e-6)           # the window of the last Kk tokens


def test_pa_kv_reorder_moves_rows():
    rng = np.random.default_rng(3)
    kc = rng.standard_normal((4, 2, 4, 8)).astype(np.float32)        # [blocks, heads, block_size, head_size]
    vc = rng.standard_normal((4, 2, 4, 8)).astype(np.float32)
    k0, v0 = kc.copy(), vc.copy()
    ps = [P(kc.shape, "k"), P(vc.shape, "v"), P([3], "bi", "i32"), P([2], "bb", "i32"), P([4], "u", "i32"), P([2], "ub", "i32")]
    n = ops.pa_kv_reorder(*ps)
    # one sequence over blocks [3, 0, 2]: token 5 (block 0, row 1) -> token 2 (block 3, row 2); token 9 (block 2, row 1) -> token 4 (block 0, row 0)
    out = run([n.output(0)], ps, [kc, vc, np.array([3, 0, 2], np.int32), np.array([0, 3], np.int32), np.array([5, 2, 9, 4], np.int32), np.array([0, 2], np.int32)])[0]
    assert out.dtype == np.uint8
    np.testing.assert_array_equal(kc[3, :, 2], k0[0, :, 1])
    np.testing.assert_array_equal(vc[0, :, 0], v0[2, :, 1])
    untouched = np.ones(kc.shape, bool)
    untouched[3, :, 2] = False
    untouched[0, :, 0] = False
    np.testing.assert_array_equal(kc[untouched], k0[untouched])


def test_augru_cell_and_sequence():
    torch.manual_seed(4)
    B, S, I, H = 3, 4, 5, 6
    x, h0 = torch.randn(B, S, I), torch.randn(B, H)
    W, R, b = torch.randn(3 * H, I) * 0.3, torch.randn(3 * H, H) * 0.3, torch.randn(3 * H) * 0.1
    a = torch.rand(B, S, 1)

    def step(xt, h, at):
        z = torch.sigmoid(xt @ W[:H].t() + h @ R[:H].t() + b[:H])
        r = torch.sigmoid(xt @ W[H:2 * H].t() + h @ R[H:2 * H].t() + b[H:2 * H])
        hh = torch.tanh(xt @ W[2 * H:].t() + (r * h) @ R[2 * H:].t() + b[2 * H:])
        zz = (1 - at) * z
        return (1 - zz) * hh + zz * h
    ps = [P([B, I], "x"), P([B, H], "h"), P(W.shape, "W"), P(R.shape, "R"), P(b.shape, "b"), P([B, 1], "a")]
    n = ops.augru_cell(*ps, hidden_size=H)
    got = run([n.output(0)], ps, [x[:, 0].numpy(), h0.numpy(), W.numpy(), R.numpy(), b.numpy(), a[:, 0].numpy()])[0]
    np.testing.assert_allclose(got, step(x[:, 0], h0, a[:, 0]).numpy(), rtol=1e-4, atol=1e-5)
    lens = np.array([4, 2, 3], np.int32)
    ps = [P([B, S, I], "x"), P([B, 1, H], "h"), P([B], "l", "i32"), P([1, 3 * H, I], "W"), P([1, 3 * H, H], "R"), P([1, 3 * H], "b"), P([B, S, 1], "a")]
    n = ops.augru_sequence(*ps, hidden_size=H)
    y, hn = run([n.output(0), n.output(1)], ps, [x.numpy(), h0[:, None].numpy(), lens, W[None].numpy(), R[None].numpy(), b[None].numpy(), a.numpy()])
    assert y.shape == (B, 1, S, H) and hn.shape == (B, 1, H)
    for bi in range(B):
        h = h0[bi:bi + 1]
        for t in range(int(lens[bi])):
            h = step(x[bi:bi + 1, t], h, a[bi:bi + 1, t])
            np.testing.assert_allclose(y[bi, 0, t], h[0].numpy(), rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(hn[bi, 0], h[0].numpy(), rtol=1e-4, atol=1e-5)
        assert (y[bi, 0, int(lens[bi]):] == 0).all()


def _pa(feeds, Hk, S):
    """A PagedAttentionExtension node over Parameters for every given input (28 inputs, absent ones are empty constants)."""
    from openvino_b200._graph import make_op
    types = {np.dtype("float32"): "f32", np.dtype("int32"): "i32", np.dtype("uint8"): "u8"}
    ps, ins = [], []
    for i, f in enumerate(feeds):
        p = ops.parameter(list(f.shape), types[f.dtype], "in%d" % i)
        ps.append(p)
        ins.append(p)
    n = make_op("PagedAttentionExtension", ins, {}, version="extension")
    n.get_rt_info()["num_k_heads"] = Hk
    return n, ps


def test_paged_attention_scores_and_key_rerotation():
    rng = np.random.default_rng(11)
    Hq, Hk, S, bs = 2, 1, 8, 4
    past, new = 5, 3
    T = new
    q = rng.standard_normal((T, Hq * S)).astype(np.float32)
    k = rng.standard_normal((T, Hk * S)).astype(np.float32)
    v = rng.standard_normal((T, Hk * S)).astype(np.float32)
    kc = rng.standard_normal((4, Hk, bs, S)).astype(np.float32)
    vc = rng.standard_normal((4, Hk, bs, S)).astype(np.float32)
    blocks = np.array([2, 0], np.int32)                       # logical block 0 -> physical 2, block 1 -> physical 0
    e_f, e_i = np.zeros((0,), np.float32), np.zeros((0,), np.int32)
    # table of (cos | sin) rows; row 1 turns every pair by 0.3 rad
    half = S // 2
    lut = np.stack([np.concatenate([np.ones(half), np.zeros(half)]), np.concatenate([np.full(half, np.cos(0.3)), np.full(half, np.sin(0.3))])]).astype(np.float32)

    def feeds(score_win, rot):
        f = [q, k, v, kc.copy(), vc.copy(), np.array([past], np.int32), np.array([0, new], np.int32), blocks, np.array([0, 2], np.int32),
             np.array(1.0 / np.sqrt(S), np.float32), np.array(0, np.int32), e_f, np.array(past + new, np.int32),
             np.array(score_win, np.int32)]
        f += ([np.array([2], np.int32), np.array([1], np.int32), lut] if rot else [e_i, e_i, e_f])
        f += [e_f, np.array(0, np.int32), np.array(0, np.int32), e_f, e_i, e_i, e_i, e_i, e_i, np.zeros((0,), np.uint8), e_i]
        return f

    def reference(score_win, rot):
        kfull = np.concatenate([kc[2, 0], kc[0, 0]])[:past + new].copy()
        vfull = np.concatenate([vc[2, 0], vc[0, 0]])[:past + new].copy()
        kfull[past:], vfull[past:] = k, v
        out = np.zeros((T, Hq * S), np.float32)
        scores = np.zeros(past + new, np.float32)
        for i in range(new):
            qpos = past + i
            keys = kfull[:qpos + 1].copy()
            if rot:                                            # cached keys of physical block 2 (positions 0..3) are turned
                x0, x1 = keys[:4, :half].copy(), keys[:4, half:].copy()
                keys[:4, :half] = x0 * np.cos(0.3) - x1 * np.sin(0.3)
                keys[:4, half:] = x0 * np.sin(0.3) + x1 * np.cos(0.3)
            for h in range(Hq):
                logit = keys @ q[i, h * S:(h + 1) * S] / np.sqrt(S)
                w = np.exp(logit - logit.max())
                w /= w.sum()
                out[i, h * S:(h + 1) * S] = w @ vfull[:qpos + 1]
                if score_win != 0 and (score_win < 0 or new - i <= score_win):
                    scores[:qpos + 1] += w
        return out, scores
    for score_win, rot in ((2, False), (-1, True), (0, False)):
        f = feeds(score_win, rot)
        node, ps = _pa(f, Hk, S)
        m = ov.Model([node.output(0), node.output(1)], ps, "pa")
        res = ov.compile_model(m, "CPU")(f)
        ro, rs = reference(score_win, rot)
        np.testing.assert_allclose(res[0], ro, rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(res[1], rs, rtol=1e-4, atol=1e-5)
        assert res[1].shape == (past + new,)
        if score_win == 2:
            assert abs(res[1].sum() - 2 * Hq) < 1e-4           # two voting queries, every head's weights sum to one


@pytest.mark.gpu
def test_recurrent_device_kernels_match_the_restatements():
    """SelectiveSSM and GatedDeltaNet on the CUDA device run the register-resident scan kernels (csrc/cuda/recurrent.cu);
    sizes are those of a Mamba-2 block (state 128) and a gated-delta layer (key width 128), plus ragged ones."""
    from openvino_b200.ops import cuda as K
    torch.manual_seed(5)
    dev = "cuda:0"
    for b, L, H, Pd, G, S in ((2, 33, 8, 64, 2, 128), (1, 7, 3, 5, 1, 40), (1, 4, 2, 3, 2, 200)):
        A = -torch.rand(H)
        dt, B, x, C, st = torch.rand(b, L, H) * 0.5, torch.randn(b, L, G, S), torch.randn(b, L, H, Pd), torch.randn(b, L, G, S), torch.randn(b, H, Pd, S)
        ry, rs = torch_ssm(A, dt, B, x, C, st)
        y, s2 = K.selective_ssm(*(t.to(dev) for t in (A, dt, B, x, C, st)))
        torch.testing.assert_close(y.cpu(), ry, rtol=2e-4, atol=2e-4)
        torch.testing.assert_close(s2.cpu(), rs, rtol=2e-4, atol=2e-4)
        # through the device plugin's graph interpreter
        ps = [P(t.shape, "i%d" % i) for i, t in enumerate((A, dt, B, x, C, st))]
        n = ops.selective_ssm(*ps)
        cm = ov.compile_model(ov.Model([n.output(0), n.output(1)], ps, "ssm"), "CUDA", {"INFERENCE_PRECISION_HINT": "f32"})
        res = cm([t.numpy() for t in (A, dt, B, x, C, st)])
        np.testing.assert_allclose(res[0], ry.numpy(), rtol=2e-4, atol=2e-4)
        np.testing.assert_allclose(res[1], rs.numpy(), rtol=2e-4, atol=2e-4)
    for b, L, Hq, Hv, Dk, Dv in ((2, 19, 4, 8, 128, 128), (1, 6, 2, 4, 24, 5), (1, 3, 1, 2, 160, 9)):
        q, k, v = torch.randn(b, L, Hq, Dk), torch.randn(b, L, Hq, Dk), torch.randn(b, L, Hv, Dv)
        st, g, beta = torch.randn(b, Hv, Dk, Dv) * 0.1, -torch.rand(b, L, Hv), torch.rand(b, L, Hv)
        for norm in (True, False):
            if not norm:
                k = k / Dk ** 0.5            # keeps the un-normalised recurrence bounded
            ry, rs = torch_gdn(q, k, v, st, g, beta, norm)
            ps = [P(t.shape, "g%d" % i) for i, t in enumerate((q, k, v, st, g, beta))]
            n = ops.gated_delta_net(*ps, fuse_qk_l2norm=norm)
            cm = ov.compile_model(ov.Model([n.output(0), n.output(1)], ps, "gdn"), "CUDA", {"INFERENCE_PRECISION_HINT": "f32"})
            res = cm([t.numpy() for t in (q, k, v, st, g, beta)])
            np.testing.assert_allclose(res[0], ry.numpy(), rtol=5e-4, atol=5e-4)
            np.testing.assert_allclose(res[1], rs.numpy(), rtol=5e-4, atol=5e-4)


@pytest.mark.gpu
def test_paged_recurrent_forms_on_the_device_update_the_table_in_place():
    """PagedGatedDeltaNet / PagedSelectiveSSM on the CUDA device: the state table is a device tensor of the caller, the scan
    kernels run per stretch between cache-interval boundaries, snapshots land in the blocks the bookkeeping names."""
    torch.manual_seed(1)
    core = ov.Core()
    rctx = core.get_default_context("CUDA")
    begins = np.array([0, 5, 7], np.int32)
    blocks = np.array([2, 2, 4, 1, 1], np.int32)
    bbeg = np.array([0, 3, 5], np.int32)
    past, interval = np.array([3, 0], np.int32), np.array([4, 0], np.int32)
    T, Hq, Hv, Dk, Dv = 7, 2, 4, 40, 9
    q, k, v = torch.randn(T, Hq, Dk), torch.randn(T, Hq, Dk), torch.randn(T, Hv, Dv)
    g, beta = -torch.rand(T, Hv), torch.rand(T, Hv)
    table = torch.randn(5, Hv, Dv, Dk) * 0.1
    ps = [P(q.shape, "q"), P(k.shape, "k"), P(v.shape, "v"), P(table.shape, "tab"), P(g.shape, "g"), P(beta.shape, "b"),
          P([3], "sb", "i32"), P([5], "bi", "i32"), P([3], "bb", "i32"), P([2], "pt", "i32"), P([2], "ci", "i32")]
    n = ops.paged_gated_delta_net(*ps, use_qk_l2norm=True)
    cm = core.compile_model(ov.Model([n.output(0)], ps, "pgdn"), "CUDA", {"INFERENCE_PRECISION_HINT": "f32"})
    remote = rctx.create_tensor(ov.Type.f32, list(table.shape))
    remote.torch().copy_(table)
    req = cm.create_infer_request()
    for i, a in enumerate([q.numpy(), k.numpy(), v.numpy(), None, g.numpy(), beta.numpy(), begins, blocks, bbeg, past, interval]):
        req.set_input_tensor(i, remote if a is None else ov.Tensor(a))
    req.infer()
    y = req.get_output_tensor(0).data
    ref0, s_mid = torch_gdn(q[None, 0:1], k[None, 0:1], v[None, 0:1], table[2].transpose(-1, -2)[None], g[None, 0:1], beta[None, 0:1], True)
    ref0b, s_end = torch_gdn(q[None, 1:5], k[None, 1:5], v[None, 1:5], s_mid, g[None, 1:5], beta[None, 1:5], True)
    ref1, s1 = torch_gdn(q[None, 5:7], k[None, 5:7], v[None, 5:7], table[1].transpose(-1, -2)[None], g[None, 5:7], beta[None, 5:7], True)
    np.testing.assert_allclose(y, torch.cat([ref0[0], ref0b[0], ref1[0]]).numpy(), rtol=5e-4, atol=5e-5)
    tab = remote.torch().cpu()
    torch.testing.assert_close(tab[2], s_mid[0].transpose(-1, -2), rtol=5e-4, atol=5e-5)
    torch.testing.assert_close(tab[4], s_end[0].transpose(-1, -2), rtol=5e-4, atol=5e-5)
    torch.testing.assert_close(tab[1], s1[0].transpose(-1, -2), rtol=5e-4, atol=5e-5)
    torch.testing.assert_close(tab[0], table[0])

    H, Pd, G, S = 4, 6, 2, 48
    A = -torch.rand(H)
    dt, B, x, C = torch.rand(3, H), torch.randn(3, G, S), torch.randn(3, H, Pd), torch.randn(3, G, S)
    tab0 = torch.randn(4, H, Pd, S)
    ps = [P([H], "A"), P(dt.shape, "dt"), P(B.shape, "B"), P(x.shape, "x"), P(C.shape, "C"), P(tab0.shape, "t"),
          P([2], "sb", "i64"), P([3], "bi", "i64"), P([2], "bb", "i64"), P([1], "pt", "i64"), P([1], "ci", "i64")]
    n = ops.paged_selective_ssm(*ps)
    cm = core.compile_model(ov.Model([n.output(0)], ps, "pssm"), "CUDA", {"INFERENCE_PRECISION_HINT": "f32"})
    remote = rctx.create_tensor(ov.Type.f32, list(tab0.shape))
    remote.torch().copy_(tab0)
    req = cm.create_infer_request()
    # 3 new tokens after 5 processed, interval 3: one token reaches the boundary (block 1), the other two go to block 3
    for i, a in enumerate([A.numpy(), dt.numpy(), B.numpy(), x.numpy(), C.numpy(), None, np.array([0, 3]), np.array([0, 1, 3]), np.array([0, 3]), np.array([5]), np.array([3])]):
        req.set_input_tensor(i, remote if a is None else ov.Tensor(a))
    req.infer()
    y = req.get_output_tensor(0).data
    ry1, rs1 = torch_ssm(A, dt[None, :1], B[None, :1], x[None, :1], C[None, :1], tab0[0][None])
    ry2, rs2 = torch_ssm(A, dt[None, 1:], B[None, 1:], x[None, 1:], C[None, 1:], rs1)
    np.testing.assert_allclose(y, torch.cat([ry1[0], ry2[0]]).numpy(), rtol=5e-4, atol=5e-5)
    tab = remote.torch().cpu()
    torch.testing.assert_close(tab[1], rs1[0], rtol=5e-4, atol=5e-5)
    torch.testing.assert_close(tab[3], rs2[0], rtol=5e-4, atol=5e-5)
    torch.testing.assert_close(tab[2], tab0[2])


@pytest.mark.gpu
def test_paged_causal_conv_and_kv_reorder_on_the_device():
    torch.manual_seed(2)
    core = ov.Core()
    rctx = core.get_default_context("CUDA")

    def remote_of(t):
        r = rctx.create_tensor(ov.Type.f32, list(t.shape))
        r.torch().copy_(t)
        return r
    Hd, Kk, T = 6, 4, 5
    x, w, bias = torch.randn(T, Hd), torch.randn(Hd, 2, Kk), torch.randn(Hd)
    ps = [P(x.shape, "x"), P([3, Hd, Kk], "t"), P(w.shape, "w"), P(bias.shape, "b"), P([2], "sb", "i32"), P([3], "bi", "i32"), P([2], "bb", "i32"), P([1], "pt", "i32"), P([1], "ci", "i32")]
    cm = core.compile_model(ov.Model([ops.paged_causal_conv1d(*ps).output(0)], ps, "pcc"), "CUDA", {"INFERENCE_PRECISION_HINT": "f32"})
    table = remote_of(torch.zeros(3, Hd, Kk))
    req = cm.create_infer_request()
    # 5 tokens after 1 processed with interval 3: two tokens reach the boundary (block 2), the other three go to block 1
    feeds = [x.numpy(), None, w.numpy(), bias.numpy(), np.array([0, T], np.int32), np.array([0, 2, 1], np.int32), np.array([0, 3], np.int32), np.array([1], np.int32), np.array([3], np.int32)]
    for i, a in enumerate(feeds):
        req.set_input_tensor(i, table if a is None else ov.Tensor(a))
    req.infer()
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(x.t()[None], (Kk - 1, 0)), w, bias, groups=3)[0].t()
    np.testing.assert_allclose(req.get_output_tensor(0).data, ref.numpy(), rtol=1e-4, atol=1e-5)
    tab = table.torch().cpu()
    torch.testing.assert_close(tab[1], x[-Kk:].t().contiguous())
    torch.testing.assert_close(tab[2][:, -2:], x[:2].t().contiguous())

    kc, vc = torch.randn(4, 2, 4, 8), torch.randn(4, 2, 4, 8)
    ps = [P(kc.shape, "k"), P(vc.shape, "v"), P([3], "bi", "i32"), P([2], "bb", "i32"), P([4], "u", "i32"), P([2], "ub", "i32")]
    cm = core.compile_model(ov.Model([ops.pa_kv_reorder(*ps).output(0)], ps, "reorder"), "CUDA", {"INFERENCE_PRECISION_HINT": "f32"})
    rk, rv = remote_of(kc), remote_of(vc)
    req = cm.create_infer_request()
    for i, a in enumerate([rk, rv, np.array([3, 0, 2], np.int32), np.array([0, 3], np.int32), np.array([5, 2, 9, 4], np.int32), np.array([0, 2], np.int32)]):
        req.set_input_tensor(i, a if not isinstance(a, np.ndarray) else ov.Tensor(a))
    req.infer()
    k1, v1 = rk.torch().cpu(), rv.torch().cpu()
    torch.testing.assert_close(k1[3, :, 2], kc[0, :, 1])
    torch.testing.assert_close(v1[0, :, 0], vc[2, :, 1])
    assert (k1 != kc).sum() == 2 * 8 * 2 and (v1 != vc).sum() == 2 * 8 * 2
