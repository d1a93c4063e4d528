"""Shape inference, reference evaluation and IR round trip of the extended operation set (csrc/core/ops_ext.cpp),
checked against numpy / PyTorch implementations of the same operations."""
import numpy as np
import pytest
import torch

import openvino_b200 as ov
from openvino_b200 import opset as ops


def run(outputs, params, feeds, tmp_path=None):
    """Evaluate on the host device; when tmp_path is given the model first goes through save -> read."""
    outputs = outputs if isinstance(outputs, (list, tuple)) else [outputs]
    results = []
    for o in outputs:
        results.append(ops.result(o))
    m = ov.Model(results, list(params), "m")
    core = ov.Core()
    if tmp_path is not None:
        ov.serialize(m, str(tmp_path / "m.xml"), str(tmp_path / "m.bin"))
        m2 = core.read_model(str(tmp_path / "m.xml"))
        ov.serialize(m2, str(tmp_path / "n.xml"), str(tmp_path / "n.bin"))
        assert open(tmp_path / "m.xml", "rb").read() == open(tmp_path / "n.xml", "rb").read()
        m = m2
    res = core.compile_model(m, "CPU")(feeds)
    return [res[i] for i in range(len(results))]


def P(shape, dtype="f32", name="x"):
    return ops.parameter(list(shape), dtype, name)


def test_space_to_depth_and_batch_round_trips(tmp_path):
    x = np.arange(2 * 4 * 4 * 6, dtype=np.float32).reshape(2, 4, 4, 6)
    p = P(x.shape)
    t = torch.from_numpy(x)
    (d,) = run(ops.space_to_depth(p, "depth_first", 2), [p], [x], tmp_path)
    assert np.array_equal(d, torch.nn.functional.pixel_unshuffle(t, 2).numpy())
    (bf,) = run(ops.space_to_depth(p, "blocks_first", 2), [p], [x])
    ref = x.reshape(2, 4, 2, 2, 3, 2).transpose(0, 3, 5, 1, 2, 4).reshape(2, 16, 2, 3)
    assert np.array_equal(bf, ref)
    # depth_to_space undoes it
    (back,) = run(ops.depth_to_space(ops.space_to_depth(p, "blocks_first", 2), "blocks_first", 2), [p], [x])
    assert np.array_equal(back, x)
    # space_to_batch followed by batch_to_space with the same blocks and pads is the identity
    blocks, pb, pe = [1, 1, 2, 3], [0, 0, 2, 0], [0, 0, 0, 3]
    s2b = ops.space_to_batch(p, np.array(blocks), np.array(pb), np.array(pe))
    assert list(s2b.get_output_partial_shape(0).to_shape()) == [12, 4, 3, 3]
    (y,) = run(ops.batch_to_space(s2b, np.array(blocks), np.array(pb), np.array(pe)), [p], [x], tmp_path)
    assert np.array_equal(y, x)
    # against the definition: pad, reshape, transpose
    (sb,) = run(s2b, [p], [x])
    xp = np.pad(x, [(0, 0), (0, 0), (2, 0), (0, 3)])
    ref = xp.reshape(2, 4, 3, 2, 3, 3).transpose(3, 5, 0, 1, 2, 4).reshape(12, 4, 3, 3)
    assert np.array_equal(sb, ref)


def test_shuffle_reverse_reorg(tmp_path):
    x = np.random.default_rng(0).standard_normal((2, 6, 3, 2)).astype(np.float32)
    p = P(x.shape)
    (y,) = run(ops.shuffle_channels(p, 1, 3), [p], [x], tmp_path)
    assert np.array_equal(y, torch.nn.functional.channel_shuffle(torch.from_numpy(x), 3).numpy())
    seq = np.array([2, 5], dtype=np.int32)
    z = np.arange(2 * 6 * 2, dtype=np.float32).reshape(2, 6, 2)
    pz = P(z.shape)
    (r,) = run(ops.reverse_sequence(pz, seq, 0, 1), [pz], [z])
    ref = z.copy()
    ref[0, :2] = z[0, :2][::-1]
    ref[1, :5] = z[1, :5][::-1]
    assert np.array_equal(r, ref)
    w = np.arange(1 * 8 * 4 * 4, dtype=np.float32).reshape(1, 8, 4, 4)
    pw = P(w.shape)
    node = ops.reorg_yolo(pw, [2])
    assert list(node.get_output_partial_shape(0).to_shape()) == [1, 32, 2, 2]
    (ry,) = run(node, [pw], [w])
    assert sorted(ry.reshape(-1).tolist()) == sorted(w.reshape(-1).tolist())


def test_bucketize_search_sorted_eye_bitshift(tmp_path):
    v = np.array([[-1.0, 0.5, 2.0], [3.0, 7.0, 100.0]], dtype=np.float32)
    b = np.array([0.0, 2.0, 5.0], dtype=np.float32)
    p = P(v.shape)
    (r,) = run(ops.bucketize(p, b, "i32", True), [p], [v], tmp_path)
    assert np.array_equal(r, torch.bucketize(torch.from_numpy(v), torch.from_numpy(b), right=False).numpy())
    (l,) = run(ops.bucketize(p, b, "i64", False), [p], [v])
    assert np.array_equal(l, torch.bucketize(torch.from_numpy(v), torch.from_numpy(b), right=True).numpy())
    s = np.sort(np.random.default_rng(1).standard_normal((3, 9)).astype(np.float32), axis=-1)
    q = np.random.default_rng(2).standard_normal((3, 4)).astype(np.float32)
    ps, pq = P(s.shape, name="s"), P(q.shape, name="q")
    for right in (False, True):
        (o,) = run(ops.search_sorted(ps, pq, right), [ps, pq], [s, q])
        assert np.array_equal(o, torch.searchsorted(torch.from_numpy(s), torch.from_numpy(q), right=right).numpy())
    (e,) = run(ops.eye(np.array(3), np.array(4), np.array(1), np.array([2]), output_type="f32"), [], [], tmp_path)
    assert np.array_equal(e, np.stack([np.eye(3, 4, 1, dtype=np.float32)] * 2))
    a = np.array([1, 2, -8, 1024], dtype=np.int32)
    pa = P(a.shape, "i32")
    (ls,) = run(ops.bitwise_left_shift(pa, np.array([3], dtype=np.int32)), [pa], [a])
    (rs,) = run(ops.bitwise_right_shift(pa, np.array([1, 1, 2, 5], dtype=np.int32)), [pa], [a])
    assert np.array_equal(ls, a << 3) and np.array_equal(rs, a >> np.array([1, 1, 2, 5]))


def test_identity_erfinv_promote():
    x = np.array([-0.9, -0.3, 0.0, 0.5, 0.999], dtype=np.float32)
    p = P(x.shape)
    (y,) = run(ops.erfinv(ops.identity(p)), [p], [x])
    assert np.allclose(y, torch.erfinv(torch.from_numpy(x)).numpy(), rtol=1e-5, atol=1e-6)
    a, b = P([2], "i32", "a"), P([2], "f16", "b")
    n = ops.convert_promote_types(a, b)
    assert str(n.get_output_element_type(0)) == str(n.get_output_element_type(1)) and "f16" in str(n.get_output_element_type(0))
    u, s8 = P([2], "u8", "u"), P([2], "i8", "s")
    assert "i16" in str(ops.convert_promote_types(u, s8).get_output_element_type(0))


def test_lrn_grn():
    x = np.random.default_rng(3).standard_normal((2, 7, 3, 3)).astype(np.float32)
    p = P(x.shape)
    (y,) = run(ops.lrn(p, np.array([1]), alpha=1e-2, beta=0.75, bias=2.0, size=3), [p], [x])
    ref = torch.nn.functional.local_response_norm(torch.from_numpy(x), 3, alpha=1e-2, beta=0.75, k=2.0).numpy()
    assert np.allclose(y, ref, rtol=1e-5, atol=1e-6)
    (g,) = run(ops.grn(p, 0.1), [p], [x])
    assert np.allclose(g, x / np.sqrt((x * x).sum(1, keepdims=True) + 0.1), rtol=1e-5)


def test_segment_max_slice_scatter_gather_tree_unique(tmp_path):
    d = np.array([[1., 5.], [3., 2.], [7., 0.], [-1., -2.]], dtype=np.float32)
    ids = np.array([0, 0, 2, 2], dtype=np.int32)
    p = P(d.shape)
    (z,) = run(ops.segment_max(p, ids, np.array(4), fill_mode="ZERO"), [p], [d], tmp_path)
    assert np.array_equal(z, np.array([[3, 5], [0, 0], [7, 0], [0, 0]], dtype=np.float32))
    (lo,) = run(ops.segment_max(p, ids, fill_mode="LOWEST"), [p], [d])
    assert lo.shape == (3, 2) and lo[1, 0] < -1e30
    x = np.zeros((4, 6), dtype=np.float32)
    upd = np.arange(6, dtype=np.float32).reshape(2, 3) + 1
    px, pu = P(x.shape), P(upd.shape, name="u")
    (s,) = run(ops.slice_scatter(px, pu, np.array([1, 0]), np.array([3, 6]), np.array([1, 2])), [px, pu], [x, upd])
    ref = x.copy()
    ref[1:3, 0:6:2] = upd
    assert np.array_equal(s, ref)
    # beam-search back-tracking (T=3, B=1, beam=2)
    step = np.array([[[1, 2]], [[3, 4]], [[5, 6]]], dtype=np.int32)
    par = np.array([[[0, 0]], [[0, 0]], [[1, 0]]], dtype=np.int32)
    (gt,) = run(ops.gather_tree(step, par, np.array([3], dtype=np.int32), np.array(9, dtype=np.int32)), [], [])
    assert gt[:, 0, 0].tolist() == [1, 4, 5] and gt[:, 0, 1].tolist() == [1, 3, 6]
    v = np.array([3, 1, 3, 2, 1, 7], dtype=np.int64)
    pv = P(v.shape, "i64")
    u = ops.unique(pv, sorted=True)
    vals, first, rev, cnt = run([u.output(0), u.output(1), u.output(2), u.output(3)], [pv], [v])
    tu, tinv, tcnt = torch.unique(torch.from_numpy(v), sorted=True, return_inverse=True, return_counts=True)
    assert np.array_equal(vals, tu.numpy()) and np.array_equal(rev, tinv.numpy()) and np.array_equal(cnt, tcnt.numpy())
    assert first.tolist() == [1, 3, 0, 5]


def test_inverse_grouped_matmul():
    rng = np.random.default_rng(4)
    a = rng.standard_normal((3, 5, 5)).astype(np.float32) + 3 * np.eye(5, dtype=np.float32)
    p = P(a.shape)
    (inv,) = run(ops.inverse(p), [p], [a])
    assert np.allclose(inv, np.linalg.inv(a), rtol=1e-4, atol=1e-5)
    (adj,) = run(ops.inverse(p, adjoint=True), [p], [a])
    assert np.allclose(adj, np.linalg.inv(a).transpose(0, 2, 1), rtol=1e-4, atol=1e-5)
    A = rng.standard_normal((3, 4, 8)).astype(np.float32)
    B = rng.standard_normal((3, 6, 8)).astype(np.float32)
    pa, pb = P(A.shape, name="a"), P(B.shape, name="b")
    (g,) = run(ops.grouped_matmul(pa, pb), [pa, pb], [A, B])
    assert np.allclose(g, np.einsum("gmk,gnk->gmn", A, B), rtol=1e-5, atol=1e-5)
    rows = rng.standard_normal((9, 8)).astype(np.float32)
    offs = np.array([2, 2, 9], dtype=np.int32)            # expert 0: rows 0-1, expert 1: none, expert 2: rows 2-8
    pr = P(rows.shape, name="r")
    (ro,) = run(ops.grouped_matmul(pr, pb, offs), [pr, pb], [rows, B])
    ref = np.concatenate([rows[:2] @ B[0].T, rows[2:] @ B[2].T])
    assert np.allclose(ro, ref, rtol=1e-5, atol=1e-5)


def test_transposed_convolution_and_col2im(tmp_path):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 4, 5, 6)).astype(np.float32)
    w = rng.standard_normal((4, 3, 3, 3)).astype(np.float32)
    px, pw = P(x.shape), P(w.shape, name="w")
    n = ops.convolution_backprop_data(px, pw, strides=[2, 2], pads_begin=[1, 1], pads_end=[1, 1], dilations=[1, 1], output_padding=[1, 0])
    ref = torch.nn.functional.conv_transpose2d(torch.from_numpy(x), torch.from_numpy(w), stride=2, padding=1, output_padding=(1, 0)).numpy()
    assert list(n.get_output_partial_shape(0).to_shape()) == list(ref.shape)
    (y,) = run(n, [px, pw], [x, w], tmp_path)
    assert np.allclose(y, ref, rtol=1e-4, atol=1e-4)
    wg = rng.standard_normal((2, 2, 3, 3, 3)).astype(np.float32)      # groups, C/G, O/G, kh, kw
    pg = P(wg.shape, name="wg")
    (yg,) = run(ops.group_convolution_backprop_data(px, pg, strides=[1, 1], pads_begin=[0, 0], pads_end=[0, 0], dilations=[2, 1]), [px, pg], [x, wg])
    refg = torch.nn.functional.conv_transpose2d(torch.from_numpy(x), torch.from_numpy(wg.reshape(4, 3, 3, 3)), groups=2, dilation=(2, 1)).numpy()
    assert np.allclose(yg, refg, rtol=1e-4, atol=1e-4)
    # 1-D
    x1 = rng.standard_normal((1, 2, 7)).astype(np.float32)
    w1 = rng.standard_normal((2, 5, 4)).astype(np.float32)
    p1, q1 = P(x1.shape), P(w1.shape, name="w")
    (y1,) = run(ops.convolution_backprop_data(p1, q1, strides=[3], pads_begin=[0], pads_end=[0], dilations=[1]), [p1, q1], [x1, w1])
    assert np.allclose(y1, torch.nn.functional.conv_transpose1d(torch.from_numpy(x1), torch.from_numpy(w1), stride=3).numpy(), rtol=1e-4, atol=1e-4)
    # col2im == torch fold
    cols = rng.standard_normal((2, 3 * 2 * 2, 12)).astype(np.float32)
    pc = P(cols.shape)
    (im,) = run(ops.col2im(pc, np.array([4, 5]), np.array([2, 2])), [pc], [cols], tmp_path)
    assert np.allclose(im, torch.nn.functional.fold(torch.from_numpy(cols), (4, 5), (2, 2)).numpy(), rtol=1e-5, atol=1e-5)


def test_adaptive_max_pool_roi_ops_grid_sample(tmp_path):
    rng = np.random.default_rng(6)
    x = rng.standard_normal((2, 3, 7, 9)).astype(np.float32)
    p = P(x.shape)
    n = ops.adaptive_max_pool(p, np.array([3, 4]))
    vals, idx = run([n.output(0), n.output(1)], [p], [x], tmp_path)
    tv, ti = torch.nn.functional.adaptive_max_pool2d(torch.from_numpy(x), (3, 4), return_indices=True)
    assert np.array_equal(vals, tv.numpy()) and np.array_equal(idx, ti.numpy())
    # grid sample vs torch for the three modes / paddings
    grid = (rng.random((2, 5, 6, 2)).astype(np.float32) * 2.6 - 1.3)
    pg = P(grid.shape, name="g")
    for mode in ("bilinear", "nearest", "bicubic"):
        for pad in ("zeros", "border"):
            for ac in (False, True):
                (y,) = run(ops.grid_sample(p, pg, ac, mode, pad), [p, pg], [x, grid])
                ref = torch.nn.functional.grid_sample(torch.from_numpy(x), torch.from_numpy(grid), mode=mode, padding_mode=pad, align_corners=ac).numpy()
                assert np.allclose(y, ref, rtol=1e-4, atol=1e-4), (mode, pad, ac)
    # ROI align (avg, asymmetric) against a direct bilinear-average computation of one bin
    feat = np.arange(1 * 1 * 6 * 6, dtype=np.float32).reshape(1, 1, 6, 6)
    pf = P(feat.shape)
    rois = np.array([[1.0, 1.0, 4.0, 4.0]], dtype=np.float32)
    (ra,) = run(ops.roi_align(pf, rois, np.array([0], dtype=np.int32), 1, 1, 2, 1.0, "avg", "asymmetric"), [pf], [feat], tmp_path)
    # a plane a*y + b*x averages to its value at the ROI centre
    assert np.allclose(ra.reshape(-1), [6 * 2.5 + 2.5], rtol=1e-5)
    (rp,) = run(ops.roi_pooling(pf, np.array([[0, 1, 1, 4, 4]], dtype=np.float32), [2, 2], 1.0, "max"), [pf], [feat])
    assert rp.shape == (1, 1, 2, 2) and rp.reshape(-1).tolist() == [14.0, 16.0, 26.0, 28.0]


def test_non_max_suppression():
    boxes = np.array([[[0, 0, 1, 1], [0, 0.1, 1, 1.1], [0, -0.1, 1, 0.9], [0, 10, 1, 11], [0, 10.1, 1, 11.1], [0, 100, 1, 101]]], dtype=np.float32)
    scores = np.array([[[0.9, 0.75, 0.6, 0.95, 0.5, 0.3]]], dtype=np.float32)
    n = ops.non_max_suppression(boxes, scores, np.array(3), np.array(0.5, dtype=np.float32), np.array(0.0, dtype=np.float32))
    idx, sc, valid = run([n.output(0), n.output(1), n.output(2)], [], [])
    assert valid.tolist() == [3] and idx[:, 2].tolist() == [3, 0, 5]
    assert np.allclose(sc[:, 2], [0.95, 0.9, 0.3])
    import torchvision  # noqa: F401  (only when available)


def test_dft_family(tmp_path):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((2, 6, 5, 2)).astype(np.float32)
    p = P(x.shape)
    c = x[..., 0] + 1j * x[..., 1]
    (y,) = run(ops.dft(p, np.array([1, 2])), [p], [x], tmp_path)
    ref = np.fft.fftn(c, axes=(1, 2))
    assert np.allclose(y[..., 0], ref.real, atol=1e-4) and np.allclose(y[..., 1], ref.imag, atol=1e-4)
    (z,) = run(ops.idft(ops.dft(p, np.array([1, 2])), np.array([1, 2])), [p], [x])
    assert np.allclose(z, x, atol=1e-4)
    (s,) = run(ops.dft(p, np.array([1]), np.array([8])), [p], [x])
    refs = np.fft.fft(c, n=8, axis=1)
    assert np.allclose(s[..., 0], refs.real, atol=1e-4)
    r = rng.standard_normal((3, 8, 6)).astype(np.float32)
    pr = P(r.shape)
    n = ops.rdft(pr, np.array([1, 2]))
    assert list(n.get_output_partial_shape(0).to_shape()) == [3, 8, 4, 2]
    (ry,) = run(n, [pr], [r], tmp_path)
    rref = np.fft.rfftn(r, axes=(1, 2))
    assert np.allclose(ry[..., 0], rref.real, atol=1e-4) and np.allclose(ry[..., 1], rref.imag, atol=1e-4)
    (back,) = run(ops.irdft(ops.rdft(pr, np.array([1, 2])), np.array([1, 2])), [pr], [r])
    assert back.shape == r.shape and np.allclose(back, r, atol=1e-4)


def _torch_rnn_weights(mod, kind, H, reverse=False):
    sfx = "_reverse" if reverse else ""
    w_ih, w_hh = getattr(mod, "weight_ih_l0" + sfx).detach(), getattr(mod, "weight_hh_l0" + sfx).detach()
    b_ih, b_hh = getattr(mod, "bias_ih_l0" + sfx).detach(), getattr(mod, "bias_hh_l0" + sfx).detach()
    if kind == "lstm":          # torch gate order i, f, g, o -> f, i, c, o
        order = [1, 0, 2, 3]
    elif kind == "gru":         # torch r, z, n -> z, r, h
        order = [1, 0, 2]
    else:
        order = [0]
    re = lambda t: torch.cat([t[i * H:(i + 1) * H] for i in order], 0)
    return re(w_ih), re(w_hh), re(b_ih), re(b_hh)


@pytest.mark.parametrize("kind", ["lstm", "gru", "rnn"])
def test_recurrent_sequences_match_torch(kind, tmp_path):
    torch.manual_seed(0)
    B, T, I, H = 3, 5, 4, 6
    mod = {"lstm": torch.nn.LSTM, "gru": torch.nn.GRU, "rnn": torch.nn.RNN}[kind](I, H, batch_first=True, bidirectional=True)
    x = torch.randn(B, T, I)
    h0 = torch.randn(2, B, H)
    c0 = torch.randn(2, B, H)
    with torch.no_grad():
        if kind == "lstm":
            y_ref, (h_ref, c_ref) = mod(x, (h0, c0))
        else:
            y_ref, h_ref = mod(x, h0)
    Ws, Rs, Bs = [], [], []
    for rev in (False, True):
        w, r, bi, bh = _torch_rnn_weights(mod, kind, H, rev)
        Ws.append(w)
        Rs.append(r)
        if kind == "gru":       # linear_before_reset: z, r biases summed, the candidate's two biases kept apart
            Bs.append(torch.cat([bi[:2 * H] + bh[:2 * H], bi[2 * H:], bh[2 * H:]]))
        else:
            Bs.append(bi + bh)
    W, R, Bv = torch.stack(Ws).numpy(), torch.stack(Rs).numpy(), torch.stack(Bs).numpy()
    px = P(x.shape)
    lens = np.full((B,), T, dtype=np.int32)
    h0n = h0.permute(1, 0, 2).contiguous().numpy()
    if kind == "lstm":
        n = ops.lstm_sequence(px, h0n, c0.permute(1, 0, 2).contiguous().numpy(), lens, W, R, Bv, H, "bidirectional")
    elif kind == "gru":
        n = ops.gru_sequence(px, h0n, lens, W, R, Bv, H, "bidirectional", linear_before_reset=True)
    else:
        n = ops.rnn_sequence(px, h0n, lens, W, R, Bv, H, "bidirectional")
    outs = run([n.output(i) for i in range(3 if kind == "lstm" else 2)], [px], [x.numpy()], tmp_path)
    y = outs[0]                                        # [B, 2, T, H]
    assert np.allclose(y.transpose(0, 2, 1, 3).reshape(B, T, 2 * H), y_ref.numpy(), atol=1e-5)
    assert np.allclose(outs[1].transpose(1, 0, 2), h_ref.numpy(), atol=1e-5)
    if kind == "lstm":
        assert np.allclose(outs[2].transpose(1, 0, 2), c_ref.numpy(), atol=1e-5)


def test_cells_match_one_sequence_step():
    torch.manual_seed(1)
    B, I, H = 2, 3, 4
    cell = torch.nn.LSTMCell(I, H)
    x, h, c = torch.randn(B, I), torch.randn(B, H), torch.randn(B, H)
    with torch.no_grad():
        h_ref, c_ref = cell(x, (h, c))
    order = [1, 0, 2, 3]
    re = lambda t: torch.cat([t[i * H:(i + 1) * H] for i in order], 0).detach().numpy()
    px = P(x.shape)
    n = ops.lstm_cell(px, h.numpy(), c.numpy(), re(cell.weight_ih), re(cell.weight_hh), re(cell.bias_ih) + re(cell.bias_hh), H)
    ho, co = run([n.output(0), n.output(1)], [px], [x.numpy()])
    assert np.allclose(ho, h_ref.numpy(), atol=1e-5) and np.allclose(co, c_ref.numpy(), atol=1e-5)
    g = torch.nn.GRUCell(I, H)
    with torch.no_grad():
        gh = g(x, h)
    reg_ = lambda t: torch.cat([t[H:2 * H], t[:H], t[2 * H:]], 0).detach()
    bi, bh = reg_(g.bias_ih), reg_(g.bias_hh)
    bias = torch.cat([bi[:2 * H] + bh[:2 * H], bi[2 * H:], bh[2 * H:]]).numpy()
    (go,) = run(ops.gru_cell(px, h.numpy(), reg_(g.weight_ih).numpy(), reg_(g.weight_hh).numpy(), bias, H, linear_before_reset=True), [px], [x.numpy()])
    assert np.allclose(go, gh.numpy(), atol=1e-5)
    r = torch.nn.RNNCell(I, H)
    with torch.no_grad():
        rh = r(x, h)
    (ro,) = run(ops.rnn_cell(px, h.numpy(), r.weight_ih.detach().numpy(), r.weight_hh.detach().numpy(), (r.bias_ih + r.bias_hh).detach().numpy(), H), [px], [x.numpy()])
    assert np.allclose(ro, rh.numpy(), atol=1e-5)


def test_ctc_greedy_decoders(tmp_path):
    # classes: 0, 1, 2 and blank = 3
    logits = np.full((1, 6, 4), -5.0, dtype=np.float32)
    for t, c in enumerate([1, 1, 3, 1, 2, 2]):
        logits[0, t, c] = 5.0
    p = P(logits.shape)
    n = ops.ctc_greedy_decoder_seq_len(p, np.array([6], dtype=np.int32))
    cls, ln = run([n.output(0), n.output(1)], [p], [logits], tmp_path)
    assert cls[0].tolist() == [1, 1, 2, -1, -1, -1] and ln.tolist() == [3]
    n2 = ops.ctc_greedy_decoder_seq_len(p, np.array([6], dtype=np.int32), merge_repeated=False)
    cls2, ln2 = run([n2.output(0), n2.output(1)], [p], [logits])
    assert cls2[0].tolist() == [1, 1, 1, 2, 2, -1] and ln2.tolist() == [5]
    tb = logits.transpose(1, 0, 2).copy()             # [T, B, classes]
    pt = P(tb.shape)
    (old,) = run(ops.ctc_greedy_decoder(pt, np.ones((6, 1), dtype=np.float32)), [pt], [tb])
    assert old.reshape(-1).tolist() == [1, 1, 2, -1, -1, -1]


def test_embedding_bags(tmp_path):
    rng = np.random.default_rng(8)
    table = rng.standard_normal((10, 3)).astype(np.float32)
    idx = np.array([1, 2, 4, 5, 4, 3, 2, 9], dtype=np.int32)
    offs = np.array([0, 3, 3, 6], dtype=np.int32)
    w = rng.random(8).astype(np.float32)
    p = P(table.shape)
    (y,) = run(ops.embedding_bag_offsets_sum(p, idx, offs, np.array(0, dtype=np.int32), w), [p], [table], tmp_path)
    ref = torch.nn.functional.embedding_bag(torch.from_numpy(idx).long(), torch.from_numpy(table), torch.from_numpy(offs).long(), mode="sum",
                                            per_sample_weights=torch.from_numpy(w)).numpy()
    ref[1] = table[0]                                   # the empty bag takes the default row
    assert np.allclose(y, ref, atol=1e-5)
    (m,) = run(ops.embedding_bag_offsets(p, idx, offs, reduction="mean"), [p], [table])
    refm = torch.nn.functional.embedding_bag(torch.from_numpy(idx).long(), torch.from_numpy(table), torch.from_numpy(offs).long(), mode="mean").numpy()
    assert np.allclose(m, refm, atol=1e-5)
    packed = idx.reshape(4, 2)
    (pk,) = run(ops.embedding_bag_packed_sum(p, packed), [p], [table])
    assert np.allclose(pk, table[packed].sum(1), atol=1e-5)
    seg = np.array([0, 0, 0, 2, 2, 2, 3, 3], dtype=np.int32)
    (sg,) = run(ops.embedding_segments_sum(p, idx, seg, np.array(5, dtype=np.int32)), [p], [table], tmp_path)
    refs = np.zeros((5, 3), np.float32)
    for i, s in zip(idx, seg):
        refs[s] += table[i]
    assert np.allclose(sg, refs, atol=1e-5)


def test_random_ops_are_deterministic_and_in_range():
    n = ops.random_uniform(np.array([4, 1000]), np.array(2.0, dtype=np.float32), np.array(5.0, dtype=np.float32), "f32", 7, 11)
    (a,) = run(n, [], [])
    (b,) = run(ops.random_uniform(np.array([4, 1000]), np.array(2.0, dtype=np.float32), np.array(5.0, dtype=np.float32), "f32", 7, 11), [], [])
    assert np.array_equal(a, b) and a.min() >= 2.0 and a.max() < 5.0 and abs(a.mean() - 3.5) < 0.05
    (c,) = run(ops.random_uniform(np.array([4, 1000]), np.array(2.0, dtype=np.float32), np.array(5.0, dtype=np.float32), "f32", 8, 11), [], [])
    assert not np.array_equal(a, c)
    probs = np.array([[0.0, 0.2, 0.8], [1.0, 0.0, 0.0]], dtype=np.float32)
    p = P(probs.shape)
    (s,) = run(ops.multinomial(p, np.array([2000]), "i32", True, False, 3, 5), [p], [probs])
    assert s.shape == (2, 2000) and (s[1] == 0).all() and (s[0] != 0).all() and abs((s[0] == 2).mean() - 0.8) < 0.05
    (wo,) = run(ops.multinomial(p, np.array([2]), "i32", False, False, 3, 5), [p], [np.array([[0.0, 0.2, 0.8], [0.5, 0.5, 0.0]], dtype=np.float32)])
    assert sorted(wo[0].tolist()) == [1, 2] and sorted(wo[1].tolist()) == [0, 1]
