"""Detection operations and the rest of the public operation sets: shape inference, evaluation on the CPU device after
an IR round trip, compared with NumPy / PyTorch restatements or hand-computed values."""
import numpy as np
import torch

import openvino_b200 as ov
from openvino_b200 import opset as ops


def run(outputs, params, feeds):
    m = ov.Model(outputs, params, "t")
    xml, weights = ov._ovcore.serialize(m._m)
    back = ov.Model._wrap(ov._ovcore.deserialize(xml.decode(), np.frombuffer(weights, dtype=np.uint8)))
    res = ov.compile_model(back, "CPU")(feeds)
    return [res[i] for i in range(len(outputs))]


def iou(a, b, off=0.0):
    iw = min(a[2], b[2]) - max(a[0], b[0]) + off
    ih = min(a[3], b[3]) - max(a[1], b[1]) + off
    if iw <= 0 or ih <= 0:
        return 0.0
    inter = iw * ih
    return inter / ((a[2] - a[0] + off) * (a[3] - a[1] + off) + (b[2] - b[0] + off) * (b[3] - b[1] + off) - inter)


def test_every_operation_of_the_reference_opset_tables_is_registered():
    import glob
    import os
    import re
    tables = glob.glob("/root/reference/src/core/include/openvino/opsets/opset*_tbl.hpp")
    if not tables:
        import pytest
        pytest.skip("reference tree not present")
    have = {s[0] for s in ov._ovcore.op_schemas()}
    want = set()
    for f in tables:
        want |= set(re.findall(r"_OPENVINO_OP_REG\((\w{2,}),", open(f).read()))
    assert sorted(want - have) == []
    assert os.path.basename(tables[0]).startswith("opset")


def test_prior_box_order_and_values():
    n = ops.prior_box(np.array([2, 2], np.int64), np.array([32, 32], np.int64),
                      {"min_size": [16.0], "max_size": [38.46], "aspect_ratio": [2.0], "flip": True, "step": 16.0, "offset": 0.5, "variance": [0.1, 0.1, 0.2, 0.2]})
    assert list(n.get_output_shape(0)) == [2, 4 * 2 * 2 * 4]
    out = run([n], [], [])[0]
    cx = cy = 8.0
    half = [(8.0, 8.0), (np.sqrt(16 * 38.46) / 2,) * 2, (8 * np.sqrt(2.0), 8 / np.sqrt(2.0)), (8 * np.sqrt(0.5), 8 / np.sqrt(0.5))]      # min, max, ratio 2, ratio 1/2
    ref = np.array([[(cx - w) / 32, (cy - h) / 32, (cx + w) / 32, (cy + h) / 32] for w, h in half], np.float32).reshape(-1)
    np.testing.assert_allclose(out[0, :16], ref, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(out[1].reshape(-1, 4), np.tile([0.1, 0.1, 0.2, 0.2], (16, 1)), rtol=1e-6)
    # second cell of the first row is shifted by one step in x
    np.testing.assert_allclose(out[0, 16:20], ref[:4] + np.array([0.5, 0, 0.5, 0], np.float32), rtol=1e-5, atol=1e-6)
    # [min, ratios, max] order and clipping
    n2 = ops.prior_box(np.array([1, 1], np.int64), np.array([20, 20], np.int64), min_size=[16.0], max_size=[32.0], aspect_ratio=[2.0], clip=True, step=0.0, offset=0.5,
                       min_max_aspect_ratios_order=False)
    o2 = run([n2], [], [])[0]
    assert o2.shape == (2, 12) and o2.min() >= 0 and o2.max() <= 1
    np.testing.assert_allclose(o2[0, 8:12], np.clip([(10 - np.sqrt(512) / 2) / 20] * 2 + [(10 + np.sqrt(512) / 2) / 20] * 2, 0, 1), rtol=1e-5)
    # fixed sizes with a density grid: 2 x 2 centres per cell
    n3 = ops.prior_box(np.array([1, 1], np.int64), np.array([16, 16], np.int64), fixed_size=[8.0], density=[2.0], step=16.0, offset=0.5)
    o3 = run([n3], [], [])[0]
    assert o3.shape == (2, 16)
    np.testing.assert_allclose(o3[0].reshape(4, 4)[:, :2], np.array([[2, 2], [6, 2], [2, 6], [6, 6]], np.float32) / 16, rtol=1e-6)


def test_detection_output_corner_code_and_suppression():
    # 4 priors, classes {background, 1, 2}; zero deltas: boxes are the priors
    priors = np.array([[0.1, 0.1, 0.4, 0.4], [0.12, 0.1, 0.42, 0.4], [0.6, 0.6, 0.9, 0.9], [0.0, 0.5, 0.2, 0.8]], np.float32)
    variances = np.full((4, 4), 0.1, np.float32)
    prior_t = np.stack([priors.reshape(-1), variances.reshape(-1)])[None]
    conf = np.array([[0.1, 0.8, 0.1], [0.2, 0.7, 0.1], [0.1, 0.1, 0.8], [0.3, 0.3, 0.4]], np.float32).reshape(1, -1)
    loc = np.zeros((1, 16), np.float32)
    pl, pc, pp = ops.parameter([1, 16], "f32", "loc"), ops.parameter([1, 12], "f32", "conf"), ops.parameter([1, 2, 16], "f32", "pri")
    n = ops.detection_output(pl, pc, pp, {"num_classes": 3, "keep_top_k": [4], "nms_threshold": 0.5, "confidence_threshold": 0.25, "normalized": True}) \
        if False else ops.detection_output(pl, pc, pp, keep_top_k=[4], nms_threshold=0.5, confidence_threshold=0.25, normalized=True)
    assert list(n.get_output_shape(0)) == [1, 1, 4, 7]
    out = run([n], [pl, pc, pp], [loc, conf, prior_t])[0].reshape(4, 7)
    # class 1: prior 0 (0.8) suppresses prior 1 (IoU 0.88); prior 3 (0.3) stays. class 2: prior 2 (0.8), prior 3 (0.4)
    assert iou(priors[0], priors[1]) > 0.5
    got = {(int(r[1]), round(float(r[2]), 3)): r[3:] for r in out if r[0] >= 0}
    assert set(got) == {(1, 0.8), (1, 0.3), (2, 0.8), (2, 0.4)}
    np.testing.assert_allclose(got[(1, 0.8)], priors[0], rtol=1e-6)
    np.testing.assert_allclose(got[(2, 0.4)], priors[3], rtol=1e-6)
    # centre-size code: a delta of (1, 0, log 2, 0) with variance 0.1 moves the centre by 0.1 widths and scales the width by 2^0.1
    loc2 = np.zeros((1, 16), np.float32)
    loc2[0, 8:12] = [1.0, 0.0, np.log(2.0), 0.0]
    n2 = ops.detection_output(pl, pc, pp, keep_top_k=[2], nms_threshold=0.5, confidence_threshold=0.5, normalized=True, code_type="caffe.PriorBoxParameter.CENTER_SIZE")
    out2 = run([n2], [pl, pc, pp], [loc2, conf, prior_t])[0].reshape(2, 7)
    row = [r for r in out2 if int(r[1]) == 2][0]
    w = 0.3 * 2 ** 0.1
    np.testing.assert_allclose(row[3:], [0.75 + 0.03 - w / 2, 0.6, 0.75 + 0.03 + w / 2, 0.9], rtol=1e-5)
    # fewer detections than rows: the list ends with image id -1
    n3 = ops.detection_output(pl, pc, pp, keep_top_k=[4], nms_threshold=0.5, confidence_threshold=0.75, normalized=True)
    out3 = run([n3], [pl, pc, pp], [loc, conf, prior_t])[0].reshape(4, 7)
    assert out3[2, 0] == -1 and (out3[:2, 0] == 0).all()


def _np_proposals(anchors, deltas, scores, img_h, img_w, min_size, thr, pre, post, off):
    An, H, W = scores.shape
    cand = []
    for h in range(H):
        for w in range(W):
            for a in range(An):
                x0, y0, x1, y1 = anchors[(h * W + w) * An + a]
                dx, dy, dw, dh = deltas[a * 4:(a + 1) * 4, h, w]
                ww, hh = x1 - x0 + off, y1 - y0 + off
                cx, cy = x0 + 0.5 * ww, y0 + 0.5 * hh
                pw, ph = np.exp(min(dw, np.log(1000 / 16))) * ww, np.exp(min(dh, np.log(1000 / 16))) * hh
                b = [dx * ww + cx - 0.5 * pw, dy * hh + cy - 0.5 * ph, dx * ww + cx + 0.5 * pw - off, dy * hh + cy + 0.5 * ph - off]
                b = [np.clip(b[0], 0, img_w - off), np.clip(b[1], 0, img_h - off), np.clip(b[2], 0, img_w - off), np.clip(b[3], 0, img_h - off)]
                if b[2] - b[0] + off >= max(min_size, 1) and b[3] - b[1] + off >= max(min_size, 1):
                    cand.append((scores[a, h, w], b))
    cand.sort(key=lambda t: -t[0])
    cand = cand[:pre]
    keep = []
    for s, b in cand:
        if len(keep) == post:
            break
        if all(iou(b, k[1], off) <= thr for k in keep):
            keep.append((s, b))
    return keep


def test_detectron_and_batched_proposals_match_numpy():
    rng = np.random.default_rng(0)
    An, H, W = 3, 4, 5
    base = np.array([[-8, -8, 8, 8], [-16, -8, 16, 8], [-8, -16, 8, 16]], np.float32)
    anchors = np.zeros((H * W * An, 4), np.float32)
    for h in range(H):
        for w in range(W):
            anchors[(h * W + w) * An:(h * W + w + 1) * An] = base + np.array([w * 8 + 4, h * 8 + 4] * 2, np.float32)
    deltas = (rng.standard_normal((An * 4, H, W)) * 0.2).astype(np.float32)
    scores = rng.random((An, H, W)).astype(np.float32)
    info = np.array([32.0, 40.0, 1.0], np.float32)
    pi, pa, pd, ps = ops.parameter([3], "f32", "i"), ops.parameter([H * W * An, 4], "f32", "a"), ops.parameter([An * 4, H, W], "f32", "d"), ops.parameter([An, H, W], "f32", "s")
    n = ops.experimental_detectron_generate_proposals_single_image(pi, pa, pd, ps, 2.0, 0.6, 10, 30)
    rois, sc = run([n.output(0), n.output(1)], [pi, pa, pd, ps], [info, anchors, deltas, scores])
    ref = _np_proposals(anchors, deltas, scores, 32, 40, 2.0, 0.6, 30, 10, 1.0)
    assert rois.shape == (10, 4) and sc.shape == (10,)
    np.testing.assert_allclose(sc[:len(ref)], [r[0] for r in ref], rtol=1e-6)
    np.testing.assert_allclose(rois[:len(ref)], [r[1] for r in ref], rtol=1e-4, atol=1e-4)
    assert (rois[len(ref):] == 0).all()
    # batched form, normalised boxes (no +1), data-dependent row count
    B = 2
    deltas_b = (rng.standard_normal((B, An * 4, H, W)) * 0.2).astype(np.float32)
    scores_b = rng.random((B, An, H, W)).astype(np.float32)
    info_b = np.array([[32, 40, 1], [30, 36, 1]], np.float32)
    pib, pab = ops.parameter([B, 3], "f32", "i"), ops.parameter([H, W, An, 4], "f32", "a")
    pdb, psb = ops.parameter([B, An * 4, H, W], "f32", "d"), ops.parameter([B, An, H, W], "f32", "s")
    g = ops.generate_proposals(pib, pab, pdb, psb, 1.0, 0.5, 50, 6, roi_num_type="i32")
    r2, s2, num = run([g.output(0), g.output(1), g.output(2)], [pib, pab, pdb, psb], [info_b, anchors.reshape(H, W, An, 4), deltas_b, scores_b])
    assert num.dtype == np.int32 and num.sum() == len(s2) and r2.shape == (len(s2), 4)
    at = 0
    for b in range(B):
        ref = _np_proposals(anchors, deltas_b[b], scores_b[b], info_b[b, 0], info_b[b, 1], 1.0, 0.5, 50, 6, 0.0)
        assert num[b] == len(ref)
        np.testing.assert_allclose(s2[at:at + len(ref)], [r[0] for r in ref], rtol=1e-6)
        np.testing.assert_allclose(r2[at:at + len(ref)], [r[1] for r in ref], rtol=1e-4, atol=1e-4)
        at += len(ref)


def test_proposal_single_anchor_by_hand():
    # one anchor (ratio 1, scale 1, base 16 -> [0, 0, 15, 15] in pixel-inclusive corners), 2 x 2 cells, stride 16, zero deltas
    probs = np.zeros((1, 2, 2, 2), np.float32)
    probs[0, 1] = [[0.9, 0.1], [0.5, 0.7]]
    deltas = np.zeros((1, 4, 2, 2), np.float32)
    pc, pd = ops.parameter([1, 2, 2, 2], "f32", "p"), ops.parameter([1, 4, 2, 2], "f32", "d")
    n = ops.proposal(pc, pd, np.array([32, 32, 1], np.float32), 16, 10, 3, 0.5, 16, 4, [1.0], [1.0], version="opset4") if False else \
        ov._graph.make_op("Proposal", [pc, pd, ops.constant(np.array([32, 32, 1], np.float32))],
                          {"base_size": 16, "pre_nms_topn": 10, "post_nms_topn": 3, "nms_thresh": 0.5, "feat_stride": 16, "min_size": 4, "ratio": [1.0], "scale": [1.0]}, version="opset4")
    assert list(n.get_output_shape(0)) == [3, 5] and list(n.get_output_shape(1)) == [3]
    rois, sc = run([n.output(0), n.output(1)], [pc, pd], [probs, deltas])
    np.testing.assert_allclose(sc, [0.9, 0.7, 0.5], rtol=1e-6)
    np.testing.assert_allclose(rois, [[0, 0, 0, 15, 15], [0, 16, 16, 31, 31], [0, 0, 16, 15, 31]], atol=1e-4)
    n1 = ov._graph.make_op("Proposal", [pc, pd, ops.constant(np.array([32, 32, 1], np.float32))],
                           {"base_size": 16, "pre_nms_topn": 10, "post_nms_topn": 2, "nms_thresh": 0.5, "feat_stride": 16, "min_size": 4, "ratio": [1.0], "scale": [1.0], "normalize": True},
                           version="opset1")
    assert n1.get_output_size() == 1
    r1 = run([n1.output(0)], [pc, pd], [probs, deltas])[0]
    np.testing.assert_allclose(r1, [[0, 0, 0, 15 / 32, 15 / 32], [0, 0.5, 0.5, 31 / 32, 31 / 32]], atol=1e-5)


def test_detectron_prior_grid_topk_and_feature_extractor():
    pri = np.array([[-2, -2, 2, 2], [-4, -1, 4, 1]], np.float32)
    pp, pf, pim = ops.parameter([2, 4], "f32", "p"), ops.parameter([1, 3, 2, 3], "f32", "f"), ops.parameter([1, 3, 16, 24], "f32", "im")
    n = ops.experimental_detectron_prior_grid_generator(pp, pf, pim, True, 0, 0, 0.0, 0.0)
    assert list(n.get_output_shape(0)) == [12, 4]
    out = run([n], [pp, pf, pim], [pri, np.zeros((1, 3, 2, 3), np.float32), np.zeros((1, 3, 16, 24), np.float32)])[0]
    ref = np.array([pri[p] + np.array([(w + 0.5) * 8, (h + 0.5) * 8] * 2) for h in range(2) for w in range(3) for p in range(2)], np.float32)
    np.testing.assert_allclose(out, ref)
    n4 = ops.experimental_detectron_prior_grid_generator(pp, pf, pim, False, 0, 0, 4.0, 4.0)
    assert list(n4.get_output_shape(0)) == [2, 3, 2, 4]
    # top-k ROIs
    rois = np.arange(20, dtype=np.float32).reshape(5, 4)
    probs = np.array([0.1, 0.9, 0.3, 0.8, 0.2], np.float32)
    pr, pq = ops.parameter([5, 4], "f32", "r"), ops.parameter([5], "f32", "q")
    t = ops.experimental_detectron_topk_rois(pr, pq, 3)
    np.testing.assert_array_equal(run([t], [pr, pq], [rois, probs])[0], rois[[1, 3, 2]])
    # feature extractor: constant maps tell which pyramid level served a box
    l0, l1 = np.full((1, 2, 16, 16), 1.0, np.float32), np.full((1, 2, 64, 64), 2.0, np.float32)
    boxes = np.array([[4, 4, 20, 20], [0, 0, 60, 60]], np.float32) * np.array([1, 1, 1, 1], np.float32)
    boxes[1] = [0, 0, 500, 500]                        # sqrt(area) = 500 > 224 * 2: level 3 -> second (last) input
    pb, p0, p1 = ops.parameter([2, 4], "f32", "b"), ops.parameter([1, 2, 16, 16], "f32", "l0"), ops.parameter([1, 2, 64, 64], "f32", "l1")
    fe = ops.experimental_detectron_roi_feature_extractor([pb, p0, p1], 3, 2, [4, 8], False)
    feats, same = run([fe.output(0), fe.output(1)], [pb, p0, p1], [boxes, l0, l1])
    assert feats.shape == (2, 2, 3, 3)
    np.testing.assert_allclose(feats[0], 1.0)
    np.testing.assert_allclose(feats[1], 2.0)
    np.testing.assert_array_equal(same, boxes)
    # a ramp: the pooled value of a bin is the ramp at the bin centre
    ramp = np.tile(np.arange(16, dtype=np.float32), (16, 1))[None, None]
    pr1 = ops.parameter([1, 1, 16, 16], "f32", "ramp")
    pb1 = ops.parameter([1, 4], "f32", "b")
    fe2 = ops.experimental_detectron_roi_feature_extractor([pb1, pr1], 2, 2, [1], True)
    f2 = run([fe2.output(0)], [pb1, pr1], [np.array([[2, 2, 10, 10]], np.float32), ramp])[0]
    np.testing.assert_allclose(f2[0, 0], [[3.5, 7.5], [3.5, 7.5]], rtol=1e-5)


def test_detectron_detection_output():
    rois = np.array([[10, 10, 30, 30], [12, 10, 32, 30], [50, 50, 70, 70]], np.float32)
    scores = np.array([[0.1, 0.9, 0.0], [0.1, 0.8, 0.1], [0.2, 0.1, 0.7]], np.float32)
    deltas = np.zeros((3, 12), np.float32)
    pr, pd, ps = ops.parameter([3, 4], "f32", "r"), ops.parameter([3, 12], "f32", "d"), ops.parameter([3, 3], "f32", "s")
    n = ops.experimental_detectron_detection_output(pr, pd, ps, np.array([[100, 100, 1]], np.float32), 0.05, 0.5, 4.135, 3, 10, 4)
    boxes, cls, sc = run([n.output(0), n.output(1), n.output(2)], [pr, pd, ps], [rois, deltas, scores])
    assert boxes.shape == (4, 4) and cls.dtype == np.int32
    # class 1: box 0 suppresses box 1, box 2 (0.1) stays; class 2: box 2 (0.7) and box 1 (0.1)
    np.testing.assert_allclose(sc, [0.9, 0.7, 0.1, 0.1], rtol=1e-6)
    np.testing.assert_array_equal(cls, [1, 2, 1, 2])
    np.testing.assert_allclose(boxes[0], [10, 10, 30, 30], atol=1e-4)       # zero deltas keep a pixel-inclusive box
    np.testing.assert_allclose(boxes[1], [50, 50, 70, 70], atol=1e-4)


def _np_matrix_nms(boxes, scores, score_thr, post_thr, top, keep, gaussian, sigma, bg):
    out = []
    for c in range(scores.shape[0]):
        if c == bg:
            continue
        order = [i for i in np.argsort(-scores[c], kind="stable") if scores[c, i] > score_thr][:top if top >= 0 else None]
        ious = np.zeros((len(order), len(order)))
        for i in range(len(order)):
            for j in range(i):
                ious[i, j] = iou(boxes[order[i]], boxes[order[j]])
        mx = ious.max(1) if len(order) else []
        for i, bi in enumerate(order):
            d = 1.0
            for j in range(i):
                d = min(d, np.exp((mx[j] ** 2 - ious[i, j] ** 2) * sigma) if gaussian else (1 - ious[i, j]) / (1 - mx[j]))
            if scores[c, bi] * d >= post_thr:
                out.append((c, scores[c, bi] * d, bi))
    out.sort(key=lambda t: -t[1])
    return out[:keep if keep >= 0 else None]


def test_matrix_and_multiclass_nms_match_numpy():
    rng = np.random.default_rng(3)
    B, M, Cn = 2, 12, 3
    xy = rng.random((B, M, 2)).astype(np.float32) * 0.6
    wh = rng.random((B, M, 2)).astype(np.float32) * 0.4 + 0.05
    boxes = np.concatenate([xy, xy + wh], -1)
    scores = rng.random((B, Cn, M)).astype(np.float32)
    pb, ps = ops.parameter([B, M, 4], "f32", "b"), ops.parameter([B, Cn, M], "f32", "s")
    for gaussian in (False, True):
        n = ops.matrix_nms(pb, ps, sort_result_type="score", score_threshold=0.2, nms_top_k=8, keep_top_k=6, background_class=0,
                           decay_function="gaussian" if gaussian else "linear", gaussian_sigma=2.0, post_threshold=0.1, output_type="i32")
        sel, idx, valid = run([n.output(0), n.output(1), n.output(2)], [pb, ps], [boxes, scores])
        at = 0
        for b in range(B):
            ref = _np_matrix_nms(boxes[b], scores[b], 0.2, 0.1, 8, 6, gaussian, 2.0, 0)
            assert valid[b] == len(ref)
            got = sel[at:at + len(ref)]
            np.testing.assert_allclose(got[:, 1], [r[1] for r in ref], rtol=1e-5)
            np.testing.assert_array_equal(got[:, 0], [r[0] for r in ref])
            np.testing.assert_array_equal(idx[at:at + len(ref), 0], [b * M + r[2] for r in ref])
            np.testing.assert_allclose(got[:, 2:], boxes[b][[r[2] for r in ref]], rtol=1e-6)
            at += len(ref)
        assert idx.dtype == np.int32 and at == len(sel)
    # multiclass: greedy suppression per class, then the best keep_top_k of the image, rows ordered by class
    m = ops.multiclass_nms(pb, ps, sort_result_type="classid", iou_threshold=0.3, score_threshold=0.3, nms_top_k=10, keep_top_k=5, background_class=-1)
    sel, idx, valid = run([m.output(0), m.output(1), m.output(2)], [pb, ps], [boxes, scores])
    at = 0
    for b in range(B):
        ref = []
        for c in range(Cn):
            keep = []
            for i in [i for i in np.argsort(-scores[b, c], kind="stable") if scores[b, c, i] > 0.3][:10]:
                if all(iou(boxes[b, i], boxes[b, k]) <= 0.3 for k in keep):
                    keep.append(i)
            ref += [(c, scores[b, c, i], i) for i in keep]
        ref = sorted(sorted(ref, key=lambda t: -t[1])[:5], key=lambda t: (t[0], -t[1]))
        assert valid[b] == len(ref)
        np.testing.assert_array_equal(sel[at:at + len(ref), 0], [r[0] for r in ref])
        np.testing.assert_allclose(sel[at:at + len(ref), 1], [r[1] for r in ref], rtol=1e-6)
        np.testing.assert_array_equal(idx[at:at + len(ref), 0], [b * M + r[2] for r in ref])
        at += len(ref)
    # shared-box form of opset9: boxes [C, M, 4], scores [C, M], rois per image
    pbs, pss, prn = ops.parameter([Cn, M, 4], "f32", "b"), ops.parameter([Cn, M], "f32", "s"), ops.parameter([2], "i64", "n")
    ms = ops.multiclass_nms(pbs, pss, prn, iou_threshold=0.3, score_threshold=0.3)
    sel, idx, valid = run([ms.output(0), ms.output(1), ms.output(2)], [pbs, pss, prn], [np.stack([boxes[0]] * Cn), scores[0], np.array([7, 5], np.int64)])
    assert valid.sum() == len(sel) and valid.shape == (2,)
    assert set(idx[:valid[0], 0]) <= set(range(7)) and set(idx[valid[0]:, 0]) <= set(range(7, 12))


def test_nms_rotated_overlaps():
    # (cx, cy, w, h, angle): 0 and 1 are the same square, 1 turned by 90 degrees; 2 and 3 form a cross (IoU 1/7); 4 is far away
    boxes = np.array([[[10, 10, 4, 4, 0.0], [10, 10, 4, 4, np.pi / 2], [30, 30, 4, 1, 0.0], [30, 30, 4, 1, np.pi / 2], [60, 60, 2, 2, 0.3]]], np.float32)
    scores = np.array([[[0.9, 0.8, 0.7, 0.6, 0.5]]], np.float32)
    pb, ps = ops.parameter([1, 5, 5], "f32", "b"), ops.parameter([1, 1, 5], "f32", "s")

    def picked(thr):
        n = ops.nms_rotated(pb, ps, np.int64(10), np.float32(thr), np.float32(0.0))
        idx, sc, valid = run([n.output(0), n.output(1), n.output(2)], [pb, ps], [boxes, scores])
        assert valid[0] == len(idx) and sc.shape == idx.shape
        return list(idx[:, 2])
    assert picked(0.5) == [0, 2, 3, 4]          # 1/7 < 0.5: both arms of the cross stay
    assert picked(0.1) == [0, 2, 4]             # 1/7 > 0.1
    # a 45-degree square against the axis-aligned one: intersection is an octagon of area 16 * (2 sqrt2 - 2) / 1 ... checked through the op's own symmetry
    b2 = np.array([[[0, 0, 4, 4, 0.0], [0, 0, 4, 4, np.pi / 4]]], np.float32)
    inter = 16 * 2 * (np.sqrt(2) - 1)                       # regular octagon with inradius 2
    expect = inter / (32 - inter)
    pb2, ps2 = ops.parameter([1, 2, 5], "f32", "b"), ops.parameter([1, 1, 2], "f32", "s")
    for thr, kept in ((expect - 0.01, 1), (expect + 0.01, 2)):
        n = ops.nms_rotated(pb2, ps2, np.int64(10), np.float32(thr), np.float32(0.0))
        assert len(run([n.output(0)], [pb2, ps2], [b2, np.array([[[0.9, 0.8]]], np.float32)])[0]) == kept


def test_roi_align_rotated_ramp():
    H = W = 16
    ramp_x = np.tile(np.arange(W, dtype=np.float32), (H, 1))
    ramp_y = ramp_x.T.copy()
    x = np.stack([ramp_x, ramp_y])[None]
    px, pr = ops.parameter([1, 2, H, W], "f32", "x"), ops.parameter([2, 5], "f32", "r")
    n = ops.roi_align_rotated(px, pr, np.array([0, 0], np.int32), 2, 2, 2, 1.0, False)
    # box centred at (8, 8), 4 wide, 4 high: unrotated, and turned by 90 degrees
    rois = np.array([[8, 8, 4, 4, 0.0], [8, 8, 4, 4, np.pi / 2]], np.float32)
    out = run([n], [px, pr], [x, rois])[0]
    assert out.shape == (2, 2, 2, 2)
    c = 7.5                                      # pixel centres sit at integer + 0.5: the box centre in sample coordinates
    np.testing.assert_allclose(out[0, 0], [[c - 1, c + 1]] * 2, rtol=1e-5)          # x ramp: columns differ
    np.testing.assert_allclose(out[0, 1], [[c - 1] * 2, [c + 1] * 2], rtol=1e-5)    # y ramp: rows differ
    # after a quarter turn the pooled grid walks x along its rows (up to the direction of the turn)
    assert np.allclose(out[1, 0][:, 0], out[1, 0][:, 1], atol=1e-4) and abs(abs(out[1, 0][0, 0] - out[1, 0][1, 0]) - 2) < 1e-4
    assert np.allclose(out[1, 1][0], out[1, 1][1], atol=1e-4) and abs(abs(out[1, 1][0, 0] - out[1, 1][0, 1]) - 2) < 1e-4
    # clockwise_mode mirrors the turn
    n2 = ops.roi_align_rotated(px, pr, np.array([0, 0], np.int32), 2, 2, 2, 1.0, True)
    out2 = run([n2], [px, pr], [x, rois])[0]
    np.testing.assert_allclose(out2[1, 0], out[1, 0][::-1], atol=1e-4)


def test_deformable_convolution_against_conv2d():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 4, 7, 8)).astype(np.float32)
    f = rng.standard_normal((6, 2, 3, 3)).astype(np.float32)          # 2 groups
    px, pf = ops.parameter([2, 4, 7, 8], "f32", "x"), ops.parameter([6, 2, 3, 3], "f32", "f")
    off = np.zeros((2, 2 * 9 * 2, 7, 8), np.float32)                  # 2 deformable groups
    po = ops.parameter(list(off.shape), "f32", "o")
    n = ops.deformable_convolution(px, po, pf, strides=[1, 1], pads_begin=[1, 1], pads_end=[1, 1], dilations=[1, 1], group=2, deformable_group=2)
    assert list(n.get_output_shape(0)) == [2, 6, 7, 8]
    ref = torch.nn.functional.conv2d(torch.from_numpy(x), torch.from_numpy(f), padding=1, groups=2).numpy()
    np.testing.assert_allclose(run([n], [px, po, pf], [x, off, f])[0], ref, rtol=1e-4, atol=1e-4)
    # a whole-pixel offset of (+1, 0) on every tap equals the convolution of the image moved up by one row
    off1 = off.copy()
    off1[:, 0::2] = 1.0
    nb = ops.deformable_convolution(px, po, pf, strides=[1, 1], pads_begin=[1, 1], pads_end=[1, 1], dilations=[1, 1], group=2, deformable_group=2, bilinear_interpolation_pad=True)
    moved = np.zeros_like(x)
    moved[:, :, :-1] = x[:, :, 1:]
    ref1 = torch.nn.functional.conv2d(torch.from_numpy(moved), torch.from_numpy(f), padding=1, groups=2).numpy()
    got1 = run([nb], [px, po, pf], [x, off1, f])[0]
    # first row: the tap on the padding row now reads row 0; last row: the tap reads past the image
    np.testing.assert_allclose(got1[:, :, 1:-1], ref1[:, :, 1:-1], rtol=1e-4, atol=1e-4)
    # a mask halves every tap
    pm = ops.parameter([2, 18, 7, 8], "f32", "m")
    nm = ops.deformable_convolution(px, po, pf, pm, strides=[1, 1], pads_begin=[1, 1], pads_end=[1, 1], dilations=[1, 1], group=2, deformable_group=2)
    np.testing.assert_allclose(run([nm], [px, po, pf, pm], [x, off, f, np.full((2, 18, 7, 8), 0.5, np.float32)])[0], ref * 0.5, rtol=1e-4, atol=1e-4)
    # half-pixel offsets blend two rows
    offh = off.copy()
    offh[:, 0::2] = 0.5
    xs = np.zeros_like(x)
    xs[:, :, :-1] = 0.5 * (x[:, :, :-1] + x[:, :, 1:])
    refh = torch.nn.functional.conv2d(torch.from_numpy(xs), torch.from_numpy(f), padding=1, groups=2).numpy()
    goth = run([nb], [px, po, pf], [x, offh, f])[0]
    np.testing.assert_allclose(goth[:, :, 1:-2], refh[:, :, 1:-2], rtol=1e-4, atol=1e-4)


def test_deformable_psroi_pooling_and_binary_convolution():
    G, OD = 2, 3
    x = np.zeros((1, OD * G * G, 8, 8), np.float32)
    for c in range(OD * G * G):
        x[0, c] = c + 1
    px, pr = ops.parameter(list(x.shape), "f32", "x"), ops.parameter([1, 5], "f32", "r")
    n = ops.deformable_psroi_pooling(px, pr, output_dim=OD, spatial_scale=1.0, group_size=G, spatial_bins_x=2, spatial_bins_y=2)
    out = run([n], [px, pr], [x, np.array([[0, 1, 1, 6, 6]], np.float32)])[0]
    assert out.shape == (1, OD, G, G)
    np.testing.assert_allclose(out[0].reshape(-1), np.arange(1, OD * G * G + 1), rtol=1e-6)       # bin (c, ph, pw) reads plane (c * G + ph) * G + pw
    # with offsets: a shift of the bins on a ramp moves the pooled value by trans_std * roi_width * offset
    ramp = np.tile(np.arange(16, dtype=np.float32), (16, 1))
    xr = np.stack([ramp] * 4)[None]
    pxr, po = ops.parameter([1, 4, 16, 16], "f32", "x"), ops.parameter([1, 2, 2, 2], "f32", "o")
    roi = np.array([[0, 4, 4, 11, 11]], np.float32)
    base = ops.deformable_psroi_pooling(pxr, pr, output_dim=1, spatial_scale=1.0, group_size=2, spatial_bins_x=1, spatial_bins_y=1)
    moved = ops.deformable_psroi_pooling(pxr, pr, po, output_dim=1, spatial_scale=1.0, group_size=2, spatial_bins_x=1, spatial_bins_y=1, trans_std=0.5, part_size=2)
    offs = np.zeros((1, 2, 2, 2), np.float32)
    offs[0, 0] = 0.25                                        # x shift: 0.25 * 0.5 * roi width (8) = 1 pixel
    b = run([base], [pxr, pr], [xr, roi])[0]
    m = run([moved], [pxr, pr, po], [xr, roi, offs])[0]
    np.testing.assert_allclose(m - b, 1.0, rtol=1e-5)
    # binary convolution: +-1 arithmetic
    rng = np.random.default_rng(2)
    xb = rng.standard_normal((1, 3, 5, 6)).astype(np.float32)
    bits = rng.integers(0, 2, (4, 3, 3, 3)).astype(np.uint8)
    pbx = ops.parameter([1, 3, 5, 6], "f32", "x")
    packed = np.packbits(bits.reshape(-1))                   # most significant bit first
    w = ops.constant(ov.Tensor(packed, [4, 3, 3, 3], ov.Type.u1))
    bc = ops.binary_convolution(pbx, w, [1, 1], [1, 1], [1, 1], [1, 1], "xnor-popcount", 0.0)
    assert list(bc.get_output_shape(0)) == [1, 4, 5, 6]
    sx = np.where(xb > 0, 1.0, -1.0).astype(np.float32)
    sx_p = np.pad(sx, ((0, 0), (0, 0), (1, 1), (1, 1)), constant_values=-1.0)               # pad_value 0 reads as the bit 0
    ref = torch.nn.functional.conv2d(torch.from_numpy(sx_p), torch.from_numpy(np.where(bits > 0, 1.0, -1.0).astype(np.float32))).numpy()
    np.testing.assert_array_equal(run([bc], [pbx], [xb])[0], ref)


def test_string_pack_unpack_reverse_xor():
    s = np.array([["Intel", ""], ["OpenVINO", "b200"]])
    ps = ops.parameter([2, 2], "string", "s")
    u = ops.string_tensor_unpack(ps)
    b, e, sym = run([u.output(0), u.output(1), u.output(2)], [ps], [s])
    np.testing.assert_array_equal(b, [[0, 5], [5, 13]])
    np.testing.assert_array_equal(e, [[5, 5], [13, 17]])
    assert bytes(sym.tolist()) == b"IntelOpenVINOb200" and sym.dtype == np.uint8
    pb, pe, py = ops.parameter([2, 2], "i32", "b"), ops.parameter([2, 2], "i32", "e"), ops.parameter([17], "u8", "y")
    back = run([ops.string_tensor_pack(pb, pe, py)], [pb, pe, py], [b, e, sym])[0]
    assert [[v.decode() if isinstance(v, bytes) else v for v in row] for row in back.tolist()] == s.tolist()
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    px = ops.parameter([2, 3, 4], "f32", "x")
    np.testing.assert_array_equal(run([ops.reverse(px, np.array([0, 2], np.int64), "index")], [px], [x])[0], x[::-1, :, ::-1])
    np.testing.assert_array_equal(run([ops.reverse(px, np.array([False, True, False]), "mask")], [px], [x])[0], x[:, ::-1])
    a, c = np.array([True, False, True, False]), np.array([True, True, False, False])
    pa, pc = ops.parameter([4], "boolean", "a"), ops.parameter([4], "boolean", "c")
    np.testing.assert_array_equal(run([ops.logical_xor_v0(pa, pc)], [pa, pc], [a, c])[0], a ^ c)


def test_istft_inverts_stft():
    rng = np.random.default_rng(7)
    sig = rng.standard_normal((2, 96)).astype(np.float32)
    fs, step = 16, 4
    win = np.hamming(fs).astype(np.float32)
    p = ops.parameter([2, 96], "f32", "x")
    spec = ops.stft(p, win, np.int64(fs), np.int64(step), True)               # [batch, bins, frames, 2]
    inv = ops.istft(spec, win, np.int64(fs), np.int64(step), center=False, normalized=False)
    assert list(inv.get_output_shape(0)) == [2, 96]
    np.testing.assert_allclose(run([inv], [p], [sig])[0], sig, rtol=1e-4, atol=1e-4)
    # against torch.istft (centre padding removed), with a given length
    pt = torch.stft(torch.from_numpy(sig), fs, step, window=torch.from_numpy(win), center=True, return_complex=True, pad_mode="reflect")
    data = torch.view_as_real(pt).numpy().astype(np.float32)
    pd = ops.parameter(list(data.shape), "f32", "d")
    inv2 = ops.istft(pd, win, np.int64(fs), np.int64(step), np.int64(90), center=True, normalized=False)
    ref = torch.istft(pt, fs, step, window=torch.from_numpy(win), center=True, length=90).numpy()
    np.testing.assert_allclose(run([inv2], [pd], [data])[0], ref, rtol=1e-4, atol=1e-4)


def test_rgb_to_nv12_planes():
    rng = np.random.default_rng(9)
    img = rng.integers(0, 256, (1, 4, 6, 3)).astype(np.uint8)
    p = ops.parameter([1, 4, 6, 3], "u8", "x")
    two = ops.rgb_to_nv12(p, False)
    assert [list(two.get_output_shape(i)) for i in range(2)] == [[1, 4, 6, 1], [1, 2, 3, 2]]
    y, uv = run([two.output(0), two.output(1)], [p], [img])
    r, g, b = [img[..., i].astype(np.float64) for i in range(3)]
    clip = lambda a: np.clip(np.round(a), 0, 255)
    np.testing.assert_array_equal(y[..., 0], clip(0.257 * r + 0.504 * g + 0.098 * b + 16))
    u = clip(-0.148 * r - 0.291 * g + 0.439 * b + 128).reshape(1, 2, 2, 3, 2).sum((2, 4)) / 4
    v = clip(0.439 * r - 0.368 * g - 0.071 * b + 128).reshape(1, 2, 2, 3, 2).sum((2, 4)) / 4
    np.testing.assert_array_equal(uv[..., 0], np.floor(u + 0.5))          # halves round away from zero
    np.testing.assert_array_equal(uv[..., 1], np.floor(v + 0.5))
    one = ops.bgr_to_nv12(p)
    assert list(one.get_output_shape(0)) == [1, 6, 6, 1]
    whole = run([one], [p], [img[..., ::-1].copy()])[0]
    np.testing.assert_array_equal(whole[0, :4, :, 0], y[0, ..., 0])
    np.testing.assert_array_equal(whole[0, 4:, :, 0].reshape(2, 3, 2), uv[0])
    # and back: NV12 -> RGB of the result stays near the image
    pn = ops.parameter([1, 6, 6, 1], "u8", "n")
    rgb = run([ops.nv12_to_rgb(pn)], [pn], [whole])[0]
    flat = np.full((1, 4, 6, 3), 120, np.uint8)
    whole_flat = run([ops.rgb_to_nv12(p)], [p], [flat])[0]
    assert np.abs(run([ops.nv12_to_rgb(pn)], [pn], [whole_flat])[0].astype(int) - 120).max() <= 2 and rgb.shape == (1, 4, 6, 3)
