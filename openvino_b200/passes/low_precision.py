"""Low-precision transformations: FakeQuantize graphs -> integer tensors with explicit dequantisation.

Three steps, run in this order by ``LowPrecision``:

* ``CompressQuantizeWeights`` - a FakeQuantize over a constant is evaluated offline: the constant is stored as i8/u8
  and followed by ``Convert -> Subtract(zero point) -> Multiply(scale)`` (reference:
  src/common/offline_transformations/src/compress_quantize_weigths.cpp).
* ``FakeQuantizeDecomposition`` - a FakeQuantize over an activation becomes a FakeQuantize whose output interval is
  the integer range, a Convert to u8/i8, and the dequantisation chain ``Convert(f32) -> Subtract -> Multiply``
  (reference: src/common/low_precision_transformations/src/fake_quantize_decomposition.cpp).
* ``MoveDequantizationAfter`` - for MatMul and Convolution whose both inputs end in such chains the Multiply scales are
  moved behind the operation (the op then runs on integer-valued tensors and one rescale follows it), and chains pass
  through MaxPool / Reshape / Transpose / ReLU unchanged (reference: the per-operation transformations
  mat_mul.cpp, convolution.cpp, max_pool.cpp, reshape.cpp, transpose.cpp, relu.cpp of the same directory, driven by
  low_precision.cpp:230-330).

The integer-valued graph is bit-exact against the FakeQuantize form on the CPU executor up to float rounding of the
rescale, which is how the reference tests the family (LayerTransformation tests compare both forms).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np

from .. import opset as ops
from .._graph import Model, Node, Output
from . import ModelPass


def _const(o: Output) -> Optional[np.ndarray]:
    n = o.get_node()
    while n.get_type_name() == "Convert" and n.input_value(0).get_node().get_type_name() == "Constant":
        return n.input_value(0).get_node().get_data().astype(np.float32)
    if n.get_type_name() != "Constant":
        return None
    return np.asarray(n.get_data())


def _replace(old: Output, new: Output) -> None:
    for inp in list(old.get_target_inputs()):
        inp.replace_source_output(new)


def _fq_params(fq: Node) -> Optional[Tuple[np.ndarray, np.ndarray, np.ndarray, np.ndarray, int]]:
    vals = [_const(fq.input_value(i)) for i in range(1, 5)]
    if any(v is None for v in vals):
        return None
    il, ih, ol, oh = (v.astype(np.float32) for v in vals)
    return il, ih, ol, oh, int(fq.get_attribute("levels"))


class CompressQuantizeWeights(ModelPass):
    def run_on_model(self, model: Model) -> bool:
        changed = False
        for fq in model.get_ops():
            if fq.get_type_name() != "FakeQuantize":
                continue
            w = _const(fq.input_value(0))
            prm = _fq_params(fq)
            if w is None or prm is None:
                continue
            il, ih, ol, oh, levels = prm
            if levels > 256:
                continue
            w = w.astype(np.float32)
            q = np.round((np.clip(w, il, ih) - il) / np.maximum(ih - il, 1e-30) * (levels - 1))
            scale = (oh - ol) / (levels - 1)
            safe = np.where(scale == 0, 1.0, scale)
            zp = -ol / safe                                   # in units of q: value = (q - zp) * scale
            signed = bool(np.all(np.abs(zp - np.round(zp)) < 1e-3) and np.all(np.round(zp) == (levels // 2)))
            if signed:                                        # symmetric around the middle level: store i8, no zero point
                qc = ops.constant((q - levels // 2).astype(np.int8))
                deq = ops.convert(qc, "f32").output(0)
            else:
                qc = ops.constant(q.astype(np.uint8))
                deq = ops.convert(qc, "f32").output(0)
                if np.any(zp != 0):
                    deq = ops.subtract(deq, ops.constant(zp.astype(np.float32))).output(0)
            deq = ops.multiply(deq, ops.constant(scale.astype(np.float32))).output(0)
            deq.get_node().set_friendly_name(fq.get_friendly_name())
            _replace(fq.output(0), deq)
            changed = True
        if changed:
            model.validate_nodes_and_infer_types()
        return changed


class FakeQuantizeDecomposition(ModelPass):
    def run_on_model(self, model: Model) -> bool:
        changed = False
        for fq in model.get_ops():
            if fq.get_type_name() != "FakeQuantize" or _const(fq.input_value(0)) is not None:
                continue
            prm = _fq_params(fq)
            if prm is None:
                continue
            il, ih, ol, oh, levels = prm
            if levels > 256 or ol.size != 1 or oh.size != 1:
                continue                                       # per-tensor activations only
            lo, hi = float(ol.reshape(-1)[0]), float(oh.reshape(-1)[0])
            if hi <= lo:
                continue
            scale = (hi - lo) / (levels - 1)
            signed = lo < 0
            if signed:
                q_lo = float(np.round(lo / scale))
                q_hi = q_lo + levels - 1
                dtype = "i8"
            else:
                q_lo, q_hi, dtype = 0.0, float(levels - 1), "u8"
            zp = q_lo - lo / scale                             # value = (q - zp) * scale
            new_fq = ops.fake_quantize(fq.input_value(0), fq.input_value(1), fq.input_value(2),
                                       ops.constant(np.float32(q_lo)), ops.constant(np.float32(q_hi)), levels)
            q = ops.convert(new_fq, dtype)
            deq = ops.convert(q, "f32").output(0)
            if abs(zp) > 1e-6:
                deq = ops.subtract(deq, ops.constant(np.float32(zp))).output(0)
            deq = ops.multiply(deq, ops.constant(np.float32(scale))).output(0)
            deq.get_node().set_friendly_name(fq.get_friendly_name())
            _replace(fq.output(0), deq)
            changed = True
        if changed:
            model.validate_nodes_and_infer_types()
        return changed


def _dequantization(o: Output):
    """-> (integer-valued f32 output before the Multiply, scale array) when `o` is `... -> Multiply(const)`."""
    n = o.get_node()
    if n.get_type_name() != "Multiply":
        return None
    for data_i, scale_i in ((0, 1), (1, 0)):
        s = _const(n.input_value(scale_i))
        if s is None:
            continue
        src = n.input_value(data_i)
        if _from_integers(src):
            return src, s.astype(np.float32)
    return None


def _from_integers(o: Output) -> bool:
    """The value is a low-precision integer tensor behind Convert / zero-point Subtract / shape-only operations."""
    walk = o.get_node()
    for _ in range(16):
        t = walk.get_type_name()
        if t == "Convert":
            return walk.input_value(0).get_element_type().get_type_name() in ("i8", "u8", "i4", "u4")
        if t == "Subtract" or t in _PASS_THROUGH:
            walk = walk.input_value(0).get_node()
            continue
        return False
    return False


_PASS_THROUGH = ("MaxPool", "Reshape", "Transpose", "Relu", "Squeeze", "Unsqueeze")


class MoveDequantizationAfter(ModelPass):
    def run_on_model(self, model: Model) -> bool:
        changed = False
        for n in model.get_ordered_ops():
            t = n.get_type_name()
            if t in _PASS_THROUGH:
                d = _dequantization(n.input_value(0))
                if d is None or d[1].size != 1 or (t == "Relu" and float(d[1].reshape(-1)[0]) < 0):
                    continue
                src, s = d
                if t == "Relu" and src.get_node().get_type_name() == "Subtract":
                    continue                                   # ReLU commutes with a positive scale only
                moved = n.clone_with_new_inputs([src] + [n.input_value(i) for i in range(1, n.get_input_size())])
                out = ops.multiply(moved.output(0), ops.constant(s.reshape(()))).output(0)
                out.get_node().set_friendly_name(n.get_friendly_name())
                _replace(n.output(0), out)
                changed = True
            elif t in ("MatMul", "Convolution"):
                a, b = _dequantization(n.input_value(0)), _dequantization(n.input_value(1))
                if a is None or b is None or a[1].size != 1:
                    continue
                (sa_src, sa), (sb_src, sb) = a, b
                # weight scale: per tensor, or per output channel
                if t == "Convolution":
                    if not (sb.size == 1 or (sb.ndim >= 1 and sb.shape[0] == sb.size)):
                        continue
                    rank = len(n.get_output_partial_shape(0))
                    post = (sa.reshape(()) * sb.reshape(-1)).reshape([1, -1] + [1] * (rank - 2)) if sb.size > 1 else sa.reshape(()) * sb.reshape(())
                else:
                    tb = bool(n.get_attribute("transpose_b"))
                    if sb.size != 1:
                        shp = list(sb.shape)
                        out_axis = len(shp) - 2 if tb else len(shp) - 1
                        if int(np.prod(shp)) != shp[out_axis]:
                            continue
                        post = (sa.reshape(()) * sb.reshape(-1)).reshape(-1)
                    else:
                        post = sa.reshape(()) * sb.reshape(())
                moved = n.clone_with_new_inputs([sa_src, sb_src] + [n.input_value(i) for i in range(2, n.get_input_size())])
                out = ops.multiply(moved.output(0), ops.constant(np.asarray(post, dtype=np.float32))).output(0)
                out.get_node().set_friendly_name(n.get_friendly_name())
                _replace(n.output(0), out)
                changed = True
        if changed:
            model.validate_nodes_and_infer_types()
        return changed


class LowPrecision(ModelPass):
    """The whole family in pipeline order."""

    def run_on_model(self, model: Model) -> bool:
        changed = CompressQuantizeWeights().run_on_model(model)
        changed = FakeQuantizeDecomposition().run_on_model(model) or changed
        while MoveDequantizationAfter().run_on_model(model):
            changed = True
        return changed


def is_quantized(model: Model) -> bool:
    """True when the model carries FakeQuantize operations (reference: LowPrecision::isFunctionQuantized)."""
    return any(n.get_type_name() == "FakeQuantize" for n in model.get_ops())
