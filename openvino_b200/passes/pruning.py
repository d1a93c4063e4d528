"""Structured pruning: output channels whose weights are all zero are removed from the graph.

A mask (the set of dead output channels) starts at every Convolution / MatMul weight constant and is propagated
forward through operations that keep the channel axis (element-wise ops with per-channel or scalar constants, ReLU-like
activations, pooling, BatchNorm); it is consumed by the next Convolution / MatMul, whose input channels are cut to
match. When every path from the producer ends in such a consumer the channels are physically removed from the
producer's weights, the constants on the way and the consumers' weights. Role of
src/common/offline_transformations/src/pruning/{init_masks,propagate_masks,shrink_weights}.cpp.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Set, Tuple

import numpy as np

from .. import opset as ops
from .._graph import Model, Node, Output
from . import ModelPass

_KEEP_AXIS = {"Relu", "PRelu", "Sigmoid", "Tanh", "Clamp", "Elu", "Gelu", "Swish", "HSwish", "Mish", "MaxPool", "AvgPool", "Convert"}
_ELTWISE = {"Add", "Subtract", "Multiply", "Divide", "Maximum", "Minimum"}


def _weights(n: Node) -> Optional[Node]:
    w = n.input_value(1).get_node()
    return w if w.get_type_name() == "Constant" else None


def _is_zero_preserving_path_const(c: np.ndarray, channels: int) -> bool:
    return c.size == 1 or (c.size == channels and c.ndim >= 2 and c.shape[1] == channels) or (c.size == channels and c.ndim == 1)


class Pruning(ModelPass):
    def run_on_model(self, model: Model) -> bool:
        changed = False
        for conv in model.get_ordered_ops():
            if conv.get_type_name() != "Convolution":
                continue
            w = _weights(conv)
            if w is None:
                continue
            wd = np.asarray(w.get_data())
            dead = [c for c in range(wd.shape[0]) if not np.any(wd[c])]
            if not dead or len(dead) == wd.shape[0]:
                continue
            plan = self._plan(conv, wd.shape[0], dead)
            if plan is None:
                continue
            keep = np.array([c for c in range(wd.shape[0]) if c not in set(dead)])
            consts, consumers = plan
            # dead channels must be exactly zero at every consumer: an Add with a non-zero entry there keeps them alive
            self._set_const(w, wd[keep])
            for c, axis in consts:
                self._set_const(c, np.take(np.asarray(c.get_data()), keep, axis=axis))
            for cons in consumers:
                cw = _weights(cons)
                data = np.asarray(cw.get_data())
                self._set_const(cw, np.take(data, keep, axis=1))
            changed = True
        if changed:
            model.validate_nodes_and_infer_types()
        return changed

    @staticmethod
    def _set_const(node: Node, value: np.ndarray) -> None:
        new = ops.constant(np.ascontiguousarray(value))
        new.set_friendly_name(node.get_friendly_name())
        for inp in list(node.output(0).get_target_inputs()):
            inp.replace_source_output(new.output(0))

    def _plan(self, producer: Node, channels: int, dead: List[int]):
        """Walk forward from `producer`; -> (constants to slice [(node, axis)], consuming convolutions) or None."""
        consts: List[Tuple[Node, int]] = []
        consumers: List[Node] = []
        seen: Set[int] = set()
        stack = [producer.output(0)]
        while stack:
            out = stack.pop()
            for inp in out.get_target_inputs():
                n = inp.get_node()
                t = n.get_type_name()
                if t == "Convolution" and inp.get_index() == 0 and _weights(n) is not None:
                    if n not in consumers:
                        consumers.append(n)
                    continue
                if id(n._n) in seen:
                    continue
                if t in _KEEP_AXIS:
                    seen.add(id(n._n))
                    stack.append(n.output(0))
                    continue
                if t in _ELTWISE:
                    other = n.input_value(1 - inp.get_index()).get_node()
                    if other.get_type_name() != "Constant":
                        return None
                    c = np.asarray(other.get_data())
                    if not _is_zero_preserving_path_const(c, channels):
                        return None
                    if c.size == channels:
                        axis = 1 if c.ndim >= 2 else 0
                        # an additive constant must not revive a dead channel
                        if t in ("Add", "Subtract") and np.any(np.take(c, dead, axis=axis)):
                            return None
                        consts.append((other, axis))
                    elif t in ("Add", "Subtract") and float(c.reshape(-1)[0]) != 0.0:
                        return None
                    seen.add(id(n._n))
                    stack.append(n.output(0))
                    continue
                return None       # Result, Reshape, Concat ...: the channel axis is observable, keep everything
        return (consts, consumers) if consumers else None
