"""Operations defined in Python (``ov.Op``) and their registration with the native operation registry.

A sub-class names its type with ``class_type_info = DiscreteTypeInfo("MyOp", "extension")`` (or ``op_type`` /
``op_version`` attributes), implements ``validate_and_infer_types`` with ``set_output_type`` calls and, to run on the
CPU device / in constant folding, ``evaluate(outputs, inputs)``. Instances are ordinary graph nodes: they serialise to IR
with their attributes, clone, and take part in passes. Reference API: src/bindings/python/src/openvino/_op_base.py and
pyopenvino/graph/op.cpp (the PyOp trampoline); ``register_op`` is the functional form of the same thing.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from . import _ovcore as _c
from ._graph import Node, Output, as_output, _attr_to_core
from ._tensor import Tensor
from ._types import PartialShape, Type

_registered: Dict[tuple, type] = {}


class DiscreteTypeInfo:
    def __init__(self, name: str, version_id: str = "extension", parent=None):
        self.name, self.version_id, self.parent = name, version_id, parent

    def __repr__(self):
        return "<DiscreteTypeInfo %s:%s>" % (self.name, self.version_id)


def register_op(op_type: str, infer: Callable[[Node], Sequence[tuple]], evaluate: Optional[Callable] = None, version: str = "extension",
                attrs: Optional[dict] = None) -> None:
    """Register an operation type. ``infer(node) -> [(Type | name, PartialShape | dims), ...]`` per output;
    ``evaluate(node, [np.ndarray, ...]) -> [np.ndarray, ...]`` (optional); ``attrs``: attribute name -> default value
    (its Python type fixes how the attribute is parsed when a model is read back from IR)."""
    def infer_cb(core_node):
        outs = []
        for et, ps in infer(Node(core_node)):
            name = Type(et).name
            ps = ps if isinstance(ps, PartialShape) else PartialShape(list(ps))
            outs.append((name, ps._to_core()))
        return outs

    eval_cb = None
    if evaluate is not None:
        def eval_cb(core_node, packed):
            ins = [Tensor._from_core(p).data for p in packed]
            res = evaluate(Node(core_node), ins)
            if res is None:
                return None
            out = []
            for a in res:
                t = a if isinstance(a, Tensor) else Tensor(np.ascontiguousarray(a))
                out.append((np.ascontiguousarray(t.data), Type(t.element_type).name))
            return out
    _c.register_custom_op(op_type, version, infer_cb, eval_cb, {k: _attr_to_core(v) for k, v in (attrs or {}).items()})


class Op(Node):
    """Base class of Python-defined operations."""

    class_type_info: Optional[DiscreteTypeInfo] = None

    @classmethod
    def _type_and_version(cls):
        ti = cls.class_type_info
        if ti is not None:
            return ti.name, ti.version_id
        return getattr(cls, "op_type", cls.__name__), getattr(cls, "op_version", "extension")

    @classmethod
    def _ensure_registered(cls, attrs: Optional[dict] = None):
        key = cls._type_and_version()
        if _registered.get(key) is cls:
            return
        _registered[key] = cls

        def proxy(core_node):
            obj = cls.__new__(cls)
            Node.__init__(obj, core_node)
            obj._out_types = {}
            return obj

        def infer(node):
            obj = proxy(node._n)
            obj.validate_and_infer_types()
            n = max(obj._out_types) + 1 if obj._out_types else 1
            return [obj._out_types.get(i, (node.get_input_element_type(0), node.get_input_partial_shape(0))) for i in range(n)]

        def evaluate(node, ins):
            obj = proxy(node._n)
            if not obj.has_evaluate():
                return None
            outs = []
            for i in range(node.get_output_size()):
                ps = node.get_output_partial_shape(i)
                shape = list(ps.to_shape()) if ps.is_static else [0]
                outs.append(Tensor(node.get_output_element_type(i), shape))
            ok = obj.evaluate(outs, [Tensor(np.ascontiguousarray(a)) for a in ins])
            return outs if ok is not False else None

        has_eval = cls.evaluate is not Op.evaluate
        register_op(key[0], infer, evaluate if has_eval else None, key[1], attrs)

    def __init__(self, inputs: Optional[Sequence] = None, attrs: Optional[dict] = None, name: Optional[str] = None):
        cls = type(self)
        cls._ensure_registered(attrs)
        t, v = cls._type_and_version()
        ins = [as_output(i)._core() for i in (inputs or [])]
        core = _c.make_node(t, v, ins, {k: _attr_to_core(val) for k, val in (attrs or {}).items() if val is not None})
        Node.__init__(self, core)
        self._out_types = {}
        if name:
            self.set_friendly_name(name)

    # ---- the methods a sub-class implements / calls
    def validate_and_infer_types(self) -> None:
        self.set_output_type(0, self.get_input_element_type(0), self.get_input_partial_shape(0))

    def set_output_type(self, index: int, element_type, partial_shape) -> None:
        self._out_types[index] = (element_type, partial_shape)

    def evaluate(self, outputs: List[Tensor], inputs: List[Tensor]) -> bool:
        return False

    def has_evaluate(self) -> bool:
        return type(self).evaluate is not Op.evaluate

    def get_type_info(self):
        t, v = self._type_and_version()
        return DiscreteTypeInfo(t, v)

    def constructor_validate_and_infer_types(self) -> None:
        self.validate()
