"""Small public types and helpers of the reference's Python package that have no weight of their own: index / axis
containers, ``OVAny``, the extension bases, batch helpers and ``tensor_from_file``.
Reference: src/bindings/python/src/pyopenvino/{core/common.cpp,graph/{coordinate,axis_set,axis_vector,strides,any}.cpp},
src/bindings/python/src/openvino/{_ov_api.py,utils/data_helpers}."""
from __future__ import annotations

from typing import Any, Iterable, List

import numpy as np


class _IntList(list):
    """A list of integers with the constructors of the reference's containers (iterable or another instance)."""

    def __init__(self, values: Iterable[int] = ()):
        super().__init__(int(v) for v in values)

    def __repr__(self):
        return "<%s: (%s)>" % (type(self).__name__, ", ".join(str(v) for v in self))


class Coordinate(_IntList):
    pass


class CoordinateDiff(_IntList):
    pass


class Strides(_IntList):
    pass


class AxisVector(_IntList):
    pass


class AxisSet(set):
    def __init__(self, values: Iterable[int] = ()):
        super().__init__(int(v) for v in values)

    def to_vector(self) -> List[int]:
        return sorted(self)

    def __repr__(self):
        return "<AxisSet {%s}>" % ", ".join(str(v) for v in sorted(self))


class OVAny:
    """A value of any type with the accessors user code expects (``value``, ``get``, ``astype``, ``aslist``)."""

    def __init__(self, value: Any):
        self._v = value._v if isinstance(value, OVAny) else value

    @property
    def value(self):
        return self._v

    def get(self):
        return self._v

    def set(self, value) -> None:
        self._v = value

    def astype(self, t):
        if t is bool and isinstance(self._v, str):
            return self._v.strip().upper() in ("YES", "TRUE", "1", "ON")
        return t(self._v)

    def aslist(self, t=None) -> list:
        v = self._v
        if isinstance(v, str):
            v = [x for x in v.replace(",", " ").split() if x]
        v = list(v) if isinstance(v, (list, tuple, set)) else [v]
        return [t(x) for x in v] if t is not None else v

    def __eq__(self, other):
        return self._v == (other._v if isinstance(other, OVAny) else other)

    def __hash__(self):
        return hash(repr(self._v))

    def __repr__(self):
        return "<OVAny %r>" % (self._v,)


class Extension:
    """Base of the objects ``Core.add_extension`` / ``FrontEnd.add_extension`` accept."""


class OpExtension(Extension):
    """Makes an operation type known to the core, so that models which hold it can be read, built and evaluated:
    ``OpExtension(MyOp)`` with a sub-class of ``ov.Op``. The frontend form ``OpExtension("TargetOp", "SourceOp", attr_map)``
    maps a source-framework operation onto a registered operation with renamed / preset attributes."""

    def __init__(self, op, fw_type: str = None, attr_names_map: dict = None, attr_values_map: dict = None):
        self.op, self.fw_type = op, fw_type
        self.attr_names_map, self.attr_values_map = dict(attr_names_map or {}), dict(attr_values_map or {})

    def register(self) -> None:
        if isinstance(self.op, type):
            self.op._ensure_registered()


def get_batch(model):
    """Extent of the batch axis ('N' of the parameters' layouts, axis 0 without a layout); all inputs must agree."""
    from ._types import Dimension
    found = None
    for p in model.get_parameters():
        ps = p.get_output_partial_shape(0)
        if not ps.rank.is_static or len(ps) == 0:
            continue
        idx = _batch_index(p)
        d = ps[idx]
        if found is None:
            found = d
        elif found.is_static and d.is_static and found.get_length() != d.get_length():
            raise RuntimeError("model inputs disagree about the batch size")
        elif not d.is_static:
            found = d
    return found if found is not None else Dimension()


def set_batch(model, batch) -> None:
    shapes = {}
    for i, p in enumerate(model.get_parameters()):
        ps = p.get_output_partial_shape(0)
        if not ps.rank.is_static or len(ps) == 0:
            continue
        dims = list(ps)
        dims[_batch_index(p)] = batch
        shapes[i] = dims
    model.reshape(shapes)


def _batch_index(param) -> int:
    try:
        from .preprocess import Layout, layout_helpers
        lay = param.get_rt_info().get("layout_0")
        if lay:
            lay = lay if isinstance(lay, Layout) else Layout(str(lay))
            if layout_helpers.has_batch(lay):
                return int(layout_helpers.batch_idx(lay))
    except Exception:   # noqa: BLE001 - no usable layout: the first axis
        pass
    return 0


def tensor_from_file(path: str):
    """The bytes of a file as a 1-D u8 tensor."""
    from ._tensor import Tensor
    return Tensor(np.fromfile(path, dtype=np.uint8))
