"""Element types, dimensions and shapes of the Python API.

Mirrors ``ov.Type`` / ``ov.Dimension`` / ``ov.PartialShape`` / ``ov.Shape``
(src/bindings/python/src/pyopenvino/graph/types/element_type.cpp, partial_shape.cpp, dimension.cpp).
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence, Union

import numpy as np

from . import _ovcore as _c


class Type:
    """Element type. Instances are interned: ``Type.f32 is Type("f32")``."""

    _by_name = {}

    def __new__(cls, name):
        if isinstance(name, Type):
            return name
        if isinstance(name, np.dtype) or (isinstance(name, type) and issubclass(name, np.generic)):
            return cls.from_numpy(name)
        name = _canon(name)
        inst = cls._by_name.get(name)
        if inst is None:
            inst = object.__new__(cls)
            info = _c.type_info(name)
            inst.name, inst.precision, inst.bitwidth, inst.real, inst.signed, inst.quantized = info
            cls._by_name[inst.name] = inst
        return inst

    @property
    def size(self) -> int:
        return (self.bitwidth + 7) // 8

    def is_static(self) -> bool:
        return self.name != "dynamic"

    def is_dynamic(self) -> bool:
        return self.name == "dynamic"

    def is_real(self) -> bool:
        return self.real

    def is_integral(self) -> bool:
        return not self.real and self.name not in ("dynamic", "string")

    def is_signed(self) -> bool:
        return self.signed

    def get_type_name(self) -> str:
        return self.name

    def to_string(self) -> str:
        return self.name

    def to_dtype(self) -> np.dtype:
        """numpy dtype that holds the values (raw container dtype for bf16 and packed types)."""
        return np.dtype(_c.type_numpy_dtype(self.name))

    @classmethod
    def from_numpy(cls, dt) -> "Type":
        dt = np.dtype(dt)
        m = {"bool": "boolean", "float16": "f16", "float32": "f32", "float64": "f64", "int8": "i8", "int16": "i16", "int32": "i32",
             "int64": "i64", "uint8": "u8", "uint16": "u16", "uint32": "u32", "uint64": "u64"}
        if dt.name in m:
            return cls(m[dt.name])
        if dt.kind in ("U", "S", "O"):
            return cls("string")
        raise TypeError("no element type for numpy dtype %s" % dt)

    def __repr__(self):
        return "<Type: '%s'>" % ("dynamic" if self.name == "dynamic" else self.name)

    def __str__(self):
        return self.name

    def __eq__(self, other):
        if isinstance(other, Type):
            return self is other
        if isinstance(other, str):
            try:
                return self is Type(other)
            except Exception:
                return False
        return NotImplemented

    def __hash__(self):
        return hash(self.name)


def _canon(name: str) -> str:
    n = str(name)
    low = n.lower()
    alias = {"undefined": "dynamic", "bool": "boolean", "float32": "f32", "float16": "f16", "float64": "f64", "bfloat16": "bf16",
             "int8": "i8", "int16": "i16", "int32": "i32", "int64": "i64", "uint8": "u8", "uint16": "u16", "uint32": "u32",
             "uint64": "u64", "fp32": "f32", "fp16": "f16", "fp64": "f64", "bin": "u1", "unspecified": "dynamic"}
    return alias.get(low, low)


for _n in _c.type_names():
    setattr(Type, _n, Type(_n))
Type.undefined = Type.dynamic


def get_element_type(x) -> Type:
    return Type(x)


class Symbol:
    """Identity of a dynamic dimension's run-time value: dimensions whose symbols compare equal are known to be the same
    size. ``Symbol()`` makes a fresh one; shape inference makes symbols equal where operands must agree
    (``ov::Symbol``, src/core/include/openvino/core/symbol.hpp)."""

    __slots__ = ("id",)

    def __init__(self, _id: int = 0):
        from . import _ovcore as _c
        self.id = int(_id) if _id else int(_c.new_symbol())

    def root(self) -> int:
        from . import _ovcore as _c
        return int(_c.symbol_root(self.id))

    def __eq__(self, other) -> bool:
        return isinstance(other, Symbol) and self.root() == other.root()

    def __hash__(self) -> int:
        return hash(("Symbol", self.id))

    def __repr__(self) -> str:
        return "<Symbol %d>" % self.root()


class Dimension:
    """A dimension: static value, interval, or fully dynamic (``Dimension()`` / ``Dimension(-1)``)."""

    __slots__ = ("lo", "hi", "sym")

    def has_symbol(self) -> bool:
        return bool(self.sym) and self.is_dynamic

    def get_symbol(self):
        return Symbol(self.sym) if self.has_symbol() else None

    def set_symbol(self, symbol) -> None:
        self.sym = symbol.id if symbol is not None else 0

    def __init__(self, a=None, b=None):
        self.sym = 0
        if isinstance(a, Dimension):
            self.lo, self.hi, self.sym = a.lo, a.hi, a.sym
        elif isinstance(a, str):
            s = a.strip()
            if s in ("?", "-1"):
                self.lo, self.hi = 0, -1
            elif ".." in s:
                l, h = s.split("..")
                self.lo, self.hi = (int(l) if l.strip() else 0), (int(h) if h.strip() else -1)
            else:
                self.lo = self.hi = int(s)
        elif a is None:
            self.lo, self.hi = 0, -1
        elif b is None:
            a = int(a)
            self.lo, self.hi = (0, -1) if a < 0 else (a, a)
        else:
            self.lo, self.hi = int(a), int(b)

    @staticmethod
    def dynamic() -> "Dimension":
        return Dimension()

    @property
    def is_static(self) -> bool:
        return self.lo == self.hi

    @property
    def is_dynamic(self) -> bool:
        return self.lo != self.hi

    def get_length(self) -> int:
        if not self.is_static:
            raise RuntimeError("get_length() called on a dynamic dimension")
        return self.lo

    def get_min_length(self) -> int:
        return self.lo

    def get_max_length(self) -> int:
        return self.hi

    min_length = property(get_min_length)
    max_length = property(get_max_length)

    def compatible(self, other) -> bool:
        o = Dimension(other)
        lo = max(self.lo, o.lo)
        hi = o.hi if self.hi < 0 else (self.hi if o.hi < 0 else min(self.hi, o.hi))
        return hi < 0 or lo <= hi

    def same_scheme(self, other) -> bool:
        o = Dimension(other)
        return (self.is_dynamic and o.is_dynamic) or (self.is_static and o.is_static and self.lo == o.lo)

    def refines(self, other) -> bool:
        o = Dimension(other)
        return self.lo >= o.lo and (o.hi < 0 or (self.hi >= 0 and self.hi <= o.hi))

    def relaxes(self, other) -> bool:
        return Dimension(other).refines(self)

    def to_string(self) -> str:
        if self.is_static:
            return str(self.lo)
        if self.lo > 0:
            return "%d..%s" % (self.lo, self.hi if self.hi >= 0 else "")
        if self.hi >= 0:
            return "..%d" % self.hi
        return "?"

    def __len__(self):
        return self.get_length()

    def __int__(self):
        return self.get_length()

    def __eq__(self, other):
        if isinstance(other, (int, np.integer)):
            return self.is_static and self.lo == int(other)
        if isinstance(other, Dimension):
            return self.lo == other.lo and self.hi == other.hi
        return NotImplemented

    def __hash__(self):
        return hash((self.lo, self.hi))

    def __repr__(self):
        return "<Dimension: %s>" % self.to_string()

    __str__ = to_string


class PartialShape:
    """Shape whose rank and dimensions may be dynamic."""

    def __init__(self, dims=None, _rank_dynamic=False):
        self._rank_dynamic = _rank_dynamic
        if isinstance(dims, PartialShape):
            self._rank_dynamic, self._dims = dims._rank_dynamic, [Dimension(d) for d in dims._dims]
        elif isinstance(dims, str):
            parsed = _c.pshape_parse(dims)
            self._rank_dynamic = parsed is None
            self._dims = [] if parsed is None else [Dimension(l, h) for l, h in parsed]
        elif dims is None:
            self._dims = []
        else:
            self._dims = [d if isinstance(d, Dimension) else (Dimension(*d) if isinstance(d, (tuple, list)) else Dimension(d)) for d in dims]

    @staticmethod
    def dynamic(rank=None) -> "PartialShape":
        if rank is None:
            return PartialShape(None, _rank_dynamic=True)
        r = rank.get_length() if isinstance(rank, Dimension) else int(rank)
        return PartialShape([Dimension() for _ in range(r)])

    @staticmethod
    def _from_core(raw) -> "PartialShape":
        if raw is None:
            return PartialShape.dynamic()
        dims = []
        for item in raw:
            d = Dimension(item[0], item[1])
            if len(item) > 2:
                d.sym = int(item[2])
            dims.append(d)
        return PartialShape(dims)

    def _to_core(self):
        return None if self._rank_dynamic else [(d.lo, d.hi, d.sym) if d.sym else (d.lo, d.hi) for d in self._dims]

    @property
    def rank(self) -> Dimension:
        return Dimension() if self._rank_dynamic else Dimension(len(self._dims))

    @property
    def is_static(self) -> bool:
        return not self._rank_dynamic and all(d.is_static for d in self._dims)

    @property
    def is_dynamic(self) -> bool:
        return not self.is_static

    def get_shape(self) -> "Shape":
        if not self.is_static:
            raise RuntimeError("get_shape() called on a dynamic shape %s" % self)
        return Shape([d.lo for d in self._dims])

    to_shape = get_shape

    def get_min_shape(self) -> "Shape":
        return Shape([d.lo for d in self._dims])

    def get_max_shape(self) -> "Shape":
        return Shape([d.hi for d in self._dims])

    def get_dimension(self, i: int) -> Dimension:
        return self._dims[i]

    def compatible(self, other) -> bool:
        o = PartialShape(other)
        if self._rank_dynamic or o._rank_dynamic:
            return True
        return len(self._dims) == len(o._dims) and all(a.compatible(b) for a, b in zip(self._dims, o._dims))

    def same_scheme(self, other) -> bool:
        o = PartialShape(other)
        if self._rank_dynamic or o._rank_dynamic:
            return self._rank_dynamic and o._rank_dynamic
        return len(self._dims) == len(o._dims) and all(a.same_scheme(b) for a, b in zip(self._dims, o._dims))

    def refines(self, other) -> bool:
        o = PartialShape(other)
        if o._rank_dynamic:
            return True
        if self._rank_dynamic:
            return False
        return len(self._dims) == len(o._dims) and all(a.refines(b) for a, b in zip(self._dims, o._dims))

    def relaxes(self, other) -> bool:
        return PartialShape(other).refines(self)

    def to_string(self) -> str:
        if self._rank_dynamic:
            return "[...]"
        return "[" + ",".join(d.to_string() for d in self._dims) + "]"

    def __len__(self):
        if self._rank_dynamic:
            raise RuntimeError("len() of a shape with dynamic rank")
        return len(self._dims)

    def __getitem__(self, i):
        if isinstance(i, slice):
            return PartialShape(self._dims[i])
        return self._dims[i]

    def __setitem__(self, i, v):
        self._dims[i] = v if isinstance(v, Dimension) else Dimension(v)

    def __iter__(self):
        return iter(self._dims)

    def __eq__(self, other):
        if isinstance(other, (PartialShape, Shape, list, tuple)):
            o = PartialShape(other) if not isinstance(other, PartialShape) else other
            return self._rank_dynamic == o._rank_dynamic and self._dims == o._dims
        return NotImplemented

    def __hash__(self):
        return hash((self._rank_dynamic, tuple(self._dims)))

    def __repr__(self):
        return "<PartialShape: %s>" % self.to_string()

    __str__ = to_string


class Shape(list):
    """Static shape: a list of ints."""

    def __init__(self, dims: Union[Iterable[int], "Shape", str, None] = None):
        if isinstance(dims, str):
            s = dims.strip().strip("[]{}")
            dims = [int(t) for t in s.split(",") if t.strip()]
        super().__init__(int(d) for d in (dims or []))

    def to_string(self) -> str:
        return "[" + ",".join(str(d) for d in self) + "]"

    def __repr__(self):
        return "<Shape: %s>" % self.to_string()

    __str__ = to_string

    def __hash__(self):
        return hash(tuple(self))


def shape_size(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n
