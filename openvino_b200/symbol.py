"""Symbol helpers (``ov::symbol::are_equal`` / ``set_equal``, src/core/include/openvino/core/symbol.hpp)."""
from . import _ovcore as _c
from ._types import Symbol


def are_equal(a: Symbol, b: Symbol) -> bool:
    return a is not None and b is not None and a == b


def set_equal(a: Symbol, b: Symbol) -> None:
    _c.symbols_set_equal(a.id, b.id)


def ancestor_of(a: Symbol) -> Symbol:
    """The representative of the class that ``a`` belongs to."""
    return Symbol(a.root())
