"""Packing of u1 / u4 / i4 / nf4 values into bytes and back (the storage of ``ov.Tensor`` for those types): u1 most
significant bit first, 4-bit types low nibble first."""
from __future__ import annotations

import numpy as np

from .._types import Type

_BITS = {"u1": 1, "u4": 4, "i4": 4, "nf4": 4, "f4e2m1": 4}


def pack_data(array: np.ndarray, type) -> np.ndarray:
    t = Type(type)
    bits = _BITS.get(t.name)
    if bits is None:
        raise ValueError("%s is not a packed element type" % t.name)
    flat = np.asarray(array).reshape(-1)
    if bits == 1:
        return np.packbits((flat != 0).astype(np.uint8))
    v = (flat.astype(np.int64) & 0xF).astype(np.uint8)
    if v.size % 2:
        v = np.concatenate([v, np.zeros(1, np.uint8)])
    return (v[0::2] | (v[1::2] << 4)).astype(np.uint8)


def unpack_data(array: np.ndarray, type, shape) -> np.ndarray:
    t = Type(type)
    bits = _BITS.get(t.name)
    if bits is None:
        raise ValueError("%s is not a packed element type" % t.name)
    n = int(np.prod(list(shape))) if len(list(shape)) else 1
    raw = np.asarray(array, dtype=np.uint8).reshape(-1)
    if bits == 1:
        return np.unpackbits(raw)[:n].reshape(list(shape))
    v = np.empty(raw.size * 2, np.uint8)
    v[0::2], v[1::2] = raw & 0xF, raw >> 4
    v = v[:n]
    if t.name == "i4":
        return ((v.astype(np.int8) ^ 8) - 8).reshape(list(shape))
    return v.reshape(list(shape))
