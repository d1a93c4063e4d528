"""``ov.Tensor``: host tensors backed by numpy memory, device tensors backed by ``torch`` CUDA memory.

Reference: ov::Tensor (src/core/include/openvino/runtime/tensor.hpp:55-242) and its Python binding
(src/bindings/python/src/pyopenvino/core/tensor.cpp): construction from a type + shape, from a numpy array
(copy or ``shared_memory``), from an array re-interpreted as another type (packed u4/i4/..., bf16), ROI
views, ``data`` as a numpy view, settable ``shape``, ``copy_to`` / ``copy_from``, string tensors.
"""
from __future__ import annotations

import sys
from typing import Optional, Sequence

import numpy as np

from . import _ovcore as _c
from ._types import PartialShape, Shape, Type, shape_size


class Tensor:
    def __init__(self, array=None, shape=None, type=None, shared_memory: bool = False, *, begin=None, end=None):
        self._torch = None      # device tensor (torch.Tensor on CUDA) when this is a remote tensor
        self._strings = None
        if isinstance(array, Tensor) and begin is not None:
            # ROI view
            idx = tuple(slice(int(b), int(e)) for b, e in zip(begin, end))
            self._type = array._type
            self._data = array.data[idx]
            self._shape = Shape(self._data.shape)
            return
        if isinstance(array, Tensor):
            self._type, self._shape, self._data, self._strings, self._torch = array._type, Shape(array._shape), array._data, array._strings, array._torch
            return
        if isinstance(array, (Type, str)) or (array is not None and not hasattr(array, "__len__") and not hasattr(array, "shape") and shape is not None and type is None and not np.isscalar(array)):
            # Tensor(type, shape)
            self._type = Type(array)
            self._shape = Shape(shape if shape is not None else [])
            if self._type == Type.string:
                self._strings = [b""] * shape_size(self._shape)
                self._data = None
            else:
                n = _c.type_byte_size(self._type.name, shape_size(self._shape))
                self._data = self._alloc(n)
            return
        try:
            torch = sys.modules.get("torch")      # a torch tensor can only arrive if the caller imported torch already
            if torch is None:
                raise ImportError
            if isinstance(array, torch.Tensor):
                if array.is_cuda:
                    self._torch = array
                    self._type = _torch_type(array.dtype)
                    self._shape = Shape(array.shape)
                    self._data = None
                    return
                array = array.detach()
                if array.dtype == torch.bfloat16:
                    arr = array.contiguous().view(torch.int16).numpy().view(np.uint16)
                    self._type, self._shape = Type.bf16, Shape(arr.shape)
                    self._data = arr if shared_memory else arr.copy()
                    return
                array = array.numpy()
        except ImportError:
            pass
        arr = np.asarray(array)
        if arr.dtype.kind in ("U", "S", "O"):
            self._type = Type.string
            self._shape = Shape(arr.shape)
            self._strings = [s if isinstance(s, bytes) else str(s).encode() for s in arr.reshape(-1).tolist()]
            self._data = None
            return
        if type is not None:
            # re-interpret the array's memory as `type` with logical `shape`
            self._type = Type(type)
            self._shape = Shape(shape if shape is not None else arr.shape)
            need = _c.type_byte_size(self._type.name, shape_size(self._shape))
            flat = np.ascontiguousarray(arr).reshape(-1).view(np.uint8)
            if flat.nbytes < need:
                raise ValueError("array of %d bytes is too small for %s of %s" % (flat.nbytes, self._shape, self._type))
            buf = flat[:need] if shared_memory else flat[:need].copy()
            self._data = self._typed_view(buf)
            return
        self._type = Type.from_numpy(arr.dtype)
        if shared_memory:
            if not arr.flags["C_CONTIGUOUS"]:
                raise RuntimeError("shared_memory needs a C-contiguous array")
            self._data = arr
        else:
            self._data = np.array(arr, copy=True, order="C")
        self._shape = Shape(self._data.shape if shape is None else shape)
        if shape is not None:
            self._data = self._data.reshape(self._shape)

    # ------------------------------------------------------------------ helpers
    def _alloc(self, nbytes: int) -> np.ndarray:
        raw = np.zeros(max(nbytes, 0), dtype=np.uint8)
        return self._typed_view(raw)

    def _typed_view(self, raw_u8: np.ndarray) -> np.ndarray:
        t = self._type
        if t.bitwidth % 8 == 0 and t.bitwidth >= 8:
            return raw_u8.view(t.to_dtype()).reshape(self._shape)
        return raw_u8   # packed sub-byte types: flat byte container

    @staticmethod
    def _from_core(packed) -> "Tensor":
        arr, et, shape = packed
        t = Tensor.__new__(Tensor)
        t._torch = None
        t._strings = None
        t._type = Type(et)
        t._shape = Shape(shape)
        if t._type == Type.string:
            t._strings = list(arr)
            t._data = None
        else:
            t._data = arr
        return t

    def _to_core(self):
        """(array, element type name, logical shape) triple understood by the native core."""
        if self._torch is not None:
            return (self.data, self._type.name, list(self._shape))
        if self._type == Type.string:
            return (list(self._strings), "string", list(self._shape))
        return (self._data, self._type.name, list(self._shape))

    # ------------------------------------------------------------------ API
    @property
    def element_type(self) -> Type:
        return self._type

    def get_element_type(self) -> Type:
        return self._type

    @property
    def shape(self) -> Shape:
        return Shape(self._shape)

    @shape.setter
    def shape(self, new_shape):
        self.set_shape(new_shape)

    def get_shape(self) -> Shape:
        return Shape(self._shape)

    def set_shape(self, new_shape) -> None:
        new_shape = Shape(new_shape)
        if self._torch is not None:
            import torch
            self._torch = torch.empty(tuple(new_shape), dtype=self._torch.dtype, device=self._torch.device)
        elif self._type == Type.string:
            self._strings = (self._strings + [b""] * shape_size(new_shape))[: shape_size(new_shape)]
        else:
            need = _c.type_byte_size(self._type.name, shape_size(new_shape))
            if self._data is not None and self._data.nbytes >= need and self._data.flags["C_CONTIGUOUS"] and self._data.flags["OWNDATA"]:
                raw = self._data.reshape(-1).view(np.uint8)[:need]
            else:
                raw = np.zeros(need, dtype=np.uint8)
            self._shape = new_shape
            self._data = self._typed_view(raw)
        self._shape = new_shape

    @property
    def size(self) -> int:
        return shape_size(self._shape)

    def get_size(self) -> int:
        return self.size

    @property
    def byte_size(self) -> int:
        return _c.type_byte_size(self._type.name, self.size)

    def get_byte_size(self) -> int:
        return self.byte_size

    @property
    def strides(self):
        if self._data is None or self._type.bitwidth < 8:
            raise RuntimeError("strides are not defined for this tensor")
        return list(self._data.strides)

    def get_strides(self):
        return self.strides

    def is_continuous(self) -> bool:
        return self._data is None or bool(self._data.flags["C_CONTIGUOUS"])

    @property
    def data(self) -> np.ndarray:
        """numpy view of the values (raw container for bf16 / packed types; a host copy for device tensors)."""
        if self._torch is not None:
            import torch
            t = self._torch.detach()
            if t.dtype == torch.bfloat16:
                return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
            return t.cpu().numpy()
        if self._type == Type.string:
            return np.array(self._strings, dtype=object).reshape(self._shape)
        return self._data

    @property
    def bytes_data(self):
        return self.data

    @property
    def str_data(self):
        return np.array([s.decode(errors="replace") for s in self._strings], dtype=object).reshape(self._shape)

    def copy_to(self, other: "Tensor") -> None:
        other.copy_from(self)

    def copy_from(self, src) -> None:
        if not isinstance(src, Tensor):
            src = Tensor(src)
        if self._torch is not None:
            import torch
            if src._torch is not None:
                self._torch.copy_(src._torch)
            else:
                self._torch.copy_(torch.from_numpy(np.ascontiguousarray(src.data)).view(self._torch.dtype) if self._type == Type.bf16 else torch.from_numpy(np.ascontiguousarray(src.data)))
            return
        if list(src._shape) != list(self._shape):
            self.set_shape(src._shape)
        if self._type == Type.string:
            self._strings = list(src._strings)
        else:
            if src._type != self._type:
                raise RuntimeError("copy between tensors of different element types (%s -> %s)" % (src._type, self._type))
            np.copyto(self._data, src.data.reshape(self._data.shape))

    def astype(self, new_type) -> "Tensor":
        """Value-converting copy (host)."""
        new_type = Type(new_type)
        return Tensor._from_core(_c.convert_bytes(np.ascontiguousarray(self.data), self._type.name, new_type.name, list(self._shape)))

    def to_float32(self) -> np.ndarray:
        return self.astype(Type.f32).data

    def __repr__(self):
        return "<Tensor: shape%s type: %s>" % (self._shape.to_string(), self._type)

    # device tensors --------------------------------------------------------------------------
    @property
    def is_remote(self) -> bool:
        return self._torch is not None

    def torch(self):
        """The torch CUDA tensor behind a remote tensor (None for host tensors)."""
        return self._torch


def _torch_type(dt) -> Type:
    import torch
    m = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16", torch.float64: "f64", torch.int8: "i8", torch.int16: "i16",
         torch.int32: "i32", torch.int64: "i64", torch.uint8: "u8", torch.bool: "boolean"}
    if dt not in m:
        raise TypeError("no element type for torch dtype %s" % dt)
    return Type(m[dt])


def torch_dtype(t: Type):
    import torch
    m = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "f64": torch.float64, "i8": torch.int8, "i16": torch.int16,
         "i32": torch.int32, "i64": torch.int64, "u8": torch.uint8, "boolean": torch.bool}
    return m[Type(t).name]
