"""``openvino.helpers``: packing of sub-byte element types. Reference: src/bindings/python/src/openvino/helpers/packing.py."""
from .packing import pack_data, unpack_data   # noqa: F401
