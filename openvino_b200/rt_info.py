"""Run-time attributes of nodes that passes and plugins agree on (the helper functions of
src/core/include/openvino/core/rt_info/ and src/common/transformations/include/transformations/rt_info/:
decompression.hpp, disable_fp16_compression.hpp, keep_const_precision.hpp, fused_names_attribute.hpp,
original_precision_attribute.hpp, is_shape_subgraph.hpp). Keys carry the attribute's version suffix, as in serialised IR."""
from __future__ import annotations

from typing import List

from ._graph import Node

_DECOMPRESSION = "decompression_0"
_NO_FP16 = "disable_fp16_compression_0"
_KEEP_CONST = "keep_const_precision_0"
_FUSED = "fused_names_0"
_ORIG_PRECISION = "original_precision_0"
_SHAPE_SUBGRAPH = "is_shape_subgraph_0"


def mark_as_decompression(node: Node) -> None:
    """The Convert that turns a compressed constant back into the compute type: ConstantFolding leaves it alone."""
    node.rt_info[_DECOMPRESSION] = ""


def unmark_as_decompression(node: Node) -> None:
    node.rt_info.pop(_DECOMPRESSION, None)


def is_decompression(node: Node) -> bool:
    return _DECOMPRESSION in node.rt_info


def disable_fp16_compression(node: Node) -> None:
    """The node stays in fp32 when the model is converted to fp16 (precision-sensitive island)."""
    node.rt_info[_NO_FP16] = ""


def enable_fp16_compression(node: Node) -> None:
    node.rt_info.pop(_NO_FP16, None)


def fp16_compression_is_disabled(node: Node) -> bool:
    return _NO_FP16 in node.rt_info


def enable_keep_const_precision(node: Node) -> None:
    """The constant keeps its element type through precision conversions and weight compression."""
    node.rt_info[_KEEP_CONST] = ""


def disable_keep_const_precision(node: Node) -> None:
    node.rt_info.pop(_KEEP_CONST, None)


def is_keep_const_precision(node: Node) -> bool:
    return _KEEP_CONST in node.rt_info


def get_fused_names(node: Node) -> List[str]:
    v = node.rt_info.get(_FUSED)
    return [s for s in str(v).split(",") if s] if v else []


def set_original_precision(node: Node, element_type) -> None:
    node.rt_info[_ORIG_PRECISION] = str(element_type)


def get_original_precision(node: Node):
    return node.rt_info.get(_ORIG_PRECISION)


def mark_shape_subgraph(node: Node) -> None:
    node.rt_info[_SHAPE_SUBGRAPH] = ""


def is_shape_subgraph(node: Node) -> bool:
    return _SHAPE_SUBGRAPH in node.rt_info
