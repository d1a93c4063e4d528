"""openvino_b200: an inference framework for NVIDIA B200 (sm_100a) with the OpenVINO programming model.

Public API in one place, named as in ``import openvino as ov``: ``Core``, ``Model``, ``Tensor``, ``Type``,
``PartialShape``, ``convert_model``, ``save_model``, ``compile_model`` and the sub-modules ``opset``,
``properties``, ``preprocess``, ``passes``, ``frontend``, ``runtime``, ``genai``.
"""
try:
    from . import _ovcore   # noqa: F401
except ImportError:   # first import of a fresh checkout: compile the native core in-tree
    from .build import build_core as _build_core
    _build_core()
    from . import _ovcore   # noqa: F401

from ._types import Dimension, PartialShape, Shape, Symbol, Type, get_element_type   # noqa: F401
from . import symbol   # noqa: F401
from ._tensor import Tensor   # noqa: F401
from ._graph import Input, Model, Node, Output, RTMap   # noqa: F401
from ._op_base import DiscreteTypeInfo, Op, register_op   # noqa: F401
from . import opset   # noqa: F401
from . import (opset1, opset2, opset3, opset4, opset5, opset6, opset7, opset8, opset9, opset10, opset11, opset12, opset13, opset14,   # noqa: F401
               opset15, opset16, opset17)
from . import properties   # noqa: F401
from . import passes   # noqa: F401
from . import preprocess   # noqa: F401
from .preprocess import Layout, layout_helpers   # noqa: F401
from .frontend import FrontEndManager, convert_model, read_model, save_model, serialize   # noqa: F401
from .runtime.core import (AsyncInferQueue, CompiledModel, Core, InferRequest, OVDict, ProfilingInfo, VariableState, Version,   # noqa: F401
                           __version__, compile_model)
from ._compat import (AxisSet, AxisVector, Coordinate, CoordinateDiff, Extension, OpExtension, OVAny, Strides, get_batch, set_batch,   # noqa: F401
                      tensor_from_file)
from .utils.shutdown import register_shutdown_callback, shutdown, unregister_shutdown_callback   # noqa: F401

__all__ = ["AsyncInferQueue", "CompiledModel", "Core", "Dimension", "FrontEndManager", "InferRequest", "Input", "Layout", "Model", "Node",
           "OVDict", "Output", "PartialShape", "ProfilingInfo", "RTMap", "Shape", "Symbol", "Tensor", "Type", "VariableState", "Version", "compile_model",
           "convert_model", "get_element_type", "layout_helpers", "opset", "passes", "preprocess", "properties", "read_model", "register_shutdown_callback",
           "save_model", "serialize", "shutdown", "unregister_shutdown_callback"]


def get_version() -> str:
    return __version__


Any = OVAny


def __getattr__(name):
    # device-side classes live with the CUDA device (importing them pulls in torch): resolved on first use
    if name in ("RemoteContext", "RemoteTensor"):
        from .runtime import cuda_plugin
        return getattr(cuda_plugin, name)
    raise AttributeError("module %r has no attribute %r" % (__name__, name))
