"""Model input/output: ``read_model``, ``convert_model``, ``save_model``, ``serialize`` and the frontend registry.

``FrontEndManager`` resolves a frontend by name or by inspecting the model ("ir", "onnx", "pytorch"), the way
ov::frontend::FrontEndManager does (src/frontends/common/src/manager.cpp:28-276); ``read_model`` and
``convert_model`` are the two entry points built on it (src/inference/src/model_reader.cpp:230,
tools/ovc/openvino/tools/ovc/convert.py). ``save_model`` compresses fp32 weights to fp16 by default
(src/core/src/graph_util.cpp:388-418), ``serialize`` writes the graph as it is.
"""
from __future__ import annotations

import os
from typing import Any, List, Optional

import numpy as np

from .. import _ovcore as _c
from .._graph import Model
from .._tensor import Tensor


class FrontEnd:
    name = ""
    # module and name of the translator table that ConversionExtension entries go to (None: the frontend has no table)
    _table = None

    def __init__(self):
        self._extensions = []

    def __init_subclass__(cls, **kw):
        """``convert`` of every frontend also takes an ``InputModel`` (edited or not) besides the (source, weights) pair."""
        super().__init_subclass__(**kw)
        raw = cls.__dict__.get("convert")
        if raw is None:
            return

        def convert(self, input_model):
            from .input_model import InputModel
            if isinstance(input_model, InputModel):
                return input_model._m()
            return raw(self, input_model)
        convert.__doc__ = raw.__doc__
        cls.convert = convert

    def get_name(self) -> str:
        return self.name

    def supported(self, model) -> bool:
        return False

    def load(self, model, weights=None):
        """-> an ``InputModel``: places can be renamed, re-shaped and cut before ``convert`` (input_model.py)."""
        from .input_model import InputModel
        return InputModel(self, model, weights)

    def add_extension(self, extension) -> None:
        """``ConversionExtension`` (a user translator for one source operation), ``TelemetryExtension``,
        ``ProgressReporterExtension``."""
        from .input_model import ConversionExtension, op_extension_translator
        from .._compat import OpExtension
        if isinstance(extension, OpExtension):
            extension.register()
            if extension.fw_type:
                extension = ConversionExtension(extension.fw_type, op_extension_translator(extension, self.name))
        if isinstance(extension, ConversionExtension):
            if self._table is None:
                raise RuntimeError("frontend '%s' has no operation table to extend" % self.name)
            import importlib
            mod = importlib.import_module(self._table[0], __package__)
            getattr(mod, self._table[1])[extension.op_type] = extension.converter
        self._extensions.append(extension)

    def _convert_source(self, model, weights) -> Model:
        """Source + weights -> Model, reporting to the telemetry / progress extensions."""
        from .input_model import ProgressReporterExtension, TelemetryExtension
        progress = [e for e in self._extensions if isinstance(e, ProgressReporterExtension)]
        telemetry = [e for e in self._extensions if isinstance(e, TelemetryExtension)]
        for p in progress:
            p.report_progress(0.0, 1, 0)
        try:
            m = self.convert((model, weights))
        except Exception as e:   # noqa: BLE001 - reported, then re-raised
            for t in telemetry:
                t.send_error("%s: %s" % (type(e).__name__, str(e)[:200]))
            raise
        from .input_model import DecoderTransformationExtension
        for e in self._extensions:
            if isinstance(e, DecoderTransformationExtension):
                e.transformation(m)
        if telemetry:
            counts = {}
            for n in m.get_ops():
                counts[n.get_type_name()] = counts.get(n.get_type_name(), 0) + 1
            for t in telemetry:
                t.send_event("conversion", self.name)
                for k, v in sorted(counts.items()):
                    t.send_event("op_count", "%s_%s" % (self.name, k), v)
        for p in progress:
            p.report_progress(1.0, 1, 1)
        return m

    def convert(self, input_model) -> Model:
        raise NotImplementedError

    def convert_partially(self, input_model) -> Model:
        return self.convert(input_model)

    def decode(self, input_model) -> Model:
        return self.convert(input_model)

    def normalize(self, model: Model) -> None:
        model.validate_nodes_and_infer_types()

    def __repr__(self):
        return "<FrontEnd '%s'>" % self.name


class IRFrontEnd(FrontEnd):
    """IR v10/v11 xml + bin (src/frontends/ir/src/frontend.cpp:31, ir_deserializer.cpp)."""

    name = "ir"

    def supported(self, model) -> bool:
        if isinstance(model, (str, os.PathLike)):
            s = str(model)
            if s.lower().endswith(".xml"):
                return True
            return s.lstrip().startswith("<?xml") or s.lstrip().startswith("<net")
        if isinstance(model, (bytes, bytearray)):
            head = bytes(model[:64]).lstrip()
            return head.startswith(b"<?xml") or head.startswith(b"<net")
        return False

    def convert(self, input_model) -> Model:
        model, weights = input_model
        if isinstance(model, (bytes, bytearray)):
            model = bytes(model).decode()
        model = str(model)
        if model.lstrip().startswith("<"):
            w = None
            if weights is not None:
                if isinstance(weights, Tensor):
                    w = np.ascontiguousarray(weights.data).reshape(-1).view(np.uint8)
                elif isinstance(weights, (bytes, bytearray, memoryview)):
                    w = np.frombuffer(weights, dtype=np.uint8)
                elif isinstance(weights, np.ndarray):
                    w = np.ascontiguousarray(weights).reshape(-1).view(np.uint8)
                else:
                    with open(weights, "rb") as f:
                        w = np.frombuffer(f.read(), dtype=np.uint8)
            return Model._wrap(_c.deserialize(model, w))
        if not os.path.exists(model):
            raise RuntimeError("Model file %s cannot be opened!" % model)
        bin_path = str(weights) if weights is not None else ""
        return Model._wrap(_c.read_model_files(model, bin_path))


class PyTorchFrontEnd(FrontEnd):
    name = "pytorch"
    _table = (".pytorch", "_TABLE")

    def supported(self, model) -> bool:
        try:
            import torch
        except ImportError:
            return False
        return isinstance(model, (torch.nn.Module, torch.jit.ScriptFunction)) or (hasattr(model, "graph_signature") and hasattr(model, "graph")) \
            or self.supported_decoder(model)

    def supported_decoder(self, model) -> bool:
        return hasattr(model, "convert") and type(model).__name__ in ("TorchScriptPythonDecoder", "TorchFXPythonDecoder")

    def convert(self, input_model) -> Model:
        from . import pytorch
        model, kwargs = input_model
        if self.supported_decoder(model):
            return model.convert()
        module_exts = [e for e in self._extensions if isinstance(e, pytorch.ModuleExtension)]
        undo = pytorch.apply_module_extensions(model, module_exts) if module_exts and hasattr(model, "named_modules") else []
        try:
            return pytorch.convert(model, **(kwargs or {}))
        finally:
            pytorch.restore_module_extensions(undo)


class OnnxFrontEnd(FrontEnd):
    name = "onnx"
    _table = (".onnx", "_T")

    def supported(self, model) -> bool:
        if isinstance(model, (str, os.PathLike)):
            return str(model).lower().endswith(".onnx")
        return False

    def convert(self, input_model) -> Model:
        from . import onnx
        model, _ = input_model
        return onnx.convert(model)


class TensorFlowFrontEnd(FrontEnd):
    name = "tf"
    _table = (".tensorflow", "_T")

    def supported(self, model) -> bool:
        return isinstance(model, (str, os.PathLike)) and str(model).lower().endswith(".pb")

    def convert(self, input_model) -> Model:
        from . import tensorflow
        model, _ = input_model
        return tensorflow.convert(model)


class TFLiteFrontEnd(FrontEnd):
    name = "tflite"
    _table = (".tflite", "_T")

    def supported(self, model) -> bool:
        if isinstance(model, (str, os.PathLike)):
            return str(model).lower().endswith(".tflite")
        return isinstance(model, (bytes, bytearray)) and len(model) >= 8 and bytes(model[4:8]) == b"TFL3"

    def convert(self, input_model) -> Model:
        from . import tflite
        model, _ = input_model
        return tflite.load(model)


class PaddleFrontEnd(FrontEnd):
    name = "paddle"
    _table = (".paddle", "_T")

    def supported(self, model) -> bool:
        return isinstance(model, (str, os.PathLike)) and str(model).lower().endswith(".pdmodel")

    def convert(self, input_model) -> Model:
        from . import paddle
        model, weights = input_model
        return paddle.load(str(model), str(weights) if isinstance(weights, (str, os.PathLike)) else None)


class JaxFrontEnd(FrontEnd):
    name = "jax"
    _table = (".jax", "_T")

    def supported(self, model) -> bool:
        # a ClosedJaxpr: an open jaxpr with its constants
        return hasattr(model, "jaxpr") and hasattr(model, "consts") and hasattr(getattr(model, "jaxpr"), "eqns")

    def convert(self, input_model) -> Model:
        from . import jax
        model, _ = input_model
        return jax.convert(model)


class GgufFrontEnd(FrontEnd):
    name = "gguf"

    def supported(self, model) -> bool:
        if isinstance(model, (str, os.PathLike)) and str(model).lower().endswith(".gguf"):
            return True
        return False

    def convert(self, input_model) -> Model:
        from . import gguf
        model, _ = input_model
        return gguf.convert(str(model))


class FrontEndManager:
    def __init__(self):
        self._frontends = {"ir": IRFrontEnd(), "pytorch": PyTorchFrontEnd(), "onnx": OnnxFrontEnd(), "tf": TensorFlowFrontEnd(), "tflite": TFLiteFrontEnd(),
                           "paddle": PaddleFrontEnd(), "jax": JaxFrontEnd(), "gguf": GgufFrontEnd()}

    def get_available_front_ends(self) -> List[str]:
        return list(self._frontends)

    def register_front_end(self, name: str, frontend: FrontEnd) -> None:
        self._frontends[name] = frontend

    def load_by_framework(self, framework: str) -> FrontEnd:
        if framework not in self._frontends:
            raise RuntimeError("frontend '%s' is not available" % framework)
        return self._frontends[framework]

    def load_by_model(self, model) -> Optional[FrontEnd]:
        for fe in self._frontends.values():
            if fe.supported(model):
                return fe
        return None


_manager = FrontEndManager()
from .input_model import (ConversionExtension, DecoderTransformationExtension, InputModel, NodeContext, Place, ProgressReporterExtension,   # noqa: E402,F401
                          TelemetryExtension)
from .._compat import OpExtension   # noqa: E402,F401


def read_model(model, weights=None, extensions=None) -> Model:
    """Read an IR (``.xml`` path, xml text or bytes; weights as path, bytes or a u8 Tensor), an ``.onnx``, a frozen TensorFlow ``.pb``, a ``.tflite`` or a ``.gguf`` file."""
    if isinstance(model, Model):
        return model
    if hasattr(model, "read"):
        model = model.read()
    fe = _manager.load_by_model(model)
    if fe is None:
        raise RuntimeError("Unable to read the model: %s. Please check that the model format is supported (IR xml, ONNX) and the file exists"
                           % (str(model)[:200],))
    return fe.convert(fe.load(model, weights))


def convert_model(input_model, input=None, output=None, example_input=None, extension=None, verbose=False, share_weights=True, **kwargs) -> Model:
    """Convert a framework model (a ``torch.nn.Module`` / ``ExportedProgram``, or a model file path) to a ``Model``.

    ``input``: shapes to give the inputs (list in input order, ``{name: shape}`` or ``[(name, shape[, type])]``);
    ``output``: names of the values to keep as model outputs; ``example_input``: sample inputs for tracing.
    """
    if isinstance(input_model, Model):
        model = input_model
    elif _manager._frontends["jax"].supported(input_model):
        model = _manager._frontends["jax"].convert((input_model, None))
    elif _manager._frontends["pytorch"].supported(input_model):
        model = _manager._frontends["pytorch"].convert((input_model, dict(example_input=example_input, input=input, share_weights=share_weights, **kwargs)))
    else:
        model = read_model(input_model)
        if input is not None:
            from .pytorch import _input_shapes
            shapes = _input_shapes(input)
            keys = list(input.keys()) if isinstance(input, dict) else [it[0] if isinstance(it, tuple) and isinstance(it[0], str) else i for i, it in enumerate(input)]
            model.reshape({k: s for k, s in zip(keys, shapes)})
    if output:
        names = [output] if isinstance(output, str) else list(output)
        keep = []
        for nm in names:
            found = None
            for n in model.get_ops():
                for o in n.outputs():
                    if nm in o.get_names() or n.get_friendly_name() == nm:
                        found = o
                        break
                if found:
                    break
            if found is None:
                raise RuntimeError("convert_model: no value named '%s'" % nm)
            keep.append(found)
        model = Model(keep, model.get_parameters(), model.get_friendly_name())
    return model


def serialize(model: Model, xml_path: str, bin_path: str = "", version: str = "UNSPECIFIED") -> None:
    """Write the model as IR (no weight compression)."""
    v = {"UNSPECIFIED": 11, "IR_V10": 10, "IR_V11": 11}.get(str(version), 11)
    _c.save_model_files(model._m, str(xml_path), str(bin_path or ""), v)


def save_model(model: Model, output_model: str, compress_to_fp16: bool = True) -> None:
    """Write the model as IR; fp32 weights are stored as fp16 followed by a Convert unless ``compress_to_fp16=False``."""
    m = model
    if compress_to_fp16:
        m = model.clone()
        _c.compress_model_to_f16(m._m)
    out = str(output_model)
    if not out.lower().endswith(".xml"):
        raise RuntimeError("save_model: the output path must end with .xml")
    _c.save_model_files(m._m, out, "", 11)
