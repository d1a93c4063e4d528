"""``Core``, device plugins, ``CompiledModel``, ``InferRequest``, ``AsyncInferQueue``.

The user-facing runtime. ``Core`` owns a plugin registry keyed by device name, parses device strings
("CUDA.1", "AUTO:CUDA,CPU", "HETERO:CUDA,CPU", "BATCH:CUDA(8)", "MULTI:…"), merges properties, consults the
model cache and hands the model to the plugin. Plugins return a ``CompiledModel`` whose requests run a
pipeline of stages on native task executors (``_ovcore.AsyncRequest`` is the state machine).

Reference call stack: ov::Core::compile_model (src/inference/src/cpp/core.cpp:121) -> CoreImpl::compile_model
(src/inference/src/dev/core_impl.cpp:845) -> parseDeviceNameIntoConfig (:611) -> get_plugin (:669) -> cache
lookup (compile_model_and_cache :1543 / load_model_from_cache :1621) -> IPlugin::compile_model
(src/inference/dev_api/openvino/runtime/iplugin.hpp:105); requests: ISyncInferRequest
(src/inference/src/dev/isync_infer_request.cpp) + IAsyncInferRequest (iasync_infer_request.cpp:43-236).
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
import threading
import time
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

import numpy as np

from .. import _ovcore as _c
from .. import properties as props
from .._graph import Model, Node, Output
from .._tensor import Tensor
from .._types import PartialShape, Shape, Type

__version__ = "2026.0.0-b200"


class Version:
    def __init__(self, description: str, build_number: str = __version__):
        self.description, self.build_number = description, build_number
        self.major, self.minor = 2026, 0

    def __repr__(self):
        return "<Version: %s %s>" % (self.description, self.build_number)


# ======================================================================================================
# profiling
# ======================================================================================================
class ProfilingInfo:
    class Status:
        NOT_RUN, OPTIMIZED_OUT, EXECUTED = "NOT_RUN", "OPTIMIZED_OUT", "EXECUTED"

    def __init__(self, node_name, node_type, exec_type, real_time_us, cpu_time_us=None, status="EXECUTED"):
        self.node_name, self.node_type, self.exec_type = node_name, node_type, exec_type
        self.real_time = real_time_us          # microseconds
        self.cpu_time = real_time_us if cpu_time_us is None else cpu_time_us
        self.status = status

    def __repr__(self):
        return "<ProfilingInfo %s (%s) %.1f us %s>" % (self.node_name, self.node_type, self.real_time, self.status)


# ======================================================================================================
# plugin interface
# ======================================================================================================
from ..utils import log as _log, trace as _trace

class Plugin:
    """Device plugin interface (IPlugin): compile, query, import, properties."""

    device_name = ""
    description = "plugin"

    def __init__(self, core: "Core"):
        self.core = core
        self.config: Dict[str, Any] = {}

    # -- properties
    def supported_properties(self) -> List[str]:
        return [props.supported_properties, props.available_devices, props.device.full_name, props.enable_profiling,
                props.hint.performance_mode, props.hint.num_requests, props.hint.inference_precision, props.hint.execution_mode,
                props.num_streams, props.inference_num_threads, props.cache_dir, props.device.capabilities,
                props.range_for_async_infer_requests, props.range_for_streams, props.device.id]

    def set_property(self, config: dict) -> None:
        for k, v in config.items():
            if k not in self.supported_properties() and k not in (props.cache_dir,):
                raise RuntimeError("[%s] unsupported property %s" % (self.device_name, k))
            self.config[k] = v

    def get_property(self, name: str, arguments: Optional[dict] = None):
        if name == props.supported_properties:
            return self.supported_properties()
        if name == props.available_devices:
            return self.available_device_ids()
        if name == props.device.full_name:
            return self.full_name((arguments or {}).get(props.device.id, ""))
        if name == props.device.capabilities:
            return self.capabilities()
        if name == props.range_for_async_infer_requests:
            return (1, 1, 1)
        if name == props.range_for_streams:
            return (1, max(1, os.cpu_count() or 1))
        if name in self.config:
            return self.config[name]
        defaults = self.default_config()
        if name in defaults:
            return defaults[name]
        raise RuntimeError("[%s] unsupported property %s" % (self.device_name, name))

    def default_config(self) -> dict:
        return {props.enable_profiling: False, props.hint.performance_mode: "LATENCY", props.hint.num_requests: 0,
                props.hint.execution_mode: "PERFORMANCE", props.num_streams: 1, props.inference_num_threads: 0,
                props.hint.inference_precision: "f32", props.cache_dir: "", props.device.id: ""}

    def available_device_ids(self) -> List[str]:
        return [""]

    def full_name(self, device_id: str = "") -> str:
        return self.description

    def capabilities(self) -> List[str]:
        return ["FP32", "EXPORT_IMPORT"]

    # -- models
    def compile_model(self, model: Model, config: dict) -> "CompiledModel":
        raise NotImplementedError

    def query_model(self, model: Model, config: dict) -> Dict[str, str]:
        """{friendly name: device} for every operation this device can run."""
        raise NotImplementedError

    def import_model(self, blob: "ModelBlob", config: dict) -> "CompiledModel":
        model = Model._wrap(_c.deserialize(blob.xml, np.frombuffer(blob.weights, dtype=np.uint8)))
        cfg = dict(blob.header.get("config", {}))
        cfg.update(config)
        cm = self.compile_model(model, cfg)
        return cm

    def merged_config(self, config: dict) -> dict:
        cfg = self.default_config()
        cfg.update(self.config)
        cfg.update(config)
        return cfg


class _EntryLock:
    """Advisory lock on a file next to a cache entry: processes (and threads) that want the same entry take turns."""
    _thread_locks: Dict[str, threading.Lock] = {}
    _guard = threading.Lock()

    def __init__(self, path: str):
        self.path = path
        with self._guard:
            self._tl = self._thread_locks.setdefault(path, threading.Lock())
        self._f = None

    def __enter__(self):
        self._tl.acquire()
        try:
            import fcntl
            self._f = open(self.path, "a+b")
            fcntl.flock(self._f.fileno(), fcntl.LOCK_EX)
        except (ImportError, OSError):
            self._f = None        # no advisory locks on this file system: the thread lock still holds
        return self

    def __exit__(self, *exc):
        if self._f is not None:
            try:
                import fcntl
                fcntl.flock(self._f.fileno(), fcntl.LOCK_UN)
            finally:
                self._f.close()
        self._tl.release()
        return False


class ModelBlob:
    """Exported compiled model: header (json) + IR xml + weights, with a fixed magic and version.

    Plays the role of the plugin blobs behind ``CompiledModel::export_model`` / ``Core::import_model`` and of the
    model-cache entries (src/inference/src/cache_manager.hpp, src/inference/src/dev/core_impl.cpp:1543-1700): the
    header records the device, the compile configuration and the runtime build so that a stale entry is rejected.
    """

    MAGIC = b"OVB200BL"
    FORMAT = 1

    def __init__(self, header: dict, xml: str, weights: bytes):
        self.header, self.xml, self.weights = header, xml, weights

    def to_bytes(self) -> bytes:
        h = json.dumps(self.header, sort_keys=True).encode()
        x = self.xml.encode() if isinstance(self.xml, str) else bytes(self.xml)
        return b"".join([self.MAGIC, struct.pack("<IQQQ", self.FORMAT, len(h), len(x), len(self.weights)), h, x, bytes(self.weights)])

    @classmethod
    def from_bytes(cls, data) -> "ModelBlob":
        data = memoryview(data)
        if bytes(data[:8]) != cls.MAGIC:
            raise RuntimeError("not a compiled-model blob (bad magic)")
        fmt, hl, xl, wl = struct.unpack("<IQQQ", data[8:36])
        if fmt != cls.FORMAT:
            raise RuntimeError("compiled-model blob format %d is not supported (expected %d)" % (fmt, cls.FORMAT))
        if 36 + hl + xl + wl != len(data):
            raise RuntimeError("compiled-model blob is truncated")
        o = 36
        header = json.loads(bytes(data[o:o + hl])); o += hl
        xml = bytes(data[o:o + xl]).decode(); o += xl
        return cls(header, xml, bytes(data[o:o + wl]))


# ======================================================================================================
# variable state
# ======================================================================================================
class VariableState:
    def __init__(self, name: str, getter, setter, resetter):
        self._name, self._get, self._set, self._reset = name, getter, setter, resetter

    @property
    def name(self) -> str:
        return self._name

    def get_name(self) -> str:
        return self._name

    @property
    def state(self) -> Tensor:
        return self._get()

    @state.setter
    def state(self, t) -> None:
        self._set(t if isinstance(t, Tensor) else Tensor(t))

    def get_state(self) -> Tensor:
        return self._get()

    def set_state(self, t) -> None:
        self._set(t if isinstance(t, Tensor) else Tensor(t))

    def reset(self) -> None:
        self._reset()


# ======================================================================================================
# compiled model / infer request
# ======================================================================================================
class _Port:
    """ConstOutput-like description of a compiled model's input/output."""

    def __init__(self, output: Output, index: int, kind: str):
        self._o, self.index, self.kind = output, index, kind

    def __getattr__(self, item):
        return getattr(self._o, item)

    def get_node(self):
        return self._o.get_node()

    def __eq__(self, other):
        return isinstance(other, _Port) and other._o == self._o and other.kind == self.kind

    def __hash__(self):
        return hash((self._o, self.kind))

    def __repr__(self):
        return "<ConstOutput: names%s, shape%s, type: %s>" % (sorted(self._o.get_names()), self._o.get_partial_shape().to_string(), self._o.get_element_type())


class CompiledModel:
    """A model compiled for one device. Sub-classes implement ``_make_runner``: a callable
    ``run(request, inputs: List[Tensor]) -> List[Tensor]`` holding the device program for one request."""

    def __init__(self, plugin: Plugin, model: Model, config: dict, runtime_model: Optional[Model] = None):
        self.plugin = plugin
        self.model = model                       # the model as given by the user (ports, names)
        self.runtime_model = runtime_model or model
        self.config = config
        self.loaded_from_cache = False
        self._inputs = [_Port(o, i, "input") for i, o in enumerate(model.inputs)]
        self._outputs = [_Port(o, i, "output") for i, o in enumerate(model.outputs)]
        n_streams = int(config.get(props.num_streams, 1) or 1)
        if n_streams < 0:
            n_streams = max(1, (os.cpu_count() or 2) // 2) if str(config.get(props.hint.performance_mode)) == "THROUGHPUT" else 1
        self._n_streams = max(1, n_streams)
        self._executor = _c.TaskExecutor(self._n_streams, "%s_streams" % plugin.device_name)
        self._callback_executor = _c.TaskExecutor(1, "%s_callbacks" % plugin.device_name)
        self._default_request: Optional[InferRequest] = None

    # ---- ports
    @property
    def inputs(self) -> List[_Port]:
        return list(self._inputs)

    @property
    def outputs(self) -> List[_Port]:
        return list(self._outputs)

    def _find(self, ports, key, kind):
        if key is None:
            if len(ports) != 1:
                raise RuntimeError("%s() needs an index or a tensor name: the model has %d %ss" % (kind, len(ports), kind))
            return ports[0]
        if isinstance(key, int):
            if key < 0 or key >= len(ports):
                raise IndexError("%s index %d out of range" % (kind, key))
            return ports[key]
        if isinstance(key, str):
            for p in ports:
                if key in p.get_names():
                    return p
            for p in ports:
                node = p.get_node()
                if node.get_friendly_name() == key:
                    return p
                if kind == "output" and key in node.input_value(0).get_names():
                    return p
            raise RuntimeError("no %s tensor named '%s'" % (kind, key))
        if isinstance(key, _Port):
            return self._find(ports, key.index, kind) if key.kind == kind else self._raise_port(key)
        if isinstance(key, Output):
            for p in ports:
                if p._o == key or (kind == "output" and p.get_node().input_value(0) == key):
                    return p
            # a port of another (equal) model object: match by names, then by index
            for p in ports:
                if key.get_names() and key.get_names() & p.get_names():
                    return p
            raise RuntimeError("port %r does not belong to this model" % (key,))
        raise TypeError("bad %s key %r" % (kind, key))

    @staticmethod
    def _raise_port(key):
        raise RuntimeError("port %r is of the wrong kind" % (key,))

    def input(self, key=None) -> _Port:
        return self._find(self._inputs, key, "input")

    def output(self, key=None) -> _Port:
        return self._find(self._outputs, key, "output")

    # ---- requests
    def create_infer_request(self) -> "InferRequest":
        return InferRequest(self)

    def infer_new_request(self, inputs=None) -> "OVDict":
        return self.create_infer_request().infer(inputs)

    def __call__(self, inputs=None, share_inputs: bool = True, share_outputs: bool = False) -> "OVDict":
        if self._default_request is None:
            self._default_request = self.create_infer_request()
        return self._default_request.infer(inputs, share_inputs=share_inputs, share_outputs=share_outputs)

    def _make_runner(self, request: "InferRequest") -> Callable:
        raise NotImplementedError

    def _variables(self, request: "InferRequest") -> List[VariableState]:
        return []

    def release_memory(self) -> None:
        pass

    # ---- introspection
    def get_runtime_model(self) -> Model:
        """The executed graph: one node per executed primitive with execution rt_info."""
        m = self.runtime_model.clone()
        for order, n in enumerate(m.get_ops()):
            n.rt_info["layerType"] = n.get_type_name()
            n.rt_info["execOrder"] = str(order)
            n.rt_info["primitiveType"] = "%s_%s" % (self.plugin.device_name.lower(), n.get_type_name().lower())
            n.rt_info["outputPrecisions"] = ",".join(str(n.get_output_element_type(i)) for i in range(n.get_output_size()))
            n.rt_info["runtimePrecision"] = str(n.get_output_element_type(0)) if n.get_output_size() else ""
            n.rt_info["originalLayersNames"] = str(n.rt_info.get("fused_names_0", n.get_friendly_name()))
            n.rt_info["execTimeMcs"] = "not_executed"
        # execution times of the most recent profiled inference (PERF_COUNT) of the default request
        req = self._default_request
        if req is not None:
            times = {p.node_name: p.real_time for p in req.get_profiling_info()}
            for n in m.get_ops():
                t = times.get(n.get_friendly_name())
                if t is not None:
                    us = t.total_seconds() * 1e6 if hasattr(t, "total_seconds") else float(t)
                    n.rt_info["execTimeMcs"] = str(int(round(us)))
        return m

    def get_property(self, name: str):
        name = str(name)
        if name == props.supported_properties:
            return [props.supported_properties, props.model_name, props.optimal_number_of_infer_requests, props.execution_devices,
                    props.loaded_from_cache] + list(self.config.keys())
        if name == props.model_name:
            return self.model.get_friendly_name()
        if name == props.optimal_number_of_infer_requests:
            return self.optimal_number_of_infer_requests()
        if name == props.execution_devices:
            return [self.plugin.device_name]
        if name == props.loaded_from_cache:
            return self.loaded_from_cache
        if name in self.config:
            return self.config[name]
        raise RuntimeError("[%s] compiled model has no property %s" % (self.plugin.device_name, name))

    def set_property(self, config) -> None:
        cfg = props.normalize(config)
        if cfg:
            raise RuntimeError("compiled-model properties are read-only")

    def optimal_number_of_infer_requests(self) -> int:
        return self._n_streams

    def export_model(self, stream=None) -> bytes:
        xml, weights = _c.serialize(self.model._m)
        header = {"device": self.plugin.device_name, "runtime": __version__,
                  "config": {k: v for k, v in self.config.items() if isinstance(v, (str, int, float, bool))}}
        data = ModelBlob(header, xml.decode(), weights).to_bytes()
        if stream is not None:
            stream.write(data)
        return data


def _compiled_get_context(self):
    """The device context the model was compiled in (devices with device memory only)."""
    try:
        name = self.get_property(props.execution_devices)[0]
    except Exception:   # noqa: BLE001 - the property is optional
        name = self.plugin.device_name
    if str(name) == self.plugin.device_name or not hasattr(self.plugin, "core"):
        if not hasattr(self.plugin, "get_default_context"):
            raise RuntimeError("device %s has no remote context" % self.plugin.device_name)
        return self.plugin.get_default_context()
    return self.plugin.core.get_default_context(str(name).split(".")[0])


CompiledModel.get_context = _compiled_get_context


class OVDict(dict):
    """Results of an inference: addressable by output port, tensor name or index (``ov.utils.data_helpers.OVDict``)."""

    def __init__(self, ports: List[_Port], values: List[np.ndarray]):
        super().__init__(zip(ports, values))
        self._ports, self._values = ports, values

    def __getitem__(self, key):
        if isinstance(key, int):
            return self._values[key]
        if isinstance(key, str):
            for p, v in zip(self._ports, self._values):
                if key in p.get_names() or p.get_node().get_friendly_name() == key or key in p.get_node().input_value(0).get_names():
                    return v
            raise KeyError(key)
        if isinstance(key, Output):
            for p, v in zip(self._ports, self._values):
                if p._o == key:
                    return v
        return super().__getitem__(key)

    def names(self):
        return tuple(p.get_names() for p in self._ports)

    def to_dict(self):
        return dict(self)

    def to_tuple(self):
        return tuple(self._values)


class InferRequest:
    """One inference request: tensors bound to ports, synchronous and asynchronous execution."""

    def __init__(self, compiled: CompiledModel):
        self._cm = compiled
        self._in: List[Optional[Tensor]] = [None] * len(compiled._inputs)
        self._out: List[Optional[Tensor]] = [None] * len(compiled._outputs)
        self._user_out: Dict[int, Tensor] = {}
        self._profile: List[ProfilingInfo] = []
        self._req = _c.AsyncRequest()
        self._runner = compiled._make_runner(self)
        self._req.set_pipeline([(compiled._executor, self._run_stage)])
        self._req.set_cancel_hook(self._on_cancel)
        self._cancel_requested = False
        self._user_callback = None
        self._userdata = None
        self._latency = 0.0

    # ---- tensors
    def _in_index(self, key) -> int:
        return self._cm._find(self._cm._inputs, key, "input").index

    def _out_index(self, key) -> int:
        return self._cm._find(self._cm._outputs, key, "output").index

    def _locate(self, key):
        """-> ('input' | 'output', index) for a name / port that may be on either side."""
        if isinstance(key, _Port):
            return key.kind, key.index
        try:
            return "input", self._in_index(key)
        except (RuntimeError, IndexError):
            return "output", self._out_index(key)

    def _check_input(self, i: int, t: Tensor) -> None:
        port = self._cm._inputs[i]
        if port.get_element_type() != t.element_type and port.get_element_type().is_static():
            raise RuntimeError("input %d: tensor element type %s does not match the model's %s" % (i, t.element_type, port.get_element_type()))
        if not port.get_partial_shape().compatible(PartialShape(list(t.shape))):
            raise RuntimeError("input %d: tensor shape %s is not compatible with the model's %s" % (i, t.shape, port.get_partial_shape()))

    def set_tensor(self, key, tensor: Tensor) -> None:
        kind, i = self._locate(key)
        if kind == "input":
            self.set_input_tensor(i, tensor)
        else:
            self.set_output_tensor(i, tensor)

    def get_tensor(self, key) -> Tensor:
        kind, i = self._locate(key)
        return self.get_input_tensor(i) if kind == "input" else self.get_output_tensor(i)

    def set_input_tensor(self, index_or_tensor, tensor: Optional[Tensor] = None) -> None:
        if tensor is None:
            index_or_tensor, tensor = None, index_or_tensor
        i = self._in_index(index_or_tensor)
        if not isinstance(tensor, Tensor):
            tensor = Tensor(tensor)
        self._check_input(i, tensor)
        self._in[i] = tensor

    def set_input_tensors(self, index_or_tensors, tensors=None) -> None:
        """Bind a batch given as separate tensors (one per batch item): they are gathered along axis 0."""
        if tensors is None:
            index_or_tensors, tensors = None, index_or_tensors
        if isinstance(tensors, dict):
            for k, v in tensors.items():
                self.set_input_tensor(k, v)
            return
        if isinstance(index_or_tensors, (int, str)) or index_or_tensors is None and len(self._cm._inputs) == 1:
            i = self._in_index(index_or_tensors)
            arrs = [t.data if isinstance(t, Tensor) else np.asarray(t) for t in tensors]
            self.set_input_tensor(i, Tensor(np.concatenate(arrs, axis=0)))
            return
        for i, t in enumerate(tensors):
            self.set_input_tensor(i, t)

    set_tensors = set_input_tensors

    def set_output_tensor(self, index_or_tensor, tensor: Optional[Tensor] = None) -> None:
        if tensor is None:
            index_or_tensor, tensor = None, index_or_tensor
        i = self._out_index(index_or_tensor)
        port = self._cm._outputs[i]
        if port.get_element_type().is_static() and port.get_element_type() != tensor.element_type:
            raise RuntimeError("output %d: tensor element type %s does not match the model's %s" % (i, tensor.element_type, port.get_element_type()))
        self._user_out[i] = tensor
        self._out[i] = tensor

    def set_output_tensors(self, tensors) -> None:
        items = tensors.items() if isinstance(tensors, dict) else enumerate(tensors)
        for k, v in items:
            self.set_output_tensor(k, v)

    def get_input_tensor(self, index=None) -> Tensor:
        i = self._in_index(index)
        if self._in[i] is None:
            port = self._cm._inputs[i]
            ps = port.get_partial_shape()
            shape = [d.get_length() if d.is_static else 0 for d in ps] if ps.rank.is_static else [0]
            self._in[i] = Tensor(port.get_element_type() if port.get_element_type().is_static() else Type.f32, shape)
        return self._in[i]

    def get_output_tensor(self, index=None) -> Tensor:
        i = self._out_index(index)
        if self._out[i] is None:
            port = self._cm._outputs[i]
            ps = port.get_partial_shape()
            shape = [d.get_length() if d.is_static else 0 for d in ps] if ps.rank.is_static else [0]
            self._out[i] = Tensor(port.get_element_type() if port.get_element_type().is_static() else Type.f32, shape)
        return self._out[i]

    @property
    def input_tensors(self) -> List[Tensor]:
        return [self.get_input_tensor(i) for i in range(len(self._in))]

    @property
    def output_tensors(self) -> List[Tensor]:
        return [self.get_output_tensor(i) for i in range(len(self._out))]

    @property
    def model_inputs(self):
        return self._cm.inputs

    @property
    def model_outputs(self):
        return self._cm.outputs

    def get_compiled_model(self) -> CompiledModel:
        return self._cm

    @property
    def results(self) -> OVDict:
        return OVDict(self._cm._outputs, [self.get_output_tensor(i).data for i in range(len(self._out))])

    @property
    def userdata(self):
        return self._userdata

    @property
    def latency(self) -> float:
        return self._req.latency_ms()

    # ---- execution
    def _bind(self, inputs, share_inputs=True) -> None:
        if inputs is None:
            return
        if isinstance(inputs, dict):
            for k, v in inputs.items():
                self._bind_one(self._in_index(k), v, share_inputs)
        elif isinstance(inputs, (list, tuple)) and not (inputs and np.isscalar(inputs[0])):
            for i, v in enumerate(inputs):
                self._bind_one(i, v, share_inputs)
        else:
            self._bind_one(self._in_index(None), inputs, share_inputs)

    def _bind_one(self, i: int, v, share: bool) -> None:
        if not isinstance(v, Tensor):
            port = self._cm._inputs[i]
            if isinstance(v, np.ndarray):
                et = port.get_element_type()
                if et.is_static() and et.bitwidth % 8 == 0 and et.name not in ("bf16", "string") and not et.name.startswith("f8") and Type.from_numpy(v.dtype) != et:
                    v = v.astype(et.to_dtype())
                v = Tensor(v, shared_memory=share and v.flags["C_CONTIGUOUS"])
            elif np.isscalar(v) or isinstance(v, (list, tuple)):
                et = port.get_element_type()
                arr = np.asarray(v)
                if et.is_static() and et.bitwidth % 8 == 0 and et.name not in ("bf16", "string") and not et.name.startswith("f8") and arr.dtype.kind not in ("U", "S", "O"):
                    arr = arr.astype(et.to_dtype())
                v = Tensor(arr)
            else:
                v = Tensor(v)
        self._check_input(i, v)
        self._in[i] = v

    def _run_stage(self) -> None:
        if self._cancel_requested:
            raise _c.CancelledError("Infer Request was canceled")
        ins = [self.get_input_tensor(i) for i in range(len(self._in))]
        with _trace.scope("ov::phases", "InferRequest::infer::%s" % self._cm.plugin.device_name):
            outs = self._runner(self, ins)
        for i, t in enumerate(outs):
            if i in self._user_out:
                dst = self._user_out[i]
                if list(dst.shape) != list(t.shape):
                    dst.set_shape(t.shape)
                dst.copy_from(t)
                self._out[i] = dst
            else:
                self._out[i] = t

    def _on_cancel(self) -> None:
        self._cancel_requested = True

    def infer(self, inputs=None, share_inputs: bool = False, share_outputs: bool = False, *, decode_strings: bool = True) -> OVDict:
        self._bind(inputs, share_inputs)
        self._cancel_requested = False
        self._req.infer()
        res = self.results
        if not share_outputs and getattr(self, "_pinned_out", None):
            # the device keeps its results in request-owned staging memory that the next inference overwrites:
            # without share_outputs the caller gets arrays of its own
            res = OVDict(self._cm._outputs, [np.array(a, copy=True) if isinstance(a, np.ndarray) else a for a in res.to_tuple()])
        return res

    def start_async(self, inputs=None, userdata=None, share_inputs: bool = False) -> None:
        self._bind(inputs, share_inputs)
        if userdata is not None:
            self._userdata = userdata
        self._cancel_requested = False
        self._req.start_async()

    def wait(self) -> None:
        self._req.wait()

    def wait_for(self, timeout_ms: int) -> bool:
        return self._req.wait_for(int(timeout_ms))

    def cancel(self) -> None:
        self._req.cancel()

    def set_callback(self, callback: Callable, userdata=None) -> None:
        """``callback(userdata)`` runs when the request completes (also after a failure)."""
        self._user_callback = callback
        self._userdata = userdata

        def on_done(err):
            callback(self._userdata)
        self._req.set_callback(on_done if callback is not None else None)

    def get_profiling_info(self) -> List[ProfilingInfo]:
        if not self._cm.config.get(props.enable_profiling):
            raise RuntimeError("profiling is off: compile the model with PERF_COUNT=True")
        return list(self._profile)

    profiling_info = property(get_profiling_info)

    def query_state(self) -> List[VariableState]:
        return self._cm._variables(self)

    def reset_state(self) -> None:
        for v in self.query_state():
            v.reset()


class AsyncInferQueue:
    """Pool of requests; ``start_async`` takes an idle one (blocking while all are busy).

    Reference: src/bindings/python/src/pyopenvino/core/async_infer_queue.cpp:20-178.
    """

    def __init__(self, compiled_model: CompiledModel, jobs: int = 0):
        if jobs <= 0:
            jobs = compiled_model.optimal_number_of_infer_requests()
        self._requests = [compiled_model.create_infer_request() for _ in range(jobs)]
        self._idle = _c.IdleQueue(jobs)
        self._callback = None
        self._userdata = [None] * jobs
        self._error: Optional[BaseException] = None
        self._lock = threading.Lock()
        for i, r in enumerate(self._requests):
            r._req.set_callback(self._make_done(i))

    def _make_done(self, i: int):
        def done(err):
            try:
                if err is None and self._callback is not None:
                    self._callback(self._requests[i], self._userdata[i])
                elif err is not None:
                    with self._lock:
                        if self._error is None:
                            self._error = err if isinstance(err, BaseException) else RuntimeError(str(err))
            except BaseException as e:   # noqa: BLE001 - kept and re-raised from wait_all / start_async
                with self._lock:
                    if self._error is None:
                        self._error = e
            finally:
                self._idle.release(i)
        return done

    def _raise_pending(self):
        with self._lock:
            e, self._error = self._error, None
        if e is not None:
            raise e

    def set_callback(self, callback: Callable) -> None:
        self._callback = callback

    def is_ready(self) -> bool:
        self._raise_pending()
        return self._idle.is_ready()

    def get_idle_request_id(self) -> int:
        i = self._idle.get_idle()
        self._raise_pending()
        return i

    def start_async(self, inputs=None, userdata=None, share_inputs: bool = False) -> None:
        i = self._idle.acquire()
        try:
            self._raise_pending()
            self._userdata[i] = userdata
            r = self._requests[i]
            r._bind(inputs, share_inputs)
            r._cancel_requested = False
            r._req.start_async()
        except BaseException:
            self._idle.release(i)
            raise

    def wait_all(self) -> None:
        self._idle.wait_all()
        for r in self._requests:
            try:
                r._req.wait()
            except BaseException as e:   # noqa: BLE001
                with self._lock:
                    if self._error is None:
                        self._error = e
        self._raise_pending()

    @property
    def userdata(self):
        return list(self._userdata)

    def __len__(self):
        return len(self._requests)

    def __iter__(self):
        return iter(self._requests)

    def __getitem__(self, i):
        return self._requests[i]


# ======================================================================================================
# CPU device: the native reference executor
# ======================================================================================================
class CpuCompiledModel(CompiledModel):
    def _make_runner(self, request: InferRequest):
        store = _c.VariableStore()
        request._variables = store
        threads = int(self.config.get(props.inference_num_threads, 0) or 0)
        profile = bool(self.config.get(props.enable_profiling))
        rm = self.runtime_model._m

        def run(req: InferRequest, ins: List[Tensor]) -> List[Tensor]:
            outs, prof = _c.evaluate(rm, [t._to_core() for t in ins], store, threads, profile)
            if profile:
                req._profile = [ProfilingInfo(name, _type_of(self.runtime_model, name), "ref_f32", us) for name, us in prof]
            return [Tensor._from_core(o) for o in outs]
        return run

    def _variables(self, request: InferRequest) -> List[VariableState]:
        store = request._variables
        out = []
        for v in self.runtime_model.get_variables():
            vid = v.get_info().variable_id
            info = v.get_info()

            def get(vid=vid, info=info):
                packed = store.get(vid)
                if packed is None:
                    shape = [d.get_length() if d.is_static else 0 for d in info.data_shape] if info.data_shape.rank.is_static else [0]
                    return Tensor(info.data_type if info.data_type.is_static() else Type.f32, shape)
                return Tensor._from_core(packed)

            def set_(t, vid=vid):
                store.set(vid, np.ascontiguousarray(t.data), t.element_type.name, list(t.shape))

            def reset(vid=vid):
                store.erase(vid)
            out.append(VariableState(vid, get, set_, reset))
        return out


_type_cache: Dict[int, Dict[str, str]] = {}


def _type_of(model: Model, name: str) -> str:
    m = _type_cache.get(id(model))
    if m is None:
        m = {n.get_friendly_name(): n.get_type_name() for n in model.get_ops()}
        _type_cache[id(model)] = m
    return m.get(name, "")


class CpuPlugin(Plugin):
    """Host execution through the native reference executor (fp32 compute, threaded).

    Serves as the always-available fallback device and as the numerical oracle for the CUDA device; covers the
    role of the template plugin (src/plugins/template) and, functionally, of the CPU plugin (src/plugins/intel_cpu).
    """

    device_name = "CPU"
    description = "Host CPU (reference executor)"

    def capabilities(self):
        return ["FP32", "FP16", "BF16", "INT8", "BIN", "EXPORT_IMPORT"]

    def get_property(self, name, arguments=None):
        if name == props.range_for_async_infer_requests:
            return (1, max(1, os.cpu_count() or 1), 1)
        if name == props.device.full_name:
            try:
                import cpuinfo   # noqa: F401
                return cpuinfo.get_cpu_info().get("brand_raw", self.description)
            except Exception:   # noqa: BLE001
                return self.description
        return super().get_property(name, arguments)

    def compile_model(self, model: Model, config: dict) -> CompiledModel:
        cfg = self.merged_config(config)
        rm = model.clone()
        _c.run_moc_transformations(rm._m, True)
        if str(cfg.get(props.hint.performance_mode)) == "THROUGHPUT" and props.num_streams not in config and props.num_streams not in self.config:
            # stream count from the host topology (physical cores, NUMA nodes), as the reference CPU device does
            streams, _ = _c.plan_streams(_c.host_cpu_topology(), "THROUGHPUT", 0, int(cfg.get(props.inference_num_threads, 0) or 0))
            cfg[props.num_streams] = max(1, min(16, streams))
        return CpuCompiledModel(self, model, cfg, rm)

    def query_model(self, model: Model, config: dict) -> Dict[str, str]:
        return {n.get_friendly_name(): self.device_name for n in model.get_ops() if n._n.has_evaluate()}


# ======================================================================================================
# Core
# ======================================================================================================
def _parse_device(device: str):
    """'CUDA.1' -> ('CUDA', {'DEVICE_ID': '1'}); 'AUTO:CUDA,CPU' -> ('AUTO', {'MULTI_DEVICE_PRIORITIES': 'CUDA,CPU'});
    'BATCH:CUDA(8)' -> ('BATCH', {... 'CUDA(8)'})."""
    cfg = {}
    name = device.strip()
    if ":" in name:
        name, rest = name.split(":", 1)
        cfg[props.device.priorities] = rest
    elif "." in name:
        name, dev_id = name.split(".", 1)
        cfg[props.device.id] = dev_id
    return name, cfg


_DEVICE_ALIASES = {"GPU": "CUDA", "B200": "CUDA"}


class Core:
    """Entry point of the runtime: model reading, device discovery, compilation, properties."""

    def __init__(self, xml_config_file: str = ""):
        self._plugins: Dict[str, Plugin] = {}
        self._factories: Dict[str, Callable[["Core"], Plugin]] = {}
        self._core_config: Dict[str, Any] = {props.cache_dir: "", props.enable_mmap: True, props.force_tbb_terminate: False}
        self._extensions: List[Any] = []
        self._lock = threading.RLock()
        self.register_plugin_factory("CPU", CpuPlugin)
        from . import policy_plugins
        policy_plugins.register(self)
        from . import npuw
        npuw.register(self)
        self.register_plugin_factory("CUDA", _load_cuda_plugin)

    # ---- plugins
    def register_plugin_factory(self, device_name: str, factory: Callable[["Core"], Plugin]) -> None:
        self._factories[device_name] = factory

    def register_plugin(self, plugin, device_name: str, config=None) -> None:
        """Register a plugin class / factory (or a ``module:attr`` string) under ``device_name``."""
        if device_name in self._factories:
            raise RuntimeError("device %s is already registered" % device_name)
        if isinstance(plugin, str):
            mod, _, attr = plugin.partition(":")
            import importlib
            plugin = getattr(importlib.import_module(mod), attr or "Plugin")
        config = dict(config or {})
        alias = config.pop("PROXY_CONFIGURATION_ALIAS", None)
        fallback = config.pop("PROXY_CONFIGURATION_FALLBACK", None)
        config.pop("PROXY_CONFIGURATION_PRIORITY", None)
        self._factories[device_name] = plugin
        if alias:
            # the plugin stays reachable under its own name; `alias` becomes (or extends) a proxy device in front of it
            from .policy_plugins import register_proxy
            register_proxy(self, alias, [device_name] + ([fallback] if fallback else []))
        if config:
            self._get_plugin(device_name).set_property(props.normalize(config))

    def register_proxy(self, alias: str, devices) -> None:
        """Expose the plugins ``devices`` (fallback order) under the single device name ``alias``."""
        from .policy_plugins import register_proxy
        register_proxy(self, alias, list(devices))

    def unload_plugin(self, device_name: str) -> None:
        name = _DEVICE_ALIASES.get(device_name, device_name)
        if name not in self._plugins:
            raise RuntimeError("device %s is not loaded" % device_name)
        del self._plugins[name]

    def _get_plugin(self, device_name: str) -> Plugin:
        name = _DEVICE_ALIASES.get(device_name, device_name)
        with self._lock:
            p = self._plugins.get(name)
            if p is None:
                f = self._factories.get(name)
                if f is None:
                    raise RuntimeError("Device with \"%s\" name is not registered in the OpenVINO Runtime" % device_name)
                p = f(self)
                p.device_name = p.device_name or name
                self._plugins[name] = p
            return p

    @property
    def available_devices(self) -> List[str]:
        return self.get_available_devices()

    def get_available_devices(self) -> List[str]:
        out = []
        for name in self._factories:
            if name in ("AUTO", "MULTI", "HETERO", "BATCH"):
                continue
            try:
                ids = self._get_plugin(name).available_device_ids()
            except Exception:   # noqa: BLE001 - a device that cannot start is simply not available
                continue
            if len(ids) == 1:
                out.append(name)
            else:
                out.extend("%s.%s" % (name, i) for i in ids)
        return out

    def get_versions(self, device_name: str) -> Dict[str, Version]:
        name, cfg = _parse_device(device_name)
        names = [name] + [d.split("(")[0].split(".")[0] for d in cfg.get(props.device.priorities, "").split(",") if d]
        return {n: Version(self._get_plugin(n).description) for n in names}

    # ---- properties
    def set_property(self, device_or_config, config=None) -> None:
        if config is None:
            cfg = props.normalize(device_or_config)
            for k, v in cfg.items():
                self._core_config[k] = v
                if k == props.log.level:
                    _log.set_level(v)
            return
        name, dev_cfg = _parse_device(device_or_config)
        cfg = props.normalize(config)
        core_keys = {props.cache_dir, props.enable_mmap, props.force_tbb_terminate, props.cache_encryption_callbacks}
        plugin_cfg = {k: v for k, v in cfg.items() if k not in core_keys or k == props.cache_dir}
        self._get_plugin(name).set_property(plugin_cfg)

    def get_property(self, device_or_name, name=None, arguments=None):
        if name is None:
            key = str(device_or_name)
            if key == props.available_devices:
                return self.get_available_devices()
            if key not in self._core_config:
                raise RuntimeError("unknown core property %s" % key)
            return self._core_config[key]
        dev, dev_cfg = _parse_device(device_or_name)
        args = dict(dev_cfg)
        args.update(arguments or {})
        return self._get_plugin(dev).get_property(str(name), args)

    # ---- reading
    def read_model(self, model, weights=None, config=None) -> Model:
        from ..frontend import read_model as _read
        with _trace.scope("ov::ReadTime", "Core::read_model"):
            return _read(model, weights, self._extensions)

    def add_extension(self, ext) -> None:
        """An ``ov.Op`` sub-class or ``OpExtension`` (the operation becomes readable from IR), a frontend extension
        (handed to every frontend), or a list of those. Shared libraries of compiled extensions are not loaded."""
        if isinstance(ext, (list, tuple)):
            for e in ext:
                self.add_extension(e)
            return
        from .._compat import OpExtension
        from .._op_base import Op
        from ..frontend import _manager
        from ..frontend.input_model import ConversionExtension, DecoderTransformationExtension, ProgressReporterExtension, TelemetryExtension
        if isinstance(ext, str):
            raise RuntimeError("extension libraries (%s) are not loaded by this runtime: register the operation with ov.Op / OpExtension" % ext)
        if isinstance(ext, type) and issubclass(ext, Op):
            ext._ensure_registered()
        elif isinstance(ext, OpExtension) and not ext.fw_type:
            ext.register()
        elif isinstance(ext, (OpExtension, ConversionExtension, DecoderTransformationExtension, ProgressReporterExtension, TelemetryExtension)):
            for fe in _manager._frontends.values():
                try:
                    fe.add_extension(ext)
                except RuntimeError:
                    pass        # a frontend without an operation table, or another framework's operation
        self._extensions.append(ext)

    def register_plugins(self, xml_config_file: str) -> None:
        """Devices from a plugins file: ``<ie><plugins><plugin name="X" location="module:attr">`` with optional
        ``<properties><property key= value=/>``."""
        import xml.etree.ElementTree as ET
        root = ET.parse(xml_config_file).getroot()
        for pl in root.iter("plugin"):
            cfg = {p.get("key"): p.get("value") for p in pl.iter("property")}
            self.register_plugin(pl.get("location"), pl.get("name"), cfg)

    # ---- compile
    def _cache_dir(self, plugin: Plugin, cfg: dict) -> str:
        return cfg.get(props.cache_dir) or plugin.config.get(props.cache_dir) or self._core_config.get(props.cache_dir) or ""

    def compile_model(self, model, device_name: Optional[str] = None, config=None, *, weights=None) -> CompiledModel:
        if device_name is None:
            device_name = "AUTO"
        if isinstance(device_name, dict):
            device_name, config = "AUTO", device_name
        cfg = props.normalize(config)
        dev, dev_cfg = _parse_device(device_name)
        dev_cfg.update(cfg)
        cfg = dev_cfg
        # per-device sub-configs: {"DEVICE_PROPERTIES": {"CPU": {...}}} or {"CPU": {...}}
        sub = cfg.pop(props.device.properties, None) or {}
        for k in list(cfg.keys()):
            if isinstance(cfg[k], dict) and k in self._factories:
                sub[k] = cfg.pop(k)
        if dev in sub:
            cfg.update(sub.pop(dev))
        if sub:
            cfg[props.device.properties] = sub
        plugin = self._get_plugin(dev)
        if not isinstance(model, Model):
            model = self.read_model(model, weights)
        cache_dir = self._cache_dir(plugin, cfg)
        cfg.pop(props.cache_dir, None)
        callbacks = cfg.pop(props.cache_encryption_callbacks, None) or self._core_config.get(props.cache_encryption_callbacks)
        with _trace.scope("ov::LoadTime", "Core::compile_model::%s" % dev):
            if cache_dir and "EXPORT_IMPORT" in plugin.capabilities():
                cm = self._compile_with_cache(plugin, model, cfg, cache_dir, callbacks)
                _log.info("core", "compiled '%s' for %s (%s)" % (model.get_friendly_name(), dev, "cache hit" if cm.loaded_from_cache else "cache miss"))
                return cm
            cm = plugin.compile_model(model, cfg)
        _log.info("core", "compiled '%s' for %s" % (model.get_friendly_name(), dev))
        return cm

    def _cache_key(self, plugin: Plugin, model: Model, cfg: dict) -> str:
        h = hashlib.sha256()
        h.update(str(_c.model_hash(model._m)).encode())
        h.update(plugin.device_name.encode())
        h.update(__version__.encode())
        merged = plugin.merged_config(cfg)
        for k in sorted(merged):
            if isinstance(merged[k], (str, int, float, bool)):
                h.update(("%s=%s;" % (k, merged[k])).encode())
        return h.hexdigest()[:32]

    def _compile_with_cache(self, plugin: Plugin, model: Model, cfg: dict, cache_dir: str, callbacks=None) -> CompiledModel:
        """One cache entry per (model, device, compile configuration). The entry is read through a memory mapping when
        ``ENABLE_MMAP`` is on; ``CACHE_ENCRYPTION_CALLBACKS`` = (encrypt, decrypt) are applied to the stored bytes; a lock file
        per entry makes processes that want the same entry take turns, so that only the first one compiles
        (src/inference/src/cache_manager.hpp, src/inference/src/cache_guard.cpp)."""
        os.makedirs(cache_dir, exist_ok=True)
        path = os.path.join(cache_dir, self._cache_key(plugin, model, cfg) + ".blob")
        encrypt, decrypt = (callbacks if callbacks else (None, None))
        use_mmap = bool(self._core_config.get(props.enable_mmap, True)) and decrypt is None
        with _EntryLock(path + ".lock"):
            if os.path.exists(path):
                try:
                    with open(path, "rb") as f:
                        if use_mmap and os.path.getsize(path) > 0:
                            import mmap
                            data = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
                        else:
                            data = f.read()
                    if decrypt is not None:
                        data = decrypt(bytes(data))
                    blob = ModelBlob.from_bytes(data)
                    if blob.header.get("runtime") != __version__ or blob.header.get("device") != plugin.device_name:
                        raise RuntimeError("stale cache entry")
                    cm = plugin.import_model(blob, cfg)
                    cm.loaded_from_cache = True
                    return cm
                except Exception:   # noqa: BLE001 - a broken entry is removed and the model compiled afresh
                    try:
                        os.remove(path)
                    except OSError:
                        pass
            cm = plugin.compile_model(model, cfg)
            tmp = path + ".%d.tmp" % os.getpid()
            payload = cm.export_model()
            if encrypt is not None:
                payload = encrypt(bytes(payload))
            with open(tmp, "wb") as f:
                f.write(payload)
            os.replace(tmp, path)
            return cm

    def import_model(self, model_stream, device_name: str, config=None) -> CompiledModel:
        data = model_stream.read() if hasattr(model_stream, "read") else model_stream
        blob = ModelBlob.from_bytes(data)
        dev, dev_cfg = _parse_device(device_name)
        dev_cfg.update(props.normalize(config))
        return self._get_plugin(dev).import_model(blob, dev_cfg)

    def query_model(self, model: Model, device_name: str, config=None) -> Dict[str, str]:
        dev, dev_cfg = _parse_device(device_name)
        dev_cfg.update(props.normalize(config))
        return self._get_plugin(dev).query_model(model, dev_cfg)

    def create_context(self, device_name: str, params: dict):
        plugin = self._get_plugin(_parse_device(device_name)[0])
        if not hasattr(plugin, "create_context"):
            raise RuntimeError("device %s has no remote context" % device_name)
        return plugin.create_context(params)

    def get_default_context(self, device_name: str):
        plugin = self._get_plugin(_parse_device(device_name)[0])
        if not hasattr(plugin, "get_default_context"):
            raise RuntimeError("device %s has no remote context" % device_name)
        return plugin.get_default_context()


def _load_cuda_plugin(core: Core) -> Plugin:
    from .cuda_plugin import CudaPlugin
    return CudaPlugin(core)


def compile_model(model, device_name: str = "AUTO", config=None) -> CompiledModel:
    """Shortcut: ``Core().compile_model(...)``."""
    return Core().compile_model(model, device_name, config)
