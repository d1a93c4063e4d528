"""Graph API: ``Node``, ``Output``, ``Input``, ``Model`` and the generic operation factory.

Thin Python views over the native graph (``_ovcore.Node`` / ``_ovcore.Model``); every view of the same
native node compares equal. API shape follows src/bindings/python/src/pyopenvino/graph/{node,node_output,
node_input,model}.cpp and src/core/include/openvino/core/model.hpp:96-515.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Union

import numpy as np

from . import _ovcore as _c
from ._tensor import Tensor
from ._types import Dimension, PartialShape, Shape, Type


def _attr_from_core(v):
    if isinstance(v, tuple) and len(v) == 2 and isinstance(v[0], str):
        if v[0] == "__type__":
            return Type(v[1])
        if v[0] == "__pshape__":
            return PartialShape._from_core(v[1])
    if isinstance(v, dict):
        return {k: _attr_from_core(x) for k, x in v.items()}
    return v


def _attr_to_core(v):
    if isinstance(v, Type):
        return ("__type__", v.name)
    if isinstance(v, PartialShape):
        return ("__pshape__", v._to_core())
    if isinstance(v, Shape):
        return list(v)
    if isinstance(v, np.ndarray):
        return v.tolist()
    if isinstance(v, (np.integer,)):
        return int(v)
    if isinstance(v, (np.floating,)):
        return float(v)
    if isinstance(v, (np.bool_,)):
        return bool(v)
    if isinstance(v, dict):
        return {k: _attr_to_core(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)) and not (len(v) == 2 and isinstance(v[0], str) and v[0].startswith("__")):
        return [_attr_to_core(x) for x in v]
    return v


class RTMap:
    """dict-like view of a node's / port's / model's runtime info."""

    def __init__(self, getter, setter, eraser=None):
        self._get, self._set, self._erase = getter, setter, eraser

    def _d(self):
        return {k: _attr_from_core(v) for k, v in self._get().items()}

    def __getitem__(self, k):
        return self._d()[k]

    def __setitem__(self, k, v):
        self._set(k, _attr_to_core(v))

    def __delitem__(self, k):
        if self._erase is None:
            raise TypeError("this runtime info cannot erase entries")
        self._erase(k)

    def __contains__(self, k):
        return k in self._get()

    def __iter__(self):
        return iter(self._d())

    def __len__(self):
        return len(self._get())

    def keys(self):
        return self._d().keys()

    def items(self):
        return self._d().items()

    def values(self):
        return self._d().values()

    def pop(self, k, default=None):
        if k in self:
            v = self[k]
            del self[k]
            return v
        return default

    def get(self, k, default=None):
        return self._d().get(k, default)

    def __repr__(self):
        return "RTMap(%r)" % self._d()


class Output:
    """One output port of a node (a value in the graph)."""

    __slots__ = ("_n", "_i")

    def __init__(self, node, index: int = 0):
        self._n = node._n if isinstance(node, Node) else node
        self._i = int(index)

    def _core(self):
        return (self._n, self._i)

    def get_node(self) -> "Node":
        return Node(self._n)

    node = property(get_node)

    def get_index(self) -> int:
        return self._i

    index = property(get_index)

    def get_element_type(self) -> Type:
        return Type(self._n.output_type(self._i))

    element_type = property(get_element_type)

    def get_partial_shape(self) -> PartialShape:
        return PartialShape._from_core(self._n.output_shape(self._i))

    partial_shape = property(get_partial_shape)

    def get_shape(self) -> Shape:
        return self.get_partial_shape().get_shape()

    shape = property(get_shape)

    def _named(self):
        # a Result's output is the same tensor as its input: names live on the producer
        if self._n.type == "Result":
            n, i = self._n.input_source(0)
            return n, i
        return self._n, self._i

    def get_names(self) -> set:
        n, i = self._named()
        return set(n.output_names(i))

    names = property(get_names)

    def set_names(self, names) -> None:
        n, i = self._named()
        n.set_output_names(i, set(names))

    def add_names(self, names) -> None:
        n, i = self._named()
        n.set_output_names(i, set(n.output_names(i)) | set(names))

    def get_any_name(self) -> str:
        names = sorted(self.get_names())
        if not names:
            raise RuntimeError("Attempt to get a name for a Tensor without names")
        return names[0]

    any_name = property(get_any_name)

    def get_tensor(self):
        return self

    def get_target_inputs(self) -> List["Input"]:
        return [Input(Node(n), i) for n, i in self._n.output_users(self._i)]

    def get_rt_info(self) -> RTMap:
        return RTMap(lambda: self._n.output_rt_info(self._i), lambda k, v: self._n.set_output_rt_info(self._i, k, v))

    rt_info = property(get_rt_info)

    def replace(self, other: "Output") -> None:
        _c.replace_output(self._core(), as_output(other)._core())

    def __eq__(self, other):
        return isinstance(other, Output) and self._n.id == other._n.id and self._i == other._i

    def __hash__(self):
        return hash((self._n.id, self._i))

    def __repr__(self):
        return "<Output: names%s, shape%s, type: %s>" % (sorted(self.get_names()), self.get_partial_shape().to_string(), self.get_element_type())

    # arithmetic sugar (as in openvino.Node)
    def _bin(self, other, op, swap=False):
        from . import opset
        a, b = (other, self) if swap else (self, other)
        return getattr(opset, op)(a, b).output(0)

    def __add__(self, o): return self._bin(o, "add")
    def __radd__(self, o): return self._bin(o, "add", True)
    def __sub__(self, o): return self._bin(o, "subtract")
    def __rsub__(self, o): return self._bin(o, "subtract", True)
    def __mul__(self, o): return self._bin(o, "multiply")
    def __rmul__(self, o): return self._bin(o, "multiply", True)
    def __truediv__(self, o): return self._bin(o, "divide")
    def __rtruediv__(self, o): return self._bin(o, "divide", True)


class Input:
    """One input port of a node."""

    __slots__ = ("_node", "_i")

    def __init__(self, node: "Node", index: int):
        self._node, self._i = node, int(index)

    def get_node(self) -> "Node":
        return self._node

    def get_index(self) -> int:
        return self._i

    def get_source_output(self) -> Output:
        n, i = self._node._n.input_source(self._i)
        return Output(n, i)

    def replace_source_output(self, new: Output) -> None:
        self._node._n.set_input(self._i, as_output(new)._core())

    def get_element_type(self) -> Type:
        return self.get_source_output().get_element_type()

    def get_partial_shape(self) -> PartialShape:
        return self.get_source_output().get_partial_shape()

    def get_shape(self) -> Shape:
        return self.get_partial_shape().get_shape()

    def __repr__(self):
        return "<Input %d of %r>" % (self._i, self._node)


class Node:
    """An operation in the graph."""

    __slots__ = ("_n",)

    def __init__(self, core_node):
        self._n = core_node._n if isinstance(core_node, Node) else core_node

    # identity
    def __eq__(self, other):
        return isinstance(other, Node) and self._n.id == other._n.id

    def __hash__(self):
        return hash(self._n.id)

    def __repr__(self):
        outs = ", ".join(self.get_output_partial_shape(i).to_string() for i in range(self.get_output_size()))
        return "<%s: '%s' (%s)>" % (self.get_type_name(), self.get_friendly_name(), outs)

    # naming / typing
    def get_type_name(self) -> str:
        return self._n.type

    type_name = property(get_type_name)

    def get_type_info(self):
        return _TypeInfo(self._n.type, self._n.version)

    type_info = property(get_type_info)

    def get_version(self) -> str:
        return self._n.version

    def get_friendly_name(self) -> str:
        return self._n.name

    def set_friendly_name(self, name: str) -> None:
        self._n.name = name

    friendly_name = property(get_friendly_name, set_friendly_name)

    def get_name(self) -> str:
        return "%s_%d" % (self._n.type, self._n.id)

    name = property(get_name)

    # ports
    def get_input_size(self) -> int:
        return self._n.num_inputs()

    def get_output_size(self) -> int:
        return self._n.num_outputs()

    def input(self, i: int) -> Input:
        if i < 0 or i >= self._n.num_inputs():
            raise IndexError("input %d out of range" % i)
        return Input(self, i)

    def inputs(self) -> List[Input]:
        return [Input(self, i) for i in range(self._n.num_inputs())]

    def output(self, i: int = 0) -> Output:
        if i < 0 or i >= self._n.num_outputs():
            raise IndexError("output %d out of range" % i)
        return Output(self._n, i)

    def outputs(self) -> List[Output]:
        return [Output(self._n, i) for i in range(self._n.num_outputs())]

    def input_value(self, i: int) -> Output:
        return self.input(i).get_source_output()

    def input_values(self) -> List[Output]:
        return [self.input_value(i) for i in range(self.get_input_size())]

    def get_input_node(self, i: int) -> "Node":
        return self.input_value(i).get_node()

    def get_output_element_type(self, i: int = 0) -> Type:
        return Type(self._n.output_type(i))

    def get_output_partial_shape(self, i: int = 0) -> PartialShape:
        return PartialShape._from_core(self._n.output_shape(i))

    def get_output_shape(self, i: int = 0) -> Shape:
        return self.get_output_partial_shape(i).get_shape()

    def get_element_type(self) -> Type:
        return self.get_output_element_type(0)

    element_type = property(get_element_type)

    def get_input_element_type(self, i: int) -> Type:
        return self.input_value(i).get_element_type()

    def get_input_partial_shape(self, i: int) -> PartialShape:
        return self.input_value(i).get_partial_shape()

    def get_input_shape(self, i: int) -> Shape:
        return self.get_input_partial_shape(i).get_shape()

    shape = property(lambda self: self.get_output_shape(0))
    partial_shape = property(lambda self: self.get_output_partial_shape(0))

    def get_output_tensor(self, i: int = 0) -> Output:
        return self.output(i)

    def get_users(self) -> List["Node"]:
        seen, out = set(), []
        for o in self.outputs():
            for inp in o.get_target_inputs():
                if inp.get_node() not in seen:
                    seen.add(inp.get_node())
                    out.append(inp.get_node())
        return out

    # attributes
    def get_attributes(self) -> dict:
        return {k: _attr_from_core(v) for k, v in self._n.attrs().items()}

    def set_attribute(self, name: str, value) -> None:
        self._n.set_attr(name, _attr_to_core(value))

    def get_attribute(self, name: str):
        return _attr_from_core(self._n.get_attr(name))

    def __getattr__(self, item):
        # get_<attr>() / set_<attr>() sugar
        if item.startswith("get_") and self._n.has_attr(item[4:]):
            return lambda: self.get_attribute(item[4:])
        if item.startswith("set_") and self._n.has_attr(item[4:]):
            return lambda v: self.set_attribute(item[4:], v)
        raise AttributeError(item)

    def get_rt_info(self) -> RTMap:
        return RTMap(self._n.rt_info, lambda k, v: self._n.set_rt_info(k, v), self._n.erase_rt_info)

    rt_info = property(get_rt_info)

    def validate(self) -> None:
        self._n.validate()

    validate_and_infer_types = validate
    constructor_validate_and_infer_types = validate

    def clone_with_new_inputs(self, inputs) -> "Node":
        return Node(self._n.clone_with_new_inputs([as_output(i)._core() for i in inputs]))

    # constants
    def get_data(self) -> np.ndarray:
        return Tensor._from_core(self._n.constant_data()).data

    data = property(get_data)

    def get_tensor_view(self) -> Tensor:
        return Tensor._from_core(self._n.constant_data())

    tensor_view = property(get_tensor_view)

    def get_vector(self) -> np.ndarray:
        t = self.get_tensor_view()
        if t.element_type.bitwidth % 8 == 0 and t.element_type.name != "bf16" and not t.element_type.name.startswith("f8"):
            return t.data.reshape(-1)
        return t.to_float32().reshape(-1)

    def get_value_strings(self):
        return [str(v) for v in self.get_vector().tolist()]

    def get_byte_size(self) -> int:
        return self.get_tensor_view().byte_size

    # sub-graphs
    def get_function(self, index: int = 0) -> "Model":
        return Model._wrap(self._n.bodies()[index])

    def get_then_body(self) -> "Model":
        return self.get_function(0)

    def get_else_body(self) -> "Model":
        return self.get_function(1)

    # arithmetic sugar
    def __add__(self, o): return self.output(0) + o
    def __radd__(self, o): return o + self.output(0)
    def __sub__(self, o): return self.output(0) - o
    def __rsub__(self, o): return o - self.output(0)
    def __mul__(self, o): return self.output(0) * o
    def __rmul__(self, o): return o * self.output(0)
    def __truediv__(self, o): return self.output(0) / o
    def __rtruediv__(self, o): return o / self.output(0)


class _TypeInfo:
    def __init__(self, name, version):
        self.name, self.version_id = name, version

    def __repr__(self):
        return "<DiscreteTypeInfo: %s v:%s>" % (self.name, self.version_id)

    def __eq__(self, other):
        return isinstance(other, _TypeInfo) and (self.name, self.version_id) == (other.name, other.version_id)


NodeInput = Union[Node, Output, np.ndarray, int, float, list, tuple]


def as_output(x, dtype=None) -> Output:
    """Node / Output / python value -> Output (python values become Constants)."""
    if isinstance(x, Output):
        return x
    if isinstance(x, Node):
        if x.get_output_size() != 1:
            raise ValueError("%r has %d outputs: pick one with .output(i)" % (x, x.get_output_size()))
        return x.output(0)
    return constant(x, dtype).output(0)


def constant(value, dtype=None, name: Optional[str] = None, shared_memory: bool = False) -> Node:
    """Constant from a numpy array / Tensor / scalar / nested list. ``dtype`` converts the values."""
    if isinstance(value, Tensor):
        t = value
        if dtype is not None and Type(dtype) != t.element_type:
            t = t.astype(dtype)
    else:
        try:
            import sys
            torch = sys.modules.get("torch")
            if torch is None:
                raise ImportError
            if isinstance(value, torch.Tensor):
                value = Tensor(value.detach().cpu(), shared_memory=shared_memory)
        except ImportError:
            pass
        if isinstance(value, Tensor):
            t = value if dtype is None or Type(dtype) == value.element_type else value.astype(dtype)
        else:
            arr = np.asarray(value)
            if arr.dtype.kind in ("U", "S", "O"):
                t = Tensor(arr)
            else:
                if dtype is None:
                    if arr.dtype == np.float64 and not isinstance(value, np.ndarray):
                        arr = arr.astype(np.float32)
                    t = Tensor(arr, shared_memory=shared_memory and isinstance(value, np.ndarray))
                else:
                    dt = Type(dtype)
                    std = dt.bitwidth % 8 == 0 and dt.name not in ("bf16", "f8e4m3", "f8e5m2", "f8e8m0")
                    if std:
                        t = Tensor(arr.astype(dt.to_dtype()))
                    else:
                        t = Tensor(arr.astype(np.float32)).astype(dt)
    if t.element_type == Type.string:
        n = _c.make_string_constant([bytes(s) for s in t._strings], list(t.shape))
    else:
        n = _c.make_constant(np.ascontiguousarray(t.data), t.element_type.name, list(t.shape), bool(shared_memory))
    node = Node(n)
    if name:
        node.set_friendly_name(name)
    return node


def parameter(shape=None, dtype=Type.f32, name: Optional[str] = None) -> Node:
    ps = shape if isinstance(shape, PartialShape) else PartialShape(shape if shape is not None else [])
    return Node(_c.make_parameter(Type(dtype).name, ps._to_core(), name or ""))


def result(value, name: Optional[str] = None) -> Node:
    n = Node(_c.make_result(as_output(value)._core()))
    if name:
        n.set_friendly_name(name)
    return n


def make_op(op_type: str, inputs: Sequence[NodeInput], attrs: Optional[dict] = None, version: str = "", name: Optional[str] = None) -> Node:
    ins = [as_output(i)._core() for i in inputs]
    n = Node(_c.make_node(op_type, version, ins, {k: _attr_to_core(v) for k, v in (attrs or {}).items() if v is not None}))
    if name:
        n.set_friendly_name(name)
    return n


class Model:
    """A graph with Parameters, Results and Sinks (ov.Model)."""

    def __init__(self, results=None, parameters=None, name: str = "", sinks=None, *args):
        if isinstance(results, _c.Model):
            self._m = results
            return
        if isinstance(results, Model):
            self._m = results._m
            return
        # accepted forms: Model(results, params, name), Model(results, sinks, params, name)
        if isinstance(name, (list, tuple)):
            sinks, parameters, name = parameters, name, (args[0] if args else "")
        res_nodes = []
        items = results if isinstance(results, (list, tuple)) else [results]
        for r in items:
            if isinstance(r, Node) and r.get_type_name() == "Result":
                res_nodes.append(r._n)
            else:
                res_nodes.append(result(r)._n)
        sink_nodes = [s._n for s in (sinks or [])]
        params = [p._n for p in (parameters or [])]
        self._m = _c.Model(res_nodes, sink_nodes, params, name or "")

    @staticmethod
    def _wrap(core_model) -> "Model":
        m = Model.__new__(Model)
        m._m = core_model
        return m

    # names
    def get_friendly_name(self) -> str:
        return self._m.name

    def set_friendly_name(self, n: str) -> None:
        self._m.name = n

    friendly_name = property(get_friendly_name, set_friendly_name)

    def get_name(self) -> str:
        return self._m.name

    name = property(get_name)

    # structure
    def get_parameters(self) -> List[Node]:
        return [Node(p) for p in self._m.params]

    def get_results(self) -> List[Node]:
        return [Node(r) for r in self._m.results]

    def get_sinks(self) -> List[Node]:
        return [Node(s) for s in self._m.sinks]

    def get_ops(self) -> List[Node]:
        return [Node(n) for n in self._m.ordered_ops()]

    get_ordered_ops = get_ops

    parameters = property(get_parameters)
    results = property(get_results)
    sinks = property(get_sinks)

    @property
    def inputs(self) -> List[Output]:
        return [Output(p, 0) for p in self._m.params]

    @property
    def outputs(self) -> List[Output]:
        return [Output(r, 0) for r in self._m.results]

    def _find_port(self, ports, key, kind):
        if isinstance(key, int):
            if key < 0 or key >= len(ports):
                raise IndexError("%s index %d out of range" % (kind, key))
            return ports[key]
        if isinstance(key, str):
            for p in ports:
                if key in p.get_names() or (kind == "input" and p.get_node().get_friendly_name() == key):
                    return p
            for p in ports:   # results inherit the names of their producers
                if kind == "output" and key in p.get_node().input_value(0).get_names():
                    return p
            raise RuntimeError("no %s with name '%s'" % (kind, key))
        if isinstance(key, Output):
            return key
        if key is None:
            if len(ports) != 1:
                raise RuntimeError("%s() needs an index or a name: the model has %d %ss" % (kind, len(ports), kind))
            return ports[0]
        raise TypeError("bad %s key %r" % (kind, key))

    def input(self, key=None) -> Output:
        return self._find_port(self.inputs, key, "input")

    def output(self, key=None) -> Output:
        return self._find_port(self.outputs, key, "output")

    def get_output_size(self) -> int:
        return len(self._m.results)

    def get_output_element_type(self, i: int) -> Type:
        return self.outputs[i].get_element_type()

    def get_output_partial_shape(self, i: int) -> PartialShape:
        return self.outputs[i].get_partial_shape()

    def get_output_shape(self, i: int) -> Shape:
        return self.outputs[i].get_shape()

    def get_parameter_index(self, p: Node) -> int:
        for i, q in enumerate(self.get_parameters()):
            if q == p:
                return i
        return -1

    def get_result_index(self, v) -> int:
        for i, r in enumerate(self.get_results()):
            if (isinstance(v, Node) and r == v) or (isinstance(v, Output) and (r.output(0) == v or r.input_value(0) == v)):
                return i
        return -1

    def add_parameters(self, params) -> None:
        self._m.add_parameters([p._n for p in params])

    def remove_parameter(self, p: Node) -> None:
        self._m.remove_parameter(p._n)

    def add_results(self, results) -> None:
        self._m.add_results([r._n for r in results])

    def remove_result(self, r: Node) -> None:
        self._m.remove_result(r._n)

    def add_sinks(self, sinks) -> None:
        self._m.add_sinks([s._n for s in sinks])

    def remove_sink(self, s: Node) -> None:
        self._m.remove_sink(s._n)

    def add_outputs(self, outputs) -> List[Output]:
        items = outputs if isinstance(outputs, (list, tuple)) and not (len(outputs) == 2 and isinstance(outputs[0], str)) else [outputs]
        added = []
        for o in items:
            if isinstance(o, str):
                node = next(n for n in self.get_ops() if n.get_friendly_name() == o)
                o = node.output(0)
            elif isinstance(o, tuple):
                node = next(n for n in self.get_ops() if n.get_friendly_name() == o[0])
                o = node.output(o[1])
            r = result(o)
            self._m.add_results([r._n])
            added.append(r.output(0))
        return added

    def get_variables(self):
        return [_Variable(i, PartialShape._from_core(s), Type(t)) for i, s, t in self._m.variables()]

    def add_variables(self, variables) -> None:
        """Variables follow from the ReadValue / Assign pairs of the graph; adding one that no node uses changes nothing."""
        known = {v.get_info().variable_id for v in self.get_variables()}
        for v in variables:
            if v.get_info().variable_id not in known:
                self.__dict__.setdefault("_extra_variables", []).append(v)

    def remove_variable(self, variable) -> None:
        vid = variable.get_info().variable_id
        if any(v.get_info().variable_id == vid for v in self.get_variables()):
            raise RuntimeError("variable '%s' is used by ReadValue / Assign nodes of the model" % vid)
        self.__dict__["_extra_variables"] = [v for v in self.__dict__.get("_extra_variables", []) if v.get_info().variable_id != vid]

    def get_variable_by_id(self, vid):
        for v in self.get_variables():
            if v.get_info().variable_id == vid:
                return v
        return None

    # shapes
    def is_dynamic(self) -> bool:
        return self._m.is_dynamic()

    dynamic = property(is_dynamic)

    def validate_nodes_and_infer_types(self) -> None:
        self._m.validate()

    def reshape(self, partial_shapes, variables_shapes=None) -> None:
        """reshape(shape) for single-input models, or {index | name | Output: shape}."""
        if not isinstance(partial_shapes, dict):
            if len(self._m.params) != 1:
                raise RuntimeError("reshape(shape) needs a single-input model")
            partial_shapes = {0: partial_shapes}
        shapes = {}
        for k, v in partial_shapes.items():
            port = self.input(k) if not isinstance(k, Output) else k
            idx = self.get_parameter_index(port.get_node())
            ps = v if isinstance(v, PartialShape) else PartialShape(v)
            shapes[idx] = ps._to_core()
        self._m.reshape(shapes)

    def clone(self) -> "Model":
        return Model._wrap(self._m.clone())

    def get_graph_size(self) -> int:
        return self._m.graph_size()

    def evaluate(self, output_tensors, input_tensors, evaluation_context=None) -> bool:
        outs, _ = _c.evaluate(self._m, [(t if isinstance(t, Tensor) else Tensor(t))._to_core() for t in input_tensors])
        for dst, src in zip(output_tensors, outs):
            dst.copy_from(Tensor._from_core(src))
        return True

    # rt_info with path access
    def _rt(self) -> dict:
        return {k: _attr_from_core(v) for k, v in self._m.rt_info().items()}

    def get_rt_info(self, path=None):
        d = self._rt()
        if path is None:
            return RTMap(self._m.rt_info, lambda k, v: self._m.set_rt_info(k, v), self._m.erase_rt_info)
        keys = [path] if isinstance(path, str) else list(path)
        cur = d
        for k in keys:
            if not isinstance(cur, dict) or k not in cur:
                raise RuntimeError("rt_info has no path %r" % (keys,))
            cur = cur[k]
        return _RtValue(cur)

    rt_info = property(lambda self: self.get_rt_info())

    def has_rt_info(self, path) -> bool:
        keys = [path] if isinstance(path, str) else list(path)
        cur = self._rt()
        for k in keys:
            if not isinstance(cur, dict) or k not in cur:
                return False
            cur = cur[k]
        return True

    def set_rt_info(self, obj, path) -> None:
        keys = [path] if isinstance(path, str) else list(path)
        d = self._rt()
        cur = d
        for k in keys[:-1]:
            if not isinstance(cur.get(k), dict):
                cur[k] = {}
            cur = cur[k]
        cur[keys[-1]] = obj if isinstance(obj, (dict, str)) else (obj.name if isinstance(obj, Type) else str(obj) if not isinstance(obj, (int, float, bool, list)) else obj)
        top = keys[0]
        self._m.set_rt_info(top, _attr_to_core(_stringify(d[top])))

    def __repr__(self):
        return "<Model: '%s'\ninputs[\n%s\n]\noutputs[\n%s\n]>" % (
            self.get_friendly_name(), ",\n".join(repr(i) for i in self.inputs), ",\n".join(repr(o) for o in self.outputs))

    def __copy__(self):
        raise TypeError("Cannot copy 'openvino.Model'. Please, use deepcopy instead.")

    def __deepcopy__(self, memo):
        return self.clone()


def _stringify(v):
    if isinstance(v, dict):
        return {k: _stringify(x) for k, x in v.items()}
    if isinstance(v, bool):
        return "1" if v else "0"
    if isinstance(v, (list, tuple)):
        return ",".join(str(x) for x in v)
    return v if isinstance(v, str) else str(v)


class _RtValue:
    """Value stored in model rt_info (strings in IR); ``astype`` converts."""

    def __init__(self, v):
        self.value = v

    def astype(self, t):
        if t is bool:
            return str(self.value).lower() in ("1", "true", "yes")
        if t in (list,):
            return [x for x in str(self.value).split(",")]
        if isinstance(self.value, dict):
            return self.value
        return t(self.value)

    def aslist(self, t=str):
        return [t(x) for x in str(self.value).split(",") if x != ""]

    def __eq__(self, other):
        return self.value == (other.value if isinstance(other, _RtValue) else other)

    def __repr__(self):
        return "<RtInfo %r>" % (self.value,)


class _VariableInfo:
    def __init__(self, vid, shape, et):
        self.variable_id, self.data_shape, self.data_type = vid, shape, et


class _Variable:
    def __init__(self, vid, shape, et):
        self._info = _VariableInfo(vid, shape, et)

    def get_info(self):
        return self._info

    info = property(get_info)
