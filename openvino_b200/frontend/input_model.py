"""Model editing before conversion: ``InputModel`` and ``Place``, and the frontend extensions.

``fe.load(path)`` gives an ``InputModel``; its places (tensors and operations, found by name) can be given shapes and
types, and the model can be cut: ``override_all_inputs`` / ``override_all_outputs`` / ``extract_subgraph`` make any
tensors the new boundary. ``fe.convert(input_model)`` returns the edited ``Model``. The frontends of this package
translate a source graph in one walk, so an ``InputModel`` converts on first use and edits the result; places refer to
values of that graph. Role in the reference: ov::frontend::InputModel / Place
(src/frontends/common/include/openvino/frontend/input_model.hpp, place.hpp) and the extension classes of
src/frontends/common/include/openvino/frontend/extension/ (conversion.hpp, telemetry.hpp, progress_reporter.hpp).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

from .._graph import Model, Node, Output, parameter, result
from .._types import PartialShape, Type


class Place:
    """A tensor (an ``Output`` of the graph) or an operation."""

    def __init__(self, model: "InputModel", output: Optional[Output] = None, node: Optional[Node] = None):
        self._im, self._output, self._node = model, output, node

    def get_names(self) -> List[str]:
        if self._output is not None:
            names = sorted(self._output.get_names())
            return names or [self._output.get_node().get_friendly_name()]
        return [self._node.get_friendly_name()]

    def is_input(self) -> bool:
        return self._output is not None and self._output.get_node().get_type_name() == "Parameter"

    def is_output(self) -> bool:
        return self._output is not None and any(i.get_node().get_type_name() == "Result" for i in self._output.get_target_inputs())

    def is_equal(self, other: "Place") -> bool:
        return (self._output is not None and other._output is not None and self._output == other._output) or \
               (self._node is not None and self._node is other._node)

    def get_producing_operation(self) -> "Place":
        return Place(self._im, node=self._output.get_node())

    def get_consuming_operations(self) -> List["Place"]:
        return [Place(self._im, node=i.get_node()) for i in self._output.get_target_inputs()]

    def get_target_tensor(self, index: int = 0) -> "Place":
        return Place(self._im, output=self._node.output(index))

    def get_source_tensor(self, index: int = 0) -> "Place":
        return Place(self._im, output=self._node.input_value(index))

    def __repr__(self):
        return "<Place %s %s>" % ("tensor" if self._output is not None else "operation", self.get_names())


class InputModel:
    def __init__(self, frontend, source, weights=None):
        self._fe, self._source, self._weights = frontend, source, weights
        self._model: Optional[Model] = None

    # the converted graph, made on first use
    def _m(self) -> Model:
        if self._model is None:
            self._model = self._fe._convert_source(self._source, self._weights)
        return self._model

    # ---- lookup
    def get_inputs(self) -> List[Place]:
        return [Place(self, output=p.output(0)) for p in self._m().get_parameters()]

    def get_outputs(self) -> List[Place]:
        return [Place(self, output=r.input_value(0)) for r in self._m().get_results()]

    def get_place_by_tensor_name(self, name: str) -> Optional[Place]:
        for n in self._m().get_ops():
            for o in n.outputs():
                if name in o.get_names():
                    return Place(self, output=o)
        for n in self._m().get_ops():                      # tensors without a name answer to their producer's name
            if n.get_friendly_name() == name and n.get_output_size() >= 1:
                return Place(self, output=n.output(0))
        return None

    def get_place_by_operation_name(self, name: str) -> Optional[Place]:
        for n in self._m().get_ops():
            if n.get_friendly_name() == name:
                return Place(self, node=n)
        return None

    def get_place_by_operation_name_and_output_port(self, name: str, port: int) -> Optional[Place]:
        p = self.get_place_by_operation_name(name)
        return p.get_target_tensor(port) if p is not None else None

    # ---- naming, shapes, types
    def set_name_for_tensor(self, place: Place, name: str) -> None:
        place._output.set_names({name})

    def add_name_for_tensor(self, place: Place, name: str) -> None:
        place._output.set_names(set(place._output.get_names()) | {name})

    def set_partial_shape(self, place: Place, shape) -> None:
        if not place.is_input():
            raise RuntimeError("shapes can be set on input places; cut the model there first (override_all_inputs)")
        m = self._m()
        idx = m.get_parameter_index(place._output.get_node())
        m.reshape({idx: shape if isinstance(shape, PartialShape) else PartialShape(shape)})

    def get_partial_shape(self, place: Place) -> PartialShape:
        return place._output.get_partial_shape()

    def set_element_type(self, place: Place, element_type) -> None:
        if not place.is_input():
            raise RuntimeError("element types can be set on input places")
        place._output.get_node().set_attribute("element_type", element_type if isinstance(element_type, Type) else Type(element_type))
        self._m().validate_nodes_and_infer_types()

    def get_element_type(self, place: Place) -> Type:
        return place._output.get_element_type()

    # ---- cutting
    def override_all_outputs(self, outputs: Sequence[Place]) -> None:
        m = self._m()
        self._model = Model([result(p._output) for p in outputs], m.get_parameters(), m.get_friendly_name())
        self._prune_inputs()

    def override_all_inputs(self, inputs: Sequence[Place]) -> None:
        m = self._m()
        params = []
        for p in inputs:
            if p.is_input():
                params.append(p._output.get_node())
                continue
            o = p._output
            name = sorted(o.get_names())[0] if o.get_names() else o.get_node().get_friendly_name()
            np_ = parameter(o.get_partial_shape(), o.get_element_type(), name)
            np_.output(0).set_names(set(o.get_names()) or {name})
            for i in list(o.get_target_inputs()):
                i.replace_source_output(np_.output(0))
            p._output = np_.output(0)
            params.append(np_)
        self._model = Model([r.input_value(0) for r in m.get_results()], params, m.get_friendly_name())

    def extract_subgraph(self, inputs: Sequence[Place], outputs: Sequence[Place]) -> None:
        self.override_all_outputs(outputs)
        self.override_all_inputs(inputs)

    def _prune_inputs(self) -> None:
        """Parameters that no longer reach an output are dropped."""
        m = self._model
        reachable, stack = set(), [r for r in m.get_results()]
        while stack:
            n = stack.pop()
            if id(n) in reachable:
                continue
            reachable.add(id(n))
            stack.extend(n.input_value(i).get_node() for i in range(n.get_input_size()))
        keep = [p for p in m.get_parameters() if id(p) in reachable]
        if len(keep) != len(m.get_parameters()):
            self._model = Model([r.input_value(0) for r in m.get_results()], keep, m.get_friendly_name())


# ---------------------------------------------------------------------------------------------- extensions
class ConversionExtension:
    """A translator for one source operation, supplied by the user: ``ConversionExtension("MyOp", fn)``. ``fn`` has the
    signature of the frontend's own translators (it is put into that frontend's table)."""

    def __init__(self, op_type: str, converter: Callable):
        self.op_type, self.converter = op_type, converter


class TelemetryExtension:
    """Receives usage events of a conversion: ``send_event(category, action, label, value)``; the frontends report the
    operation types they met (``"op_count"``) and errors."""

    def __init__(self, event_category: str, send_event: Callable, send_error: Optional[Callable] = None, send_stack_trace: Optional[Callable] = None):
        self.event_category, self._event, self._error, self._stack = event_category, send_event, send_error, send_stack_trace

    def send_event(self, action: str, label: str, value: int = 1) -> None:
        self._event(self.event_category, action, label, value)

    def send_error(self, message: str) -> None:
        if self._error is not None:
            self._error(self.event_category, message)

    def send_stack_trace(self, trace: str) -> None:
        if self._stack is not None:
            self._stack(self.event_category, trace)


class ProgressReporterExtension:
    """``callback(progress in [0, 1], total_steps, completed_steps)`` while a model converts."""

    def __init__(self, callback: Optional[Callable] = None):
        self._cb = callback or (lambda progress, total, completed: None)

    def report_progress(self, progress: float, total_steps: int, completed_steps: int) -> None:
        if not (0.0 <= progress <= 1.0) or completed_steps > total_steps:
            raise RuntimeError("bad progress report: %r of %r (%r)" % (completed_steps, total_steps, progress))
        self._cb(progress, total_steps, completed_steps)


class NodeContext:
    """What a user translator sees of one source operation: its inputs as graph outputs and its attributes.
    ``get_input(i)``, ``get_input_size()``, ``get_attribute(name, default)``, ``get_op_type()``, ``get_name()``."""

    def __init__(self, op_type: str, inputs, attrs: Optional[dict] = None, name: str = ""):
        self._type, self._inputs, self._attrs, self._name = op_type, list(inputs), dict(attrs or {}), name

    def get_input(self, index: int) -> Output:
        return self._inputs[index]

    def get_input_size(self) -> int:
        return len(self._inputs)

    def get_attribute(self, name: str, default=None):
        return self._attrs.get(name, default)

    def has_attribute(self, name: str) -> bool:
        return name in self._attrs

    def get_op_type(self) -> str:
        return self._type

    def get_name(self) -> str:
        return self._name


class DecoderTransformationExtension:
    """A function applied to every model the frontend has converted (``fn(model)``; a true return value means changed)."""

    def __init__(self, transformation: Callable):
        self.transformation = transformation


def op_extension_translator(ext, frontend_name: str) -> Callable:
    """Translator for ``OpExtension(target, source, names_map, values_map)``: the source operation becomes one ``target``
    node over all of its inputs; attributes are taken by the names map (target name -> source name), then the fixed values."""
    from .._graph import make_op
    target = ext.op if isinstance(ext.op, str) else ext.op._type_and_version()[0]
    version = "" if isinstance(ext.op, str) else ext.op._type_and_version()[1]

    def attrs_from(source: dict) -> dict:
        out = {t: source[s] for t, s in ext.attr_names_map.items() if s in source}
        out.update(ext.attr_values_map)
        return out
    if frontend_name == "onnx":
        return lambda n, i: [o for o in make_op(target, list(i), attrs_from(n.attrs), version=version).outputs()]
    raise RuntimeError("OpExtension with a source operation is served by the ONNX frontend; frontend '%s' takes ConversionExtension" % frontend_name)
