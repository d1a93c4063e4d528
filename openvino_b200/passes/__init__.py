"""Graph passes: ``Manager``, ``ModelPass``, ``MatcherPass``/``Matcher`` with pattern nodes, and the named passes.

Python face of the native pass infrastructure. Reference API: ``openvino.passes``
(src/bindings/python/src/pyopenvino/graph/passes/{manager,model_pass,matcher_pass,pattern_ops,transformations}.cpp);
the machinery it fronts: ov::pass::Manager::run_passes (src/core/src/pass/manager.cpp:323), GraphRewrite
(src/core/src/pass/graph_rewrite.cpp:73-292) and the pattern Matcher (src/core/src/pattern/matcher.cpp:108-242).
"""
from __future__ import annotations

from typing import Callable, Iterable, List, Optional, Sequence, Union

from .. import _ovcore as _c
from .._graph import Model, Node, Output


class PassBase:
    def __init__(self, name: Optional[str] = None):
        self._name = name or type(self).__name__

    def get_name(self) -> str:
        return self._name

    def set_name(self, name: str) -> None:
        self._name = name

    def _native(self):
        raise NotImplementedError


class ModelPass(PassBase):
    """Sub-class and implement ``run_on_model(model) -> bool`` (True when the graph was changed)."""

    def run_on_model(self, model: Model) -> bool:
        raise NotImplementedError

    def _native(self):
        return _c.make_python_pass(self.get_name(), lambda core_model: bool(self.run_on_model(Model._wrap(core_model))))


class _NamedPass(PassBase):
    """A pass implemented natively, addressed by name with options."""

    native_name = ""

    def __init__(self, **options):
        super().__init__(self.native_name or type(self).__name__)
        self._options = options

    def _native(self):
        return _c.make_pass(self.native_name or type(self).__name__, self._options)

    def run_on_model(self, model: Model) -> bool:
        return self._native().run_on_model(model._m)


class ConstantFolding(_NamedPass):
    native_name = "ConstantFolding"


class NopElimination(_NamedPass):
    native_name = "NopElimination"


class BatchNormDecomposition(_NamedPass):
    native_name = "BatchNormDecomposition"


class Validate(_NamedPass):
    native_name = "Validate"


class InitNodeInfo(_NamedPass):
    native_name = "InitNodeInfo"


class FusedNamesCleanup(_NamedPass):
    native_name = "FusedNamesCleanup"


class ConvertFP32ToFP16(_NamedPass):
    native_name = "ConvertFP32ToFP16"


class CompressFloatConstants(_NamedPass):
    native_name = "CompressFloatConstants"


class MOCTransformations(_NamedPass):
    native_name = "MOCTransformations"


class RMSFusion(_NamedPass):
    native_name = "RMSFusion"


class RoPEFusion(_NamedPass):
    native_name = "RoPEFusion"


class LoraSubgraphFusion(_NamedPass):
    """main(x) + ((x @ A^T) * alpha) @ B^T with A / alpha / B read from variables -> one LoraSubgraph operation."""


class GLUFusion(_NamedPass):
    native_name = "GLUFusion"


class SDPAFusion(_NamedPass):
    native_name = "SDPAFusion"


class FuseMOEExperts(_NamedPass):
    native_name = "FuseMOEExperts"


class ConvertMatMulToFullyConnected(_NamedPass):
    native_name = "ConvertMatMulToFullyConnected"


class ConvertFullyConnectedToFullyConnectedCompressed(_NamedPass):
    native_name = "ConvertFullyConnectedToFullyConnectedCompressed"


class StatefulToStateless(_NamedPass):
    native_name = "StatefulToStateless"


class SDPAToPagedAttention(_NamedPass):
    native_name = "SDPAToPagedAttention"

    def __init__(self, use_block_indices_inputs=False, use_score_outputs=False, allow_score_aggregation=False, allow_cache_rotation=False,
                 allow_xattention=False, allow_adaptive_rkv=False, allow_qq_bias=False):
        super().__init__(use_block_indices_inputs=use_block_indices_inputs, use_score_outputs=use_score_outputs,
                         allow_score_aggregation=allow_score_aggregation, allow_cache_rotation=allow_cache_rotation,
                         allow_xattention=allow_xattention, allow_adaptive_rkv=allow_adaptive_rkv, allow_qq_bias=allow_qq_bias)


class ConvertPrecision(ModelPass):
    """``ConvertPrecision(from_type, to_type)``: re-types parameters, constants and operations. Converting f32 to f16 with
    ``keep_precision_sensitive_in_fp32`` (the default) leaves the nodes marked ``disable_fp16_compression`` in fp32: a
    Convert to f32 goes in front of every input of such an island and a Convert back behind its outputs
    (transformations/convert_precision.cpp together with align_mixed_fp32_fp16_types.cpp in the reference)."""

    def __init__(self, from_type="f32", to_type="f16", keep_precision_sensitive_in_fp32: bool = True):
        super().__init__("ConvertPrecision")
        self._from, self._to, self._keep = str(from_type), str(to_type), bool(keep_precision_sensitive_in_fp32)

    def run_on_model(self, model: Model) -> bool:
        from .. import opset as ops
        from .. import rt_info as rt
        if self._keep and self._from == "f32" and self._to == "f16":
            island = [n for n in model.get_ordered_ops() if rt.fp16_compression_is_disabled(n) and n.get_type_name() not in ("Parameter", "Result")]
            members = set(island)
            for n in island:
                for k in range(n.get_input_size()):
                    src = n.input_value(k)
                    p = src.get_node()
                    if p in members or src.get_element_type().name != "f32" or p.get_type_name() == "Constant":
                        continue
                    cvt = ops.convert(src, "f32")              # stays f32: the producer's output becomes f16 below
                    rt.disable_fp16_compression(cvt)
                    n.input(k).replace_source_output(cvt.output(0))
                for o in n.outputs():
                    if o.get_element_type().name != "f32":
                        continue
                    outside = [i for i in o.get_target_inputs() if i.get_node() not in members and not rt.fp16_compression_is_disabled(i.get_node())]
                    if outside:
                        back = ops.convert(o, "f32")           # unmarked: the native pass re-targets it to f16
                        for i in outside:
                            i.replace_source_output(back.output(0))
        return bool(_c.make_pass("ConvertPrecision", {"from": self._from, "to": self._to}).run_on_model(model._m))


class CompressWeights(_NamedPass):
    native_name = "CompressWeights"

    def __init__(self, mode: str = "int4_asym", group_size: int = 128, ratio: float = 1.0, all_layers: bool = False):
        super().__init__(mode=mode, group_size=group_size, ratio=ratio, all_layers=all_layers)


class MarkSugraphsToKeepInMixedPrecision(ModelPass):
    """Marks the operations whose fp16 evaluation loses too much (``disable_fp16_compression``), so that a later
    ``ConvertPrecision`` f32 -> f16 leaves them in fp32 and puts Converts at the island's borders:

    * exponent sums: ``Exp`` and everything between it and the ``ReduceSum`` / ``ReduceMean`` that accumulates it, the
      reduction itself and the division / multiplication that normalises by it (soft-max written out, log-sum-exp);
    * variance-style normalisations: ``ReduceMean`` / ``ReduceSum`` of squares up to the ``Sqrt`` / ``Power`` /
      ``Divide`` that applies it (layer norm, RMS norm, L2 normalisation written out), and ``MVN`` / ``NormalizeL2``.

    Role in the reference: transformations/fp16_compression/mark_subgraphs_to_keep_in_mixed_precision.cpp."""

    _THROUGH = {"Add", "Subtract", "Multiply", "Divide", "Convert", "Reshape", "Squeeze", "Unsqueeze", "Transpose", "Broadcast", "Maximum", "Power", "Sqrt",
                "Negative", "Abs", "Clamp"}
    _REDUCE = {"ReduceSum", "ReduceMean"}

    def run_on_model(self, model) -> bool:
        from .. import rt_info as rt
        marked = set()

        def consumers(n):
            return [i.get_node() for o in n.outputs() for i in o.get_target_inputs()]

        def mark_down_to_reduce(start):
            """start .. element-wise .. Reduce .. normalising consumer: mark the whole path when it reaches a reduction."""
            path_marks, stack, seen = [], [(start, [start])], set()
            while stack:
                n, path = stack.pop()
                if id(n) in seen or len(path) > 12:
                    continue
                seen.add(id(n))
                for c in consumers(n):
                    t = c.get_type_name()
                    if t in self._REDUCE:
                        path_marks.extend(path + [c])
                        # the consumers that apply the reduced value (divide by the sum, multiply by 1 / sqrt(mean + eps) ...)
                        frontier = [c]
                        for _ in range(6):
                            nxt = []
                            for f in frontier:
                                for cc in consumers(f):
                                    if cc.get_type_name() in self._THROUGH and cc not in path_marks:
                                        path_marks.append(cc)
                                        nxt.append(cc)
                            frontier = nxt
                    elif t in self._THROUGH:
                        stack.append((c, path + [c]))
            return path_marks

        for n in model.get_ordered_ops():
            t = n.get_type_name()
            if t in ("MVN", "NormalizeL2"):
                marked.add(n)
            elif t == "Exp":
                marked.update(mark_down_to_reduce(n))
            elif t in ("Multiply", "Power") and n.get_output_element_type(0).is_real():
                # squares: x * x or x ^ 2 on the way to a mean / sum
                ins = [n.input_value(i) for i in range(n.get_input_size())]
                is_square = (t == "Multiply" and len(ins) == 2 and ins[0] == ins[1]) or \
                            (t == "Power" and ins[1].get_node().get_type_name() == "Constant" and ins[1].get_node().get_tensor_view().size == 1
                             and float(ins[1].get_node().get_tensor_view().to_float32().reshape(-1)[0]) == 2.0)
                if is_square:
                    marked.update(mark_down_to_reduce(n))
        for n in marked:
            if n.get_type_name() not in ("Parameter", "Result", "Constant"):
                rt.disable_fp16_compression(n)
        return bool(marked)


class SymbolicPropagation(ModelPass):
    """Gives every dynamic dimension of the model's Parameters a fresh symbol (dimensions that already carry one keep
    it) and re-runs shape inference, so that the symbols travel to every value that inherits the dimension; where
    operands must agree (Concat, element-wise with equal dimensions) their symbols become one class
    (src/common/transformations/src/transformations/symbolic_transformations/symbolic_optimizations.cpp, SymbolicPropagation)."""

    def run_on_model(self, model) -> bool:
        from .._types import Symbol
        shapes = {}
        for i, p in enumerate(model.get_parameters()):
            ps = p.get_output_partial_shape(0)
            if ps.rank.is_dynamic:
                continue
            touched = False
            for d in ps:
                if d.is_dynamic and not d.has_symbol():
                    d.set_symbol(Symbol())
                    touched = True
            if touched:
                shapes[i] = ps
        if shapes:
            model.reshape(shapes)            # re-runs shape inference: the symbols travel with the dimensions
        return bool(shapes)


class MakeStateful(ModelPass):
    """Turn (Parameter, Result) pairs into ReadValue/Assign. Pairs are tensor names or nodes."""

    def __init__(self, pairs):
        super().__init__("MakeStateful")
        items = pairs.items() if isinstance(pairs, dict) else pairs
        self._pairs = []
        for p, r in items:
            pn = p if isinstance(p, str) else (sorted(p.output(0).get_names()) or [p.get_friendly_name()])[0]
            rn = r if isinstance(r, str) else (sorted(r.input_value(0).get_names()) or [r.get_friendly_name()])[0]
            self._pairs.append((pn, rn))

    def run_on_model(self, model: Model) -> bool:
        return _c.make_stateful(model._m, self._pairs)


class LowLatency2(ModelPass):
    """Turns the back edges of TensorIterator / Loop nodes into model state: the initial value of every merged input is
    read through ``ReadValue`` and the value after the last iteration is stored with ``Assign``, so a recurrent network
    that is fed one chunk of the sequence per inference carries its hidden state from one call to the next
    (``reset_state`` starts a new sequence). With ``use_const_initializer`` the ReadValue starts from zeros of the
    initial value's shape instead of the original initial-value sub-graph. Reference: src/core/src/pass/low_latency.cpp."""

    def __init__(self, use_const_initializer: bool = True):
        super().__init__("LowLatency2")
        self.use_const_initializer = use_const_initializer

    def run_on_model(self, model: Model) -> bool:
        import numpy as np
        from .. import opset as ops
        changed = False
        sinks = []
        for n in model.get_ordered_ops():
            if n.get_type_name() not in ("TensorIterator", "Loop"):
                continue
            at = n.get_attributes()
            back = list(at.get("back_edges") or [])
            if not back:
                continue
            in_map = list(at.get("input_map") or [])
            out_map = list(at.get("output_map") or [])
            for k in range(0, len(back), 2):
                ridx, pidx = int(back[k]), int(back[k + 1])
                port = next((int(in_map[j]) for j in range(0, len(in_map), 3) if int(in_map[j + 1]) == pidx and int(in_map[j + 2]) < 0), None)
                if port is None:
                    continue
                init = n.input_value(port)
                var_id = "%s/variable_%d" % (n.get_friendly_name(), k // 2)
                if any(s_.get_type_name() == "Assign" and s_.get_attributes().get("variable_id") == var_id for s_ in model.get_sinks()):
                    continue                                     # already converted
                ps = init.get_partial_shape()
                if self.use_const_initializer and ps.is_static:
                    zeros = np.zeros(list(ps.to_shape()), dtype=init.get_element_type().to_dtype())
                    start = ops.constant(zeros).output(0)
                else:
                    start = init
                rv = ops.read_value(start, variable_id=var_id, variable_type=init.get_element_type().name, variable_shape=ps)
                n.input(port).replace_source_output(rv.output(0))
                # node output that carries the value of the last iteration (added when the model does not expose it)
                j = next((q // 2 for q in range(0, len(out_map), 2) if int(out_map[q]) == ridx and int(out_map[q + 1]) < 0), None)
                if j is None:
                    out_map += [ridx, -1]
                    n.set_attribute("output_map", [int(v) for v in out_map])
                    n.validate()
                    j = len(out_map) // 2 - 1
                sinks.append(ops.assign(n.output(j), variable_id=var_id))
                changed = True
        if changed:
            model.add_sinks(sinks)
            model.validate_nodes_and_infer_types()
        return changed


class Serialize(ModelPass):
    def __init__(self, path_to_xml: str, path_to_bin: str = "", version: str = "UNSPECIFIED"):
        super().__init__("Serialize")
        self.xml, self.bin, self.version = path_to_xml, path_to_bin, version

    def run_on_model(self, model: Model) -> bool:
        from ..frontend import serialize
        serialize(model, self.xml, self.bin, self.version)
        return False


class VisualizeTree(ModelPass):
    """Writes the graph in Graphviz dot format."""

    def __init__(self, file_name: str = "model.dot"):
        super().__init__("VisualizeTree")
        self.file_name = file_name

    def run_on_model(self, model: Model) -> bool:
        lines = ["digraph model {", "  node [shape=box, fontsize=10];"]
        ids = {}
        for i, n in enumerate(model.get_ops()):
            ids[n] = "n%d" % i
            shapes = ", ".join(n.get_output_partial_shape(k).to_string() for k in range(n.get_output_size()))
            lines.append('  n%d [label="%s\\n%s\\n%s"];' % (i, n.get_friendly_name().replace('"', "'"), n.get_type_name(), shapes))
        for n in model.get_ops():
            for k in range(n.get_input_size()):
                src = n.input_value(k).get_node()
                lines.append("  %s -> %s;" % (ids[src], ids[n]))
        lines.append("}")
        with open(self.file_name, "w") as f:
            f.write("\n".join(lines))
        return False


# ------------------------------------------------------------------------------------------------ patterns
class _Pattern:
    def __init__(self, native):
        self._p = native

    def output(self, i: int = 0) -> "_Pattern":
        return self


def _pred(pred):
    if pred is None:
        return None
    return lambda pair: bool(pred(Output(pair[0], pair[1])))


def _types(t) -> List[str]:
    items = t if isinstance(t, (list, tuple)) else [t]
    return [str(x).split(".")[-1] if not str(x).startswith("opset") else str(x).split(".")[-1] for x in items]


def _pins(inputs) -> list:
    return [i._p if isinstance(i, _Pattern) else i for i in (inputs or [])]


class AnyInput(_Pattern):
    def __init__(self, predicate: Optional[Callable[[Output], bool]] = None):
        super().__init__(_c.pattern_any(_pred(predicate)))


class WrapType(_Pattern):
    """Matches a node of one of the given types (``"opset13.Relu"`` or ``"Relu"``) whose inputs match ``inputs``."""

    def __init__(self, type_names, inputs=None, predicate=None):
        if callable(inputs) and predicate is None:
            inputs, predicate = None, inputs
        if isinstance(inputs, _Pattern):
            inputs = [inputs]
        super().__init__(_c.pattern_type(_types(type_names), _pins(inputs), _pred(predicate)))


class Optional(_Pattern):   # noqa: A001 - name fixed by the API it mirrors
    """Matches the node when present, otherwise matches its first input pattern directly."""

    def __init__(self, type_names, inputs=None, predicate=None):
        if isinstance(inputs, _Pattern):
            inputs = [inputs]
        super().__init__(_c.pattern_optional(_types(type_names), _pins(inputs), _pred(predicate)))


class Or(_Pattern):
    def __init__(self, alternatives: Sequence[_Pattern]):
        super().__init__(_c.pattern_or(_pins(alternatives)))


def any_input(predicate=None) -> AnyInput:
    return AnyInput(predicate)


def wrap_type(type_names, inputs=None, predicate=None) -> WrapType:
    return WrapType(type_names, inputs, predicate)


# predicates (src/core/include/openvino/pass/pattern/op/pattern.hpp)
def consumers_count(n: int):
    return lambda o: len(o.get_target_inputs()) == n


def has_static_shape():
    return lambda o: o.get_partial_shape().is_static


def has_static_rank():
    return lambda o: o.get_partial_shape().rank.is_static


def has_static_dim(i: int):
    return lambda o: o.get_partial_shape().rank.is_static and len(o.get_partial_shape()) > i and o.get_partial_shape()[i].is_static


def rank_equals(r: int):
    return lambda o: o.get_partial_shape().rank.is_static and len(o.get_partial_shape()) == r


def type_matches(t):
    return lambda o: o.get_element_type() == t


def type_matches_any(ts):
    return lambda o: any(o.get_element_type() == t for t in ts)


class Matcher:
    """Matches a pattern against a graph value; after a successful ``match`` gives the pattern -> value map."""

    def __init__(self, pattern: _Pattern, name: str = ""):
        self._pattern = pattern
        self._m = _c.Matcher(pattern._p, name)

    @classmethod
    def _wrap(cls, native) -> "Matcher":
        m = cls.__new__(cls)
        m._m, m._pattern = native, None
        return m

    def get_name(self) -> str:
        return self._m.name

    def match(self, value) -> bool:
        from .._graph import as_output
        return self._m.match(as_output(value)._core())

    def get_match_root(self) -> Node:
        return Node(self._m.get_match_root())

    def get_match_value(self) -> Output:
        n, i = self._m.get_match_value()
        return Output(n, i)

    def get_match_nodes(self) -> List[Node]:
        return [Node(n) for n in self._m.get_matched_nodes()]

    def get_pattern_value_map(self) -> "_PatternMap":
        return _PatternMap(self._m)


class _PatternMap:
    def __init__(self, native_matcher):
        self._m = native_matcher

    def __contains__(self, p: _Pattern) -> bool:
        return self._m.has(p._p)

    def __getitem__(self, p: _Pattern) -> Output:
        n, i = self._m.at(p._p)
        return Output(n, i)


class MatcherPass(PassBase):
    """``MatcherPass(matcher, callback)`` or sub-class calling ``register_matcher(matcher, callback)``.
    ``callback(matcher) -> bool`` may rewrite the graph around the match root."""

    def __init__(self, matcher: Optional[Matcher] = None, callback: Optional[Callable[[Matcher], bool]] = None):
        super().__init__()
        self._matcher, self._callback = matcher, callback
        self._new_nodes: List[Node] = []

    def register_matcher(self, matcher: Matcher, callback: Callable[[Matcher], bool]) -> None:
        self._matcher, self._callback = matcher, callback
        if matcher.get_name():
            self.set_name(matcher.get_name())

    def register_new_node(self, node: Node) -> Node:
        self._new_nodes.append(node)
        return node

    def _native(self):
        if self._matcher is None:
            raise RuntimeError("MatcherPass has no matcher registered")
        cb = self._callback
        return _c.make_matcher_pass(self.get_name(), self._matcher._pattern._p, lambda native: bool(cb(Matcher._wrap(native))))

    def run_on_model(self, model: Model) -> bool:
        return self._native().run_on_model(model._m)


class GraphRewrite(PassBase):
    """Runs several matcher passes over the graph."""

    def __init__(self, passes: Iterable[MatcherPass] = ()):
        super().__init__()
        self._passes = list(passes)

    def add_matcher(self, p: MatcherPass) -> MatcherPass:
        self._passes.append(p)
        return p

    def _native(self):
        natives = [p._native() for p in self._passes]
        return _c.make_python_pass(self.get_name(), lambda core_model: any([n.run_on_model(core_model) for n in natives]))


BackwardGraphRewrite = GraphRewrite


class Manager:
    """Ordered list of passes; ``run_passes(model)`` applies them and re-validates the graph in between."""

    def __init__(self):
        self._pm = _c.PassManager()
        self._passes: List[PassBase] = []

    def register_pass(self, p, *args, **kwargs) -> PassBase:
        if isinstance(p, type):
            p = p(*args, **kwargs)
        if isinstance(p, str):
            native, wrapper = _c.make_pass(p, kwargs), None
        else:
            native, wrapper = p._native(), p
        self._pm.add(native)
        self._passes.append(wrapper)
        return wrapper

    def set_per_pass_validation(self, new_state: bool) -> None:
        self._pm.validate_after_each = bool(new_state)

    def disable(self, name: str) -> None:
        self._pm.disable(name)

    def enable(self, name: str) -> None:
        self._pm.enable(name)

    def run_passes(self, model: Model) -> bool:
        from ..utils import trace
        with trace.scope("ov::pass", "Manager::run_passes"):
            changed = self._pm.run(model._m)
        if trace.enabled():
            # one event per pass, laid end to end inside the manager's scope
            import threading
            import time
            t = time.perf_counter_ns()
            for name, ms, _ in reversed(list(self._pm.timings())):
                t -= int(ms * 1e6)
                trace._events.append(("ov::pass", str(name), t, int(ms * 1e6), threading.get_ident()))
        return changed

    def get_timings(self):
        """[(pass name, milliseconds, changed)] of the last run."""
        return list(self._pm.timings())


def available_passes() -> List[str]:
    return list(_c.available_passes())


class Version:
    """IR version selector of ``Serialize`` (``Version.UNSPECIFIED`` writes the newest the model needs)."""
    UNSPECIFIED = "UNSPECIFIED"
    IR_V10 = "IR_V10"
    IR_V11 = "IR_V11"
