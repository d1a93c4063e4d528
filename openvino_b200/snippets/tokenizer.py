"""Snippet tokenisation: connected groups of element-wise operations (optionally with Softmax / reductions over the
innermost axis) are cut out of a model and replaced by one ``Subgraph`` operation that owns them as a body model.

A node joins the group of one of its producers when that cannot close a cycle through nodes outside the group; groups
do not merge with each other, so a node's set of upstream groups is final once it has been visited, and the cycle test
is a set lookup. Every member must produce the group's full shape, or that shape with an innermost extent of 1 (per-row
values such as reduction results); what broadcasts in from outside (bias rows, per-row scales, scalars) stays an input.
Scalar constants are copied into the body, everything else that a member reads from outside becomes a body parameter.

The ``Subgraph`` operation evaluates on the host through the NumPy executor of its linear IR and on the CUDA device
through a generated kernel (runtime.py). Role of the reference's tokeniser and Subgraph operation
(src/common/snippets/src/pass/{collapse_subgraph,tokenization}.cpp, src/common/snippets/src/op/subgraph.cpp).
"""
from __future__ import annotations

import itertools
from typing import Dict, List, Optional, Sequence, Set, Tuple

import numpy as np

from .._graph import Model, Node, Output, make_op, parameter, result
from .._op_base import register_op
from .._types import PartialShape
from .op_table import OPS, REDUCE_OPS

_FLOATS = ("f32", "f16", "bf16")
_BODIES: Dict[int, "SnippetBody"] = {}
_next_id = itertools.count(1)
_registered = False


class SnippetBody:
    """What a Subgraph node owns: the body model and the compiled forms per broadcast signature."""

    def __init__(self, body: Model, names: List[str]):
        self.body = body
        self.fused_names = names
        self.lowered: Dict[tuple, object] = {}        # in_kinds -> LinearIR
        self.kernels: Dict[tuple, object] = {}        # in_kinds -> CudaKernel

    def linear_ir(self, kinds: Tuple[str, ...]):
        from .lowered import lower
        lir = self.lowered.get(kinds)
        if lir is None:
            lir = self.lowered[kinds] = lower(self.body, kinds)
        return lir


def body_of(node: Node) -> SnippetBody:
    return _BODIES[int(node.get_attributes()["body_id"])]


# --------------------------------------------------------------------------------------------- run-time canonical form
def classify(shapes: Sequence[Sequence[int]], out_shape: Sequence[int]) -> Optional[Tuple[Tuple[str, ...], int, int]]:
    """Inputs of a snippet against its full output shape -> (kind per input, rows, cols), or None when an input
    broadcasts in a way the 2-D form cannot express."""
    D = list(out_shape)
    if not D:
        D = [1]
    cols = int(D[-1])
    rows = int(np.prod(D[:-1], dtype=np.int64)) if len(D) > 1 else 1
    kinds = []
    for s in shapes:
        s = [1] * (len(D) - len(s)) + [int(v) for v in s]
        if len(s) != len(D):
            return None
        if s == D:
            kinds.append("full" if not all(v == 1 for v in s) or rows * cols == 1 else "scalar")
        elif all(v == 1 for v in s):
            kinds.append("scalar")
        elif all(v == 1 for v in s[:-1]) and s[-1] == cols:
            kinds.append("row")
        elif s[:-1] == D[:-1] and s[-1] == 1:
            kinds.append("col")
        else:
            return None
    return tuple(kinds), rows, cols


def full_shape(shapes: Sequence[Sequence[int]]) -> List[int]:
    """NumPy broadcast of the input shapes: the iteration domain of a snippet."""
    return list(np.broadcast_shapes(*[tuple(int(v) for v in s) for s in shapes])) if shapes else []


def _host_eval(node: Node, ins: List[np.ndarray]) -> List[np.ndarray]:
    from .emit_numpy import run_numpy
    sb = body_of(node)
    body = sb.body
    shapes = [list(a.shape) for a in ins]
    outs_ps = _infer_outputs(sb, shapes)
    D = full_shape(shapes + [s for _, s in outs_ps])
    got = classify(shapes, D)
    if got is None:
        raise RuntimeError("Subgraph %s: inputs %s do not fit the 2-D broadcast forms" % (node.get_friendly_name(), shapes))
    kinds, rows, cols = got
    lir = sb.linear_ir(kinds)
    form = {"full": (rows, cols), "row": (1, cols), "col": (rows, 1), "scalar": (1, 1)}
    arrs = []
    for a, k, t in zip(ins, kinds, lir.in_types):
        a = np.asarray(a)
        if t == "bf16" and a.dtype == np.uint16:
            a = (a.astype(np.uint32) << 16).view(np.float32)
        arrs.append(a.astype(np.float32).reshape(form[k]))
    res = run_numpy(lir, arrs, rows, cols)
    outs = []
    for r, (t, shape) in zip(res, outs_ps):
        r = r.reshape(shape)
        if t == "bf16":
            r = (np.ascontiguousarray(r, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
            from .._tensor import Tensor
            outs.append(Tensor(r, list(shape), "bf16"))
            continue
        outs.append(r.astype({"f32": np.float32, "f16": np.float16, "boolean": np.bool_}[t]))
    return outs


def _infer_outputs(sb: SnippetBody, in_shapes: Sequence[Sequence[int]]) -> List[Tuple[str, List[int]]]:
    body = sb.body
    params = body.get_parameters()
    body.reshape({i: PartialShape([int(v) for v in s]) for i, s in enumerate(in_shapes)})
    return [(str(r.get_input_element_type(0)), [int(v) for v in r.get_input_shape(0)]) for r in body.get_results()]


def ensure_registered() -> None:
    global _registered
    if _registered:
        return

    def infer(node: Node):
        sb = body_of(node)
        body = sb.body
        params = body.get_parameters()
        body.reshape({i: node.get_input_partial_shape(i) for i in range(len(params))})
        return [(r.get_input_element_type(0), r.get_input_partial_shape(0)) for r in body.get_results()]

    register_op("Subgraph", infer, _host_eval, version="SnippetsOpset", attrs={"body_id": 0})
    _registered = True


# --------------------------------------------------------------------------------------------- tokenisation
def _reduces_last_axis(n: Node) -> bool:
    rank = n.get_input_partial_shape(0).rank
    if not rank.is_static or rank.get_length() < 1:
        return False
    r = rank.get_length()
    t = n.get_type_name()
    if t == "Softmax":
        ax = int(n.get_attributes().get("axis", -1))
        return ax in (-1, r - 1)
    axes_node = n.input_value(1).get_node()
    if axes_node.get_type_name() != "Constant" or not bool(n.get_attributes().get("keep_dims", False)):
        return False
    axes = [int(v) for v in np.asarray(axes_node.get_data()).reshape(-1)]
    return len(axes) == 1 and axes[0] in (-1, r - 1)


def _is_scalar_const(n: Node) -> bool:
    return n.get_type_name() == "Constant" and int(np.prod(list(n.get_output_shape(0)) or [1])) == 1 and str(n.get_output_element_type(0)) in _FLOATS + ("i32", "i64", "boolean")


def _eligible(n: Node) -> bool:
    t = n.get_type_name()
    if t in OPS:
        pass
    elif t in REDUCE_OPS or t == "Softmax":
        if not _reduces_last_axis(n):
            return False
    else:
        return False
    for o in n.outputs():
        et = str(o.get_element_type())
        if et not in _FLOATS and not (et == "boolean" and OPS.get(t) is not None and OPS[t].boolean):
            return False
        if not o.get_partial_shape().rank.is_static:
            return False
    n_data = 1 if (t in REDUCE_OPS) else n.get_input_size()
    for k in range(n_data):
        et = str(n.get_input_element_type(k))
        if et not in _FLOATS + ("boolean",) and not _is_scalar_const(n.input_value(k).get_node()):
            return False
    if t == "Convert" and str(n.get_input_element_type(0)) not in _FLOATS + ("boolean",):
        return False
    return True


def _same_dims(a: PartialShape, b: PartialShape, upto: Optional[int] = None) -> bool:
    da, db = list(a), list(b)
    if len(da) != len(db):
        return False
    for x, y in list(zip(da, db))[:upto]:
        if x.is_static != y.is_static:
            return False
        if x.is_static and x.get_length() != y.get_length():
            return False
        if not x.is_static and (x.get_symbol() if hasattr(x, "get_symbol") else None) != (y.get_symbol() if hasattr(y, "get_symbol") else None):
            pass        # two dynamic extents: equality is checked again when the snippet runs
    return True


def _fits(domain: PartialShape, shape: PartialShape) -> bool:
    """``shape`` is the group's full shape, or that with an innermost extent of 1."""
    if _same_dims(domain, shape):
        return True
    d = list(shape)
    return len(d) == len(list(domain)) and len(d) >= 1 and d[-1].is_static and d[-1].get_length() == 1 and _same_dims(domain, shape, len(d) - 1)


class _Group:
    def __init__(self, gid: int, domain: PartialShape):
        self.id, self.domain, self.nodes = gid, domain, []


def tokenize(model: Model, min_ops: int = 2, skip=None) -> int:
    """Collapse groups of at least ``min_ops`` operations into Subgraph nodes; returns how many were made.
    ``skip(node) -> bool`` keeps a node out (the device plugin passes the operations it already fuses elsewhere)."""
    ensure_registered()
    group_of: Dict[Node, _Group] = {}
    upstream: Dict[Node, Set[int]] = {}           # groups a node depends on (its own included)
    groups: List[_Group] = []
    readers: Dict[Tuple[Node, int], List[_Group]] = {}      # value -> groups that read it from outside
    for n in model.get_ordered_ops() if hasattr(model, "get_ordered_ops") else model.get_ops():
        deps: Set[int] = set()
        producers = [n.input_value(k).get_node() for k in range(n.get_input_size())]
        for p in producers:
            deps |= upstream.get(p, set())
        ok = _eligible(n) and not (skip is not None and skip(n))
        if ok:
            out_ps = n.get_output_partial_shape(0)
            placed = None
            for p in producers:
                g = group_of.get(p)
                if g is None or placed is not None:
                    continue
                # the other inputs must not depend on this group through nodes outside it
                others = [q for q in producers if group_of.get(q) is not g]
                if any(g.id in upstream.get(q, set()) for q in others):
                    continue
                # the value handed over must be one the body can hold: a reduce may widen nothing, a member fits the domain
                if not _fits(g.domain, out_ps):
                    # a wider result (a per-row group meeting a full tensor) would change the group's domain: keep it simple
                    continue
                placed = g
            if placed is None:
                # no producer to join: a group that reads one of the same values (a sibling) will do, under the same two rules
                for k in range(n.get_input_size()):
                    o = n.input_value(k)
                    for g in readers.get((o.get_node(), o.get_index()), []):
                        if placed is None and _fits(g.domain, out_ps) and not any(g.id in upstream.get(q, set()) for q in producers):
                            placed = g
            if placed is None:
                if n.get_type_name() in REDUCE_OPS:
                    dom = n.get_input_partial_shape(0)
                else:
                    dom = out_ps
                placed = _Group(len(groups) + 1, dom)
                groups.append(placed)
            for k in range(n.get_input_size()):
                o = n.input_value(k)
                if group_of.get(o.get_node()) is not placed and not _is_scalar_const(o.get_node()):
                    lst = readers.setdefault((o.get_node(), o.get_index()), [])
                    if placed not in lst:
                        lst.append(placed)
            placed.nodes.append(n)
            group_of[n] = placed
            deps.add(placed.id)
        upstream[n] = deps
    made = 0
    for g in groups:
        real = [n for n in g.nodes if n.get_type_name() != "Convert"]
        if len(g.nodes) < min_ops or not real:
            continue
        if _collapse(model, g):
            made += 1
    if made:
        model.validate_nodes_and_infer_types()
    return made


def _collapse(model: Model, g: _Group) -> bool:
    members = set(g.nodes)
    ext_inputs: List[Output] = []
    body_params: List[Node] = []
    mapping: Dict[Tuple[Node, int], Output] = {}

    def body_value(o: Output) -> Output:
        src = o.get_node()
        key = (src, o.get_index())
        if key in mapping:
            return mapping[key]
        if _is_scalar_const(src):
            mapping[key] = src.clone_with_new_inputs([]).output(0)        # same element type and value, owned by the body
            return mapping[key]
        p = parameter(o.get_partial_shape(), o.get_element_type(), "in%d" % len(body_params))
        body_params.append(p)
        ext_inputs.append(o)
        mapping[key] = p.output(0)
        return mapping[key]

    if len(members) == 0:
        return False
    for n in g.nodes:                       # already in topological order
        t = n.get_type_name()
        ins = []
        for k in range(n.get_input_size()):
            o = n.input_value(k)
            if t in REDUCE_OPS and k == 1:
                from .._graph import constant
                ins.append(constant(np.asarray(o.get_node().get_data())).output(0))
                continue
            ins.append(mapping[(o.get_node(), o.get_index())] if o.get_node() in members else body_value(o))
        clone = make_op(t, ins, dict(n.get_attributes()), version=n.get_version())
        clone.set_friendly_name(n.get_friendly_name())
        for i in range(n.get_output_size()):
            mapping[(n, i)] = clone.output(i)
    if len(body_params) > 12:
        return False
    # outputs: member values read outside the group (or by a Result)
    outs: List[Tuple[Node, int]] = []
    for n in g.nodes:
        for i, o in enumerate(n.outputs()):
            if any(inp.get_node() not in members for inp in o.get_target_inputs()):
                outs.append((n, i))
    if not outs or len(outs) > 12:
        return False
    body = Model([result(mapping[k]) for k in outs], body_params, "snippet_body")
    bid = next(_next_id)
    _BODIES[bid] = SnippetBody(body, [n.get_friendly_name() for n in g.nodes])
    sub = make_op("Subgraph", ext_inputs, {"body_id": bid}, version="SnippetsOpset")
    sub.set_friendly_name(g.nodes[-1].get_friendly_name())
    sub.get_rt_info()["fused_names_0"] = ",".join(n.get_friendly_name() for n in g.nodes)
    for k, (n, i) in enumerate(outs):
        old = n.output(i)
        names = old.get_names()
        for inp in list(old.get_target_inputs()):
            if inp.get_node() not in members:
                inp.replace_source_output(sub.output(k))
        if names:
            sub.output(k).set_names(set(names))
    return True
