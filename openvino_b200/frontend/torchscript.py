"""TorchScript front end: a traced or scripted ``torch.jit.ScriptModule`` / ``ScriptFunction`` -> ``Model``.

The graph of the (frozen, inlined) module is walked once. ``aten::`` nodes are looked up in the same translator table
as the ``torch.export`` path (``frontend/pytorch.py``): a node is presented to a translator as positional arguments and
keyword-only arguments split by its operator schema, which is how an exported graph presents the same operator.
``prim::`` plumbing (constants, list / tuple construction and unpacking, ``NumToTensor``, ``aten::size`` / ``aten::Int``
shape arithmetic) is evaluated here; integer shape values stay symbolic (``ShapeOf`` / ``Gather`` sub-graphs), so a traced
model keeps dynamic dimensions when it is given dynamic input shapes.

Role in the reference: the TorchScript decoder src/bindings/python/src/openvino/frontend/pytorch/ts_decoder.py and the
node walk of src/frontends/pytorch/src/translate_session.cpp.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from .. import opset as ops
from .._graph import Model, Node, Output, as_output
from .._tensor import Tensor
from .._types import PartialShape, Type
from ..opset import constant, parameter, result
from . import pytorch as P
from .pytorch import ConversionError


class _Args:
    """What a translator sees of a TorchScript node: ``args`` / ``kwargs`` of graph values and python values."""

    def __init__(self, name: str, args: list, kwargs: dict, target: str = ""):
        self.name, self.args, self.kwargs, self.target = name, tuple(args), kwargs, target
        self.meta: Dict[str, Any] = {}


def _schema_key(node) -> str:
    """``aten::add`` with overload ``Tensor`` -> ``aten.add.Tensor`` (the key of the translator table)."""
    kind = node.kind()
    ns, name = kind.split("::", 1)
    overload = ""
    try:
        sch = node.schema()
        if "(" in sch:
            head = sch.split("(", 1)[0]
            if "." in head.split("::", 1)[-1]:
                overload = head.split("::", 1)[-1].split(".", 1)[1]
    except RuntimeError:
        pass
    return "%s.%s.%s" % (ns, name, overload or "default")


def _kwarg_only_names(node) -> Optional[List[Optional[str]]]:
    """Per input of the node: its name when it is keyword-only in the operator schema, else None."""
    try:
        sch = node.schema()
    except RuntimeError:
        return None
    if "(" not in sch:
        return None
    inner = sch[sch.index("(") + 1:sch.rindex(") ->")] if ") ->" in sch else sch[sch.index("(") + 1:]
    out: List[Optional[str]] = []
    kw = False
    depth = 0
    cur = ""
    parts = []
    for ch in inner:
        if ch in "([":
            depth += 1
        elif ch in ")]":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        parts.append(cur.strip())
    for part in parts:
        if part == "*":
            kw = True
            continue
        name = part.split("=")[0].strip().split(" ")[-1]
        out.append(name if kw else None)
    return out


def _const_value(node):
    """Python value / tensor of a prim::Constant."""
    import torch
    if not node.hasAttribute("value") and not node.hasAttributes():
        return None
    out_t = node.output().type()
    kind = out_t.kind()
    if kind == "NoneType":
        return None
    v = node.output().toIValue()
    if isinstance(v, torch.Tensor):
        return v
    return v


def _tensor_constant(t, share: bool) -> Output:
    return constant(Tensor(t.detach().contiguous(), shared_memory=share), shared_memory=share).output(0)


_DTYPE_BY_INDEX = None


def _scalar_type(idx):
    """TorchScript passes dtypes as the integer codes of c10::ScalarType."""
    import torch
    global _DTYPE_BY_INDEX
    if _DTYPE_BY_INDEX is None:
        _DTYPE_BY_INDEX = {0: torch.uint8, 1: torch.int8, 2: torch.int16, 3: torch.int32, 4: torch.int64, 5: torch.float16, 6: torch.float32,
                           7: torch.float64, 11: torch.bool, 15: torch.bfloat16}
    return _DTYPE_BY_INDEX.get(idx, idx)


_DTYPE_ARGS = {"dtype"}
# operators that only traced graphs contain -> the exported-graph operator with the same leading arguments
_ALIASES = {"aten._convolution.default": "aten.convolution.default", "aten._convolution.deprecated": "aten.convolution.default"}
_ALIAS_ARGC = {"aten._convolution.default": 9, "aten._convolution.deprecated": 9}     # arguments the target operator takes


def from_script(module, example_input=None, input=None, share_weights: bool = True) -> Model:
    """``torch.jit.ScriptModule`` / ``ScriptFunction`` (or an ``nn.Module`` plus ``example_input``, traced here) -> ``Model``."""
    import torch
    if isinstance(module, torch.nn.Module) and not isinstance(module, torch.jit.ScriptModule):
        if example_input is None:
            raise ConversionError("tracing a torch module needs example_input")
        ex = tuple(example_input) if isinstance(example_input, (list, tuple)) else (example_input,)
        module = module.eval()
        with torch.no_grad():
            module = torch.jit.trace(module, ex, strict=False, check_trace=False)
    if isinstance(module, torch.jit.ScriptModule):
        module = module.eval()
        try:
            module = torch.jit.freeze(module)
        except RuntimeError:
            pass
        graph = module.graph
        self_value = next(iter(graph.inputs())) if module is not None else None
        skip_self = True
    else:
        graph = module.graph
        self_value, skip_self = None, False
    torch._C._jit_pass_inline(graph)

    values: Dict[Any, Any] = {}      # torch._C.Value (by unique id) -> Output | python value | list | module object
    ctx = P.Ctx()
    params: List[Node] = []
    shapes = P._input_shapes(input) if input is not None else None
    ex_list = list(example_input) if isinstance(example_input, (list, tuple)) else ([example_input] if example_input is not None else [])
    gi = list(graph.inputs())
    if skip_self:
        values[gi[0].unique()] = module
        gi = gi[1:]
    for i, v in enumerate(gi):
        name = v.debugName()
        t = v.type()
        dtype, dims = torch.float32, None
        if i < len(ex_list) and isinstance(ex_list[i], torch.Tensor):
            dtype, dims = ex_list[i].dtype, list(ex_list[i].shape)
        if hasattr(t, "scalarType") and t.kind() == "TensorType":
            if t.dtype() is not None:
                dtype = t.dtype()
            if dims is None and t.sizes() is not None:
                dims = list(t.sizes())
        if shapes is not None and i < len(shapes):
            dims = list(shapes[i])
        if dims is None:
            raise ConversionError("input %s has no known shape: pass example_input or input=[shapes]" % name)
        p = parameter(PartialShape(dims), P._ov_type(dtype), name)
        p.output(0).set_names({name})
        params.append(p)
        values[v.unique()] = p.output(0)

    def val(v):
        return values[v.unique()]

    def to_output(x, like: Optional[Output] = None) -> Output:
        if isinstance(x, torch.Tensor):
            return _tensor_constant(x, share_weights)
        return ctx.out(x, like)

    def run_nodes(nodes):
        for node in nodes:
            run_node(node)

    def run_node(node):
        kind = node.kind()
        outs = list(node.outputs())
        if kind == "prim::If":
            # a condition known at conversion time (shape arithmetic on static dimensions) selects the branch to inline
            cond = val(node.input())
            if not isinstance(cond, (bool, int)):
                raise ConversionError("prim::If on a value that is not known at conversion time")
            blk = list(node.blocks())[0 if cond else 1]
            run_nodes(blk.nodes())
            for o, b in zip(outs, blk.outputs()):
                values[o.unique()] = val(b)
        elif kind == "prim::Constant":
            v = _const_value(node)
            values[outs[0].unique()] = _tensor_constant(v, share_weights) if isinstance(v, torch.Tensor) else v
        elif kind == "prim::GetAttr":
            obj = val(node.input())
            attr = getattr(obj, node.s("name"))
            values[outs[0].unique()] = _tensor_constant(attr, share_weights) if isinstance(attr, torch.Tensor) else attr
        elif kind in ("prim::ListConstruct", "prim::TupleConstruct"):
            values[outs[0].unique()] = [val(i) for i in node.inputs()]
        elif kind in ("prim::ListUnpack", "prim::TupleUnpack"):
            seq = val(node.input())
            if not isinstance(seq, (list, tuple)) or len(seq) != len(outs):
                raise ConversionError("%s of a value that is not a %d-element sequence" % (kind, len(outs)))
            for o, x in zip(outs, seq):
                values[o.unique()] = x
        elif kind in ("prim::NumToTensor", "aten::Int", "aten::ScalarImplicit", "aten::IntImplicit", "aten::FloatImplicit", "aten::Float",
                      "prim::dtype_passthrough", "aten::alias", "aten::detach", "aten::contiguous", "prim::device"):
            src = val(next(iter(node.inputs()))) if kind != "prim::device" else "cpu"
            if kind == "aten::Float" and isinstance(src, Output) and src.get_element_type() != Type.f32:
                src = ops.convert(src, Type.f32).output(0)
            values[outs[0].unique()] = src
        elif kind == "aten::size":
            ins = [val(i) for i in node.inputs()]
            x = to_output(ins[0])
            shape = ops.shape_of(x, Type.i64).output(0)
            if len(ins) == 1:
                ps = x.get_partial_shape()
                values[outs[0].unique()] = [int(d.get_length()) if d.is_static else ops.gather(shape, np.array(i, dtype=np.int64), np.array(0, dtype=np.int64)).output(0)
                                            for i, d in enumerate(ps)] if ps.rank.is_static else shape
            else:
                dim = ins[1]
                ps = x.get_partial_shape()
                if ps.rank.is_static and isinstance(dim, int) and ps[dim % ps.rank.get_length()].is_static:
                    values[outs[0].unique()] = int(ps[dim % ps.rank.get_length()].get_length())
                else:
                    values[outs[0].unique()] = ops.gather(shape, to_output(dim), np.array(0, dtype=np.int64)).output(0)
        elif kind == "aten::len":
            seq = val(node.input())
            values[outs[0].unique()] = len(seq)
        elif kind == "aten::__getitem__":
            seq, idx = [val(i) for i in node.inputs()]
            if isinstance(seq, (list, tuple)) and isinstance(idx, int):
                values[outs[0].unique()] = seq[idx]
            else:
                values[outs[0].unique()] = ops.gather(to_output(seq), to_output(idx), np.array(0, dtype=np.int64)).output(0)
        elif kind.startswith("aten::") or kind.startswith("prim::") and kind in ("prim::min", "prim::max"):
            key = _schema_key(node)
            ins = [val(i) for i in node.inputs()]
            inplace = key.split(".")[1].endswith("_") and not key.split(".")[1].startswith("__")
            fn = P._TABLE.get(_ALIASES.get(key, key))
            if fn is None and inplace:
                fn = P._TABLE.get(key.replace("_.", ".", 1))
            if fn is None:
                base = ".".join(key.split(".")[:2])
                cands = [k for k in P._TABLE if k.startswith(base + ".")]
                if len(cands) == 1:
                    fn = P._TABLE[cands[0]]
            # python-level integer arithmetic on shape values
            if fn is None or all(isinstance(x, (int, float, bool)) for x in ins):
                name = key.split(".")[1]
                pyops = {"add": "add", "sub": "sub", "mul": "mul", "div": "truediv", "floordiv": "floordiv", "remainder": "mod", "eq": "eq", "ne": "ne",
                         "lt": "lt", "le": "le", "gt": "gt", "ge": "ge"}
                if name in pyops and len(ins) >= 2 and all(isinstance(x, (int, float, bool)) for x in ins[:2]):
                    values[outs[0].unique()] = P._python_scalar_op(pyops[name], ins[:2])
                    return
                if name in pyops and fn is None:
                    fn = P._TABLE.get({"add": "add", "sub": "sub", "mul": "mul", "div": "truediv", "floordiv": "floordiv"}.get(name, ""))
            if fn is None:
                raise ConversionError("no translator for %s (%s)" % (kind, key))
            kw_names = _kwarg_only_names(node) or [None] * len(ins)
            args, kwargs = [], {}
            for x, kwn in zip(ins, kw_names + [None] * (len(ins) - len(kw_names))):
                if kwn is not None:
                    kwargs[kwn] = _scalar_type(x) if kwn in _DTYPE_ARGS and isinstance(x, int) else x
                else:
                    args.append(x)
            # positional dtype arguments (aten::to.dtype, aten::softmax.int ...) carry ScalarType codes
            try:
                sch = node.schema()
                pos_names = [p_.split("=")[0].strip().split(" ")[-1] for p_ in sch[sch.index("(") + 1:].split("*")[0].split(",") if p_.strip()]
                for i_, nm in enumerate(pos_names):
                    if nm in _DTYPE_ARGS and i_ < len(args) and isinstance(args[i_], int):
                        args[i_] = _scalar_type(args[i_])
            except (RuntimeError, ValueError):
                pass
            if key in _ALIAS_ARGC:
                args = args[:_ALIAS_ARGC[key]]
            out = fn(ctx, _Args(outs[0].debugName() if outs else kind, args, kwargs, key))
            if isinstance(out, Node):
                out = out.output(0) if out.get_output_size() == 1 or len(outs) == 1 else [out.output(i) for i in range(out.get_output_size())]
            if len(outs) == 1:
                values[outs[0].unique()] = out
            else:
                seq = list(out) if isinstance(out, (list, tuple)) else [out]
                for o, x in zip(outs, seq):
                    values[o.unique()] = x
            if inplace and ins:
                first = next(iter(node.inputs()))
                values[first.unique()] = values[outs[0].unique()]
        else:
            raise ConversionError("TorchScript node %s is not supported" % kind)

    run_nodes(graph.nodes())

    flat: List[Output] = []

    def walk(x):
        if isinstance(x, (list, tuple)):
            for y in x:
                walk(y)
        elif isinstance(x, dict):
            for y in x.values():
                walk(y)
        elif x is not None:
            flat.append(to_output(x))
    for v in graph.outputs():
        walk(val(v))
    results = []
    for i, o in enumerate(flat):
        if not o.get_names():
            o.set_names({"output_%d" % i})
        results.append(result(o))
    return Model(results, params, "Model")
