"""Linear IR of a snippet and its loop structure.

A snippet body (a small ``Model`` of element-wise operations, optionally with Softmax / reductions over the innermost
axis) is lowered to a flat list of expressions over a 2-D iteration domain [rows, cols] (all outer axes collapsed into
rows). Every expression has a *domain*: ``full`` (one value per element) or ``col`` (one value per row: per-row inputs,
scalars, reduction results and what is computed from those alone).

The loop manager then splits the work of one row into *stages*. A reduction needs a whole pass over the row before its
result can be used, so an expression's stage is the number of reductions on the longest path behind it. Stage ``k``
becomes one loop over the columns that (re)computes the full-domain expressions needed by the reductions and the
stores of that stage; independent reductions of one stage share the loop (loop fusion). Values of earlier loops are
recomputed instead of being kept (the row is still in L1 / L2), which is what keeps the register footprint flat.
Inside a loop, virtual registers are assigned by liveness so that structurally equal snippets give equal text.

Role of the reference's lowered IR (src/common/snippets/include/snippets/lowered/{linear_ir,expression,loop_manager}.hpp,
pass/{mark_loops,fuse_loops,assign_registers,softmax_decomposition}.cpp).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .op_table import OPS, REDUCE_OPS

FULL, COL = "full", "col"


@dataclass
class Expr:
    id: int
    kind: str                      # param | scalar | op | reduce | inv_cols
    op: str = ""                   # operation type (kind op) or reduction name (kind reduce)
    args: Tuple[int, ...] = ()
    attrs: dict = field(default_factory=dict)
    value: float = 0.0             # kind scalar
    index: int = -1                # kind param: input position
    domain: str = FULL
    stage: int = 0                 # loop in which the value is computed (reduce: accumulated)
    avail: int = 0                 # first loop that may read the value


@dataclass
class Store:
    output: int                    # output position
    value: int                     # expression id
    domain: str = FULL
    stage: int = 0


@dataclass
class Loop:
    """One pass over the columns of a row."""
    index: int
    prologue: List[int]            # col-domain expressions evaluated once per row before the pass
    body: List[int]                # full-domain expressions evaluated per element, in order
    reduces: List[int]             # reductions accumulated in this pass
    stores: List[Store]
    regs: Dict[int, int] = field(default_factory=dict)      # expression id -> virtual register inside the body
    readback: List[int] = field(default_factory=list)       # kept values of earlier passes that this pass reads back


@dataclass
class LinearIR:
    exprs: List[Expr]
    stores: List[Store]
    loops: List[Loop]
    epilogue: List[int]            # col-domain expressions needed only by col-domain stores after the last loop
    in_types: List[str]
    out_types: List[str]
    in_kinds: Tuple[str, ...]      # per input: full | row | col | scalar
    loops_kept: List[Loop] = field(default_factory=list)   # the same passes when `kept` values stay in registers between them
    kept: List[int] = field(default_factory=list)

    @property
    def has_reduce(self) -> bool:
        return any(e.kind == "reduce" for e in self.exprs)

    def dump(self) -> str:
        lines = []
        for e in self.exprs:
            lines.append("%%%d = %s %s(%s) %s stage=%d" % (e.id, e.kind, e.op or (e.value if e.kind == "scalar" else e.index),
                                                        ", ".join("%%%d" % a for a in e.args), e.domain, e.stage))
        for lp in self.loops:
            lines.append("loop %d: prologue %s body %s reduces %s stores %s" % (lp.index, lp.prologue, lp.body, lp.reduces, [(s.output, s.value) for s in lp.stores]))
        return "\n".join(lines)


class _Builder:
    def __init__(self):
        self.exprs: List[Expr] = []

    def add(self, kind, **kw) -> int:
        e = Expr(len(self.exprs), kind, **kw)
        if kind == "op":
            e.domain = COL if all(self.exprs[a].domain == COL for a in e.args) else FULL
        elif kind == "reduce":
            e.domain = COL
        self.exprs.append(e)
        return e.id

    def divide(self, x: int, d: int, attrs=None) -> int:
        """x / d; with a per-row d (the sum of a Softmax) it becomes x * (1 / d): one division per row, not per element."""
        if self.exprs[x].domain == FULL and self.exprs[d].domain == COL:
            return self.add("op", op="Multiply", args=(x, self.add("op", op="Reciprocal", args=(d,))))
        return self.add("op", op="Divide", args=(x, d), attrs=attrs or {})


def _const_scalar(node) -> Optional[float]:
    if node.get_type_name() != "Constant":
        return None
    data = np.asarray(node.get_data())
    if data.size != 1:
        return None
    if str(node.get_output_element_type(0)) == "bf16" and data.dtype == np.uint16:       # raw bf16 bits
        return float((data.astype(np.uint32) << 16).view(np.float32).reshape(-1)[0])
    return float(np.asarray(data, dtype=np.float64).reshape(-1)[0])


def lower(body, in_kinds: Sequence[str]) -> LinearIR:
    """Body model + how every input broadcasts at run time -> linear IR with loops.

    ``in_kinds[i]`` is ``full`` ([rows, cols]), ``row`` ([1, cols]: same for every row), ``col`` ([rows, 1]) or
    ``scalar``. Softmax is decomposed into max / exp / sum / divide; ReduceMean into a sum times 1 / cols."""
    b = _Builder()
    value_of: Dict[tuple, int] = {}           # (node, port) -> expression id
    params = body.get_parameters()
    for i, p in enumerate(params):
        dom = FULL if in_kinds[i] in ("full", "row") else COL
        value_of[(p, 0)] = b.add("param", index=i, domain=dom)
    for n in body.get_ordered_ops() if hasattr(body, "get_ordered_ops") else body.get_ops():
        t = n.get_type_name()
        if t in ("Parameter", "Result"):
            continue
        if t == "Constant":
            v = _const_scalar(n)
            if v is None:
                raise ValueError("snippet bodies hold scalar constants only; %s is not one" % n.get_friendly_name())
            value_of[(n, 0)] = b.add("scalar", value=v, domain=COL)
            continue
        args = [value_of[(n.input_value(k).get_node(), n.input_value(k).get_index())] for k in range(n.get_input_size())]
        attrs = dict(n.get_attributes())
        if t == "Softmax":
            m = b.add("reduce", op="max", args=(args[0],))
            d = b.add("op", op="Subtract", args=(args[0], m))
            e = b.add("op", op="Exp", args=(d,))
            s = b.add("reduce", op="sum", args=(e,))
            value_of[(n, 0)] = b.divide(e, s)
        elif t in REDUCE_OPS:
            r = b.add("reduce", op=REDUCE_OPS[t], args=(args[0],))     # args[1] is the axes constant, checked by the tokenizer
            if t == "ReduceMean":
                inv = b.add("inv_cols", domain=COL)
                r = b.add("op", op="Multiply", args=(r, inv))
            value_of[(n, 0)] = r
        else:
            if t not in OPS:
                raise ValueError("operation %s cannot be part of a snippet" % t)
            if t == "Convert":
                attrs = {"destination_type": str(n.get_output_element_type(0))}
            value_of[(n, 0)] = b.divide(args[0], args[1], attrs) if t == "Divide" else b.add("op", op=t, args=tuple(args[:OPS[t].arity]), attrs=attrs)
    exprs = b.exprs
    # domains and stages
    for e in exprs:
        if e.kind == "op":
            e.domain = COL if all(exprs[a].domain == COL for a in e.args) else FULL
            e.stage = max(exprs[a].avail for a in e.args)
            e.avail = e.stage
        elif e.kind == "reduce":
            e.domain = COL
            e.stage = exprs[e.args[0]].avail
            e.avail = e.stage + 1
    stores = []
    for k, r in enumerate(body.get_results()):
        src = r.input_value(0)
        vid = value_of[(src.get_node(), src.get_index())]
        stores.append(Store(k, vid, exprs[vid].domain, exprs[vid].avail))
    loops, epilogue = _plan_loops(exprs, stores, set())
    # values worth keeping in registers from the pass that computes them to the later passes that read them again
    kept = _values_to_keep(exprs, stores)
    loops_kept = _plan_loops(exprs, stores, kept)[0] if kept else []
    return LinearIR(exprs, stores, loops, epilogue, [str(p.get_output_element_type(0)) for p in params],
                    [str(r.get_input_element_type(0)) for r in body.get_results()], tuple(in_kinds), loops_kept, sorted(kept))


def _values_to_keep(exprs: List[Expr], stores: List[Store], limit: int = 6) -> set:
    """Full-domain results that a later pass reads: recomputing them costs their whole cone of operations again, keeping
    them costs VEC registers per value and iteration. Inputs are not kept (a load is as cheap as a register move)."""
    kept = set()
    for e in exprs:
        if e.kind != "op" or e.domain != FULL:
            continue
        later = any(x.kind in ("op", "reduce") and e.id in x.args and x.stage > e.stage for x in exprs) or any(s.value == e.id and s.stage > e.stage for s in stores)
        if later:
            kept.add(e.id)
    if len(kept) > limit:
        return set()
    return kept


def _plan_loops(exprs: List[Expr], stores: List[Store], kept: set):
    """Passes over a row. With ``kept`` values a later pass reads them back instead of walking into their arguments."""
    n_loops = 1 + max([e.stage for e in exprs if e.kind == "reduce"] + [s.stage for s in stores if s.domain == FULL] + [0])
    loops: List[Loop] = []
    done_col: set = set()
    for k in range(n_loops):
        reduces = [e.id for e in exprs if e.kind == "reduce" and e.stage == k]
        lstores = [s for s in stores if s.domain == FULL and s.stage == k]
        need: set = set()
        stack = [exprs[r].args[0] for r in reduces] + [s.value for s in lstores]
        # a kept value is written in the pass of its own stage even if nothing else of that pass reads it
        stack += [i for i in kept if exprs[i].stage == k]
        col_need: set = set()
        while stack:
            i = stack.pop()
            e = exprs[i]
            if e.domain == COL:
                col_need.add(i)
                continue
            if i in need:
                continue
            need.add(i)
            if i in kept and e.stage < k:
                continue                      # read back, not recomputed
            stack.extend(e.args)
        # col-domain values read by this loop (and whatever col-domain values they are computed from), once per row
        stack = sorted(col_need)
        seen: set = set()
        while stack:
            i = stack.pop()
            if i in seen or i in done_col:
                continue
            seen.add(i)
            if exprs[i].kind == "op":
                stack.extend(exprs[i].args)
        prologue = sorted(i for i in seen if exprs[i].kind in ("op", "scalar", "inv_cols", "param"))
        done_col |= set(prologue)
        lp = Loop(k, prologue, sorted(need), reduces, lstores)
        lp.readback = sorted(i for i in need if i in kept and exprs[i].stage < k)
        _assign_registers(lp, exprs)
        loops.append(lp)
    # col-domain stores (a reduction result that leaves the snippet) and their inputs
    stack = [s.value for s in stores if s.domain == COL]
    seen = set()
    while stack:
        i = stack.pop()
        if i in seen or i in done_col:
            continue
        seen.add(i)
        if exprs[i].kind == "op":
            stack.extend(exprs[i].args)
    epilogue = sorted(i for i in seen if exprs[i].kind != "reduce")
    return loops, epilogue


def _assign_registers(lp: Loop, exprs: List[Expr]) -> None:
    """Linear-scan numbering of the per-element values of a loop body: a register is reused after the last reader."""
    last_use: Dict[int, int] = {}
    for pos, i in enumerate(lp.body):
        for a in exprs[i].args:
            if a in lp.body:
                last_use[a] = pos
    for r in lp.reduces:
        last_use[exprs[r].args[0]] = len(lp.body)
    for s in lp.stores:
        last_use[s.value] = len(lp.body)
    free: List[int] = []
    next_reg = 0
    for pos, i in enumerate(lp.body):
        # registers of arguments that die here can be reused by the result
        for a in exprs[i].args:
            if a in lp.regs and last_use.get(a, -1) == pos and lp.regs[a] not in free:
                free.append(lp.regs[a])
        if free:
            free.sort()
            lp.regs[i] = free.pop(0)
        else:
            lp.regs[i] = next_reg
            next_reg += 1
