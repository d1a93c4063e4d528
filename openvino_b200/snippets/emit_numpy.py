"""NumPy executor of a snippet's linear IR: walks the loops the way the generated kernel does (one pass per stage,
recomputation included), whole rows at a time. It is the host implementation of the ``Subgraph`` operation and the
check of the lowering itself."""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np

from .lowered import COL, FULL, LinearIR
from .op_table import OPS, REDUCTIONS

_NP = {"f32": np.float32, "f16": np.float16, "boolean": np.bool_, "u8": np.uint8, "i32": np.int32, "i64": np.int64}


def _to_bf16_f32(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return u.view(np.float32)


def run_numpy(lir: LinearIR, inputs: Sequence[np.ndarray], rows: int, cols: int) -> List[np.ndarray]:
    """``inputs[i]`` is a 2-D array already in its broadcast form ([rows, cols], [1, cols], [rows, 1] or [1, 1]);
    bf16 data arrives as fp32. Returns 2-D fp32 arrays rounded to the output types ([rows, cols] or [rows, 1])."""
    ex = lir.exprs
    row_vals: Dict[int, np.ndarray] = {}           # col-domain values: [rows, 1]

    def col_value(i: int) -> np.ndarray:
        e = ex[i]
        if e.kind == "scalar":
            return np.full((rows, 1), e.value, np.float32)
        if e.kind == "inv_cols":
            return np.full((rows, 1), 1.0 / cols, np.float32)
        if e.kind == "param":
            return np.broadcast_to(np.asarray(inputs[e.index], dtype=np.float32), (rows, 1))
        return OPS[e.op].np_fn(e.attrs, *[row_vals[a] for a in e.args]).astype(np.float32)

    outs: List[np.ndarray] = [None] * len(lir.stores)
    for lp in lir.loops:
        for i in lp.prologue:
            row_vals[i] = col_value(i)
        vals: Dict[int, np.ndarray] = {}
        for i in lp.body:
            e = ex[i]
            if e.kind == "param":
                vals[i] = np.broadcast_to(np.asarray(inputs[e.index], dtype=np.float32), (rows, cols))
            else:
                args = [vals[a] if ex[a].domain == FULL else row_vals[a] for a in e.args]
                with np.errstate(all="ignore"):
                    vals[i] = np.asarray(OPS[e.op].np_fn(e.attrs, *args), dtype=np.float32)
                    vals[i] = np.broadcast_to(vals[i], (rows, cols))
        for r in lp.reduces:
            src = ex[r].args[0]
            v = vals[src] if ex[src].domain == FULL else np.broadcast_to(row_vals[src], (rows, cols))
            row_vals[r] = REDUCTIONS[ex[r].op][1](v, axis=1, keepdims=True).astype(np.float32)
        for s in lp.stores:
            outs[s.output] = vals[s.value]
    for i in lir.epilogue:
        if i not in row_vals:
            row_vals[i] = col_value(i)
    for s in lir.stores:
        if s.domain == COL:
            outs[s.output] = row_vals[s.value]
    res = []
    for o, t in zip(outs, lir.out_types):
        o = np.ascontiguousarray(o, dtype=np.float32)
        if t == "bf16":
            o = _to_bf16_f32(o)
        elif t == "f16":
            o = o.astype(np.float16).astype(np.float32)
        elif t == "boolean":
            o = (o != 0).astype(np.float32)
        res.append(o)
    return res
