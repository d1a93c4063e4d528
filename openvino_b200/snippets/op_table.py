"""Operations a snippet may contain: how each is evaluated by the NumPy executor and how the CUDA emitter writes it.

Every value inside a snippet is an fp32 scalar per element (16-bit inputs are widened on load, results narrowed on
store; booleans are 0.0 / 1.0), so one table serves every element type. When every input and output of a snippet is a 16-bit type the emitter sets
``_fast`` in the attributes: sigmoid-shaped functions then cost one ``tanh.approx`` (relative error about 5e-4, below
the resolution of the stored values) instead of an exponential and a reciprocal. Role of the emitter tables of the reference
(src/common/snippets/include/snippets/target_machine.hpp, src/plugins/intel_cpu/src/emitters/snippets/x64/cpu_generator.cpp).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, NamedTuple, Optional

import numpy as np


class OpDef(NamedTuple):
    arity: int
    np_fn: Callable            # (attrs, *arrays) -> array
    cuda: Callable             # (attrs, *arg names) -> C expression
    boolean: bool = False      # result is a truth value


def _erf(x):
    # Abramowitz-Stegun 7.1.26 is not accurate enough for fp32 checks: use math.erf element-wise
    return np.vectorize(math.erf, otypes=[np.float32])(x)


def _f(v) -> str:
    """A float attribute as a C literal."""
    v = float(v)
    if math.isinf(v):
        return "INFINITY" if v > 0 else "-INFINITY"
    if math.isnan(v):
        return "NAN"
    return "%sf" % repr(float(np.float32(v)))


def _gelu_np(a, x):
    if str(a.get("approximation_mode", "ERF")).upper() == "TANH":
        return 0.5 * x * (1 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    return 0.5 * x * (1 + _erf(x * 0.7071067811865476))


def _gelu_cu(a, x):
    if str(a.get("approximation_mode", "ERF")).upper() == "TANH":
        if a.get("_fast"):
            return "(0.5f * %s * (1.0f + tanh_fast(0.7978845608028654f * (%s + 0.044715f * %s * %s * %s))))" % (x, x, x, x, x)
        return "(0.5f * %s * (1.0f + tanhf(0.7978845608028654f * (%s + 0.044715f * %s * %s * %s))))" % (x, x, x, x, x)
    return "(0.5f * %s * (1.0f + erff(%s * 0.70710678118654752f)))" % (x, x)


def _round_to(a, x):
    t = str(a.get("destination_type", "f32"))
    if t == "f16":
        return x.astype(np.float16).astype(np.float32)
    if t == "bf16":
        u = x.astype(np.float32).view(np.uint32)
        u = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
        return u.view(np.float32)
    if t == "boolean":
        return (x != 0).astype(np.float32)
    return x


def _round_to_cu(a, x):
    t = str(a.get("destination_type", "f32"))
    if t == "f16":
        return "__half2float(__float2half_rn(%s))" % x
    if t == "bf16":
        return "__bfloat162float(__float2bfloat16_rn(%s))" % x
    if t == "boolean":
        return "((%s) != 0.0f ? 1.0f : 0.0f)" % x
    return x


def _cmp(sym):
    return OpDef(2, lambda a, x, y, s=sym: eval("x %s y" % s).astype(np.float32), lambda a, x, y, s=sym: "((%s %s %s) ? 1.0f : 0.0f)" % (x, s, y), True)


OPS: Dict[str, OpDef] = {
    "Relu": OpDef(1, lambda a, x: np.maximum(x, 0), lambda a, x: "fmaxf(%s, 0.0f)" % x),
    "Sigmoid": OpDef(1, lambda a, x: 1 / (1 + np.exp(-x)),
                     lambda a, x: ("(0.5f * tanh_fast(0.5f * %s) + 0.5f)" % x) if a.get("_fast") else ("__fdividef(1.0f, 1.0f + __expf(-%s))" % x)),
    "Tanh": OpDef(1, lambda a, x: np.tanh(x), lambda a, x: ("tanh_fast(%s)" if a.get("_fast") else "tanhf(%s)") % x),
    "Exp": OpDef(1, lambda a, x: np.exp(x), lambda a, x: "__expf(%s)" % x),
    "Log": OpDef(1, lambda a, x: np.log(x), lambda a, x: "__logf(%s)" % x),
    "Sqrt": OpDef(1, lambda a, x: np.sqrt(x), lambda a, x: "sqrtf(%s)" % x),
    "Abs": OpDef(1, lambda a, x: np.abs(x), lambda a, x: "fabsf(%s)" % x),
    "Negative": OpDef(1, lambda a, x: -x, lambda a, x: "(-%s)" % x),
    "Floor": OpDef(1, lambda a, x: np.floor(x), lambda a, x: "floorf(%s)" % x),
    "Ceiling": OpDef(1, lambda a, x: np.ceil(x), lambda a, x: "ceilf(%s)" % x),
    "Erf": OpDef(1, lambda a, x: _erf(x), lambda a, x: "erff(%s)" % x),
    "Sin": OpDef(1, lambda a, x: np.sin(x), lambda a, x: "sinf(%s)" % x),
    "Cos": OpDef(1, lambda a, x: np.cos(x), lambda a, x: "cosf(%s)" % x),
    "Gelu": OpDef(1, _gelu_np, _gelu_cu),
    "Swish": OpDef(1, lambda a, x: x / (1 + np.exp(-x)),
                   lambda a, x: ("(%s * (0.5f * tanh_fast(0.5f * %s) + 0.5f))" % (x, x)) if a.get("_fast") else ("__fdividef(%s, 1.0f + __expf(-%s))" % (x, x))),
    "HSwish": OpDef(1, lambda a, x: x * np.clip(x + 3, 0, 6) / 6, lambda a, x: "(%s * fminf(fmaxf(%s + 3.0f, 0.0f), 6.0f) * (1.0f / 6.0f))" % (x, x)),
    "HSigmoid": OpDef(1, lambda a, x: np.clip(x + 3, 0, 6) / 6, lambda a, x: "(fminf(fmaxf(%s + 3.0f, 0.0f), 6.0f) * (1.0f / 6.0f))" % x),
    "Mish": OpDef(1, lambda a, x: x * np.tanh(np.log1p(np.exp(x))), lambda a, x: "(%s * tanhf(log1pf(__expf(%s))))" % (x, x)),
    "SoftPlus": OpDef(1, lambda a, x: np.where(x > 20, x, np.log1p(np.exp(np.minimum(x, 20)))), lambda a, x: "(%s > 20.0f ? %s : log1pf(__expf(%s)))" % (x, x, x)),
    "Elu": OpDef(1, lambda a, x: np.where(x > 0, x, float(a.get("alpha", 1.0)) * (np.exp(np.minimum(x, 0)) - 1)),
                 lambda a, x: "(%s > 0.0f ? %s : %s * (__expf(%s) - 1.0f))" % (x, x, _f(a.get("alpha", 1.0)), x)),
    "Clamp": OpDef(1, lambda a, x: np.clip(x, float(a["min"]), float(a["max"])), lambda a, x: "fminf(fmaxf(%s, %s), %s)" % (x, _f(a["min"]), _f(a["max"]))),
    "Convert": OpDef(1, _round_to, _round_to_cu),
    "Reciprocal": OpDef(1, lambda a, x: 1.0 / x, lambda a, x: "(1.0f / %s)" % x),          # made by the lowering, never tokenised
    "LogicalNot": OpDef(1, lambda a, x: (x == 0).astype(np.float32), lambda a, x: "((%s) == 0.0f ? 1.0f : 0.0f)" % x, True),
    "Add": OpDef(2, lambda a, x, y: x + y, lambda a, x, y: "(%s + %s)" % (x, y)),
    "Subtract": OpDef(2, lambda a, x, y: x - y, lambda a, x, y: "(%s - %s)" % (x, y)),
    "Multiply": OpDef(2, lambda a, x, y: x * y, lambda a, x, y: "(%s * %s)" % (x, y)),
    "Divide": OpDef(2, lambda a, x, y: x / y, lambda a, x, y: "(%s / %s)" % (x, y)),
    "Maximum": OpDef(2, lambda a, x, y: np.maximum(x, y), lambda a, x, y: "fmaxf(%s, %s)" % (x, y)),
    "Minimum": OpDef(2, lambda a, x, y: np.minimum(x, y), lambda a, x, y: "fminf(%s, %s)" % (x, y)),
    "Power": OpDef(2, lambda a, x, y: np.power(x, y), lambda a, x, y: "powf(%s, %s)" % (x, y)),
    "SquaredDifference": OpDef(2, lambda a, x, y: (x - y) ** 2, lambda a, x, y: "((%s - %s) * (%s - %s))" % (x, y, x, y)),
    "PRelu": OpDef(2, lambda a, x, y: np.where(x >= 0, x, x * y), lambda a, x, y: "(%s >= 0.0f ? %s : %s * %s)" % (x, x, x, y)),
    "Greater": _cmp(">"), "GreaterEqual": _cmp(">="), "Less": _cmp("<"), "LessEqual": _cmp("<="), "Equal": _cmp("=="), "NotEqual": _cmp("!="),
    "LogicalAnd": OpDef(2, lambda a, x, y: ((x != 0) & (y != 0)).astype(np.float32), lambda a, x, y: "((%s != 0.0f && %s != 0.0f) ? 1.0f : 0.0f)" % (x, y), True),
    "LogicalOr": OpDef(2, lambda a, x, y: ((x != 0) | (y != 0)).astype(np.float32), lambda a, x, y: "((%s != 0.0f || %s != 0.0f) ? 1.0f : 0.0f)" % (x, y), True),
    "Select": OpDef(3, lambda a, c, x, y: np.where(c != 0, x, y), lambda a, c, x, y: "(%s != 0.0f ? %s : %s)" % (c, x, y)),
}

# reductions over the innermost axis: (identity, NumPy reduction, C combine expression, name of the block reduction)
REDUCTIONS = {
    "max": (-math.inf, np.max, lambda acc, v: "fmaxf(%s, %s)" % (acc, v), "block_max"),
    "sum": (0.0, np.sum, lambda acc, v: "(%s + %s)" % (acc, v), "block_sum"),
}

REDUCE_OPS = {"ReduceMax": "max", "ReduceSum": "sum", "ReduceMean": "sum"}


def supported(type_name: str) -> Optional[OpDef]:
    return OPS.get(type_name)
