"""Timing of generated snippet kernels on the CUDA device:

    python -m openvino_b200.snippets.bench [--rows 32768] [--cols 4096] [--dtype f16] [--iters 20]

Two bodies: an element-wise chain (multiply by a row vector, add, Swish, maximum with the negated input) and a row-wise
chain (bias row, GELU, per-row scale, clamp, Softmax, residual add). Inputs are larger than L2; CUDA events around each
launch, median of ``iters``; achieved bandwidth counts every input and output once."""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

import openvino_b200 as ov
from openvino_b200 import opset as ops


def _models(rows: int, cols: int, dtype: str):
    npdt = {"f16": np.float16, "f32": np.float32}[dtype]
    x = ops.parameter([rows, cols], dtype, "x")
    y = ops.parameter([cols], dtype, "y")
    z = ops.swish(ops.add(ops.multiply(x, y), npdt(0.25)))
    ew = ov.Model([ops.maximum(z, ops.negative(x))], [x, y], "elementwise_chain")
    x2 = ops.parameter([rows, cols], dtype, "x")
    s2 = ops.parameter([rows, 1], dtype, "s")
    bias = ops.constant(np.linspace(-1, 1, cols).astype(npdt))
    h = ops.clamp(ops.multiply(ops.gelu(ops.add(x2, bias), "TANH"), s2), -2.0, 2.0)
    rw = ov.Model([ops.add(ops.softmax(h, 1), x2)], [x2, s2], "rowwise_chain")
    return ew, rw


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--dtype", default="f16")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    core = ov.Core()
    tdt = {"f16": torch.float16, "f32": torch.float32}[args.dtype]
    esz = 2 if args.dtype == "f16" else 4
    for model in _models(args.rows, args.cols, args.dtype):
        cm = core.compile_model(model, "CUDA", {"SNIPPETS_MODE": "ENABLE", "INFERENCE_PRECISION_HINT": args.dtype})
        node = next(n for n in cm.get_runtime_model().get_ops() if n.get_type_name() == "Subgraph")
        from openvino_b200.runtime.cuda_plugin import _OPS
        from openvino_b200.snippets.runtime import run_subgraph
        # inputs of the Subgraph node in its own order: parameters of the model, then constants that stayed outside the body
        feeds = []
        for k in range(node.get_input_size()):
            src = node.input_value(k).get_node()
            shape = [int(d) for d in node.get_input_shape(k)]
            if src.get_type_name() == "Constant":
                feeds.append(torch.as_tensor(np.asarray(src.get_data())).to("cuda").to(tdt))
            else:
                feeds.append(torch.randn(shape, device="cuda").to(tdt))
        ctx = cm.program.ctx
        for _ in range(3):
            run_subgraph(node, feeds, ctx, _OPS)
        times = []
        for _ in range(args.iters):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            run_subgraph(node, feeds, ctx, _OPS)
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b))
        ms = float(np.median(times))
        nbytes = sum(int(t.numel()) for t in feeds) * esz + args.rows * args.cols * esz
        print(json.dumps({"kernel": "snippet:" + model.get_friendly_name(), "rows": args.rows, "cols": args.cols, "dtype": args.dtype, "ms": ms,
                          "gbs": nbytes / ms / 1e6, "note": "one generated kernel per launch (output allocation included)"}))


if __name__ == "__main__":
    main()
