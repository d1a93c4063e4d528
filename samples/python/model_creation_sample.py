#!/usr/bin/env python3
"""Builds a small convolutional classifier with the opset factories, saves it as IR and runs it.

usage: model_creation_sample.py [device] [out.xml]
Flow of samples/python/model_creation_sample/model_creation_sample.py (weights are random instead of a LeNet file).
"""
import sys

import numpy as np

import openvino_b200 as ov
from openvino_b200 import opset as ops


def create_model(rng) -> ov.Model:
    x = ops.parameter([1, 1, 28, 28], "f32", "image")
    w1 = rng.standard_normal((8, 1, 5, 5)).astype(np.float32) * 0.1
    y = ops.relu(ops.add(ops.convolution(x, w1, [1, 1], [0, 0], [0, 0], [1, 1]), np.zeros((1, 8, 1, 1), np.float32)))
    y = ops.max_pool(y, [2, 2], [1, 1], [0, 0], [0, 0], [2, 2]).output(0)
    w2 = rng.standard_normal((16, 8, 5, 5)).astype(np.float32) * 0.1
    y = ops.relu(ops.convolution(y, w2, [1, 1], [0, 0], [0, 0], [1, 1]))
    y = ops.max_pool(y, [2, 2], [1, 1], [0, 0], [0, 0], [2, 2]).output(0)
    y = ops.reshape(y, np.array([1, -1], dtype=np.int64), False)
    fc = rng.standard_normal((10, 16 * 4 * 4)).astype(np.float32) * 0.1
    y = ops.softmax(ops.matmul(y, fc, False, True), 1)
    y.output(0).set_names({"prob"})
    return ov.Model([ops.result(y)], [x], "lenet_like")


def main() -> int:
    device = sys.argv[1] if len(sys.argv) > 1 else "CPU"
    rng = np.random.default_rng(0)
    model = create_model(rng)
    if len(sys.argv) > 2:
        ov.save_model(model, sys.argv[2], compress_to_fp16=False)
        print("saved", sys.argv[2])
    compiled = ov.Core().compile_model(model, device)
    digit = rng.uniform(0, 1, (1, 1, 28, 28)).astype(np.float32)
    probs = compiled(digit)["prob"].reshape(-1)
    for c in np.argsort(probs)[::-1][:3]:
        print(f"class {c}: {probs[c]:.5f}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
