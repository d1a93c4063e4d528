#!/usr/bin/env python3
"""Asynchronous classification of several tensors through AsyncInferQueue with a completion callback.

usage: classification_sample_async.py <model.xml> <count> [device]
Flow of samples/python/classification_sample_async/classification_sample_async.py (inputs are random tensors).
"""
import sys

import numpy as np

import openvino_b200 as ov


def main() -> int:
    if len(sys.argv) < 3:
        print(__doc__)
        return 1
    model_path, count = sys.argv[1], int(sys.argv[2])
    device = sys.argv[3] if len(sys.argv) > 3 else "CPU"
    core = ov.Core()
    compiled = core.compile_model(core.read_model(model_path), device, {"PERFORMANCE_HINT": "THROUGHPUT"})
    shape = [d if d > 0 else 1 for d in compiled.input(0).get_partial_shape().get_min_shape()]
    rng = np.random.default_rng(0)
    results = {}

    def done(request, userdata):
        probs = request.get_output_tensor(0).data.reshape(-1)
        results[userdata] = int(np.argmax(probs))

    queue = ov.AsyncInferQueue(compiled)
    queue.set_callback(done)
    for i in range(count):
        queue.start_async({0: rng.standard_normal(shape).astype(np.float32)}, userdata=i)
    queue.wait_all()
    for i in range(count):
        print(f"input {i}: class {results[i]}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
