#!/usr/bin/env python3
"""Synchronous classification of one tensor: read -> pre-process -> compile -> infer -> top-10.

usage: hello_classification.py <model.xml|.onnx|.gguf> <input.npy | "random"> [device]
Flow of samples/python/hello_classification/hello_classification.py; the image is an ``.npy`` array of shape HxWx3
(uint8) because this package carries no image decoder.
"""
import sys

import numpy as np

import openvino_b200 as ov
from openvino_b200.preprocess import PrePostProcessor, ResizeAlgorithm


def main() -> int:
    if len(sys.argv) < 3:
        print(__doc__)
        return 1
    model_path, image_path = sys.argv[1], sys.argv[2]
    device = sys.argv[3] if len(sys.argv) > 3 else "CPU"
    core = ov.Core()
    model = core.read_model(model_path)
    if len(model.inputs) != 1 or len(model.outputs) != 1:
        print("the sample supports single-input, single-output models")
        return 1
    if image_path == "random":
        image = np.random.default_rng(0).integers(0, 255, (224, 224, 3), dtype=np.uint8)
    else:
        image = np.load(image_path)
    tensor = np.expand_dims(image, 0)
    ppp = PrePostProcessor(model)
    ppp.input().tensor().set_shape(list(tensor.shape)).set_element_type(ov.Type.u8).set_layout(ov.Layout("NHWC"))
    ppp.input().preprocess().resize(ResizeAlgorithm.RESIZE_LINEAR)
    ppp.input().model().set_layout(ov.Layout("NCHW"))
    ppp.output().tensor().set_element_type(ov.Type.f32)
    model = ppp.build()
    compiled = core.compile_model(model, device)
    probs = compiled.infer_new_request({0: tensor})[compiled.output(0)].reshape(-1)
    top = np.argsort(probs)[-10:][::-1]
    print(f"Image path: {image_path}\nTop 10 results:\nclass_id probability\n--------------------")
    for c in top:
        print(f"{c:<8d} {probs[c]:.7f}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
