"""compile_tool: compile a model for a device ahead of time and write the device's blob.

    python -m openvino_b200.tools.compile_tool -m model.xml -d CPU -o model.blob [-c config.json | -p KEY=VALUE ...]
                                               [--shape "name[1,3,224,224]"] [--check]

The blob is what ``Core.import_model(open(path, "rb").read(), device)`` takes back; ``--check`` does that import right after
writing and runs one inference on zeros through both, comparing the outputs. Role of
src/plugins/intel_npu/tools/compile_tool/main.cpp (offline compilation into a file that the runtime imports).
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import numpy as np

from .ovc import parse_input


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="compile_tool", description=__doc__.splitlines()[0])
    ap.add_argument("-m", "--model", required=True)
    ap.add_argument("-d", "--device", default="CPU")
    ap.add_argument("-o", "--output", default=None, help="blob path (default: the model's name with .blob)")
    ap.add_argument("-c", "--config", default=None, help="JSON file with the device configuration")
    ap.add_argument("-p", "--property", action="append", default=[], metavar="KEY=VALUE")
    ap.add_argument("--shape", default=None, help='static shapes, "name[dims],name[dims]" or "[dims]" in input order')
    ap.add_argument("--check", action="store_true", help="import the blob back and compare one inference")
    a = ap.parse_args(argv)

    import openvino_b200 as ov
    core = ov.Core()
    model = core.read_model(a.model)
    if a.shape:
        spec = parse_input(a.shape)
        model.reshape(spec if isinstance(spec, dict) else {i: s for i, s in enumerate(spec)})
    config = {}
    if a.config:
        with open(a.config) as f:
            config.update(json.load(f))
    for kv in a.property:
        if "=" not in kv:
            ap.error("-p expects KEY=VALUE, got %r" % kv)
        k, v = kv.split("=", 1)
        config[k] = v
    t0 = time.perf_counter()
    compiled = core.compile_model(model, a.device, config)
    t1 = time.perf_counter()
    blob = compiled.export_model()
    out = a.output or (a.model.rsplit(".", 1)[0] + ".blob")
    with open(out, "wb") as f:
        f.write(blob)
    print("compiled for %s in %.1f ms; %d bytes -> %s" % (a.device, (t1 - t0) * 1e3, len(blob), out))
    if a.check:
        back = core.import_model(blob, a.device, config)
        feeds = []
        for port in compiled.inputs:
            ps = port.get_partial_shape()
            if not ps.is_static:
                print("check skipped: input %s has a dynamic shape %s (give --shape)" % (port.get_any_name(), ps))
                return 0
            feeds.append(np.zeros([d.get_length() for d in ps], port.get_element_type().to_dtype()))
        r0, r1 = compiled(feeds), back(feeds)
        for i in range(len(compiled.outputs)):
            if not np.allclose(np.asarray(r0[i], dtype=np.float64), np.asarray(r1[i], dtype=np.float64), rtol=1e-5, atol=1e-6, equal_nan=True):
                print("check FAILED: output %d of the imported blob differs" % i)
                return 1
        print("check ok: %d output(s) equal" % len(compiled.outputs))
    return 0


if __name__ == "__main__":
    sys.exit(main())
