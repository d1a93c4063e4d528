"""ovc: convert a model file to IR from the command line.

    python -m openvino_b200.tools.ovc model.onnx --output_model out.xml [--input "x[1,3,224,224]"] [--output name]
                                                 [--compress_to_fp16 True|False] [--verbose]

Accepts what ``convert_model`` accepts as a file: IR ``.xml``, ``.onnx``, frozen TensorFlow ``.pb``, ``.gguf``. ``--input``
takes comma-separated entries ``name[shape]`` or ``[shape]`` (``?`` or ``-1`` for a dynamic dimension) in input order.
Role of tools/ovc/openvino/tools/ovc/main.py (the command-line face of ``ov.convert_model`` + ``ov.save_model``).
"""
from __future__ import annotations

import argparse
import os
import re
import sys


def parse_input(spec: str):
    """"a[1,3,?,224],b[2]" or "[1,3,224,224]" -> dict name -> dims, or list of dims in input order."""
    entries = re.findall(r"([^,\[\]]*)\[([^\]]*)\]", spec)
    if not entries:
        raise ValueError("--input: expected name[shape] entries, got %r" % spec)
    named, plain = {}, []
    for name, dims in entries:
        shape = [-1 if d.strip() in ("?", "-1") else int(d) for d in dims.split(",") if d.strip()]
        if name.strip():
            named[name.strip()] = shape
        else:
            plain.append(shape)
    if named and plain:
        raise ValueError("--input: give names for all inputs or for none")
    return named or plain


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ovc", description=__doc__.splitlines()[0])
    ap.add_argument("input_model")
    ap.add_argument("--output_model", default=None, help="path of the .xml to write (default: <input name>.xml in the current directory)")
    ap.add_argument("--input", default=None)
    ap.add_argument("--output", default=None, help="comma-separated names of the values to keep as outputs")
    ap.add_argument("--compress_to_fp16", default="True", choices=["True", "False", "true", "false"])
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args(argv)
    import openvino_b200 as ov
    if not os.path.exists(a.input_model):
        print("[ ERROR ] model file %s does not exist" % a.input_model, file=sys.stderr)
        return 1
    try:
        model = ov.convert_model(a.input_model, input=parse_input(a.input) if a.input else None,
                                 output=[o.strip() for o in a.output.split(",")] if a.output else None)
    except Exception as e:
        print("[ ERROR ] conversion failed: %s" % e, file=sys.stderr)
        return 1
    out = a.output_model or os.path.splitext(os.path.basename(a.input_model))[0] + ".xml"
    if not out.lower().endswith(".xml"):
        out = os.path.join(out, os.path.splitext(os.path.basename(a.input_model))[0] + ".xml")
        os.makedirs(os.path.dirname(out), exist_ok=True)
    ov.save_model(model, out, compress_to_fp16=a.compress_to_fp16.lower() == "true")
    if a.verbose:
        for p in model.inputs:
            print("input  %s %s %s" % (p.get_any_name(), p.get_element_type(), p.get_partial_shape()))
        for p in model.outputs:
            print("output %s %s %s" % (p.get_any_name(), p.get_element_type(), p.get_partial_shape()))
    print("[ SUCCESS ] XML file: %s" % os.path.abspath(out))
    print("[ SUCCESS ] BIN file: %s" % os.path.abspath(out[:-4] + ".bin"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
