"""benchmark_app: measure latency / throughput of a model on a device.

    python -m openvino_b200.benchmark_app -m model.xml -d CPU -hint throughput -t 10
    python -m openvino_b200.benchmark_app -m model.xml -d CUDA -api sync -niter 200 -pc

Follows the reference tool (tools/benchmark_tool/openvino/tools/benchmark/main.py, benchmark.py:80-190): read -> optional
reshape -> compile with a performance hint -> fill inputs with random data -> warm-up -> sync loop or AsyncInferQueue
loop bounded by ``-niter`` and/or ``-t`` -> latency percentiles and throughput, optional per-layer counters (``-pc``) and a
JSON report (``-report_type``).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from typing import Dict, List

import numpy as np

import openvino_b200 as ov
from openvino_b200 import properties as props


def parse_shapes(text: str) -> Dict[str, List[int]]:
    """"input[1,3,224,224],other[1,10]" or "[1,3,224,224]" (single input)."""
    out = {}
    text = text.strip()
    if not text:
        return out
    import re
    for name, dims in re.findall(r"([^\[\],]*)\[([^\]]*)\]", text):
        out[name.strip()] = [int(d) if d.strip() not in ("?", "-1") else -1 for d in dims.split(",") if d.strip()]
    return out


def fill_inputs(compiled, rng) -> List[np.ndarray]:
    feeds = []
    for port in compiled.inputs:
        ps = port.get_partial_shape()
        if ps.is_dynamic:
            raise SystemExit("input %s has a dynamic shape %s: give -shape" % (sorted(port.get_names()), ps))
        shape = list(ps.get_shape())
        et = port.get_element_type()
        if et.is_real():
            feeds.append(rng.standard_normal(shape).astype(et.to_dtype() if et.name in ("f32", "f16", "f64") else np.float32))
        elif et.name == "boolean":
            feeds.append(rng.integers(0, 2, shape).astype(bool))
        else:
            feeds.append(rng.integers(0, 10, shape).astype(et.to_dtype()))
    return feeds


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="benchmark_app", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("-m", "--path_to_model", required=True)
    ap.add_argument("-d", "--target_device", default="CPU")
    ap.add_argument("-hint", "--perf_hint", default="throughput", choices=["throughput", "tput", "latency", "cumulative_throughput", "ctput", "none"])
    ap.add_argument("-api", "--api_type", default="async", choices=["sync", "async"])
    ap.add_argument("-niter", "--number_iterations", type=int, default=0)
    ap.add_argument("-t", "--time", type=float, default=0.0, help="seconds")
    ap.add_argument("-nireq", "--number_infer_requests", type=int, default=0)
    ap.add_argument("-nstreams", "--number_streams", type=int, default=0)
    ap.add_argument("-nthreads", "--number_threads", type=int, default=0)
    ap.add_argument("-b", "--batch_size", type=int, default=0)
    ap.add_argument("-shape", default="")
    ap.add_argument("-infer_precision", default="")
    ap.add_argument("-cache_dir", default="")
    ap.add_argument("-pc", "--perf_counts", action="store_true")
    ap.add_argument("-report_type", default="", choices=["", "no_counters", "average_counters", "detailed_counters"])
    ap.add_argument("-report_folder", default=".")
    ap.add_argument("-seed", type=int, default=0)
    a = ap.parse_args(argv)

    print("[Step 1/8] Loading the runtime: openvino_b200 %s" % ov.get_version())
    core = ov.Core()
    print("[Step 2/8] Reading model %s" % a.path_to_model)
    t0 = time.perf_counter()
    model = core.read_model(a.path_to_model)
    print("           read in %.1f ms" % ((time.perf_counter() - t0) * 1e3))
    shapes = parse_shapes(a.shape)
    if shapes or a.batch_size:
        print("[Step 3/8] Reshaping")
        new = {}
        for i, p in enumerate(model.inputs):
            names = p.get_names()
            given = next((s for n, s in shapes.items() if n in names or (n == "" and len(model.inputs) == 1)), None)
            dims = given if given is not None else [d.get_length() if d.is_static else -1 for d in p.get_partial_shape()]
            if a.batch_size and dims:
                dims = [a.batch_size] + list(dims[1:])
            new[i] = dims
        model.reshape(new)
    cfg = {}
    hint = {"tput": "THROUGHPUT", "throughput": "THROUGHPUT", "latency": "LATENCY", "ctput": "CUMULATIVE_THROUGHPUT",
            "cumulative_throughput": "CUMULATIVE_THROUGHPUT"}.get(a.perf_hint)
    if hint:
        cfg[props.hint.performance_mode] = hint
    if a.number_streams:
        cfg[props.num_streams] = a.number_streams
    if a.number_threads:
        cfg[props.inference_num_threads] = a.number_threads
    if a.infer_precision:
        cfg[props.hint.inference_precision] = a.infer_precision
    if a.perf_counts or a.report_type in ("average_counters", "detailed_counters"):
        cfg[props.enable_profiling] = True
    if a.cache_dir:
        core.set_property({props.cache_dir: a.cache_dir})
    print("[Step 4/8] Compiling for %s with %s" % (a.target_device, cfg))
    t0 = time.perf_counter()
    compiled = core.compile_model(model, a.target_device, cfg)
    compile_ms = (time.perf_counter() - t0) * 1e3
    print("           compiled in %.1f ms; execution devices %s" % (compile_ms, compiled.get_property(props.execution_devices)))
    nireq = a.number_infer_requests or (1 if a.api_type == "sync" else compiled.get_property(props.optimal_number_of_infer_requests))
    print("[Step 5/8] Creating %d infer request(s), filling inputs with random data" % nireq)
    rng = np.random.default_rng(a.seed)
    feeds = fill_inputs(compiled, rng)
    niter, seconds = a.number_iterations, a.time
    if not niter and not seconds:
        seconds = 10.0
    print("[Step 6/8] Warm-up")
    first = compiled.create_infer_request()
    t0 = time.perf_counter()
    first.infer(feeds)
    print("           first inference took %.2f ms" % ((time.perf_counter() - t0) * 1e3))
    print("[Step 7/8] Measuring (%s API, %s)" % (a.api_type, ("%d iterations" % niter) if niter else ("%.1f s" % seconds)))
    latencies: List[float] = []
    start = time.perf_counter()
    done = 0

    def more() -> bool:
        if niter and done >= niter:
            return False
        if seconds and (time.perf_counter() - start) >= seconds and not (niter and done < niter):
            return False
        return True
    last_request = first
    if a.api_type == "sync":
        while more():
            t1 = time.perf_counter()
            first.infer(feeds)
            latencies.append((time.perf_counter() - t1) * 1e3)
            done += 1
    else:
        queue = ov.AsyncInferQueue(compiled, nireq)
        queue.set_callback(lambda req, userdata: latencies.append(req.latency))
        while more():
            queue.start_async(feeds)
            done += 1
        queue.wait_all()
        last_request = queue[0]
    total = time.perf_counter() - start
    print("[Step 8/8] Results")
    latencies.sort()
    pct = lambda q: latencies[min(len(latencies) - 1, int(q * len(latencies)))] if latencies else float("nan")
    batch = feeds[0].shape[0] if feeds and feeds[0].ndim else 1
    report = {"device": a.target_device, "api": a.api_type, "iterations": done, "duration_ms": total * 1e3, "nireq": nireq,
              "compile_ms": compile_ms, "latency_ms": {"median": pct(0.5), "avg": statistics.fmean(latencies) if latencies else None,
                                                         "min": latencies[0] if latencies else None, "max": latencies[-1] if latencies else None,
                                                         "p90": pct(0.9), "p99": pct(0.99)},
              "throughput_fps": done * batch / total}
    print("Count:          %d iterations" % done)
    print("Duration:       %.2f ms" % (total * 1e3))
    print("Latency:        median %.3f ms, avg %.3f ms, min %.3f ms, max %.3f ms" % (pct(0.5), report["latency_ms"]["avg"] or 0, latencies[0], latencies[-1]))
    print("Throughput:     %.2f FPS" % report["throughput_fps"])
    if cfg.get(props.enable_profiling):
        info = last_request.get_profiling_info()
        by_type: Dict[str, float] = {}
        for p in info:
            by_type[p.node_type] = by_type.get(p.node_type, 0.0) + p.real_time
        print("Performance counters of the last request (us by operation type):")
        for t, us in sorted(by_type.items(), key=lambda kv: -kv[1])[:20]:
            print("  %-32s %10.1f" % (t, us))
        report["counters_us_by_type"] = by_type
        if a.report_type == "detailed_counters":
            report["counters"] = [{"name": p.node_name, "type": p.node_type, "exec": p.exec_type, "us": p.real_time, "status": p.status} for p in info]
    if a.report_type:
        import os
        path = os.path.join(a.report_folder, "benchmark_report.json")
        with open(path, "w") as f:
            json.dump(report, f, indent=1)
        print("Report written to %s" % path)
    return 0


if __name__ == "__main__":
    sys.exit(main())
