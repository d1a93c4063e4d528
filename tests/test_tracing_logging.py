"""Phase tracing, logging sink, execution-graph rt_info, serving metrics report."""
import json

import numpy as np

import openvino_b200 as ov
from openvino_b200 import opset as ops, properties as props
from openvino_b200.utils import log, trace


def _model():
    x = ops.parameter([2, 8], "f32", "x")
    w = np.random.default_rng(0).standard_normal((4, 8)).astype(np.float32)
    return ov.Model([ops.result(ops.relu(ops.matmul(x, w, False, True)))], [x], "m")


def test_scopes_are_recorded_and_dumped(tmp_path):
    trace.clear()
    trace.enable(True)
    try:
        core = ov.Core()
        path = str(tmp_path / "m.xml")
        ov.serialize(_model(), path)
        m = core.read_model(path)
        cm = core.compile_model(m, "CPU")
        cm(np.zeros((2, 8), np.float32))
        pm = ov.passes.Manager()
        pm.register_pass("ConstantFolding")
        pm.run_passes(m)
    finally:
        trace.enable(False)
    names = {(d, n) for d, n, *_ in trace.events()}
    assert ("ov::ReadTime", "Core::read_model") in names and ("ov::LoadTime", "Core::compile_model::CPU") in names
    assert ("ov::phases", "InferRequest::infer::CPU") in names and ("ov::pass", "Manager::run_passes") in names
    assert any(d == "ov::pass" and n == "ConstantFolding" for d, n in names)
    out = str(tmp_path / "trace.json")
    assert trace.dump_chrome_trace(out) == len(trace.events())
    data = json.load(open(out))
    assert all(e["ph"] == "X" and e["dur"] >= 0 for e in data["traceEvents"])
    assert trace.summary()[("ov::phases", "InferRequest::infer::CPU")]["count"] == 1
    n = len(trace.events())
    core.compile_model(_model(), "CPU")          # tracing off: nothing is recorded
    assert len(trace.events()) == n


def test_log_level_and_callback():
    lines = []
    log.set_log_callback(lines.append)
    try:
        core = ov.Core()
        core.set_property({props.log.level: "INFO"})
        assert log.get_level() == "INFO"
        core.compile_model(_model(), "CPU")
        assert any("compiled 'm' for CPU" in l and l.startswith("[INFO]") for l in lines)
        core.set_property({props.log.level: "ERR"})
        n = len(lines)
        core.compile_model(_model(), "CPU")
        assert len(lines) == n
    finally:
        log.reset_log_callback()
        log.set_level("WARNING")


def test_runtime_model_carries_execution_info():
    cm = ov.Core().compile_model(_model(), "CPU", {props.enable_profiling: True})
    cm(np.ones((2, 8), np.float32))
    rm = cm.get_runtime_model()
    mm = [n for n in rm.get_ops() if n.get_type_name() == "MatMul"][0]
    assert mm.rt_info["layerType"] == "MatMul" and mm.rt_info["runtimePrecision"] == "f32"
    assert mm.rt_info["execTimeMcs"].isdigit() and "originalLayersNames" in mm.rt_info


def test_metrics_report():
    from openvino_b200.genai.pipeline import GenerationResult, PipelineMetrics
    m = PipelineMetrics(steps=5, prefill_steps=1, decode_steps=4, generated_tokens=8)
    res = [GenerationResult(0, [1, 2], 0.010, 0.002), GenerationResult(1, [3, 4], 0.030, 0.004)]
    r = m.report(res, kv_blocks_total=100, kv_blocks_free=75)
    assert r["decode_steps"] == 4 and abs(r["kv_block_utilisation"] - 0.25) < 1e-9
    assert abs(r["ttft_ms"]["p50"] - 20.0) < 1e-6 and r["tpot_ms"]["p99"] <= 4.0 + 1e-6
    json.dumps(r)
