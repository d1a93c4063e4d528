"""The Python samples run end to end on the CPU device."""
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SAMPLES = os.path.join(ROOT, "samples", "python")


def _run(script, *args):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, os.path.join(SAMPLES, script), *args], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    return r.stdout


def test_model_creation_then_async_and_sync_classification(tmp_path):
    xml = str(tmp_path / "lenet.xml")
    out = _run("model_creation_sample.py", "CPU", xml)
    assert "saved" in out and out.count("class ") == 3 and os.path.exists(xml)
    out = _run("classification_sample_async.py", xml, "4")
    assert out.count("class ") == 4
    out = _run("hello_query_device.py")
    assert "CPU :" in out and "FULL_DEVICE_NAME" in out


def test_hello_classification_with_preprocessing(tmp_path):
    import openvino_b200 as ov
    from openvino_b200 import opset as ops
    x = ops.parameter([1, 3, 16, 16], "f32", "image")
    w = np.random.default_rng(0).standard_normal((6, 3, 3, 3)).astype(np.float32) * 0.01
    y = ops.reduce_mean(ops.relu(ops.convolution(x, w, [1, 1], [1, 1], [1, 1], [1, 1])), np.array([2, 3]), False)
    xml = str(tmp_path / "c.xml")
    ov.serialize(ov.Model([ops.result(ops.softmax(y, 1))], [x], "c"), xml)
    img = str(tmp_path / "img.npy")
    np.save(img, np.random.default_rng(1).integers(0, 255, (40, 30, 3), dtype=np.uint8))
    out = _run("hello_classification.py", xml, img)
    assert "Top 10 results" in out and len([l for l in out.splitlines() if l[:1].isdigit()]) == 6
