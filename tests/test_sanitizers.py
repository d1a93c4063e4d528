"""The native core under sanitizers, and the thread model of the peer-memory protocols under ThreadSanitizer.

``build.build_native_test`` compiles the C++ core, the C API and one test driver from ``tests/native`` into an
executable of its own (no Python in the process, so no preloaded sanitizer runtime is needed):

* ``core_smoke.cpp``          - model read / reshape / compile / threaded inference / save, and the scheduler with preemption
                                and prefix cache; under ASan + UBSan;
* ``runtime_threads.cpp``     - executors, asynchronous requests (busy, cancel, failing stage), the idle queue, the
                                scheduler shared by two threads; under TSan;
* ``comm_protocol_model.cpp`` - W threads run the all-reduce protocols of the fused GEMM epilogue (two-hop packets,
                                one-shot packets, fence + flags, in-switch barrier) with the kernels' index arithmetic,
                                including a rank that skips a step (the others time out with a status, the next step
                                works); under TSan.
"""
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

import openvino_b200 as ov
from openvino_b200 import build
from openvino_b200 import opset as ops

NATIVE = Path(__file__).resolve().parent / "native"


def _model(path):
    x = ops.parameter([1, 3, 8, 8], "f32", "data")
    w = (np.arange(4 * 3 * 3 * 3, dtype=np.float32).reshape(4, 3, 3, 3) - 50.0) / 100
    c = ops.convolution(x, ops.constant(w), [1, 1], [1, 1], [1, 1], [1, 1])
    r = ops.relu(ops.add(c, ops.constant(np.ones((1, 4, 1, 1), np.float32))))
    p = ops.max_pool(r, [2, 2], [1, 1], [0, 0], [0, 0], [2, 2]) if hasattr(ops, "max_pool") else r
    out = p.output(0) if hasattr(p, "output") else p
    m = ov.Model([ops.result(out)], [x], "smoke")
    ov.serialize(m, str(path), str(path)[:-4] + ".bin")


def _run(exe, args, env_extra):
    env = dict(os.environ, **env_extra)
    return subprocess.run([str(exe), *map(str, args)], capture_output=True, text=True, timeout=900, env=env)


def test_core_smoke_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    exe = build.build_native_test(NATIVE / "core_smoke.cpp", "address")
    _model(tmp_path / "m.xml")
    r = _run(exe, [tmp_path / "m.xml", tmp_path / "out.xml"], {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "print_stacktrace=1"})
    assert r.returncode == 0 and "CORE_SMOKE_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-6000:])
    assert "ERROR: AddressSanitizer" not in r.stderr and "runtime error" not in r.stderr, r.stderr[-6000:]


def test_runtime_threads_under_thread_sanitizer():
    # executors, asynchronous requests, the idle queue and the scheduler (the translation units that own threads and locks)
    exe = build.build_native_test(NATIVE / "runtime_threads.cpp", "thread", core_subset=("runtime", "sched", "types"))
    r = _run(exe, [], {"TSAN_OPTIONS": "halt_on_error=1"})
    assert r.returncode == 0 and "RUNTIME_THREADS_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-6000:])
    assert "WARNING: ThreadSanitizer" not in r.stderr, r.stderr[-6000:]


def test_comm_protocol_model_under_thread_sanitizer():
    exe = build.build_native_test(NATIVE / "comm_protocol_model.cpp", "thread", core_subset=())
    r = _run(exe, [], {"TSAN_OPTIONS": "halt_on_error=1"})
    assert r.returncode == 0 and "COMM_MODEL_OK" in r.stdout, (r.stdout[-3000:], r.stderr[-6000:])
    assert "WARNING: ThreadSanitizer" not in r.stderr, r.stderr[-6000:]
