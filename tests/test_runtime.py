"""Core / CompiledModel / InferRequest / AsyncInferQueue behaviour, model cache, policy devices.

Mirrors the behaviour suites of the reference (src/tests/functional/plugin/shared/include/behavior/ov_infer_request/*,
ov_plugin/caching_tests.hpp, ov_plugin/properties_tests.hpp) on the CPU device.
"""
import io
import os
import threading
import time

import numpy as np
import pytest

import openvino_b200 as ov
from openvino_b200 import Model, Tensor, Type
from openvino_b200 import opset as ops
from openvino_b200 import properties as props
from openvino_b200.runtime.core import CompiledModel, CpuPlugin, Plugin


def mlp(batch=1, name="mlp"):
    rng = np.random.default_rng(0)
    x = ops.parameter([batch, 16], "f32", "x")
    x.output(0).set_names({"x"})
    h = ops.relu(ops.matmul(x, rng.standard_normal((32, 16)).astype(np.float32), False, True), name="hidden")
    y = ops.matmul(h, rng.standard_normal((4, 32)).astype(np.float32), False, True, name="logits")
    y.output(0).set_names({"y"})
    return Model([y], [x], name)


def ref(x):
    rng = np.random.default_rng(0)
    w1 = rng.standard_normal((32, 16)).astype(np.float32)
    w2 = rng.standard_normal((4, 32)).astype(np.float32)
    return np.maximum(x @ w1.T, 0) @ w2.T


@pytest.fixture()
def core():
    return ov.Core()


def test_devices_and_versions(core):
    assert "CPU" in core.available_devices
    assert "CPU" in core.get_versions("CPU")
    assert set(core.get_versions("HETERO:CPU")) == {"HETERO", "CPU"}
    with pytest.raises(RuntimeError, match="not registered"):
        core.compile_model(mlp(), "NOPE")


def test_properties(core):
    sp = core.get_property("CPU", props.supported_properties)
    assert props.enable_profiling in sp and props.num_streams in sp
    assert core.get_property("CPU", props.hint.performance_mode) == "LATENCY"
    core.set_property("CPU", {props.hint.performance_mode: props.PerformanceMode.THROUGHPUT})
    assert core.get_property("CPU", props.hint.performance_mode) == "THROUGHPUT"
    core.set_property("CPU", props.num_streams(3))
    cm = core.compile_model(mlp(), "CPU")
    assert cm.get_property(props.num_streams) == 3 and cm.get_property(props.optimal_number_of_infer_requests) == 3
    assert cm.get_property(props.model_name) == "mlp" and cm.get_property(props.execution_devices) == ["CPU"]
    with pytest.raises(RuntimeError):
        core.set_property("CPU", {"NO_SUCH_PROPERTY": 1})
    with pytest.raises(RuntimeError):
        core.get_property("CPU", "NO_SUCH_PROPERTY")
    with pytest.raises(RuntimeError):
        cm.set_property({props.num_streams: 1})
    assert isinstance(core.get_property("CPU", props.device.full_name), str)


def test_infer_variants(core):
    cm = core.compile_model(mlp(), "CPU")
    x = np.random.default_rng(1).standard_normal((1, 16)).astype(np.float32)
    want = ref(x)
    for res in (cm(x), cm([x]), cm({"x": x}), cm({0: x}), cm({cm.input(0): x}), cm.infer_new_request({"x": x})):
        np.testing.assert_allclose(res[0], want, rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(res["y"], want, rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(res[cm.output(0)], want, rtol=1e-5, atol=1e-5)
    req = cm.create_infer_request()
    req.set_tensor("x", Tensor(x))
    req.infer()
    np.testing.assert_allclose(req.get_tensor("y").data, want, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(req.get_output_tensor().data, want, rtol=1e-5, atol=1e-5)
    assert req.latency > 0
    assert cm.input("x").get_shape() == [1, 16] and cm.output().get_element_type() == Type.f32


def test_tensor_checks(core):
    cm = core.compile_model(mlp(), "CPU")
    req = cm.create_infer_request()
    with pytest.raises(RuntimeError, match="shape"):
        req.set_input_tensor(Tensor(np.zeros((2, 16), np.float32)))
    with pytest.raises(RuntimeError, match="element type"):
        req.set_input_tensor(Tensor(np.zeros((1, 16), np.int32)))
    with pytest.raises((RuntimeError, IndexError)):
        req.get_tensor("nope")
    # numpy inputs of another dtype are converted to the model's type
    np.testing.assert_allclose(cm(np.ones((1, 16), np.float64))[0], ref(np.ones((1, 16), np.float32)), rtol=1e-5)


def test_user_output_tensor_is_filled(core):
    cm = core.compile_model(mlp(), "CPU")
    req = cm.create_infer_request()
    out = Tensor(Type.f32, [1, 4])
    req.set_output_tensor(0, out)
    x = np.ones((1, 16), np.float32)
    req.infer({"x": x})
    np.testing.assert_allclose(out.data, ref(x), rtol=1e-5)
    assert req.get_output_tensor(0) is out


def test_dynamic_model_reshapes_per_inference(core):
    m = mlp()
    m.reshape({0: [-1, 16]})
    assert m.is_dynamic()
    cm = core.compile_model(m, "CPU")
    for b in (1, 3, 7):
        x = np.random.default_rng(b).standard_normal((b, 16)).astype(np.float32)
        out = cm(x)[0]
        assert out.shape == (b, 4)
        np.testing.assert_allclose(out, ref(x), rtol=1e-4, atol=1e-4)
    m2 = mlp()
    m2.reshape([5, 16])
    assert m2.output(0).get_shape() == [5, 4]


def test_async_callback_and_wait(core):
    cm = core.compile_model(mlp(), "CPU")
    req = cm.create_infer_request()
    seen = []
    req.set_callback(lambda ud: seen.append((ud, threading.get_ident())), "tag")
    x = np.ones((1, 16), np.float32)
    req.start_async({"x": x})
    req.wait()
    assert seen and seen[0][0] == "tag"
    np.testing.assert_allclose(req.results[0], ref(x), rtol=1e-5)
    req.start_async({"x": x}, userdata="second")
    assert req.wait_for(10_000)
    assert seen[-1][0] == "second"


class SlowCompiled(CompiledModel):
    def _make_runner(self, request):
        def run(req, ins):
            for _ in range(50):
                if req._cancel_requested:
                    raise RuntimeError("stopped early")
                time.sleep(0.01)
            return [Tensor(np.zeros((1, 4), np.float32))]
        return run


class SlowPlugin(Plugin):
    device_name = "SLOW"

    def compile_model(self, model, config):
        return SlowCompiled(self, model, self.merged_config(config))

    def query_model(self, model, config):
        return {n.get_friendly_name(): "SLOW" for n in model.get_ops()}


def test_busy_and_cancel(core):
    core.register_plugin(SlowPlugin, "SLOW")
    cm = core.compile_model(mlp(), "SLOW")
    req = cm.create_infer_request()
    req.start_async({"x": np.zeros((1, 16), np.float32)})
    with pytest.raises(RuntimeError, match="busy"):
        req.start_async()
    with pytest.raises(RuntimeError, match="busy"):
        req.infer()
    assert req.wait_for(1) is False
    req.cancel()
    with pytest.raises(RuntimeError):
        req.wait()
    # usable again afterwards
    req.start_async()
    req.wait()
    with pytest.raises(RuntimeError, match="already registered"):
        core.register_plugin(SlowPlugin, "SLOW")
    core.unload_plugin("SLOW")


def test_exception_in_inference_reaches_wait(core):
    class Failing(CpuPlugin):
        device_name = "FAIL"

        def compile_model(self, model, config):
            cm = super().compile_model(model, config)
            cm._make_runner = lambda request: (lambda req, ins: (_ for _ in ()).throw(ValueError("boom")))
            return cm
    core.register_plugin(Failing, "FAIL")
    req = core.compile_model(mlp(), "FAIL").create_infer_request()
    with pytest.raises(Exception, match="boom"):
        req.infer({"x": np.zeros((1, 16), np.float32)})
    req.start_async()
    with pytest.raises(Exception, match="boom"):
        req.wait()


def test_async_infer_queue(core):
    cm = core.compile_model(mlp(), "CPU", {props.num_streams: 2})
    q = ov.AsyncInferQueue(cm, 3)
    assert len(q) == 3
    got = {}
    lock = threading.Lock()

    def done(request, userdata):
        with lock:
            got[userdata] = request.results[0].copy()
    q.set_callback(done)
    xs = [np.random.default_rng(i).standard_normal((1, 16)).astype(np.float32) for i in range(12)]
    for i, x in enumerate(xs):
        q.start_async({"x": x}, userdata=i)
    q.wait_all()
    assert sorted(got) == list(range(12))
    for i, x in enumerate(xs):
        np.testing.assert_allclose(got[i], ref(x), rtol=1e-4, atol=1e-4)
    assert q.is_ready()

    def bad(request, userdata):
        raise KeyError("from callback")
    q.set_callback(bad)
    q.start_async({"x": xs[0]})
    with pytest.raises(KeyError):
        q.wait_all()


def test_profiling(core):
    cm = core.compile_model(mlp(), "CPU", {props.enable_profiling: True})
    req = cm.create_infer_request()
    req.infer({"x": np.zeros((1, 16), np.float32)})
    info = req.get_profiling_info()
    types = {p.node_type for p in info}
    assert "MatMul" in types and all(p.real_time >= 0 for p in info) and all(p.status == "EXECUTED" for p in info)
    with pytest.raises(RuntimeError):
        core.compile_model(mlp(), "CPU").create_infer_request().get_profiling_info()
    rt = cm.get_runtime_model()
    assert all("layerType" in n.rt_info for n in rt.get_ops())


def test_export_import_and_cache(core, tmp_path):
    m = mlp()
    cm = core.compile_model(m, "CPU")
    blob = cm.export_model()
    cm2 = core.import_model(io.BytesIO(blob), "CPU")
    x = np.ones((1, 16), np.float32)
    np.testing.assert_array_equal(cm2(x)[0], cm(x)[0])
    with pytest.raises(RuntimeError, match="magic"):
        core.import_model(b"garbage-bytes-not-a-blob-at-all-0000000000", "CPU")
    with pytest.raises(RuntimeError, match="truncated"):
        core.import_model(blob[:-5], "CPU")
    cache = str(tmp_path / "cache")
    core.set_property({props.cache_dir: cache})
    a = core.compile_model(m, "CPU")
    assert a.get_property(props.loaded_from_cache) is False and len([f for f in os.listdir(cache) if f.endswith(".blob")]) == 1
    b = core.compile_model(m, "CPU")
    assert b.get_property(props.loaded_from_cache) is True
    np.testing.assert_array_equal(a(x)[0], b(x)[0])
    # another configuration or another model gives another entry
    core.compile_model(m, "CPU", {props.num_streams: 2})
    core.compile_model(mlp(2, "other"), "CPU")
    assert len([f for f in os.listdir(cache) if f.endswith(".blob")]) == 3
    # a corrupt entry is replaced, not fatal
    entry = sorted(os.listdir(cache))[0]
    with open(os.path.join(cache, entry), "wb") as f:
        f.write(b"broken")
    for mm in (m, mlp(2, "other")):
        core.compile_model(mm, "CPU")
    core.compile_model(m, "CPU", {props.num_streams: 2})
    assert len([f for f in os.listdir(cache) if f.endswith(".blob")]) == 3


def test_stateful_model_and_variable_state(core):
    x = ops.parameter([1, 4], "f32", "x")
    rv = ops.read_value(ops.constant(np.zeros((1, 4), np.float32)), "acc", "f32", [1, 4])
    s = ops.add(rv, x)
    asg = ops.assign(s, "acc")
    m = Model([ops.result(s)], [x], "stateful", [asg])
    cm = core.compile_model(m, "CPU")
    req = cm.create_infer_request()
    one = np.ones((1, 4), np.float32)
    assert (req.infer({"x": one})[0] == 1).all()
    assert (req.infer({"x": one})[0] == 2).all()
    states = req.query_state()
    assert [s.name for s in states] == ["acc"]
    assert (states[0].state.data == 2).all()
    states[0].state = Tensor(np.full((1, 4), 10, np.float32))
    assert (req.infer({"x": one})[0] == 11).all()
    req.reset_state()
    assert (req.infer({"x": one})[0] == 1).all()
    # states are per request
    other = cm.create_infer_request()
    assert (other.infer({"x": one})[0] == 1).all()


def test_auto_and_multi(core):
    m = mlp()
    x = np.ones((1, 16), np.float32)
    auto = core.compile_model(m, "AUTO:CPU")
    assert auto.get_property(props.execution_devices) == ["CPU"]
    np.testing.assert_allclose(auto(x)[0], ref(x), rtol=1e-5)
    assert core.compile_model(m)  # default device is AUTO
    multi = core.compile_model(m, "MULTI:CPU,CPU")
    assert multi.get_property(props.execution_devices) == ["CPU", "CPU"]
    reqs = [multi.create_infer_request() for _ in range(4)]
    for r in reqs:
        np.testing.assert_allclose(r.infer({"x": x})[0], ref(x), rtol=1e-5)
    ct = core.compile_model(m, "AUTO:CPU", {props.hint.performance_mode: "CUMULATIVE_THROUGHPUT"})
    np.testing.assert_allclose(ct(x)[0], ref(x), rtol=1e-5)


def test_auto_falls_back_when_a_device_fails(core):
    class Broken(Plugin):
        device_name = "BROKEN"

        def compile_model(self, model, config):
            raise RuntimeError("cannot compile")

        def query_model(self, model, config):
            return {}
    core.register_plugin(Broken, "BROKEN")
    cm = core.compile_model(mlp(), "AUTO:BROKEN,CPU")
    assert cm.get_property(props.execution_devices) == ["CPU"]

    class FailsAtRuntime(CpuPlugin):
        device_name = "FLAKY"

        def compile_model(self, model, config):
            cm = super().compile_model(model, config)
            cm._make_runner = lambda request: (lambda req, ins: (_ for _ in ()).throw(RuntimeError("device lost")))
            return cm
    core.register_plugin(FailsAtRuntime, "FLAKY")
    cm = core.compile_model(mlp(), "AUTO:FLAKY,CPU")
    x = np.ones((1, 16), np.float32)
    np.testing.assert_allclose(cm(x)[0], ref(x), rtol=1e-5)
    assert cm.get_property(props.execution_devices) == ["FLAKY", "CPU"]


def test_proxy_device_aliases_plugins_with_fallback(core):
    class Broken(Plugin):
        device_name = "LOWLEVEL_A"

        def compile_model(self, model, config):
            raise RuntimeError("driver too old")

        def query_model(self, model, config):
            return {}

    class TwoDevices(CpuPlugin):
        device_name = "LOWLEVEL_B"

        def available_device_ids(self):
            return ["0", "1"]

    # two low-level plugins behind one name; the second is the fallback of the first
    core.register_plugin(Broken, "LOWLEVEL_A", {"PROXY_CONFIGURATION_ALIAS": "ACCEL"})
    core.register_plugin(TwoDevices, "LOWLEVEL_B", {"PROXY_CONFIGURATION_ALIAS": "ACCEL"})
    assert core.get_property("ACCEL", "PROXY_FALLBACK_ORDER") == ["LOWLEVEL_A", "LOWLEVEL_B"]
    assert core.get_property("ACCEL", props.available_devices) == ["0", "1", "2"]
    x = np.ones((1, 16), np.float32)
    cm = core.compile_model(mlp(), "ACCEL")          # device 0 belongs to the broken plugin: falls back
    np.testing.assert_allclose(cm(x)[0], ref(x), rtol=1e-5)
    cm = core.compile_model(mlp(), "ACCEL.2")        # third device = second device of the second plugin
    np.testing.assert_allclose(cm(x)[0], ref(x), rtol=1e-5)
    with pytest.raises(RuntimeError, match="no device with id 5"):
        core.compile_model(mlp(), "ACCEL.5")
    core.register_proxy("ONLY_BROKEN", ["LOWLEVEL_A"])
    with pytest.raises(RuntimeError, match="driver too old"):
        core.compile_model(mlp(), "ONLY_BROKEN")


def test_hetero_splits_by_supported_ops(core):
    class NoRelu(CpuPlugin):
        device_name = "NORELU"

        def query_model(self, model, config):
            return {k: "NORELU" for k, v in super().query_model(model, config).items()
                    if next(n for n in model.get_ops() if n.get_friendly_name() == k).get_type_name() != "Relu"}
    core.register_plugin(NoRelu, "NORELU")
    m = mlp()
    q = core.query_model(m, "HETERO:NORELU,CPU")
    assert q["hidden"] == "CPU" and q["logits"] == "NORELU"
    cm = core.compile_model(m, "HETERO:NORELU,CPU")
    assert [s.device for s in cm.subs] == ["NORELU", "CPU", "NORELU"]
    assert cm.get_property(props.execution_devices) == ["CPU", "NORELU"]
    x = np.random.default_rng(3).standard_normal((1, 16)).astype(np.float32)
    np.testing.assert_allclose(cm(x)[0], ref(x), rtol=1e-5, atol=1e-5)
    # manual affinity wins
    m2 = mlp()
    for n in m2.get_ops():
        if n.get_type_name() == "MatMul":
            n.rt_info["affinity"] = "CPU"
    cm2 = core.compile_model(m2, "HETERO:NORELU,CPU")
    assert {s.device for s in cm2.subs} == {"CPU"}


def test_hetero_pipeline_parallel_splits_by_memory_and_round_trips_the_partition(core):
    """MODEL_DISTRIBUTION_POLICY = PIPELINE_PARALLEL: contiguous runs of operations per device, sized by the devices'
    memory; the exported blob restores the same partition without querying the devices."""
    class Stage(CpuPlugin):
        device_name = "STAGE_A"
    class StageB(CpuPlugin):
        device_name = "STAGE_B"
    core.register_plugin(Stage, "STAGE_A")
    core.register_plugin(StageB, "STAGE_B")
    rng = np.random.default_rng(5)
    x = ops.parameter([2, 32], "f32", "x")
    h = x
    ws = []
    for i in range(8):
        w = rng.standard_normal((32, 32)).astype(np.float32) * 0.2
        ws.append(w)
        h = ops.relu(ops.matmul(h, w, False, True, name="fc%d" % i), name="act%d" % i)
    m = Model([h], [x], "deep")
    xin = rng.standard_normal((2, 32)).astype(np.float32)
    want = xin
    for w in ws:
        want = np.maximum(want @ w.T, 0)
    cfg = {props.hint.model_distribution_policy: "PIPELINE_PARALLEL",
           props.device.properties: {"STAGE_A": {"PIPELINE_MEMORY_BYTES": 3}, "STAGE_B": {"PIPELINE_MEMORY_BYTES": 1}}}
    cm = core.compile_model(m, "HETERO:STAGE_A,STAGE_B", cfg)
    assert [s.device for s in cm.subs] == ["STAGE_A", "STAGE_B"]          # one cut, devices in list order
    on_a = sum(1 for k, v in cm.affinity.items() if v == "STAGE_A" and k.startswith("fc"))
    assert on_a == 6                                                     # 3 : 1 of the eight equal layers
    np.testing.assert_allclose(cm(xin)[0], want, rtol=1e-4, atol=1e-5)
    # equal memory: an even split
    cm_eq = core.compile_model(m, "HETERO:STAGE_A,STAGE_B", {props.hint.model_distribution_policy: "PIPELINE_PARALLEL"})
    assert sum(1 for k, v in cm_eq.affinity.items() if v == "STAGE_A" and k.startswith("fc")) == 4
    # export / import keeps the partition
    blob = cm.export_model()
    cm2 = core.import_model(blob, "HETERO:STAGE_A,STAGE_B")
    assert cm2.affinity == cm.affinity and [s.device for s in cm2.subs] == ["STAGE_A", "STAGE_B"]
    np.testing.assert_allclose(cm2(xin)[0], want, rtol=1e-4, atol=1e-5)


def test_auto_batching(core):
    m = mlp()
    cm = core.compile_model(m, "BATCH:CPU(4)", {props.auto_batch_timeout: 200})
    assert cm.get_property(props.optimal_number_of_infer_requests) >= 4
    reqs = [cm.create_infer_request() for _ in range(4)]
    xs = [np.random.default_rng(i).standard_normal((1, 16)).astype(np.float32) for i in range(4)]
    for r, x in zip(reqs, xs):
        r.start_async({"x": x})
    for r, x in zip(reqs, xs):
        r.wait()
        np.testing.assert_allclose(r.results[0], ref(x), rtol=1e-4, atol=1e-4)
    assert cm.collector.num_batched_runs == 1
    # a lone request is served after the timeout
    np.testing.assert_allclose(cm(xs[0])[0], ref(xs[0]), rtol=1e-4, atol=1e-4)
    assert cm.collector.num_batched_runs == 2


def test_shutdown_runs_callbacks_in_reverse_order_once(core):
    order = []
    h1 = ov.register_shutdown_callback(lambda: order.append("first"), "first")
    ov.register_shutdown_callback(lambda: (_ for _ in ()).throw(RuntimeError("boom")), "failing")
    ov.register_shutdown_callback(lambda: order.append("last"), "last")
    h4 = ov.register_shutdown_callback(lambda: order.append("removed"), "removed")
    assert ov.unregister_shutdown_callback(h4) and not ov.unregister_shutdown_callback(h4)
    cm = core.compile_model(mlp(), "BATCH:CPU(2)", {props.auto_batch_timeout: 50})     # owns a collector thread
    thread = cm.collector.thread
    assert thread.is_alive()
    ran = ov.shutdown()
    assert order == ["last", "first"] and "failing" in ran and "BATCH collector thread" in ran
    thread.join(timeout=5)
    assert not thread.is_alive()
    assert ov.shutdown() == [] and h1 > 0


def test_cache_encryption_lock_and_mmap(core, tmp_path):
    """Entries pass through the user's (encrypt, decrypt) pair; a plain entry is read through a memory mapping; threads
    that ask for the same entry take turns, so one of them compiles and the others import."""
    import threading
    x = ops.parameter([2, 4], "f32", "x")
    m = Model([ops.relu(ops.add(x, np.float32(1)))], [x], "enc")
    cache = str(tmp_path / "c1")
    key = 0x5A
    enc = (lambda b: bytes(v ^ key for v in b), lambda b: bytes(v ^ key for v in b))
    a = core.compile_model(m, "CPU", {props.cache_dir: cache, props.cache_encryption_callbacks: enc})
    entry = [f for f in os.listdir(cache) if f.endswith(".blob")]
    assert len(entry) == 1 and not open(os.path.join(cache, entry[0]), "rb").read().startswith(b"OVB200BL")
    b = core.compile_model(m, "CPU", {props.cache_dir: cache, props.cache_encryption_callbacks: enc})
    assert a.get_property(props.loaded_from_cache) is False and b.get_property(props.loaded_from_cache) is True
    xin = np.array([[-3, 0, 1, 2], [5, -1, -2, 0]], np.float32)
    np.testing.assert_array_equal(b([xin])[0], np.maximum(xin + 1, 0))
    # reading the encrypted entry without the callbacks cannot work: it is dropped and the model compiled again
    c = core.compile_model(m, "CPU", {props.cache_dir: cache})
    assert c.get_property(props.loaded_from_cache) is False
    # plain entries, several threads at once
    cache2 = str(tmp_path / "c2")
    got = []
    def worker():
        got.append(core.compile_model(m, "CPU", {props.cache_dir: cache2}).get_property(props.loaded_from_cache))
    ts = [threading.Thread(target=worker) for _ in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert sorted(got) == [False, True, True, True]
    assert len([f for f in os.listdir(cache2) if f.endswith(".blob")]) == 1
