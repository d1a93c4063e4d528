"""Policy devices that wrap hardware devices: AUTO, MULTI, HETERO and BATCH.

* ``AUTO[:dev,…]``   picks one device from a priority list by performance hint and falls back to the next when a
  compile or an inference fails (src/plugins/auto: plugin.cpp, auto_schedule.cpp, cumulative_schedule.cpp).
  ``PERFORMANCE_HINT=CUMULATIVE_THROUGHPUT`` turns it into MULTI.
* ``MULTI:dev,…``    compiles on every device and deals requests round-robin.
* ``HETERO:dev,…``   assigns every operation to the first device in the list that supports it (``query_model``),
  cuts the graph into per-device sub-models and runs them in dependency order
  (src/plugins/hetero/src/subgraph_collector.cpp, graph splitting; sync_infer_request.cpp).
* ``BATCH:dev(N)``   gathers up to N single requests (or waits ``AUTO_BATCH_TIMEOUT`` ms) and runs them as one
  batched inference (src/plugins/auto_batch/src/{plugin,compiled_model,sync_infer_request}.cpp).
"""
from __future__ import annotations

import re
import threading
import time
from typing import Dict, List, Optional

import numpy as np

from .. import _ovcore as _c
from .. import properties as props
from .._graph import Model, Node, Output, parameter, result
from .._tensor import Tensor
from .._types import PartialShape
from .core import CompiledModel, InferRequest, Plugin, ProfilingInfo, VariableState


def _split_devices(text: str) -> List[str]:
    return [d.strip() for d in re.split(r",(?![^()]*\))", text or "") if d.strip()]


def _default_priorities(core) -> List[str]:
    names = []
    for n in ("CUDA", "CPU"):
        try:
            if core._get_plugin(n).available_device_ids():
                names.append(n)
        except Exception:   # noqa: BLE001 - unavailable device
            pass
    return names or ["CPU"]


def _device_config(cfg: dict, device: str) -> dict:
    """Config to pass down to ``device``: common hints plus its DEVICE_PROPERTIES entry."""
    passthrough = (props.hint.performance_mode, props.hint.num_requests, props.enable_profiling, props.hint.inference_precision,
                   props.hint.execution_mode, props.num_streams, props.inference_num_threads)
    out = {k: v for k, v in cfg.items() if k in passthrough}
    sub = cfg.get(props.device.properties) or {}
    out.update(sub.get(device.split(".")[0].split("(")[0], {}))
    return out


# ---------------------------------------------------------------------------------------------- AUTO / MULTI
class _DelegatingCompiledModel(CompiledModel):
    """Compiled model made of compiled models on real devices; requests delegate to one of them."""

    def __init__(self, plugin, model, config, compiled: List[CompiledModel], devices: List[str], candidates=None):
        super().__init__(plugin, model, config, compiled[0].runtime_model)
        self.compiled, self.devices = compiled, devices
        self._candidates = candidates or []      # devices still available for runtime fallback (AUTO)
        self._rr = 0
        self._lock = threading.Lock()

    def optimal_number_of_infer_requests(self) -> int:
        return sum(c.optimal_number_of_infer_requests() for c in self.compiled)

    def get_property(self, name):
        if str(name) == props.execution_devices:
            return list(self.devices)
        if str(name) == props.device.priorities:
            return ",".join(self.devices + self._candidates)
        try:
            return super().get_property(name)
        except RuntimeError:
            return self.compiled[0].get_property(name)

    def _pick(self) -> int:
        with self._lock:
            i = self._rr % len(self.compiled)
            self._rr += 1
            return i

    def _make_runner(self, request: InferRequest):
        state = {"idx": self._pick(), "inner": None}

        def inner():
            if state["inner"] is None:
                state["inner"] = self.compiled[state["idx"]].create_infer_request()
            return state["inner"]
        request._delegate = inner

        def run(req: InferRequest, ins: List[Tensor]) -> List[Tensor]:
            while True:
                r = inner()
                try:
                    for i, t in enumerate(ins):
                        r._in[i] = t
                    outs = r._runner(r, ins)
                    req._profile = r._profile
                    return outs
                except Exception:   # noqa: BLE001 - runtime fallback to the next candidate device
                    if not self._fallback(state):
                        raise
        return run

    def _fallback(self, state) -> bool:
        if not self.config.get(props.intel_auto.enable_runtime_fallback, True):
            return False
        with self._lock:
            while self._candidates:
                dev = self._candidates.pop(0)
                try:
                    cm = self.plugin.core.compile_model(self.model, dev, _device_config(self.config, dev))
                except Exception:   # noqa: BLE001
                    continue
                self.compiled.append(cm)
                self.devices.append(dev)
                state["idx"], state["inner"] = len(self.compiled) - 1, None
                return True
        return False

    def _variables(self, request):
        return request._delegate().query_state()


class AutoPlugin(Plugin):
    device_name = "AUTO"
    description = "Automatic device selection"

    def supported_properties(self):
        return super().supported_properties() + [props.device.priorities, props.device.properties, props.hint.model_priority,
                                                 props.intel_auto.enable_startup_fallback, props.intel_auto.enable_runtime_fallback,
                                                 props.intel_auto.schedule_policy, props.intel_auto.device_bind_buffer, props.log.level]

    def capabilities(self):
        return ["FP32", "FP16", "BF16", "INT8"]

    def _priorities(self, cfg) -> List[str]:
        devs = _split_devices(cfg.get(props.device.priorities, ""))
        exclude = [d[1:] for d in devs if d.startswith("-")]
        devs = [d for d in devs if not d.startswith("-")]
        if not devs:
            devs = [d for d in _default_priorities(self.core) if d not in exclude]
        return devs

    def compile_model(self, model: Model, config: dict) -> CompiledModel:
        cfg = self.merged_config(config)
        devs = self._priorities(cfg)
        if str(cfg.get(props.hint.performance_mode)) == "CUMULATIVE_THROUGHPUT":
            return MultiPlugin.compile_on_all(self, model, cfg, devs)
        errors = []
        for i, dev in enumerate(devs):
            try:
                cm = self.core.compile_model(model, dev, _device_config(cfg, dev))
            except Exception as e:   # noqa: BLE001 - try the next device of the list
                errors.append("%s: %s" % (dev, e))
                continue
            return _DelegatingCompiledModel(self, model, cfg, [cm], [dev], candidates=devs[i + 1:])
        raise RuntimeError("[AUTO] no device could compile the model: " + "; ".join(errors))

    def query_model(self, model, config):
        cfg = self.merged_config(config)
        for dev in self._priorities(cfg):
            try:
                return self.core.query_model(model, dev, _device_config(cfg, dev))
            except Exception:   # noqa: BLE001
                continue
        return {}


class MultiPlugin(AutoPlugin):
    device_name = "MULTI"
    description = "Multi-device round-robin execution"

    @staticmethod
    def compile_on_all(plugin, model, cfg, devs) -> CompiledModel:
        compiled, used, errors = [], [], []
        for dev in devs:
            try:
                compiled.append(plugin.core.compile_model(model, dev, _device_config(cfg, dev)))
                used.append(dev)
            except Exception as e:   # noqa: BLE001
                errors.append("%s: %s" % (dev, e))
        if not compiled:
            raise RuntimeError("[%s] no device could compile the model: %s" % (plugin.device_name, "; ".join(errors)))
        return _DelegatingCompiledModel(plugin, model, cfg, compiled, used)

    def compile_model(self, model, config):
        cfg = self.merged_config(config)
        return self.compile_on_all(self, model, cfg, self._priorities(cfg))


# ---------------------------------------------------------------------------------------------- HETERO
class _SubModel:
    def __init__(self, device: str, model: Model, input_sources: List[tuple], output_keys: List[tuple]):
        self.device, self.model = device, model
        self.input_sources = input_sources      # per sub-model input: ("param", index) | ("value", (node id, port))
        self.output_keys = output_keys          # per sub-model output: (node id, port) of the original graph
        self.compiled: Optional[CompiledModel] = None


def split_by_affinity(model: Model, affinity: Dict[str, str]) -> List[_SubModel]:
    """Cut ``model`` into sub-models so that every sub-model runs on one device.

    Each operation gets a stage: the largest producer stage, plus one when the producer runs on another device.
    Operations with the same (stage, device) form a sub-model; sub-models are returned in stage order, so each one
    only consumes model inputs and outputs of earlier sub-models.
    """
    ops = model.get_ops()
    params = model.get_parameters()
    stage: Dict[Node, int] = {}
    dev_of: Dict[Node, str] = {}
    for n in ops:
        t = n.get_type_name()
        if t in ("Parameter", "Constant", "Result"):
            continue
        d = affinity.get(n.get_friendly_name())
        if d is None:
            raise RuntimeError("[HETERO] no device supports operation %r" % n)
        s = 0
        for src in n.input_values():
            p = src.get_node()
            if p in stage:
                s = max(s, stage[p] if dev_of[p] == d else stage[p] + 1)
        stage[n], dev_of[n] = s, d
    groups: Dict[tuple, List[Node]] = {}
    for n in ops:
        if n in stage:
            groups.setdefault((stage[n], dev_of[n]), []).append(n)
    result_sources = {r.input_value(0) for r in model.get_results()}
    subs = []
    for key in sorted(groups):
        members = groups[key]
        member_set = set(members)
        new_of: Dict[Output, Output] = {}
        sub_params, input_sources = [], []

        def map_input(src: Output) -> Output:
            if src in new_of:
                return new_of[src]
            p = src.get_node()
            if p.get_type_name() == "Constant":
                c = p.clone_with_new_inputs([])
                new_of[src] = c.output(0)
                return new_of[src]
            np_ = parameter(src.get_partial_shape(), src.get_element_type(), p.get_friendly_name() if p.get_type_name() == "Parameter" else "")
            if src.get_names():
                np_.output(0).set_names(src.get_names())
            sub_params.append(np_)
            input_sources.append(("param", params.index(p)) if p.get_type_name() == "Parameter" else ("value", (p._n.id, src.get_index())))
            new_of[src] = np_.output(0)
            return new_of[src]

        for n in members:
            clone = n.clone_with_new_inputs([map_input(s) for s in n.input_values()])
            clone.set_friendly_name(n.get_friendly_name())
            for i in range(n.get_output_size()):
                new_of[n.output(i)] = clone.output(i)
        sub_results, output_keys = [], []
        for n in members:
            for i in range(n.get_output_size()):
                o = n.output(i)
                external = o in result_sources or any(u.get_node() not in member_set for u in o.get_target_inputs())
                if external:
                    sub_results.append(result(new_of[o]))
                    output_keys.append((n._n.id, i))
        sm = Model(sub_results, sub_params, "%s_sub%d_%s" % (model.get_friendly_name(), len(subs), key[1]))
        subs.append(_SubModel(key[1], sm, input_sources, output_keys))
    return subs


class HeteroCompiledModel(CompiledModel):
    def __init__(self, plugin, model, config, subs: List[_SubModel], split_model: Model):
        super().__init__(plugin, model, config)
        self.subs = subs
        params = split_model.get_parameters()     # node ids in the sub-model maps refer to the model that was split
        self._result_sources = []
        for r in split_model.get_results():
            src = r.input_value(0)
            p = src.get_node()
            self._result_sources.append(("param", params.index(p)) if p.get_type_name() == "Parameter" else ("value", (p._n.id, src.get_index())))

    def get_property(self, name):
        if str(name) == props.execution_devices:
            return sorted({s.device for s in self.subs})
        return super().get_property(name)

    def export_model(self, stream=None) -> bytes:
        from .core import ModelBlob, __version__
        xml, weights = _c.serialize(self.model._m)
        header = {"device": self.plugin.device_name, "runtime": __version__, "affinity": dict(getattr(self, "affinity", {}) or {}),
                  "config": {k: v for k, v in self.config.items() if isinstance(v, (str, int, float, bool))}}
        data = ModelBlob(header, xml.decode(), weights).to_bytes()
        if stream is not None:
            stream.write(data)
        return data

    def _make_runner(self, request):
        inner = [s.compiled.create_infer_request() for s in self.subs]

        def run(req, ins):
            values = {}
            prof = []
            for s, r in zip(self.subs, inner):
                sub_in = [ins[src[1]] if src[0] == "param" else values[src[1]] for src in s.input_sources]
                for i, t in enumerate(sub_in):
                    r._in[i] = t
                outs = r._runner(r, sub_in)
                prof.extend(r._profile)
                for k, t in zip(s.output_keys, outs):
                    values[k] = t
            req._profile = prof
            return [ins[src[1]] if src[0] == "param" else values[src[1]] for src in self._result_sources]
        return run


class HeteroPlugin(Plugin):
    device_name = "HETERO"
    description = "Heterogeneous execution across devices"

    def supported_properties(self):
        return super().supported_properties() + [props.device.priorities, props.device.properties, props.hint.model_distribution_policy]

    def _device_memory(self, dev: str, cfg: dict) -> float:
        """Memory a device offers to the pipeline split: its DEVICE_PROPERTIES entry "PIPELINE_MEMORY_BYTES" when given,
        else what the device reports (GPU_DEVICE_TOTAL_MEM_SIZE), else an equal share."""
        sub = (cfg.get(props.device.properties) or {}).get(dev.split(".")[0].split("(")[0], {})
        if "PIPELINE_MEMORY_BYTES" in sub:
            return float(sub["PIPELINE_MEMORY_BYTES"])
        for key in ("GPU_DEVICE_TOTAL_MEM_SIZE", "DEVICE_TOTAL_MEM_SIZE"):
            try:
                v = self.core.get_property(dev, key)
                if v:
                    return float(v)
            except Exception:   # noqa: BLE001 - the device has no such property
                pass
        return 1.0

    def _assign_pipeline(self, model: Model, cfg: dict, devs: List[str], supported: Dict[str, set]) -> Dict[str, str]:
        """``MODEL_DISTRIBUTION_POLICY = PIPELINE_PARALLEL``: the operations, in topological order, are cut into one
        contiguous run per device so that every device receives a share of the constant (weight) bytes in proportion to
        its memory; an operation that its device cannot run goes to the first device of the list that can. The activations
        cross a device border once per cut (src/plugins/hetero/src/plugin.cpp, get_model_distribution_policy and the
        memory-ratio walk of query_model_update)."""
        mem = [self._device_memory(d, cfg) for d in devs]
        if all(m == 1.0 for m in mem):
            mem = [1.0] * len(devs)
        ops_ = [n for n in model.get_ordered_ops() if n.get_type_name() not in ("Parameter", "Constant", "Result")]
        weight = []
        for n in ops_:
            w = 0
            for src in n.input_values():
                p = src.get_node()
                if p.get_type_name() == "Convert" and p.input_value(0).get_node().get_type_name() == "Constant":
                    p = p.input_value(0).get_node()
                if p.get_type_name() == "Constant":
                    ps = src.get_partial_shape() if p is src.get_node() else p.output(0).get_partial_shape()
                    cnt = 1
                    for d in ps:
                        cnt *= int(d.get_length())
                    w += cnt * max(1, p.output(0).get_element_type().bitwidth) // 8
            weight.append(max(w, 1))
        total, acc, di = float(sum(weight)), 0.0, 0
        bounds = []
        run = 0.0
        for m_ in mem:
            run += m_ / sum(mem)
            bounds.append(run * total)
        affinity: Dict[str, str] = {}
        for n, w in zip(ops_, weight):
            while di < len(devs) - 1 and acc + w / 2.0 > bounds[di]:
                di += 1
            acc += w
            name = n.get_friendly_name()
            a = n.rt_info.get("affinity")
            if a:
                affinity[name] = str(a)
            elif name in supported[devs[di]]:
                affinity[name] = devs[di]
            else:
                for d in devs:
                    if name in supported[d]:
                        affinity[name] = d
                        break
        return affinity

    def _assign(self, model: Model, cfg: dict) -> Dict[str, str]:
        devs = _split_devices(cfg.get(props.device.priorities, ""))
        if not devs:
            raise RuntimeError("[HETERO] needs a device list: HETERO:CUDA,CPU")
        if "PIPELINE_PARALLEL" in str(cfg.get(props.hint.model_distribution_policy, "") or ""):
            supported = {}
            for dev in devs:
                try:
                    supported[dev] = set(self.core.query_model(model, dev, _device_config(cfg, dev)))
                except Exception:   # noqa: BLE001 - a device that cannot answer supports nothing
                    supported[dev] = set()
            return self._assign_pipeline(model, cfg, devs, supported)
        # a user-given per-node "affinity" rt_info wins over the automatic assignment
        affinity: Dict[str, str] = {}
        for n in model.get_ops():
            a = n.rt_info.get("affinity")
            if a:
                affinity[n.get_friendly_name()] = str(a)
        for dev in devs:
            try:
                supported = self.core.query_model(model, dev, _device_config(cfg, dev))
            except Exception:   # noqa: BLE001 - a device that cannot answer supports nothing
                continue
            for name in supported:
                affinity.setdefault(name, dev)
        return affinity

    def query_model(self, model, config):
        return self._assign(model, self.merged_config(config))

    def compile_model(self, model, config, affinity: Optional[Dict[str, str]] = None):
        cfg = self.merged_config(config)
        work = model.clone()
        affinity = dict(affinity) if affinity is not None else self._assign(work, cfg)
        subs = split_by_affinity(work, affinity)
        for s in subs:
            s.compiled = self.core.compile_model(s.model, s.device, _device_config(cfg, s.device))
        cm = HeteroCompiledModel(self, model, cfg, subs, work)
        cm.affinity = affinity
        return cm

    def import_model(self, blob, config):
        """The exported blob carries the partition (operation -> device): the import compiles the same sub-models on the
        same devices without asking the devices again (src/plugins/hetero/src/compiled_model.cpp, the constructor
        from a stream)."""
        model = Model._wrap(_c.deserialize(blob.xml, np.frombuffer(blob.weights, dtype=np.uint8)))
        cfg = dict(blob.header.get("config", {}))
        cfg.update(config)
        return self.compile_model(model, cfg, affinity=blob.header.get("affinity"))


# ---------------------------------------------------------------------------------------------- BATCH
class _BatchCollector:
    """Gathers single requests into one batched inference."""

    def __init__(self, compiled_batched: CompiledModel, batch: int, timeout_ms: float, batched_inputs: List[bool], batched_outputs: List[bool]):
        self.batch, self.timeout = batch, timeout_ms / 1000.0
        self.request = compiled_batched.create_infer_request()
        self.batched_inputs, self.batched_outputs = batched_inputs, batched_outputs
        self.pending: List[dict] = []
        self.cv = threading.Condition()
        self.stop = False
        self.num_batched_runs = 0
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()
        self._register_shutdown()

    def _register_shutdown(self) -> None:
        import weakref
        from ..utils.shutdown import register_shutdown_callback
        ref = weakref.ref(self)
        register_shutdown_callback(lambda: ref() and ref().close(), "BATCH collector thread")

    def submit(self, ins: List[Tensor]) -> List[Tensor]:
        item = {"ins": ins, "done": threading.Event(), "outs": None, "err": None}
        with self.cv:
            self.pending.append(item)
            self.cv.notify_all()
        item["done"].wait()
        if item["err"] is not None:
            raise item["err"]
        return item["outs"]

    def _loop(self):
        while True:
            with self.cv:
                while not self.pending and not self.stop:
                    self.cv.wait()
                if self.stop:
                    return
                deadline = time.monotonic() + self.timeout
                while len(self.pending) < self.batch and not self.stop:
                    left = deadline - time.monotonic()
                    if left <= 0:
                        break
                    self.cv.wait(left)
                items, self.pending = self.pending[:self.batch], self.pending[self.batch:]
            try:
                self._run(items)
            except Exception as e:   # noqa: BLE001 - delivered to every request of the batch
                for it in items:
                    it["err"] = e
            for it in items:
                it["done"].set()

    def _run(self, items):
        n = len(items)
        ins = []
        for i, batched in enumerate(self.batched_inputs):
            if not batched:
                ins.append(items[0]["ins"][i])
                continue
            arrs = [it["ins"][i].data for it in items]
            if n < self.batch:   # pad the tail of an incomplete batch with copies of the last item
                arrs = arrs + [arrs[-1]] * (self.batch - n)
            ins.append(Tensor(np.concatenate(arrs, axis=0)))
        r = self.request
        for i, t in enumerate(ins):
            r._in[i] = t
        outs = r._runner(r, ins)
        self.num_batched_runs += 1
        for k, it in enumerate(items):
            res = []
            for o, batched in zip(outs, self.batched_outputs):
                if batched:
                    per = o.shape[0] // self.batch
                    res.append(Tensor(np.ascontiguousarray(o.data[k * per:(k + 1) * per])))
                else:
                    res.append(o)
            it["outs"] = res

    def close(self):
        with self.cv:
            self.stop = True
            self.cv.notify_all()


class BatchCompiledModel(CompiledModel):
    def __init__(self, plugin, model, config, collector: _BatchCollector, batched: CompiledModel):
        config = dict(config)
        config[props.num_streams] = collector.batch * max(1, batched.optimal_number_of_infer_requests())   # requests wait inside a stream
        super().__init__(plugin, model, config, batched.runtime_model)
        self.collector, self.batched = collector, batched

    def optimal_number_of_infer_requests(self) -> int:
        return self.collector.batch * max(1, self.batched.optimal_number_of_infer_requests())

    def get_property(self, name):
        if str(name) == props.execution_devices:
            return self.batched.get_property(name)
        return super().get_property(name)

    def _make_runner(self, request):
        return lambda req, ins: self.collector.submit(ins)

    def __del__(self):
        try:
            self.collector.close()
        except Exception:   # noqa: BLE001
            pass


class BatchPlugin(Plugin):
    device_name = "BATCH"
    description = "Automatic batching"

    def supported_properties(self):
        return super().supported_properties() + [props.device.priorities, props.auto_batch_timeout, props.device.properties]

    def default_config(self):
        d = super().default_config()
        d[props.auto_batch_timeout] = 1000
        return d

    def compile_model(self, model: Model, config: dict) -> CompiledModel:
        cfg = self.merged_config(config)
        spec = cfg.get(props.device.priorities, "")
        m = re.match(r"^([^()]+)(?:\((\d+)\))?$", spec.strip())
        if not m:
            raise RuntimeError("[BATCH] device string must look like BATCH:CUDA(8)")
        dev, batch = m.group(1), int(m.group(2) or 0)
        if batch <= 0:
            try:
                batch = int(self.core.get_property(dev, props.optimal_batch_size))
            except Exception:   # noqa: BLE001
                batch = 8
        batched_inputs, shapes = [], {}
        for i, p in enumerate(model.inputs):
            ps = p.get_partial_shape()
            if ps.is_dynamic:
                raise RuntimeError("[BATCH] dynamic models are not batched automatically")
            is_b = len(ps) > 0 and ps[0].get_length() == 1
            batched_inputs.append(is_b)
            if is_b:
                shapes[i] = [batch] + [d.get_length() for d in ps[1:]]
        if not any(batched_inputs):
            raise RuntimeError("[BATCH] the model has no input with batch dimension 1")
        big = model.clone()
        big.reshape(shapes)
        batched_outputs = []
        for o_small, o_big in zip(model.outputs, big.outputs):
            s, b = o_small.get_shape(), o_big.get_shape()
            batched_outputs.append(len(s) > 0 and len(b) > 0 and b[0] == s[0] * batch and list(b[1:]) == list(s[1:]))
        compiled = self.core.compile_model(big, dev, _device_config(cfg, dev))
        collector = _BatchCollector(compiled, batch, float(cfg.get(props.auto_batch_timeout, 1000)), batched_inputs, batched_outputs)
        return BatchCompiledModel(self, model, cfg, collector, compiled)

    def query_model(self, model, config):
        cfg = self.merged_config(config)
        dev = re.sub(r"\(\d+\)$", "", cfg.get(props.device.priorities, "").strip())
        return self.core.query_model(model, dev, {})


class ProxyPlugin(Plugin):
    """One device name in front of several plugins, with a fallback order.

    The proxy numbers the devices of its plugins consecutively ("GPU.0", "GPU.1" may belong to different plugins),
    forwards every call to the plugin that owns the addressed device and, when that plugin cannot compile the model,
    tries the remaining plugins in order. Role of src/plugins/proxy/src/plugin.cpp (alias / fallback / priority
    configuration of src/plugins/proxy/dev_api/openvino/proxy/properties.hpp).
    """

    description = "proxy"

    def __init__(self, core, alias: str, order: List[str]):
        super().__init__(core)
        self.device_name = alias
        self.order = list(order)

    def add_fallback(self, device: str, priority: Optional[int] = None) -> None:
        if device not in self.order:
            self.order.insert(len(self.order) if priority is None else max(0, min(priority, len(self.order))), device)

    def _devices(self) -> List[tuple]:
        out = []
        for name in self.order:
            try:
                ids = self.core._get_plugin(name).available_device_ids()
            except Exception:
                continue
            out += [(name, i) for i in ids]
        return out

    def available_device_ids(self) -> List[str]:
        return [str(i) for i in range(len(self._devices()))]

    def _target(self, config: dict) -> List[tuple]:
        """(plugin, device id) candidates: the addressed device first, then one device of every later plugin."""
        devs = self._devices()
        if not devs:
            raise RuntimeError("[%s] none of the devices behind the proxy is available: %s" % (self.device_name, self.order))
        idx = int(str(config.get(props.device.id, self.config.get(props.device.id, "")) or 0))
        if idx >= len(devs):
            raise RuntimeError("[%s] no device with id %d (have %d)" % (self.device_name, idx, len(devs)))
        first = devs[idx]
        rest = []
        for name in self.order[self.order.index(first[0]) + 1:]:
            cand = [d for d in devs if d[0] == name]
            if cand:
                rest.append(cand[0])
        return [first] + rest

    def supported_properties(self) -> List[str]:
        return super().supported_properties() + ["PROXY_FALLBACK_ORDER"]

    def get_property(self, name: str, arguments: Optional[dict] = None):
        if name == "PROXY_FALLBACK_ORDER":
            return list(self.order)
        if name in (props.supported_properties, props.available_devices):
            return super().get_property(name, arguments)
        plugin, dev_id = self._target(dict(arguments or {}))[0]
        args = dict(arguments or {})
        args[props.device.id] = dev_id
        return self.core._get_plugin(plugin).get_property(name, args)

    def set_property(self, config: dict) -> None:
        for k, v in config.items():
            if k == props.device.id:
                self.config[k] = v
                continue
            for name in self.order:
                try:
                    self.core._get_plugin(name).set_property({k: v})
                except RuntimeError:
                    pass

    def compile_model(self, model: Model, config: dict):
        errors = []
        cfg = {k: v for k, v in config.items() if k != props.device.id}
        for plugin, dev_id in self._target(config):
            try:
                sub = dict(cfg)
                if dev_id not in ("", None):
                    sub[props.device.id] = dev_id
                return self.core._get_plugin(plugin).compile_model(model, sub)
            except Exception as e:          # the next plugin in the fallback order gets its chance
                errors.append("%s: %s" % (plugin, e))
        raise RuntimeError("[%s] no plugin behind the proxy could compile the model: %s" % (self.device_name, "; ".join(errors)))

    def query_model(self, model, config):
        plugin, _ = self._target(config)[0]
        return {k: self.device_name for k in self.core._get_plugin(plugin).query_model(model, {}).keys()}

    def import_model(self, blob, config):
        plugin, _ = self._target(config)[0]
        return self.core._get_plugin(plugin).import_model(blob, config)


def register_proxy(core, alias: str, devices: List[str]) -> ProxyPlugin:
    """Put ``devices`` (plugin names, highest priority first) behind the device name ``alias``."""
    existing = core._plugins.get(alias)
    if isinstance(existing, ProxyPlugin):
        for d in devices:
            existing.add_fallback(d)
        return existing
    core._factories[alias] = lambda c, a=alias, d=list(devices): ProxyPlugin(c, a, d)
    core._plugins.pop(alias, None)
    return core._get_plugin(alias)


def register(core) -> None:
    core.register_plugin_factory("AUTO", AutoPlugin)
    core.register_plugin_factory("MULTI", MultiPlugin)
    core.register_plugin_factory("HETERO", HeteroPlugin)
    core.register_plugin_factory("BATCH", BatchPlugin)
