"""NPUW-style compilation on top of any device: repeated blocks of a model (the layers of a transformer) are found by
structure, folded into ONE function body that is compiled once, and called once per block with that block's weights;
weights go through a per-device *weights bank* so that equal constants (tied embeddings, position tables, the prefill
and the generate variant of one network) are held once.

* ``find_repeated_blocks(model)``  - the periodic region of the operation list and a node-by-node isomorphism check;
* ``fold_repeated_blocks(model)``  - rewrites the model: every block becomes a ``FunctionCall`` node (inputs: what the
  block reads from outside, then its weights in body order) that refers to the shared body;
* ``WeightsBank``                  - content-addressed constants per device; ``dedupe_constants(model)`` uses it;
* ``NpuwPlugin`` (device ``NPUW``) - ``compile_model(model, "NPUW", {"NPUW_DEVICES": "CPU"})``: bank, fold, then compile
  on the backing device. ``FunctionCall`` evaluates on the host through the body compiled on the backing device and on
  the CUDA device through the body's own graph program.

Reference: src/plugins/intel_npu/src/plugin/npuw/partitioning/online/ (repeated-block detection by node meta-description),
partitioning/partitioning.cpp (function folding, closures), weights_bank.cpp, compiled_model.cpp.
"""
from __future__ import annotations

import hashlib
import itertools
import threading
from typing import Dict, List, Optional, Tuple

import numpy as np

from .. import properties as props
from .._graph import Model, Node, Output, constant, make_op, parameter, result
from .._op_base import register_op
from .._types import PartialShape
from .core import CompiledModel, Plugin

_FUNCS: Dict[int, "FoldedFunction"] = {}
_next_id = itertools.count(1)
_registered = False


# ------------------------------------------------------------------------------------------------- weights bank
class WeightsBank:
    """Constants by content. ``intern`` returns the array already held for the same bytes, shape and type."""
    _banks: Dict[str, "WeightsBank"] = {}
    _lock = threading.Lock()

    def __init__(self, device: str):
        self.device = device
        self._store: Dict[tuple, np.ndarray] = {}
        self.hits = 0
        self.bytes_saved = 0

    @classmethod
    def for_device(cls, device: str) -> "WeightsBank":
        with cls._lock:
            b = cls._banks.get(device)
            if b is None:
                b = cls._banks[device] = WeightsBank(device)
            return b

    @staticmethod
    def key_of(arr: np.ndarray, et: str) -> tuple:
        a = np.ascontiguousarray(arr)
        return (et, tuple(a.shape), hashlib.sha1(a.view(np.uint8).reshape(-1)).hexdigest())

    def intern(self, arr: np.ndarray, et: str) -> Tuple[np.ndarray, bool]:
        k = self.key_of(arr, et)
        with self._lock:
            have = self._store.get(k)
            if have is not None:
                self.hits += 1
                self.bytes_saved += have.nbytes
                return have, True
            self._store[k] = arr
            return arr, False

    def __len__(self):
        return len(self._store)


def dedupe_constants(model: Model, bank: Optional[WeightsBank] = None, min_bytes: int = 64) -> int:
    """Constants with equal content become one node (and one array in the bank); returns how many were removed."""
    first: Dict[tuple, Node] = {}
    removed = 0
    for n in model.get_ops():
        if n.get_type_name() != "Constant":
            continue
        et = str(n.get_output_element_type(0))
        if et == "string":
            continue
        data = np.asarray(n.get_data())
        if data.nbytes < min_bytes:
            continue
        key = WeightsBank.key_of(data, et)
        if bank is not None:
            bank.intern(data, et)
        keep = first.get(key)
        if keep is None:
            first[key] = n
            continue
        for inp in list(n.output(0).get_target_inputs()):
            inp.replace_source_output(keep.output(0))
        removed += 1
    return removed


# ------------------------------------------------------------------------------------------------- repeated blocks
_NEVER_FOLDED = ("ReadValue", "Assign", "If", "Loop", "TensorIterator", "Subgraph", "FunctionCall")


def _attrs_key(n: Node) -> str:
    return repr(sorted((k, repr(v)) for k, v in n.get_attributes().items()))


def _signature(n: Node) -> tuple:
    """Meta-description of a node: its type, attributes, result types / ranks and what kind of value feeds each input.
    Operations that own state or a body never match another node: a shared function cannot hold them."""
    if n.get_type_name() in _NEVER_FOLDED:
        return ("unique", n.get_name())
    ins = []
    for k in range(n.get_input_size()):
        o = n.input_value(k)
        p = o.get_node()
        if p.get_type_name() == "Constant":
            ins.append(("c", str(o.get_element_type()), tuple(int(d) for d in o.get_shape())))
        else:
            ins.append(("n", o.get_index()))
    outs = tuple((str(o.get_element_type()), o.get_partial_shape().to_string()) for o in n.outputs())
    return (n.get_type_name(), n.get_version(), _attrs_key(n), tuple(ins), outs)


class Blocks:
    """R instances of a block of L operations: ``nodes[r][j]`` is operation j of instance r."""

    def __init__(self, nodes: List[List[Node]]):
        self.nodes = nodes
        self.count, self.length = len(nodes), len(nodes[0])


def find_repeated_blocks(model: Model, min_ops: int = 4, min_repeats: int = 2) -> Optional[Blocks]:
    ops_ = [n for n in model.get_ops() if n.get_type_name() not in ("Constant", "Parameter", "Result")]
    sig = [_signature(n) for n in ops_]
    ids: Dict[tuple, int] = {}
    seq = [ids.setdefault(s, len(ids)) for s in sig]
    n = len(seq)
    # candidate periods: distances between successive occurrences of each signature
    periods: Dict[int, int] = {}
    last: Dict[int, int] = {}
    for i, s in enumerate(seq):
        if s in last:
            d = i - last[s]
            periods[d] = periods.get(d, 0) + 1
        last[s] = i
    best = None
    for L, votes in sorted(periods.items(), key=lambda kv: -kv[1])[:8]:
        if L < min_ops:
            continue
        # longest run with seq[i] == seq[i + L]
        run_start, i = None, 0
        runs = []
        while i + L < n:
            if seq[i] == seq[i + L]:
                if run_start is None:
                    run_start = i
            elif run_start is not None:
                runs.append((run_start, i))
                run_start = None
            i += 1
        if run_start is not None:
            runs.append((run_start, n - L))
        for s, e in runs:
            reps = (e - s) // L + 1
            if reps >= min_repeats and (best is None or reps * L > best[2] * best[1]):
                best = (s, L, reps)
    if best is None:
        return None
    s, L, R = best
    # the run may start anywhere inside a block: try every alignment and keep the first that is a true isomorphism
    for shift in range(L):
        start = s + shift
        reps = R if start + R * L <= n else R - 1
        while reps >= min_repeats:
            nodes = [ops_[start + r * L:start + (r + 1) * L] for r in range(reps)]
            if _isomorphic(nodes):
                return Blocks(nodes)
            reps -= 1
    return None


def _isomorphic(nodes: List[List[Node]]) -> bool:
    L = len(nodes[0])
    pos = [{n: j for j, n in enumerate(blk)} for blk in nodes]
    for r in range(1, len(nodes)):
        for j in range(L):
            a, b = nodes[0][j], nodes[r][j]
            if a.get_type_name() != b.get_type_name() or a.get_input_size() != b.get_input_size() or _attrs_key(a) != _attrs_key(b):
                return False
            for k in range(a.get_input_size()):
                oa, ob = a.input_value(k), b.input_value(k)
                pa, pb = oa.get_node(), ob.get_node()
                ia, ib = pos[0].get(pa), pos[r].get(pb)
                if (ia is None) != (ib is None):
                    return False
                if ia is not None:
                    if ia != ib or oa.get_index() != ob.get_index():
                        return False
                    continue
                ca, cb = pa.get_type_name() == "Constant", pb.get_type_name() == "Constant"
                if ca != cb:
                    return False
                if ca and (str(oa.get_element_type()) != str(ob.get_element_type()) or list(oa.get_shape()) != list(ob.get_shape())):
                    return False
                if not ca and (str(oa.get_element_type()) != str(ob.get_element_type()) or oa.get_partial_shape().to_string() != ob.get_partial_shape().to_string()):
                    return False
    return True


class FoldedFunction:
    """The shared body of the folded blocks and its compiled forms per device."""

    def __init__(self, body: Model, n_external: int, n_closure: int):
        self.body, self.n_external, self.n_closure = body, n_external, n_closure
        self.device = "CPU"
        self.device_config: dict = {}
        self._compiled = None
        self._request_local = threading.local()
        self.calls = 0
        self.compiles = 0

    def request(self, core):
        if self._compiled is None:
            self._compiled = core.compile_model(self.body, self.device, self.device_config)
            self.compiles += 1
        r = getattr(self._request_local, "r", None)
        if r is None:
            r = self._request_local.r = self._compiled.create_infer_request()
        return r


def function_of(node: Node) -> FoldedFunction:
    return _FUNCS[int(node.get_attributes()["function_id"])]


def ensure_registered() -> None:
    global _registered
    if _registered:
        return

    def infer(node: Node):
        f = function_of(node)
        f.body.reshape({i: node.get_input_partial_shape(i) for i in range(f.n_external)})
        return [(r.get_input_element_type(0), r.get_input_partial_shape(0)) for r in f.body.get_results()]

    def evaluate(node: Node, ins):
        from .core import Core
        f = function_of(node)
        f.calls += 1
        req = f.request(Core())
        res = req.infer(list(ins))
        return [res[i] for i in range(len(f.body.get_results()))]

    register_op("FunctionCall", infer, evaluate, version="NPUWOpset", attrs={"function_id": 0})
    _registered = True


def _small_equal_constant(instances: List[Node]) -> bool:
    """A constant that every block holds with the same small content stays inside the body."""
    a = np.asarray(instances[0].get_data())
    if a.size > 16:
        return False
    return all(np.array_equal(a, np.asarray(c.get_data())) for c in instances[1:])


def fold_repeated_blocks(model: Model, min_ops: int = 4, min_repeats: int = 2) -> Optional[FoldedFunction]:
    """Fold the repeated blocks of ``model`` in place; returns the shared function or None when there is nothing to fold."""
    ensure_registered()
    blocks = find_repeated_blocks(model, min_ops, min_repeats)
    if blocks is None:
        return None
    R, L = blocks.count, blocks.length
    pos = [{n: j for j, n in enumerate(blk)} for blk in blocks.nodes]
    # inputs of the body in block-0 order: externals first (deduplicated per producer output), then closure constants
    ext_slots: List[Tuple[int, int]] = []            # (j, k) of the first read
    ext_index: Dict[Tuple[int, int], int] = {}       # (j, k) -> external slot
    clo_slots: List[Tuple[int, int]] = []
    kept_consts: Dict[Tuple[int, int], Node] = {}
    seen_ext: Dict[Tuple[Node, int], int] = {}
    for j, n in enumerate(blocks.nodes[0]):
        for k in range(n.get_input_size()):
            o = n.input_value(k)
            p = o.get_node()
            if p in pos[0]:
                continue
            if p.get_type_name() == "Constant":
                inst = [blocks.nodes[r][j].input_value(k).get_node() for r in range(R)]
                if _small_equal_constant(inst):
                    kept_consts[(j, k)] = p
                else:
                    clo_slots.append((j, k))
                continue
            key = (p, o.get_index())
            if key in seen_ext:
                # the same outside value read twice: the other blocks must read one value twice as well
                s = seen_ext[key]
                j0, k0 = ext_slots[s]
                ok = all(blocks.nodes[r][j].input_value(k) == blocks.nodes[r][j0].input_value(k0) for r in range(R))
                if ok:
                    ext_index[(j, k)] = s
                    continue
            seen_ext[key] = len(ext_slots)
            ext_index[(j, k)] = len(ext_slots)
            ext_slots.append((j, k))
    # outputs: (j, port) read outside its block in any instance
    out_slots: List[Tuple[int, int]] = []
    for r in range(R):
        for j, n in enumerate(blocks.nodes[r]):
            for port, o in enumerate(n.outputs()):
                if (j, port) not in out_slots and any(inp.get_node() not in pos[r] for inp in o.get_target_inputs()):
                    out_slots.append((j, port))
    out_slots.sort()
    if not out_slots:
        return None
    # body model from block 0
    mapping: Dict[Tuple[int, int], Output] = {}
    params: List[Node] = []
    ext_params: List[Node] = []
    for s, (j, k) in enumerate(ext_slots):
        o = blocks.nodes[0][j].input_value(k)
        p = parameter(o.get_partial_shape(), o.get_element_type(), "ext%d" % s)
        ext_params.append(p)
    clo_params: List[Node] = []
    for s, (j, k) in enumerate(clo_slots):
        o = blocks.nodes[0][j].input_value(k)
        clo_params.append(parameter(o.get_partial_shape(), o.get_element_type(), "w%d" % s))
    params = ext_params + clo_params
    clo_index = {jk: s for s, jk in enumerate(clo_slots)}
    for j, n in enumerate(blocks.nodes[0]):
        ins = []
        for k in range(n.get_input_size()):
            o = n.input_value(k)
            p = o.get_node()
            if p in pos[0]:
                ins.append(mapping[(pos[0][p], o.get_index())])
            elif (j, k) in kept_consts:
                ins.append(kept_consts[(j, k)].clone_with_new_inputs([]).output(0))
            elif (j, k) in clo_index:
                ins.append(clo_params[clo_index[(j, k)]].output(0))
            else:
                ins.append(ext_params[ext_index[(j, k)]].output(0))
        clone = make_op(n.get_type_name(), ins, dict(n.get_attributes()), version=n.get_version())
        clone.set_friendly_name("block/" + n.get_friendly_name())
        for port in range(n.get_output_size()):
            mapping[(j, port)] = clone.output(port)
    body = Model([result(mapping[s]) for s in out_slots], params, "npuw_function")
    f = FoldedFunction(body, len(ext_slots), len(clo_slots))
    fid = next(_next_id)
    _FUNCS[fid] = f
    # calls: blocks in order, so that a block reading the one before it finds the call already made
    replaced: Dict[Tuple[int, int, int], Output] = {}
    for r in range(R):
        args: List[Output] = []
        for (j, k) in ext_slots:
            o = blocks.nodes[r][j].input_value(k)
            args.append(o)
        for (j, k) in clo_slots:
            args.append(blocks.nodes[r][j].input_value(k))
        call = make_op("FunctionCall", args, {"function_id": fid}, version="NPUWOpset")
        call.set_friendly_name("npuw_block_%d" % r)
        for s, (j, port) in enumerate(out_slots):
            old = blocks.nodes[r][j].output(port)
            names = old.get_names()
            for inp in list(old.get_target_inputs()):
                if inp.get_node() not in pos[r]:
                    inp.replace_source_output(call.output(s))
            if names:
                call.output(s).set_names(set(names))
    model.validate_nodes_and_infer_types()
    f.blocks = R
    f.block_ops = L
    return f


# ------------------------------------------------------------------------------------------------- the device
class NpuwCompiledModel(CompiledModel):
    def __init__(self, plugin, model, config, inner: CompiledModel, function: Optional[FoldedFunction], bank: WeightsBank, removed: int):
        super().__init__(plugin, model, config, inner.runtime_model)
        self.inner, self.function, self.bank, self.constants_removed = inner, function, bank, removed

    def get_property(self, name):
        n = str(name)
        if n == props.execution_devices:
            return ["NPUW"] + list(self.inner.get_property(props.execution_devices))
        if n == "NPUW_FOLDED_BLOCKS":
            return getattr(self.function, "blocks", 0) if self.function else 0
        if n == "NPUW_BANK_SIZE":
            return len(self.bank)
        try:
            return super().get_property(name)
        except RuntimeError:
            return self.inner.get_property(name)

    def _make_runner(self, request):
        inner = self.inner.create_infer_request()
        request._delegate = lambda: inner

        def run(req, ins):
            for i, t in enumerate(ins):
                inner._in[i] = t
            outs = inner._runner(inner, ins)
            req._profile = inner._profile
            return outs
        return run

    def _variables(self, request):
        return request._delegate().query_state()


class NpuwPlugin(Plugin):
    device_name = "NPUW"
    description = "Repeated-block folding and weights bank over another device"

    def supported_properties(self):
        return super().supported_properties() + ["NPUW_DEVICES", "NPUW_FOLD", "NPUW_ONLINE_MIN_SIZE", "NPUW_ONLINE_KEEP_BLOCKS", "NPUW_WEIGHTS_BANK", props.device.priorities,
                                                 "NPUW_LLM", "NPUW_LLM_MAX_PROMPT_LEN", "NPUW_LLM_MIN_RESPONSE_LEN", "NPUW_LLM_PREFILL_CHUNK_SIZE",
                                                 "NPUW_LLM_GENERATE_VARIANTS", "NPUW_LLM_PREFIX_CACHING"]

    def default_config(self):
        d = super().default_config()
        d.update({"NPUW_DEVICES": "CPU", "NPUW_FOLD": "YES", "NPUW_ONLINE_MIN_SIZE": 4, "NPUW_ONLINE_KEEP_BLOCKS": 2, "NPUW_WEIGHTS_BANK": "shared",
                  "NPUW_LLM": "NO", "NPUW_LLM_MAX_PROMPT_LEN": 1024, "NPUW_LLM_MIN_RESPONSE_LEN": 128, "NPUW_LLM_PREFILL_CHUNK_SIZE": 0,
                  "NPUW_LLM_GENERATE_VARIANTS": "", "NPUW_LLM_PREFIX_CACHING": "NO"})
        return d

    def compile_model(self, model: Model, config: dict) -> CompiledModel:
        cfg = self.merged_config(config)
        dev = str(cfg.get(props.device.priorities) or cfg.get("NPUW_DEVICES") or "CPU").split(",")[0]
        bank = WeightsBank.for_device("%s/%s" % (dev, cfg.get("NPUW_WEIGHTS_BANK", "shared")))
        if str(cfg.get("NPUW_LLM", "NO")).upper() in ("YES", "TRUE", "1"):
            from .npuw_llm import NpuwLlmCompiledModel, is_llm
            if not is_llm(model):
                raise RuntimeError("[NPUW] NPUW_LLM needs a stateful decoder with input_ids / attention_mask / position_ids inputs")
            inner_cfg = {k: v for k, v in cfg.items() if not str(k).startswith("NPUW_") and k != props.device.priorities and k in config}
            return NpuwLlmCompiledModel(self, model, cfg, dev, inner_cfg, bank)
        work = model.clone()
        removed = dedupe_constants(work, bank)
        f = None
        if str(cfg.get("NPUW_FOLD", "YES")).upper() in ("YES", "TRUE", "1"):
            f = fold_repeated_blocks(work, int(cfg.get("NPUW_ONLINE_MIN_SIZE", 4)), int(cfg.get("NPUW_ONLINE_KEEP_BLOCKS", 2)))
            if f is not None:
                f.device = dev
        inner_cfg = {k: v for k, v in cfg.items() if not str(k).startswith("NPUW_") and k != props.device.priorities and k in config}
        inner = self.core.compile_model(work, dev, inner_cfg)
        return NpuwCompiledModel(self, model, cfg, inner, f, bank, removed)

    def query_model(self, model, config):
        cfg = self.merged_config(config)
        dev = str(cfg.get(props.device.priorities) or cfg.get("NPUW_DEVICES") or "CPU").split(",")[0]
        return {k: "NPUW" for k in self.core.query_model(model, dev, {})}


def register(core) -> None:
    ensure_registered()
    core.register_plugin_factory("NPUW", NpuwPlugin)
