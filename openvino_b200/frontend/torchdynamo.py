"""``torch.compile`` backend: ``torch.compile(model, backend="openvino_b200", options={"device": "CPU"})``.

Dynamo hands the backend an fx graph of torch-level calls. It is lowered to aten operators (``make_fx`` with the core
decompositions), the nodes that the PyTorch front end can translate are grouped into partitions
(``CapabilityBasedPartitioner``), every partition is converted, compiled for the chosen device and replaced by a call
into its compiled model; nodes without a translator stay in eager PyTorch between the partitions. Compiled partitions
are cached per input signature (shapes and dtypes), so a recompilation by dynamo with new shapes compiles anew.

Options: ``device`` (default "CPU"), ``config`` (properties for ``compile_model``), ``min_partition_size`` (partitions with
fewer operators stay eager, default 1), ``aot_decompositions`` (default True).

Role in the reference: src/bindings/python/src/openvino/frontend/pytorch/torchdynamo/{backend.py, partition.py,
execute.py, op_support.py}; the backend is also registered under the reference's name "openvino" when no other package
registered that name.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import numpy as np

_registered = False


class _CompiledPartition:
    """One supported sub-graph: converted and compiled on first call per input signature."""

    def __init__(self, gm, options: dict):
        self.gm, self.options = gm, options
        self.cache: Dict[tuple, Any] = {}
        self.fallback = False

    def __call__(self, *args):
        import torch
        if self.fallback:
            return self.gm(*args)
        key = tuple((tuple(a.shape), str(a.dtype)) if isinstance(a, torch.Tensor) else ("py", a) for a in args)
        entry = self.cache.get(key)
        if entry is None:
            try:
                entry = self._compile(args)
            except Exception as e:      # noqa: BLE001 - an unsupported corner keeps the partition in eager mode
                from ..utils import log
                log.warn("torchdynamo", "partition stays in eager mode: %s: %s" % (type(e).__name__, str(e)[:200]))
                self.fallback = True
                return self.gm(*args)
            self.cache[key] = entry
        compiled, n_tensor_outputs, out_struct = entry
        tensors = [a for a in args if isinstance(a, torch.Tensor)]
        dev = tensors[0].device if tensors else torch.device("cpu")
        feeds = [t.detach().cpu().contiguous().numpy() if t.dtype != torch.bfloat16 else t.detach().cpu().float().numpy() for t in tensors]
        outs = compiled(feeds)
        res = [torch.from_numpy(np.ascontiguousarray(outs[i])).to(dev) for i in range(n_tensor_outputs)]
        return out_struct(res)

    def _compile(self, args):
        import torch
        from .. import Core
        from . import pytorch as P
        model = P.from_fx(self.gm, list(args), share_weights=True)
        # bf16 inputs are fed as fp32
        core = Core()
        compiled = core.compile_model(model, self.options.get("device", "CPU"), dict(self.options.get("config") or {}))
        out_node = next(n for n in self.gm.graph.nodes if n.op == "output")
        spec = out_node.args[0]

        def count(a):
            if isinstance(a, (list, tuple)):
                return sum(count(x) for x in a)
            return 0 if a is None else 1

        def build(a, it):
            if isinstance(a, (list, tuple)):
                return type(a)(build(x, it) for x in a)
            return None if a is None else next(it)
        n_out = count(spec)
        return compiled, n_out, (lambda res: build(spec, iter(res)))


def _supported(node) -> bool:
    from . import pytorch as P
    if node.op != "call_function":
        return False
    name = P._target_name(node.target)
    return name in P._TABLE


def compile_fx(gm, example_inputs: Sequence[Any], options: Optional[dict] = None):
    """The backend function proper; returns a callable with the signature of ``gm.forward``."""
    import torch
    from torch.fx.experimental.proxy_tensor import make_fx
    from torch.fx.passes.infra.partitioner import CapabilityBasedPartitioner
    from torch.fx.passes.operator_support import OperatorSupport
    options = dict(options or {})
    decomp = {}
    if options.get("aot_decompositions", True):
        from torch._decomp import core_aten_decompositions
        decomp = core_aten_decompositions()
        from . import pytorch as P
        # keep the operators that have a translator of their own whole
        decomp = {k: v for k, v in decomp.items() if str(k) not in P._TABLE}
    with torch.no_grad():
        aten_gm = make_fx(gm, decomposition_table=decomp, tracing_mode="fake", _allow_non_fake_inputs=True)(*example_inputs)

    class Support(OperatorSupport):
        def is_node_supported(self, submodules, node) -> bool:
            return _supported(node)

    part = CapabilityBasedPartitioner(aten_gm, Support(), allows_single_node_partition=True)
    partitions = [p for p in part.propose_partitions() if len(p.nodes) >= int(options.get("min_partition_size", 1))]
    fused = part.fuse_partitions(partitions) if partitions else aten_gm
    n_compiled = 0
    for name, sub in list(fused.named_children()):
        if name.startswith("fused_") and isinstance(sub, torch.fx.GraphModule):
            setattr(fused, name, _wrap(_CompiledPartition(sub, options)))
            n_compiled += 1
    fused.recompile()
    fused._ovb_partitions = n_compiled

    def run(*args):
        with torch.no_grad():
            return fused(*args)
    run._ovb_partitions = n_compiled
    run._ovb_graph = fused
    return run


def _wrap(partition: _CompiledPartition):
    import torch

    class _Module(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.partition = partition

        def forward(self, *args):
            return self.partition(*args)
    return _Module()


def backend(gm, example_inputs, options: Optional[dict] = None, **kwargs):
    return compile_fx(gm, example_inputs, options or kwargs.get("options"))


def register() -> None:
    """Register the backend with dynamo (idempotent). Called when the package is imported and torch is present."""
    global _registered
    if _registered:
        return
    try:
        from torch._dynamo import register_backend
        from torch._dynamo.backends.registry import list_backends
    except Exception:      # noqa: BLE001 - torch without dynamo
        return
    register_backend(name="openvino_b200", compiler_fn=backend)
    try:
        if "openvino" not in list_backends(exclude_tags=()):
            register_backend(name="openvino", compiler_fn=backend)
    except Exception:      # noqa: BLE001
        pass
    _registered = True
