"""Tensor-parallel partitioning of a generic (fused) graph: every rank gets its own shard of the model.

Works on the device graph after the fusion passes (``FullyConnected`` / ``ScaledDotProductAttention`` form):

* attention: the FullyConnected nodes that feed the query / key / value inputs of an SDPA are split by output channels
  (heads), the head count in the ``Reshape`` constants on the way is divided by the world size, and the
  FullyConnected that consumes the attention output is split by input channels and followed by an ``AllReduce``;
* MLP: ``FullyConnected -> (bias, activation) -> FullyConnected`` pairs are split column-wise / row-wise the same way.

Per-channel constants between a column-split FullyConnected and its consumer (biases, scales) are sliced with it.
``AllReduce`` is an operation of this package (sum over the ranks of ``torch.distributed``; NCCL on the CUDA device,
gloo on the host). The reference partitions only on the CPU plugin and only FullyConnected (split + all-gather by
memcpy per socket, src/plugins/intel_cpu/src/nodes/fullyconnected.cpp:336-425, enabled by
``MODEL_DISTRIBUTION_POLICY=TENSOR_PARALLEL``); the same property switches this pass on.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Set, Tuple

import numpy as np

from .. import opset as ops
from .._graph import Model, Node, Output, make_op
from .._op_base import register_op

_ELEMENTWISE = {"Add", "Subtract", "Multiply", "Divide", "Gelu", "Relu", "Swish", "Sigmoid", "Tanh", "Erf", "Convert", "Clamp", "HSwish", "Mish", "Power"}
_SHAPE_OPS = {"Reshape", "Transpose"}
_registered = False


def _all_reduce_eval(node, ins):
    x = np.ascontiguousarray(ins[0])
    import sys
    torch = sys.modules.get("torch")
    if torch is None:
        import torch
    dist = torch.distributed
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.from_numpy(x.copy())
        dist.all_reduce(t)
        return [t.numpy()]
    return [x]


def ensure_registered() -> None:
    global _registered
    if not _registered:
        register_op("AllReduce", lambda n: [(n.get_input_element_type(0), n.get_input_partial_shape(0))], _all_reduce_eval,
                    version="ie_internal_opset", attrs={"reduction": "sum"})
        _registered = True


def _const_node(o: Output) -> Optional[Node]:
    n = o.get_node()
    if n.get_type_name() == "Convert":
        n = n.input_value(0).get_node()
    return n if n.get_type_name() == "Constant" else None


def _replace_const(o: Output, value: np.ndarray, like: Node) -> None:
    """Re-point every use of the constant behind `o` (directly or through a Convert) at `value`."""
    n = o.get_node()
    new = ops.constant(np.ascontiguousarray(value))
    new.set_friendly_name(like.get_friendly_name())
    if n.get_type_name() == "Convert":
        n.input(0).replace_source_output(new.output(0))
        n.validate()
    else:
        for inp in list(o.get_target_inputs()):
            inp.replace_source_output(new.output(0))


def _is_fc(n: Node) -> bool:
    return n.get_type_name() == "FullyConnected" and _const_node(n.input_value(1)) is not None


def _trace_back_to_fc(o: Output, path: List[Node]) -> Optional[Node]:
    """Walk producers through shape-only and per-channel element-wise operations up to a FullyConnected."""
    for _ in range(12):
        n = o.get_node()
        t = n.get_type_name()
        if _is_fc(n):
            return n
        if t in _SHAPE_OPS or (t in _ELEMENTWISE and (n.get_input_size() == 1 or _const_node(n.input_value(1)) is not None)):
            path.append(n)
            o = n.input_value(0)
            continue
        return None
    return None


def _trace_forward_to_fc(o: Output, path: List[Node]) -> Optional[Node]:
    for _ in range(12):
        users = o.get_target_inputs()
        if len(users) != 1:
            return None
        n = users[0].get_node()
        t = n.get_type_name()
        if _is_fc(n) and users[0].get_index() == 0:
            return n
        if t in _SHAPE_OPS or (t in _ELEMENTWISE and users[0].get_index() == 0 and (n.get_input_size() == 1 or _const_node(n.input_value(1)) is not None)):
            path.append(n)
            o = n.output(0)
            continue
        return None
    return None


def _split_rows(fc: Node, rank: int, world: int) -> Tuple[int, int]:
    """Column-parallel: keep the output channels [lo, hi) of the weight [N, K] (and of a fused bias)."""
    wn = _const_node(fc.input_value(1))
    w = np.asarray(wn.get_data())
    N = w.shape[0]
    lo, hi = rank * N // world, (rank + 1) * N // world
    _replace_const(fc.input_value(1), w[lo:hi], wn)
    if fc.get_input_size() > 2:
        bn = _const_node(fc.input_value(2))
        if bn is not None and int(np.prod(bn.get_output_shape(0) or [0])) == N:
            _replace_const(fc.input_value(2), np.asarray(bn.get_data()).reshape(-1)[lo:hi], bn)
    return N, hi - lo


def _split_cols(fc: Node, rank: int, world: int) -> None:
    """Row-parallel: keep the input channels [lo, hi) of the weight [N, K]; a fused bias is divided by the world size
    (the all-reduce adds it up again)."""
    wn = _const_node(fc.input_value(1))
    w = np.asarray(wn.get_data())
    K = w.shape[1]
    lo, hi = rank * K // world, (rank + 1) * K // world
    _replace_const(fc.input_value(1), w[:, lo:hi], wn)
    if fc.get_input_size() > 2:
        bn = _const_node(fc.input_value(2))
        if bn is not None and int(np.prod(bn.get_output_shape(0) or [0])) > 0:
            b = np.asarray(bn.get_data())
            _replace_const(fc.input_value(2), (b.astype(np.float32) / world).astype(b.dtype), bn)


def _fix_path(path: List[Node], N: int, Nloc: int, rank: int, world: int) -> None:
    """Adapt the operations between a column-split FullyConnected and its consumer to the local channel count."""
    for n in path:
        t = n.get_type_name()
        if t == "Reshape":
            sn = _const_node(n.input_value(1))
            if sn is None:
                raise RuntimeError("tensor-parallel partitioning needs constant Reshape targets (%s)" % n.get_friendly_name())
            v = [int(x) for x in np.asarray(sn.get_data()).reshape(-1)]
            done = False
            for i in range(len(v) - 1, -1, -1):           # [.., H, D] with H * D = N  ->  H / world ;  [.., N] -> N / world
                tail = int(np.prod(v[i + 1:])) if i + 1 < len(v) else 1
                if v[i] > 0 and tail > 0 and v[i] * tail == N and v[i] % world == 0:
                    v[i] //= world
                    done = True
                    break
            if done:
                _replace_const(n.input_value(1), np.array(v, dtype=np.asarray(sn.get_data()).dtype), sn)
        elif t in _ELEMENTWISE and n.get_input_size() > 1:
            cn = _const_node(n.input_value(1))
            c = np.asarray(cn.get_data())
            if c.size == N and c.shape[-1] == N:
                lo = rank * N // world
                _replace_const(n.input_value(1), c[..., lo:lo + Nloc], cn)


def tensor_parallel_partition(model: Model, rank: int, world: int) -> int:
    """Rewrite `model` in place into the shard of `rank`; returns the number of AllReduce operations inserted."""
    if world <= 1:
        return 0
    ensure_registered()
    taken: Set[int] = set()
    inserted = 0

    def finish_row_parallel(fc: Node) -> None:
        nonlocal inserted
        _split_cols(fc, rank, world)
        users = list(fc.output(0).get_target_inputs())
        ar = make_op("AllReduce", [fc.output(0)], {"reduction": "sum"}, version="ie_internal_opset", name=fc.get_friendly_name() + "/all_reduce")
        for u in users:
            u.replace_source_output(ar.output(0))
        inserted += 1

    order = model.get_ordered_ops()
    # ---- attention blocks
    for sdpa in order:
        if sdpa.get_type_name() != "ScaledDotProductAttention":
            continue
        plans = []
        ok = True
        for i in range(3):
            path: List[Node] = []
            fc = _trace_back_to_fc(sdpa.input_value(i), path)
            if fc is None or id(fc._n) in taken:
                ok = False
                break
            plans.append((fc, path))
        out_path: List[Node] = []
        fo = _trace_forward_to_fc(sdpa.output(0), out_path) if ok else None
        if not ok or fo is None or id(fo._n) in taken or len({id(p[0]._n) for p in plans}) != 3:
            continue
        N = int(np.asarray(_const_node(plans[0][0].input_value(1)).get_data()).shape[0])
        if N % world or any(int(np.asarray(_const_node(p[0].input_value(1)).get_data()).shape[0]) % world for p in plans):
            continue
        for fc, path in plans:
            n_full, n_loc = _split_rows(fc, rank, world)
            _fix_path(path, n_full, n_loc, rank, world)
            taken.add(id(fc._n))
        _fix_path(out_path, N, N // world, rank, world)
        finish_row_parallel(fo)
        taken.add(id(fo._n))
    # ---- MLP pairs
    for up in order:
        if not _is_fc(up) or id(up._n) in taken:
            continue
        path = []
        down = _trace_forward_to_fc(up.output(0), path)
        if down is None or id(down._n) in taken or any(p.get_type_name() in _SHAPE_OPS for p in path):
            continue
        N = int(np.asarray(_const_node(up.input_value(1)).get_data()).shape[0])
        if N % world or N < 2 * world:
            continue
        n_full, n_loc = _split_rows(up, rank, world)
        _fix_path(path, n_full, n_loc, rank, world)
        finish_row_parallel(down)
        taken.update((id(up._n), id(down._n)))
    model.validate_nodes_and_infer_types()
    return inserted
