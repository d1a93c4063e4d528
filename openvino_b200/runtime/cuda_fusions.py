"""Device-specific graph fusions of the CUDA plugin, run after the common and LLM fusion passes.

* ``FullyConnected -> Add(constant [N])`` : the bias becomes the FullyConnected's third input (added in the GEMM epilogue);
* ``FullyConnected -> Gelu / Relu / Swish`` : the activation is recorded on the node (``fused_activation`` in rt_info)
  and applied in the GEMM epilogue;
* ``MVN(last axis) -> Multiply(gamma) -> Add(beta)`` : one ``LayerNormFused`` operation (own kernel).

Role of the post-op fusing passes of the reference GPU plugin (src/plugins/intel_gpu/src/graph/graph_optimizer/
prepare_primitive_fusing.cpp: fuse_bias, fuse_activations, fuse_simple_primitives).
"""
from __future__ import annotations

from typing import Optional

import numpy as np

from .. import opset as ops
from .._graph import Model, Node, Output, make_op
from .._op_base import register_op

_registered = False


def ensure_registered() -> None:
    global _registered
    if _registered:
        return

    def ln_eval(node, ins):
        x, g, b = ins[0].astype(np.float32), ins[1].astype(np.float32), ins[2].astype(np.float32)
        eps = float(node.get_attributes()["eps"])
        mu = x.mean(-1, keepdims=True)
        var = ((x - mu) ** 2).mean(-1, keepdims=True)
        return [((x - mu) / np.sqrt(var + eps) * g + b).astype(ins[0].dtype)]

    register_op("LayerNormFused", lambda n: [(n.get_input_element_type(0), n.get_input_partial_shape(0))], ln_eval,
                version="ie_internal_opset", attrs={"eps": 1e-5})
    _registered = True


def _const(o: Output) -> Optional[Node]:
    n = o.get_node()
    if n.get_type_name() == "Convert":
        n = n.input_value(0).get_node()
    return n if n.get_type_name() == "Constant" else None


def _single_user(o: Output):
    users = o.get_target_inputs()
    return users[0] if len(users) == 1 else None


def _replace(old: Output, new: Output) -> None:
    for inp in list(old.get_target_inputs()):
        inp.replace_source_output(new)


def fuse_fc_bias_and_activation(model: Model) -> int:
    count = 0
    for fc in model.get_ordered_ops():
        if fc.get_type_name() != "FullyConnected":
            continue
        N = fc.get_output_partial_shape(0)
        if not N.rank.is_static or not N[-1].is_static:
            continue
        n_out = N[-1].get_length()
        cur = fc
        has_bias = fc.get_input_size() > 2 and int(np.prod(fc.input_value(2).get_shape() or [0])) > 0 if fc.get_input_size() > 2 and fc.input_value(2).get_partial_shape().is_static else False
        user = _single_user(cur.output(0))
        if not has_bias and user is not None and user.get_node().get_type_name() == "Add":
            add = user.get_node()
            other = add.input_value(1 - user.get_index())
            cn = _const(other)
            if cn is not None and int(np.prod(cn.get_output_shape(0) or [1])) == n_out and list(cn.get_output_shape(0))[-1:] == [n_out]:
                bias = ops.reshape(other, np.array([n_out], dtype=np.int64), False).output(0)
                new_fc = fc.clone_with_new_inputs([fc.input_value(0), fc.input_value(1), bias])
                new_fc.set_friendly_name(fc.get_friendly_name())
                for k, v in fc.get_rt_info().items():
                    new_fc.get_rt_info()[k] = v
                _replace(add.output(0), new_fc.output(0))
                cur = new_fc
                count += 1
        user = _single_user(cur.output(0))
        if user is not None and "fused_activation" not in cur.get_rt_info():
            act = user.get_node()
            t = act.get_type_name()
            name = None
            if t == "Gelu":
                name = "gelu_tanh" if str(act.get_attributes().get("approximation_mode", "ERF")).upper() == "TANH" else "gelu_erf"
            elif t == "Relu":
                name = "relu"
            elif t == "Swish" and act.get_input_size() == 1:
                name = "silu"
            if name is not None:
                cur.get_rt_info()["fused_activation"] = name
                _replace(act.output(0), cur.output(0))
                count += 1
    return count


def fuse_layer_norm(model: Model) -> int:
    ensure_registered()
    count = 0
    for mvn in model.get_ordered_ops():
        if mvn.get_type_name() != "MVN":
            continue
        at = mvn.get_attributes()
        axes = _const(mvn.input_value(1))
        x = mvn.input_value(0)
        rank = x.get_partial_shape().rank
        if axes is None or not rank.is_static or not at.get("normalize_variance") or str(at.get("eps_mode", "")).lower() != "inside_sqrt":
            continue
        ax = [int(a) for a in np.asarray(axes.get_data()).reshape(-1)]
        if len(ax) != 1 or ax[0] % rank.get_length() != rank.get_length() - 1:
            continue
        last = x.get_partial_shape()[-1]
        if not last.is_static:
            continue
        C = last.get_length()
        u1 = _single_user(mvn.output(0))
        if u1 is None or u1.get_node().get_type_name() != "Multiply":
            continue
        mul = u1.get_node()
        gamma = mul.input_value(1 - u1.get_index())
        u2 = _single_user(mul.output(0))
        if _const(gamma) is None or u2 is None or u2.get_node().get_type_name() != "Add":
            continue
        add = u2.get_node()
        beta = add.input_value(1 - u2.get_index())
        if _const(beta) is None or int(np.prod(gamma.get_shape())) != C or int(np.prod(beta.get_shape())) != C:
            continue
        shp = np.array([C], dtype=np.int64)
        ln = make_op("LayerNormFused", [x, ops.reshape(gamma, shp, False), ops.reshape(beta, shp, False)], {"eps": float(at["eps"])},
                     version="ie_internal_opset", name=add.get_friendly_name())
        _replace(add.output(0), ln.output(0))
        count += 1
    return count


def run(model: Model) -> int:
    n = fuse_fc_bias_and_activation(model) + fuse_layer_norm(model)
    if n:
        from ..passes import ConstantFolding
        ConstantFolding().run_on_model(model)          # the reshaped bias / gamma / beta constants
        model.validate_nodes_and_infer_types()
    return n
