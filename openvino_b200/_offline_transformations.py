"""Offline model transformations (``openvino._offline_transformations``).

Reference entry points: src/bindings/python/src/pyopenvino/core/offline_transformations.cpp:34-190.
"""
from __future__ import annotations

from . import _ovcore as _c
from ._graph import Model
from . import passes as _passes


def apply_moc_transformations(model: Model, cf: bool = True, smart_reshape: bool = False) -> None:
    _c.run_moc_transformations(model._m, bool(cf))


def apply_moc_legacy_transformations(model: Model, params_with_custom_types=None) -> None:
    _c.run_moc_transformations(model._m, True)


def apply_low_latency_transformation(model: Model, use_const_initializer: bool = True) -> None:
    _passes.LowLatency2(use_const_initializer).run_on_model(model)


def apply_pruning_transformation(model: Model) -> None:
    from .passes.pruning import Pruning
    Pruning().run_on_model(model)


def apply_make_stateful_transformation(model: Model, param_res_names) -> None:
    _passes.MakeStateful(param_res_names).run_on_model(model)


def compress_model_transformation(model: Model) -> None:
    _c.compress_model_to_f16(model._m)


def compress_quantize_weights_transformation(model: Model) -> None:
    from .passes.low_precision import CompressQuantizeWeights
    CompressQuantizeWeights().run_on_model(model)


def convert_sequence_to_tensor_iterator_transformation(model: Model) -> None:
    model.validate_nodes_and_infer_types()


def apply_fused_names_cleanup(model: Model) -> None:
    _passes.FusedNamesCleanup().run_on_model(model)


def paged_attention_transformation(model: Model, use_block_indices_inputs: bool = False, use_score_outputs: bool = False,
                                   allow_score_aggregation: bool = False, allow_cache_rotation: bool = False,
                                   allow_xattention: bool = False, allow_adaptive_rkv: bool = False, allow_qq_bias: bool = False) -> None:
    _c.sdpa_to_paged_attention(model._m, dict(use_block_indices_inputs=use_block_indices_inputs, use_score_outputs=use_score_outputs,
                                              allow_score_aggregation=allow_score_aggregation, allow_cache_rotation=allow_cache_rotation,
                                              allow_xattention=allow_xattention, allow_adaptive_rkv=allow_adaptive_rkv, allow_qq_bias=allow_qq_bias))


def stateful_to_stateless_transformation(model: Model) -> None:
    _c.stateful_to_stateless(model._m)
