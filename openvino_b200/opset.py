"""Operation factories (``ov.opset1`` … ``ov.opset16`` style): ``opset.matmul(a, b, False, True)`` and so on.

Every factory accepts Nodes, Outputs or plain Python / numpy values (which become Constants) for its inputs,
attribute values positionally or by keyword, and ``name=`` for the friendly name. The signatures follow the
reference Python factories (src/bindings/python/src/openvino/opset*/ops.py); they are generated from the
compact table below instead of one hand-written function per operation.

Table line: ``python_name OpType[@opsetN] : input … [optional_input] … *variadic | attribute[=default] …``.
An attribute written ``py_name>ir_name`` is exposed as ``py_name`` and stored as ``ir_name``.
"""
from __future__ import annotations

import sys
import types as _pytypes
from typing import Optional

import numpy as np

from ._graph import Model, Node, Output, as_output, constant, make_op, parameter, result
from ._types import PartialShape, Type

_SPEC = """
gather_matmul GatherMatmul@ie_internal_opset : A B indices [bias]
gather_matmul_compressed GatherMatmulCompressed@ie_internal_opset : A B indices bias weight_scales [weight_zero_points]
grouped_matmul_compressed GroupedMatMulCompressed@ie_internal_opset : *inputs
fully_connected_quantized FullyConnectedQuantized@ie_internal_opset : X W bias weight_scales weight_zero_points input_scales input_zero_points output_scales output_zero_points | output_type=dynamic
fully_connected_quantized_legacy FullyConnectedQuantizedLegacy@ie_internal_opset : X W bias deq_scales [deq_zero_points] | output_type=dynamic
group_query_attention GroupQueryAttention@ie_internal_opset : *inputs | num_heads kv_num_heads scale=0.0 do_rotary=False rotary_interleaved=False local_window_size=-1 smooth_softmax=False
vl_sdpa VLSDPA@ie_internal_opset : q k v cu_seqlens | order_q=[] order_k=[] order_v=[] order_out=[]
selective_ssm SelectiveSSM@ie_internal_opset : A dt B x C recurrent_state
gated_delta_net GatedDeltaNet@ie_internal_opset : query key value recurrent_state gate beta | fuse_qk_l2norm=False q_l2_norm_eps=1e-6 k_l2_norm_eps=1e-6
paged_selective_ssm PagedSelectiveSSM@ie_internal_opset : A dt B x C recurrent_state_table subsequence_begins la_block_indices la_block_indices_begins num_processed_tokens cache_interval
paged_gated_delta_net PagedGatedDeltaNet@ie_internal_opset : query key value recurrent_state_table gate beta subsequence_begins la_block_indices la_block_indices_begins processed_tokens cache_interval | use_qk_l2norm=False q_l2_norm_eps=1e-6 k_l2_norm_eps=1e-6
paged_causal_conv1d PagedCausalConv1D@ie_internal_opset : input_embeds conv_state_table conv_weight conv_bias subsequence_begins la_block_indices la_block_indices_begins processed_tokens cache_interval
pa_kv_reorder PaKVReorder@ie_internal_opset : key_cache value_cache block_indices block_indices_begins block_update_indices block_update_indices_begins
augru_cell AUGRUCell@ie_internal_opset : X initial_hidden_state W R B A | hidden_size activations=[] activations_alpha=[] activations_beta=[] clip=0.0 linear_before_reset=False
augru_sequence AUGRUSequence@ie_internal_opset : X initial_hidden_state sequence_lengths W R B A | hidden_size direction=forward activations=[] activations_alpha=[] activations_beta=[] clip=0.0 linear_before_reset=False
prior_box PriorBox : layer_shape image_shape | min_size=[] max_size=[] aspect_ratio=[] density=[] fixed_ratio=[] fixed_size=[] clip=False flip=False step=0.0 offset=0.0 variance=[] scale_all_sizes=True min_max_aspect_ratios_order=True
detection_output DetectionOutput : box_logits class_preds proposals [aux_class_preds] [aux_box_preds] | background_label_id=0 top_k=-1 variance_encoded_in_target=False keep_top_k=[1] code_type=caffe.PriorBoxParameter.CORNER share_location=True nms_threshold=0.0 confidence_threshold=0.0 clip_after_nms=False clip_before_nms=False decrease_label_id=False normalized=False input_height=1 input_width=1 objectness_score=0.0
proposal Proposal : class_probs bbox_deltas image_shape | base_size pre_nms_topn post_nms_topn nms_thresh feat_stride min_size ratio scale clip_before_nms=True clip_after_nms=False normalize=False box_size_scale=1.0 box_coordinate_scale=1.0 framework=
generate_proposals GenerateProposals : im_info anchors deltas scores | min_size nms_threshold pre_nms_count post_nms_count normalized=True nms_eta=1.0 roi_num_type=i64
experimental_detectron_prior_grid_generator ExperimentalDetectronPriorGridGenerator : priors feature_map image | flatten=True h=0 w=0 stride_x=0.0 stride_y=0.0
experimental_detectron_detection_output ExperimentalDetectronDetectionOutput : input_rois input_deltas input_scores input_im_info | score_threshold nms_threshold max_delta_log_wh num_classes post_nms_count max_detections_per_image class_agnostic_box_regression=False deltas_weights=[10.0,10.0,5.0,5.0]
experimental_detectron_generate_proposals_single_image ExperimentalDetectronGenerateProposalsSingleImage : im_info anchors deltas scores | min_size nms_threshold post_nms_count pre_nms_count
experimental_detectron_roi_feature_extractor ExperimentalDetectronROIFeatureExtractor : *inputs | output_size sampling_ratio pyramid_scales aligned=False
experimental_detectron_topk_rois ExperimentalDetectronTopKROIs : input_rois rois_probs | max_rois=0
deformable_convolution DeformableConvolution : data offsets filters [mask] | strides pads_begin pads_end dilations auto_pad=explicit group=1 deformable_group=1 bilinear_interpolation_pad=False
deformable_psroi_pooling DeformablePSROIPooling : feature_maps coords [offsets] | output_dim spatial_scale group_size=1 mode=bilinear_deformable spatial_bins_x=1 spatial_bins_y=1 trans_std=1.0 part_size=1
matrix_nms MatrixNms : boxes scores | sort_result_type=none sort_result_across_batch=False output_type=i64 score_threshold=0.0 nms_top_k=-1 keep_top_k=-1 background_class=-1 decay_function=linear gaussian_sigma=2.0 post_threshold=0.0 normalized=True
multiclass_nms MulticlassNms : boxes scores [roisnum] | sort_result_type=none sort_result_across_batch=False output_type=i64 iou_threshold=0.0 score_threshold=0.0 nms_top_k=-1 keep_top_k=-1 background_class=-1 nms_eta=1.0 normalized=True
nms_rotated NMSRotated : boxes scores max_output_boxes_per_class iou_threshold score_threshold | sort_result_descending=True output_type=i64 clockwise=True
roi_align_rotated ROIAlignRotated : data rois batch_indices | pooled_h pooled_w sampling_ratio spatial_scale clockwise_mode=False
binary_convolution BinaryConvolution : data filters | strides pads_begin pads_end dilations mode=xnor-popcount pad_value=0.0 auto_pad=explicit
string_tensor_pack StringTensorPack : begins ends symbols
string_tensor_unpack StringTensorUnpack : data
reverse Reverse : data axis | mode=index
istft ISTFT : data window frame_size frame_step [signal_length] | center=False normalized=False
logical_xor_v0 Xor : a b | auto_broadcast=numpy
rgb_to_nv12 RGBtoNV12 : arg | single_plane=True
bgr_to_nv12 BGRtoNV12 : arg | single_plane=True
identity Identity : data
nv12_to_rgb NV12toRGB : arg [arg_uv]
nv12_to_bgr NV12toBGR : arg [arg_uv]
i420_to_rgb I420toRGB : arg [arg_u] [arg_v]
i420_to_bgr I420toBGR : arg [arg_u] [arg_v]
prior_box_clustered PriorBoxClustered : output_size image_size | width height step=0.0 step_w=0.0 step_h=0.0 clip=True offset=0.0 variance=[]
psroi_pooling PSROIPooling : input coords | output_dim group_size spatial_scale spatial_bins_x=1 spatial_bins_y=1 mode=average
fake_convert FakeConvert : data scale [shift] | destination_type=f8e4m3
sparse_fill_empty_rows SparseFillEmptyRows : values dense_shape indices default_value
extract_image_patches ExtractImagePatches : image | sizes strides rates auto_pad=valid
region_yolo RegionYolo : input | coords classes num>num do_softmax mask axis end_axis anchors=[]
ctc_loss CTCLoss : logits logit_length labels label_length [blank_index] | preprocess_collapse_repeated=False ctc_merge_repeated=True unique=False
stft STFT : data window frame_size frame_step | transpose_frames=False
erfinv ErfInv : x
bitwise_left_shift BitwiseLeftShift : a b | auto_broadcast=numpy
bitwise_right_shift BitwiseRightShift : a b | auto_broadcast=numpy
convert_promote_types ConvertPromoteTypes : left right | promote_unsafe=False pytorch_scalar_promotion=False u64_integer_promotion_target=f32
space_to_depth SpaceToDepth : data | mode block_size=1
space_to_batch SpaceToBatch : data block_shape pads_begin pads_end
batch_to_space BatchToSpace : data block_shape crops_begin crops_end
shuffle_channels ShuffleChannels : data | axis group=1
reverse_sequence ReverseSequence : input seq_lengths | batch_axis seq_axis
reorg_yolo ReorgYolo : input | stride
bucketize Bucketize : data buckets | output_type=i64 with_right_bound=True
search_sorted SearchSorted : sorted_sequence values | right_mode=False output_type=i64
eye Eye : num_rows num_columns diagonal_index [batch_shape] | output_type
random_uniform RandomUniform : output_shape min_val max_val | output_type global_seed=0 op_seed=0 alignment=TENSORFLOW
multinomial Multinomial : probs num_samples | convert_type with_replacement log_probs global_seed=0 op_seed=0
lrn LRN : data axes | alpha=1.0 beta=0.5 bias=1.0 size=5
grn GRN : data | bias
segment_max SegmentMax : data segment_ids [num_segments] | fill_mode=ZERO
slice_scatter SliceScatter : data updates start stop step [axes]
gather_tree GatherTree : step_ids parent_idx max_seq_len end_token
unique Unique : data [axis] | sorted=True index_element_type=i64 count_element_type=i64
inverse Inverse : data | adjoint=False
grouped_matmul GroupedMatMul : mat_a mat_b [offsets]
convolution_backprop_data ConvolutionBackpropData : data filters [output_shape] | strides pads_begin=[] pads_end=[] dilations=[] auto_pad=explicit output_padding=[]
group_convolution_backprop_data GroupConvolutionBackpropData : data filters [output_shape] | strides pads_begin=[] pads_end=[] dilations=[] auto_pad=explicit output_padding=[]
col2im Col2Im : data output_size kernel_size | strides=[1,1] dilations=[1,1] pads_begin=[0,0] pads_end=[0,0]
adaptive_max_pool AdaptiveMaxPool : data output_shape | index_element_type=i64
roi_align ROIAlign : data rois batch_indices | pooled_h pooled_w sampling_ratio spatial_scale mode aligned_mode=asymmetric
roi_pooling ROIPooling : input coords | output_size spatial_scale method=max
grid_sample GridSample : data grid | align_corners=False mode=bilinear padding_mode=zeros
non_max_suppression NonMaxSuppression : boxes scores [max_output_boxes_per_class] [iou_threshold] [score_threshold] [soft_nms_sigma] | box_encoding=corner sort_result_descending=True output_type=i64
dft DFT : data axes [signal_size]
idft IDFT : data axes [signal_size]
rdft RDFT : data axes [signal_size]
irdft IRDFT : data axes [signal_size]
lstm_cell LSTMCell : X initial_hidden_state initial_cell_state W R [B] | hidden_size activations=[] activations_alpha=[] activations_beta=[] clip=0.0
gru_cell GRUCell : X initial_hidden_state W R [B] | hidden_size activations=[] activations_alpha=[] activations_beta=[] clip=0.0 linear_before_reset=False
rnn_cell RNNCell : X initial_hidden_state W R [B] | hidden_size activations=[] activations_alpha=[] activations_beta=[] clip=0.0
lstm_sequence LSTMSequence : X initial_hidden_state initial_cell_state sequence_lengths W R B | hidden_size direction activations=[] activations_alpha=[] activations_beta=[] clip=0.0
gru_sequence GRUSequence : X initial_hidden_state sequence_lengths W R B | hidden_size direction activations=[] activations_alpha=[] activations_beta=[] clip=0.0 linear_before_reset=False
rnn_sequence RNNSequence : X initial_hidden_state sequence_lengths W R B | hidden_size direction activations=[] activations_alpha=[] activations_beta=[] clip=0.0
ctc_greedy_decoder CTCGreedyDecoder : data sequence_mask | merge_repeated>ctc_merge_repeated=True
ctc_greedy_decoder_seq_len CTCGreedyDecoderSeqLen : data sequence_length [blank_index] | merge_repeated=True classes_index_type=i32 sequence_length_type=i32
embedding_bag_offsets_sum EmbeddingBagOffsetsSum : emb_table indices offsets [default_index] [per_sample_weights]
embedding_bag_packed_sum EmbeddingBagPackedSum : emb_table indices [per_sample_weights]
embedding_bag_offsets EmbeddingBagOffsets : emb_table indices offsets [default_index] [per_sample_weights] | reduction=sum
embedding_bag_packed EmbeddingBagPacked : emb_table indices [per_sample_weights] | reduction=sum
embedding_segments_sum EmbeddingSegmentsSum : emb_table indices segment_ids num_segments [default_index] [per_sample_weights]
abs Abs : x
acos Acos : x
acosh Acosh : x
adaptive_avg_pool AdaptiveAvgPool : data output_shape
add Add : a b | auto_broadcast=numpy
asin Asin : x
asinh Asinh : x
assign Assign : new_value | variable_id
atan Atan : x
atanh Atanh : x
avg_pool AvgPool : data | strides pads_begin pads_end kernel_shape>kernel exclude_pad>exclude-pad rounding_type=floor auto_pad=explicit
batch_norm_inference BatchNormInference : data gamma beta mean variance | epsilon
bitwise_and BitwiseAnd : a b | auto_broadcast=numpy
bitwise_not BitwiseNot : x
bitwise_or BitwiseOr : a b | auto_broadcast=numpy
bitwise_xor BitwiseXor : a b | auto_broadcast=numpy
broadcast Broadcast : data target_shape [axes_mapping] | broadcast_spec>mode=numpy
ceiling Ceiling : x
ceil Ceiling : x
clamp Clamp : data | min_value>min max_value>max
concat Concat : *nodes | axis
convert Convert : data | destination_type
convert_like ConvertLike : data like
convolution Convolution : data filters | strides pads_begin pads_end dilations auto_pad=explicit
cos Cos : x
cosh Cosh : x
cum_sum CumSum : arg axis | exclusive=False reverse=False
cumsum CumSum : arg axis | exclusive=False reverse=False
depth_to_space DepthToSpace : data | mode block_size=1
divide Divide : a b | auto_broadcast=numpy
einsum Einsum : *inputs | equation
elu Elu : data | alpha
equal Equal : a b | auto_broadcast=numpy
erf Erf : x
exp Exp : x
fake_quantize FakeQuantize : data input_low input_high output_low output_high | levels auto_broadcast=numpy
floor Floor : x
floor_mod FloorMod : a b | auto_broadcast=numpy
gather Gather : data indices axis | batch_dims=0
gather_elements GatherElements : data indices | axis=0
gather_nd GatherND : data indices | batch_dims=0
gelu Gelu : x | approximation_mode=erf
greater Greater : a b | auto_broadcast=numpy
greater_equal GreaterEqual : a b | auto_broadcast=numpy
group_convolution GroupConvolution : data filters | strides pads_begin pads_end dilations auto_pad=explicit
group_normalization GroupNormalization : data scale bias | num_groups epsilon
hard_sigmoid HardSigmoid : data alpha beta
hsigmoid HSigmoid : x
hswish HSwish : x
interpolate Interpolate : image scales_or_sizes [axes] | mode shape_calculation_mode pads_begin=[] pads_end=[] coordinate_transformation_mode=half_pixel nearest_mode=round_prefer_floor antialias=False cube_coeff=-0.75
is_finite IsFinite : x
is_inf IsInf : x | detect_negative=True detect_positive=True
is_nan IsNaN : x
less Less : a b | auto_broadcast=numpy
less_equal LessEqual : a b | auto_broadcast=numpy
log Log : x
log_softmax LogSoftmax : data | axis
logical_and LogicalAnd : a b | auto_broadcast=numpy
logical_not LogicalNot : x
logical_or LogicalOr : a b | auto_broadcast=numpy
logical_xor LogicalXor : a b | auto_broadcast=numpy
matmul MatMul : a b | transpose_a=False transpose_b=False
max_pool MaxPool : data | strides dilations pads_begin pads_end kernel_shape>kernel rounding_type=floor auto_pad=explicit index_element_type=i64 axis=0
maximum Maximum : a b | auto_broadcast=numpy
minimum Minimum : a b | auto_broadcast=numpy
mish Mish : x
mod Mod : a b | auto_broadcast=numpy
multiply Multiply : a b | auto_broadcast=numpy
mvn MVN : data axes | normalize_variance eps eps_mode
negative Negative : x
non_zero NonZero : data | output_type=i64
normalize_l2 NormalizeL2 : data axes | eps eps_mode
not_equal NotEqual : a b | auto_broadcast=numpy
one_hot OneHot : indices depth on_value off_value | axis
pad Pad : arg pads_begin pads_end [arg_pad_value] | pad_mode=constant
power Power : a b | auto_broadcast=numpy
prelu PRelu : data slope
range Range : start stop step | output_type=i64
read_value ReadValue : [init_value] | variable_id variable_type=dynamic variable_shape=None
reduce_l1 ReduceL1 : node reduction_axes | keep_dims=False
reduce_l2 ReduceL2 : node reduction_axes | keep_dims=False
reduce_logical_and ReduceLogicalAnd : node reduction_axes | keep_dims=False
reduce_logical_or ReduceLogicalOr : node reduction_axes | keep_dims=False
reduce_max ReduceMax : node reduction_axes | keep_dims=False
reduce_mean ReduceMean : node reduction_axes | keep_dims=False
reduce_min ReduceMin : node reduction_axes | keep_dims=False
reduce_prod ReduceProd : node reduction_axes | keep_dims=False
reduce_sum ReduceSum : node reduction_axes | keep_dims=False
relu Relu : x
reshape Reshape : node output_shape | special_zero=False
roll Roll : data shift axes
round Round : data | mode=half_to_even
scaled_dot_product_attention ScaledDotProductAttention : query key value [attention_mask] [scale] [sink] | causal=False
scatter_elements_update ScatterElementsUpdate : data indices updates axis | reduction=none use_init_val=True
scatter_nd_update ScatterNDUpdate : data indices updates | reduction=none
scatter_update ScatterUpdate : data indices updates axis
select Select : cond then_node else_node | auto_broadcast=numpy
selu Selu : data alpha lambda_value
shape_of ShapeOf : data | output_type=i64
sigmoid Sigmoid : x
sign Sign : x
sin Sin : x
sinh Sinh : x
slice Slice : data start stop step [axes]
softmax Softmax : data | axis
softplus SoftPlus : x
softsign SoftSign : x
split Split : data axis | num_splits
sqrt Sqrt : x
squared_difference SquaredDifference : a b | auto_broadcast=numpy
squeeze Squeeze : data [axes] | allow_axis_skip=False
strided_slice StridedSlice : data begin end [strides] | begin_mask end_mask new_axis_mask=[] shrink_axis_mask=[] ellipsis_mask=[]
subtract Subtract : a b | auto_broadcast=numpy
swish Swish : data [beta]
tan Tan : x
tanh Tanh : x
tile Tile : data repeats
topk TopK : data k | axis mode sort index_element_type=i32 stable=False
transpose Transpose : data input_order
unsqueeze Unsqueeze : data axes
variadic_split VariadicSplit : data axis split_lengths
"""

_LITERALS = {"True": True, "False": False, "None": None, "[]": []}


def _parse_default(text):
    if text in _LITERALS:
        v = _LITERALS[text]
        return list(v) if isinstance(v, list) else v
    if text.startswith("[") and text.endswith("]"):      # list literal: [1,1]
        return [_parse_default(t) for t in text[1:-1].split(",") if t]
    try:
        return int(text)
    except ValueError:
        pass
    try:
        return float(text)
    except ValueError:
        return text


_REQUIRED = object()
_TYPE_ATTRS = {"destination_type", "output_type", "index_element_type", "variable_type", "compute_type", "convert_type", "count_element_type",
               "classes_index_type", "sequence_length_type", "u64_integer_promotion_target"}


def _make_factory(py_name, op_type, version, inputs, attrs):
    req_inputs = [i for i in inputs if not i.startswith("[") and not i.startswith("*")]
    opt_inputs = [i[1:-1] for i in inputs if i.startswith("[")]
    variadic = next((i[1:] for i in inputs if i.startswith("*")), None)
    attr_specs = []
    for a in attrs:
        default = _REQUIRED
        if "=" in a:
            a, d = a.split("=", 1)
            default = _parse_default(d)
        py, ir = (a.split(">") + [None])[:2] if ">" in a else (a, a)
        attr_specs.append((py, ir, default))

    def factory(*args, name: Optional[str] = None, **kwargs):
        args = list(args)
        ins = []
        if variadic is not None:
            first = kwargs.pop(variadic) if variadic in kwargs else args.pop(0)
            ins = list(first)
        else:
            for n in req_inputs:
                if n in kwargs:
                    ins.append(kwargs.pop(n))
                elif args:
                    ins.append(args.pop(0))
                else:
                    raise TypeError("%s() missing input '%s'" % (py_name, n))
            for n in opt_inputs:
                if n in kwargs:
                    v = kwargs.pop(n)
                    if v is not None:
                        ins.append(v)
                elif args and args[0] is None:
                    args.pop(0)
                elif args and not isinstance(args[0], (str, bool, Type)):
                    ins.append(args.pop(0))
        # the detection factories of the reference take their attributes as one dict: ``prior_box(layer, image, attrs)``
        if args and isinstance(args[0], dict):
            kwargs.update(args.pop(0))
        elif isinstance(kwargs.get("attrs"), dict):
            kwargs.update(kwargs.pop("attrs"))
        values = {}
        for py, ir, default in attr_specs:
            if py in kwargs:
                v = kwargs.pop(py)
            elif ir in kwargs:
                v = kwargs.pop(ir)
            elif args:
                v = args.pop(0)
            elif default is _REQUIRED:
                raise TypeError("%s() missing attribute '%s'" % (py_name, py))
            else:
                v = default
            if ir in _TYPE_ATTRS and v is not None:
                v = Type(v)
            if ir == "variable_shape":
                v = PartialShape.dynamic() if v is None else (v if isinstance(v, PartialShape) else PartialShape(v))
            if isinstance(v, str) and ir in ("auto_pad", "auto_broadcast", "mode", "rounding_type", "pad_mode", "eps_mode", "sort",
                                              "reduction", "shape_calculation_mode", "coordinate_transformation_mode", "nearest_mode"):
                v = v.lower()
            if isinstance(v, str) and ir == "approximation_mode":
                v = v.upper()
            values[ir] = v
        if args or kwargs:
            raise TypeError("%s() got unexpected arguments %r %r" % (py_name, args, kwargs))
        return make_op(op_type, ins, values, version=version, name=name)

    factory.__name__ = py_name
    factory.__qualname__ = py_name
    factory._spec = (py_name, op_type, version, list(inputs), list(attrs))
    sig = ", ".join(inputs + [a for a in attrs])
    factory.__doc__ = "Create a %s operation. Arguments: %s, name=None." % (op_type, sig)
    return factory


def _build():
    mod = sys.modules[__name__]
    for line in _SPEC.strip().splitlines():
        line = line.strip()
        if not line:
            continue
        head, _, rest = line.partition(":")
        py_name, op = head.split()
        version = ""
        if "@" in op:
            op, version = op.split("@")
        ins_txt, _, attr_txt = rest.partition("|")
        setattr(mod, py_name, _make_factory(py_name, op, version, ins_txt.split(), attr_txt.split()))


_build()


def export_versioned(namespace: dict, number: int) -> None:
    """Fill ``namespace`` with the factories of ``opset<number>``: an operation appears when some version of it is at most
    that set, and the factory then creates the newest such version (``opset1.softmax`` makes Softmax-1, ``opset8.softmax``
    Softmax-8). Hand-written builders and helpers are shared by all sets. Reference: src/bindings/python/src/openvino/opsetN/."""
    from . import _ovcore as _c
    versions: dict = {}
    for sch in _c.op_schemas():
        t, v = sch[0], sch[1]
        if v.startswith("opset") and v[5:].isdigit():
            versions.setdefault(t, []).append(int(v[5:]))
    mod = sys.modules[__name__]
    for name, obj in vars(mod).items():
        if name.startswith("_"):
            continue
        spec = getattr(obj, "_spec", None)
        if spec is None:
            if callable(obj) or isinstance(obj, type):
                namespace.setdefault(name, obj)
            continue
        py_name, op_type, version, inputs, attrs = spec
        have = versions.get(op_type)
        if version or not have:                      # pinned to a set (internal operations) or not versioned: as is
            if not version.startswith("opset") or int(version[5:] or 0) <= number:
                namespace[name] = obj
            continue
        best = max((v for v in have if v <= number), default=None)
        if best is None:
            continue
        namespace[name] = _make_factory(py_name, op_type, "opset%d" % best, inputs, attrs)


# ---------------------------------------------------------------------------- factories that need hand-written logic
def if_op(condition, name: Optional[str] = None) -> "IfBuilder":
    return IfBuilder(condition, name)


class _SubgraphBuilder:
    """Shared port-map bookkeeping of If / Loop / TensorIterator builders.

    Port maps are stored as flat integer lists: ``input_map`` triples ``(node input, body parameter index, slice axis
    or -1)``, ``output_map`` pairs ``(body result index, concatenation axis or -1)`` in node-output order, and
    ``back_edges`` pairs ``(body result index, body parameter index)``. Sliced inputs and concatenated outputs walk
    their axis front to back, one element per iteration.
    """

    def __init__(self, op_type, inputs, name):
        self._type = op_type
        self._inputs = [as_output(i) for i in inputs]
        self._name = name
        self._bodies = []
        self._maps = {"input_map": [], "output_map": [], "else_input_map": [], "else_output_map": [], "back_edges": []}
        self._attrs = {}
        self._num_outputs = 0
        self._node = None

    def _add_input(self, value) -> int:
        o = as_output(value)
        for i, e in enumerate(self._inputs):
            if e == o:
                return i
        self._inputs.append(o)
        return len(self._inputs) - 1

    def _finish(self) -> Node:
        attrs = dict(self._attrs)
        for k, v in self._maps.items():
            attrs[k] = [int(x) for e in v for x in e]
        from . import _ovcore as _c
        from ._graph import _attr_to_core
        n = _c.make_node(self._type, "", [i._core() for i in self._inputs], {k: _attr_to_core(v) for k, v in attrs.items()}, False)
        n.set_bodies([b._m for b in self._bodies])
        n.validate()
        node = Node(n)
        if self._name:
            node.set_friendly_name(self._name)
        self._node = node
        return node


class IfBuilder(_SubgraphBuilder):
    """``If`` with then/else bodies: set bodies, map inputs/outputs, then ``build()``."""

    def __init__(self, condition, name=None):
        super().__init__("If", [condition], name)
        self._bodies = [None, None]

    def set_then_body(self, body: Model):
        self._bodies[0] = body

    def set_else_body(self, body: Model):
        self._bodies[1] = body

    def set_input(self, value, then_parameter: Optional[Node], else_parameter: Optional[Node]):
        port = self._add_input(value)
        if then_parameter is not None:
            self._maps["input_map"].append((port, self._bodies[0].get_parameter_index(then_parameter), -1))
        if else_parameter is not None:
            self._maps["else_input_map"].append((port, self._bodies[1].get_parameter_index(else_parameter), -1))

    def set_output(self, then_result: Node, else_result: Node) -> int:
        idx = self._num_outputs
        self._num_outputs += 1
        self._maps["output_map"].append((self._bodies[0].get_result_index(then_result), -1))
        self._maps["else_output_map"].append((self._bodies[1].get_result_index(else_result), -1))
        return idx

    def build(self) -> Node:
        return self._finish()


class LoopBuilder(_SubgraphBuilder):
    """``Loop`` (trip count + condition) or ``TensorIterator`` (``op_type="TensorIterator"``)."""

    def __init__(self, trip_count=None, execution_condition=None, name=None, op_type="Loop"):
        ins = [] if op_type == "TensorIterator" else [trip_count, execution_condition]
        super().__init__(op_type, ins, name)
        self._attrs = {"current_iteration_input": -1, "body_condition_output": -1}

    def set_function(self, body: Model):
        self._bodies = [body]

    set_body = set_function

    def set_special_body_ports(self, current_iteration_input: int, body_condition_output: int):
        self._attrs["current_iteration_input"] = int(current_iteration_input)
        self._attrs["body_condition_output"] = int(body_condition_output)

    def set_invariant_input(self, body_parameter: Node, value):
        port = self._add_input(value)
        self._maps["input_map"].append((port, self._bodies[0].get_parameter_index(body_parameter), -1))

    def set_merged_input(self, body_parameter: Node, initial_value, successive_value):
        port = self._add_input(initial_value)
        pidx = self._bodies[0].get_parameter_index(body_parameter)
        self._maps["input_map"].append((port, pidx, -1))
        ridx = self._bodies[0].get_result_index(as_output(successive_value))
        if ridx < 0:
            raise ValueError("the successive value is not a Result of the body")
        self._maps["back_edges"].append((ridx, pidx))

    def set_sliced_input(self, body_parameter: Node, value, start: int = 0, stride: int = 1, part_size: int = 1, end: int = -1, axis: int = 0):
        if (start, stride, part_size, end) != (0, 1, 1, -1):
            raise ValueError("sliced inputs walk the whole axis front to back, one element per iteration")
        port = self._add_input(value)
        self._maps["input_map"].append((port, self._bodies[0].get_parameter_index(body_parameter), int(axis)))

    def get_iter_value(self, body_value, iteration: int = -1) -> int:
        ridx = self._bodies[0].get_result_index(as_output(body_value))
        idx = self._num_outputs
        self._num_outputs += 1
        if iteration != -1:
            raise ValueError("only the value of the last iteration (-1) can be taken")
        self._maps["output_map"].append((ridx, -1))
        return idx

    def get_concatenated_slices(self, body_value, start: int = 0, stride: int = 1, part_size: int = 1, end: int = -1, axis: int = 0) -> int:
        if (start, stride, part_size, end) != (0, 1, 1, -1):
            raise ValueError("concatenated outputs collect every iteration front to back")
        ridx = self._bodies[0].get_result_index(as_output(body_value))
        idx = self._num_outputs
        self._num_outputs += 1
        self._maps["output_map"].append((ridx, int(axis)))
        return idx

    def build(self) -> Node:
        return self._finish()


def loop(trip_count, execution_condition, name=None) -> LoopBuilder:
    return LoopBuilder(trip_count, execution_condition, name)


def tensor_iterator(name=None) -> LoopBuilder:
    return LoopBuilder(name=name, op_type="TensorIterator")


def _internal(op_type, inputs, attrs, name=None):
    return make_op(op_type, [i for i in inputs if i is not None], attrs, name=name)


def rms_norm(data, gamma, epsilon: float = 1e-6, name=None) -> Node:
    """Fused RMS normalisation over the last axis (internal ``RMS`` op)."""
    return _internal("RMS", [data, gamma], {"epsilon": float(epsilon)}, name)


def rope(data, cos, sin, position_ids=None, name=None, **config) -> Node:
    """Fused rotary embedding (internal ``RoPE`` op); ``config`` holds the layout flags."""
    return _internal("RoPE", [data, cos, sin, position_ids], config, name)


def fully_connected(x, weight, bias=None, output_type="dynamic", name=None) -> Node:
    return _internal("FullyConnected", [x, weight, bias], {"output_type": Type(output_type)}, name)


def fully_connected_compressed(x, weight, bias, scale, zero_point=None, output_type="dynamic", name=None) -> Node:
    return _internal("FullyConnectedCompressed", [x, weight, bias, scale, zero_point], {"output_type": Type(output_type)}, name)


def paged_attention(inputs, write_kv_cache: bool = True, name=None) -> Node:
    """``PagedAttentionExtension``: 13 mandatory inputs (query, key, value, key_cache, value_cache, past_lens,
    subsequence_begins, block_indices, block_indices_begins, scale, sliding_window, alibi_slopes, max_context_len)
    and up to 28 with rotation / xattention / adaptive-RKV / sink / token-type inputs."""
    return make_op("PagedAttentionExtension", list(inputs), {"write_kv_cache": bool(write_kv_cache)}, name=name)


# re-exports so that ``from openvino_b200.opset import constant, parameter``
def type_relaxed(base_type: str, inputs, input_data_types=(), output_data_types=(), base_version: str = "", name=None, **attrs) -> Node:
    """``base_type`` applied to ``inputs`` with its type rules seeing ``input_data_types`` and its outputs declared as
    ``output_data_types`` (ov::op::TypeRelaxed<Base> of the reference, src/core/include/openvino/op/util/... ov_ops/type_relaxed.hpp).
    An empty string or "dynamic" in either list leaves that port as it is."""
    spell = lambda t: t if isinstance(t, str) else Type(t).get_type_name()
    a = dict(attrs, base_type=base_type, base_version=base_version, input_data_types=[spell(t) for t in input_data_types],
             output_data_types=[spell(t) for t in output_data_types])
    return make_op("TypeRelaxed", list(inputs), a, version="type_relaxed_opset", name=name)


__all__ = [n for n in dir() if not n.startswith("_")]
