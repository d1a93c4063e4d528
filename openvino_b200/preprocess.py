"""Pre/post-processing embedded into the model graph (``ov.preprocess.PrePostProcessor``) and ``Layout``.

``PrePostProcessor(model)`` collects, per input, what the user tensor looks like (element type, layout, colour
format, spatial size), a list of steps (convert type / layout / colour, mean, scale, resize, crop, pad, custom)
and the layout the model expects; ``build()`` inserts the matching operations after new Parameters (and before
new Results for outputs) and returns the model.

Reference: src/core/src/preprocess/pre_post_process.cpp (build at :244), preprocess_steps_impl.cpp (one lambda per
step), color_utils.cpp; Layout: src/core/src/layout.cpp.
"""
from __future__ import annotations

import enum
import re
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

from . import opset as ops
from ._graph import Model, Node, Output, as_output, constant, parameter, result
from ._types import Dimension, PartialShape, Type


# ------------------------------------------------------------------------------------------------ Layout
class Layout:
    """Named dimensions: ``Layout("NCHW")``, ``Layout("N...C")``, ``Layout("[batch, ?, height, width]")``."""

    _ALIASES = {"BATCH": "N", "CHANNELS": "C", "CHANNEL": "C", "HEIGHT": "H", "WIDTH": "W", "DEPTH": "D"}

    def __init__(self, text: str = ""):
        if isinstance(text, Layout):
            self._left, self._right, self._dynamic = list(text._left), list(text._right), text._dynamic
            return
        text = text.strip()
        self._dynamic = False
        names: List[str] = []
        if text.startswith("["):
            if not text.endswith("]"):
                raise ValueError("bad layout '%s'" % text)
            names = [t.strip() for t in text[1:-1].split(",")] if text[1:-1].strip() else []
        else:
            i = 0
            while i < len(text):
                if text.startswith("...", i):
                    names.append("...")
                    i += 3
                else:
                    names.append(text[i])
                    i += 1
        names = [self._ALIASES.get(n.upper(), n.upper()) if n not in ("?", "...") else n for n in names]
        if names.count("...") > 1:
            raise ValueError("layout '%s' has more than one '...'" % text)
        for n in names:
            if n not in ("?", "...") and not re.fullmatch(r"[A-Z0-9_]+", n):
                raise ValueError("bad dimension name '%s' in layout '%s'" % (n, text))
        known = [n for n in names if n not in ("?", "...")]
        if len(set(known)) != len(known):
            raise ValueError("layout '%s' repeats a dimension name" % text)
        if "..." in names:
            k = names.index("...")
            self._left, self._right, self._dynamic = names[:k], names[k + 1:], True
        else:
            self._left, self._right = names, []

    @staticmethod
    def scalar() -> "Layout":
        return Layout("")

    def empty(self) -> bool:
        return not self._left and not self._right and not self._dynamic

    def has_name(self, name: str) -> bool:
        name = self._ALIASES.get(name.upper(), name.upper())
        return name in self._left or name in self._right

    def get_index_by_name(self, name: str) -> int:
        """Index from the front (>= 0) or, for names after '...', from the back (< 0)."""
        name = self._ALIASES.get(name.upper(), name.upper())
        if name in self._left:
            return self._left.index(name)
        if name in self._right:
            return self._right.index(name) - len(self._right)
        raise ValueError("layout %s has no dimension '%s'" % (self, name))

    def rank(self) -> Optional[int]:
        return None if self._dynamic else len(self._left)

    def names(self) -> List[str]:
        return self._left + (["..."] if self._dynamic else []) + self._right

    def to_string(self) -> str:
        if self.empty():
            return "[]"
        return "[" + ",".join(self.names()) + "]"

    def __eq__(self, other):
        if isinstance(other, str):
            other = Layout(other)
        return isinstance(other, Layout) and self.names() == other.names()

    def __hash__(self):
        return hash(tuple(self.names()))

    def __repr__(self):
        return "<Layout: %s>" % self.to_string()

    __str__ = to_string


class layout_helpers:
    @staticmethod
    def _idx(layout, name):
        return Layout(layout).get_index_by_name(name)

    @staticmethod
    def has_batch(layout): return Layout(layout).has_name("N")
    @staticmethod
    def batch_idx(layout): return layout_helpers._idx(layout, "N")
    @staticmethod
    def has_channels(layout): return Layout(layout).has_name("C")
    @staticmethod
    def channels_idx(layout): return layout_helpers._idx(layout, "C")
    @staticmethod
    def has_depth(layout): return Layout(layout).has_name("D")
    @staticmethod
    def depth_idx(layout): return layout_helpers._idx(layout, "D")
    @staticmethod
    def has_height(layout): return Layout(layout).has_name("H")
    @staticmethod
    def height_idx(layout): return layout_helpers._idx(layout, "H")
    @staticmethod
    def has_width(layout): return Layout(layout).has_name("W")
    @staticmethod
    def width_idx(layout): return layout_helpers._idx(layout, "W")

    @staticmethod
    def get_layout(port: Output) -> Layout:
        node = port.get_node()
        info = node.rt_info.get("layout_0")
        return Layout(info) if info else Layout()

    @staticmethod
    def set_layout(port: Output, layout) -> None:
        port.get_node().rt_info["layout_0"] = Layout(layout).to_string()


def _permutation(src: Layout, dst: Layout, rank: int) -> List[int]:
    """order such that transpose(x_in_src_layout, order) is in dst layout."""
    if src.empty() or dst.empty() or src == dst:
        return list(range(rank))
    s, d = src.names(), dst.names()
    if "..." in s or "..." in d or len(s) != len(d) or len(s) != rank:
        raise RuntimeError("cannot convert layout %s to %s for rank %d" % (src, dst, rank))
    if "?" in s or "?" in d or set(s) != set(d):
        raise RuntimeError("layouts %s and %s do not name the same dimensions" % (src, dst))
    return [s.index(n) for n in d]


# ------------------------------------------------------------------------------------------------ enums
class ColorFormat(enum.Enum):
    UNDEFINED = 0
    NV12_SINGLE_PLANE = 1
    NV12_TWO_PLANES = 2
    I420_SINGLE_PLANE = 3
    I420_THREE_PLANES = 4
    RGB = 5
    BGR = 6
    GRAY = 7
    RGBX = 8
    BGRX = 9


class ResizeAlgorithm(enum.Enum):
    RESIZE_LINEAR = 0
    RESIZE_CUBIC = 1
    RESIZE_NEAREST = 2
    RESIZE_BILINEAR_PILLOW = 3
    RESIZE_BICUBIC_PILLOW = 4


class PaddingMode(enum.Enum):
    CONSTANT = "constant"
    EDGE = "edge"
    REFLECT = "reflect"
    SYMMETRIC = "symmetric"


# ------------------------------------------------------------------------------------------------ info objects
class _TensorInfo:
    def __init__(self):
        self.element_type: Optional[Type] = None
        self.layout: Optional[Layout] = None
        self.color_format = ColorFormat.UNDEFINED
        self.sub_names: List[str] = []
        self.spatial: Optional[tuple] = None        # (h, w) static
        self.spatial_dynamic = False
        self.shape: Optional[PartialShape] = None
        self.memory_type: Optional[str] = None

    def set_element_type(self, t):
        self.element_type = Type(t)
        return self

    def set_layout(self, layout):
        self.layout = Layout(layout)
        return self

    def set_color_format(self, fmt: ColorFormat, sub_names: Sequence[str] = ()):
        self.color_format, self.sub_names = fmt, list(sub_names)
        return self

    def set_spatial_static_shape(self, height: int, width: int):
        self.spatial, self.spatial_dynamic = (int(height), int(width)), False
        return self

    def set_spatial_dynamic_shape(self):
        self.spatial, self.spatial_dynamic = None, True
        return self

    def set_shape(self, shape):
        self.shape = shape if isinstance(shape, PartialShape) else PartialShape(shape)
        return self

    def set_from(self, tensor):
        self.element_type = Type(tensor.element_type) if hasattr(tensor, "element_type") else Type.from_numpy(tensor.dtype)
        self.shape = PartialShape(list(tensor.shape))
        return self

    def set_memory_type(self, memory_type: str):
        self.memory_type = memory_type
        return self


class _ModelInfo:
    def __init__(self):
        self.layout: Optional[Layout] = None

    def set_layout(self, layout):
        self.layout = Layout(layout)
        return self


class _State:
    """What flows through the steps: the current values (one per colour plane), layout and colour format."""

    def __init__(self, values: List[Output], layout: Layout, color: ColorFormat):
        self.values, self.layout, self.color = values, layout, color

    @property
    def value(self) -> Output:
        if len(self.values) != 1:
            raise RuntimeError("this step needs a single-plane tensor: convert the colour format first")
        return self.values[0]


class _Steps:
    def __init__(self):
        self._steps: List[Callable[[_State, dict], None]] = []

    def _add(self, fn):
        self._steps.append(fn)
        return self

    # -- type / layout
    def convert_element_type(self, t=None):
        def step(st: _State, ctx):
            target = Type(t) if t is not None else ctx["model_type"]
            st.values = [v if v.get_element_type() == target else ops.convert(v, target).output(0) for v in st.values]
        return self._add(step)

    def convert_layout(self, dst=None):
        def step(st: _State, ctx):
            v = st.value
            rank = len(v.get_partial_shape())
            if isinstance(dst, (list, tuple)):
                order = list(dst)
                names = st.layout.names()
                new_layout = Layout("[" + ",".join(names[i] for i in order) + "]") if len(names) == len(order) and "..." not in names else st.layout
            else:
                target = Layout(dst) if dst is not None else ctx["model_layout"]
                if target is None or target.empty():
                    return
                order = _permutation(st.layout, target, rank)
                new_layout = target
            if order != list(range(rank)):
                st.values = [ops.transpose(v, np.array(order, dtype=np.int64)).output(0)]
            st.layout = new_layout
        return self._add(step)

    def reverse_channels(self):
        def step(st: _State, ctx):
            v = st.value
            axis = st.layout.get_index_by_name("C")
            c = v.get_partial_shape()[axis].get_length()
            idx = constant(np.arange(c - 1, -1, -1, dtype=np.int64))
            st.values = [ops.gather(v, idx, constant(np.array(axis, dtype=np.int64))).output(0)]
            if st.color in (ColorFormat.RGB, ColorFormat.BGR):
                st.color = ColorFormat.BGR if st.color == ColorFormat.RGB else ColorFormat.RGB
        return self._add(step)

    # -- arithmetic
    def _per_channel(self, st: _State, values) -> Output:
        v = st.value
        et = v.get_element_type()
        if not et.is_real():
            raise RuntimeError("mean/scale need a floating-point tensor: add convert_element_type(f32) before")
        if np.isscalar(values):
            return constant(np.array(values, dtype=np.float32), et).output(0)
        vals = np.asarray(values, dtype=np.float32)
        rank = len(v.get_partial_shape())
        axis = st.layout.get_index_by_name("C")
        if axis < 0:
            axis += rank
        shape = [1] * rank
        shape[axis] = vals.size
        return constant(vals.reshape(shape), et).output(0)

    def mean(self, values):
        def step(st: _State, ctx):
            st.values = [ops.subtract(st.value, self._per_channel(st, values)).output(0)]
        return self._add(step)

    def scale(self, values):
        def step(st: _State, ctx):
            st.values = [ops.divide(st.value, self._per_channel(st, values)).output(0)]
        return self._add(step)

    def clamp(self, min_value: float, max_value: float):
        return self._add(lambda st, ctx: setattr(st, "values", [ops.clamp(st.value, float(min_value), float(max_value)).output(0)]))

    def custom(self, fn: Callable[[Output], Output]):
        def step(st: _State, ctx):
            st.values = [as_output(fn(st.value))]
        return self._add(step)

    # -- geometry
    def resize(self, alg: ResizeAlgorithm, dst_height: Optional[int] = None, dst_width: Optional[int] = None):
        def step(st: _State, ctx):
            v = st.value
            rank = len(v.get_partial_shape())
            h_ax, w_ax = st.layout.get_index_by_name("H"), st.layout.get_index_by_name("W")
            h_ax, w_ax = (h_ax + rank) % rank, (w_ax + rank) % rank
            if dst_height is not None:
                h, w = int(dst_height), int(dst_width)
            else:
                ms, ml = ctx["model_shape"], ctx["model_layout"]
                if ml is None or ml.empty():
                    raise RuntimeError("resize() without a size needs the model layout")
                mh, mw = ms[ml.get_index_by_name("H")], ms[ml.get_index_by_name("W")]
                if mh.is_dynamic or mw.is_dynamic:
                    raise RuntimeError("resize() without a size needs static model height and width")
                h, w = mh.get_length(), mw.get_length()
            mode = {ResizeAlgorithm.RESIZE_LINEAR: "linear", ResizeAlgorithm.RESIZE_CUBIC: "cubic", ResizeAlgorithm.RESIZE_NEAREST: "nearest",
                    ResizeAlgorithm.RESIZE_BILINEAR_PILLOW: "bilinear_pillow", ResizeAlgorithm.RESIZE_BICUBIC_PILLOW: "bicubic_pillow"}[alg]
            ct = "asymmetric" if mode == "nearest" else "half_pixel"
            st.values = [ops.interpolate(v, np.array([h, w], dtype=np.int64), np.array([h_ax, w_ax], dtype=np.int64), mode, "sizes",
                                         [0] * rank, [0] * rank, ct, "floor").output(0)]
        return self._add(step)

    def crop(self, begin: Sequence[int], end: Sequence[int]):
        def step(st: _State, ctx):
            n = len(begin)
            st.values = [ops.slice(st.value, np.array(begin, dtype=np.int64), np.array(end, dtype=np.int64), np.ones(n, dtype=np.int64),
                                   np.arange(n, dtype=np.int64)).output(0)]
        return self._add(step)

    def pad(self, pads_begin: Sequence[int], pads_end: Sequence[int], value=0.0, mode: PaddingMode = PaddingMode.CONSTANT):
        def step(st: _State, ctx):
            v = st.value
            pv = constant(np.array(value), v.get_element_type())
            st.values = [ops.pad(v, np.array(pads_begin, dtype=np.int64), np.array(pads_end, dtype=np.int64), pv, mode.value).output(0)]
        return self._add(step)

    # -- colour
    def convert_color(self, dst: ColorFormat):
        def step(st: _State, ctx):
            _convert_color(st, dst)
        return self._add(step)


def _yuv_to_rgb(y: Output, u: Output, v: Output, et: Type) -> Output:
    """BT.601 limited-range YUV -> RGB on NHWC planes broadcast to the luma size; result clipped to [0, 255]."""
    f = lambda o: o if o.get_element_type() == Type.f32 else ops.convert(o, Type.f32).output(0)
    c = lambda x: constant(np.array(x, dtype=np.float32))
    yy = ops.multiply(ops.subtract(f(y), c(16.0)), c(1.164))
    uu = ops.subtract(f(u), c(128.0))
    vv = ops.subtract(f(v), c(128.0))
    r = ops.add(yy, ops.multiply(vv, c(1.596)))
    g = ops.subtract(ops.subtract(yy, ops.multiply(uu, c(0.391))), ops.multiply(vv, c(0.813)))
    b = ops.add(yy, ops.multiply(uu, c(2.018)))
    rgb = ops.clamp(ops.concat([r.output(0), g.output(0), b.output(0)], -1), 0.0, 255.0)
    if et.is_real():
        return rgb.output(0) if et == Type.f32 else ops.convert(rgb, et).output(0)
    return ops.convert(ops.round(rgb, "half_to_even"), et).output(0)


def _upsample2(x: Output) -> Output:
    """Nearest 2x upsample over H and W of an NHWC plane."""
    return ops.interpolate(x, np.array([2.0, 2.0], dtype=np.float32), np.array([1, 2], dtype=np.int64), "nearest", "scales",
                           [0, 0, 0, 0], [0, 0, 0, 0], "asymmetric", "floor").output(0)


def _convert_color(st: _State, dst: ColorFormat) -> None:
    src = st.color
    if src == dst:
        return
    if src in (ColorFormat.NV12_SINGLE_PLANE, ColorFormat.NV12_TWO_PLANES, ColorFormat.I420_SINGLE_PLANE, ColorFormat.I420_THREE_PLANES):
        if dst not in (ColorFormat.RGB, ColorFormat.BGR):
            raise RuntimeError("YUV input converts to RGB or BGR only")
        i64 = lambda v: constant(np.array(v, dtype=np.int64))
        et = st.values[0].get_element_type()
        if src in (ColorFormat.NV12_SINGLE_PLANE, ColorFormat.I420_SINGLE_PLANE):
            x = st.value                                   # [N, H*3/2, W, 1]
            shp = x.get_partial_shape()
            if shp[1].is_dynamic or shp[2].is_dynamic:
                raise RuntimeError("single-plane YUV conversion needs static height and width")
            h, w = shp[1].get_length() * 2 // 3, shp[2].get_length()
            y = ops.slice(x, i64([0]), i64([h]), i64([1]), i64([1])).output(0)
            rest = ops.slice(x, i64([h]), i64([h * 3 // 2]), i64([1]), i64([1])).output(0)
            if src == ColorFormat.NV12_SINGLE_PLANE:
                uv = ops.reshape(rest, i64([0, h // 2, w // 2, 2]), True).output(0)
                planes = [y, uv]
            else:
                flat = ops.reshape(rest, i64([0, 2, h // 2, w // 2]), True)
                u = ops.reshape(ops.slice(flat, i64([0]), i64([1]), i64([1]), i64([1])), i64([0, h // 2, w // 2, 1]), True).output(0)
                v = ops.reshape(ops.slice(flat, i64([1]), i64([2]), i64([1]), i64([1])), i64([0, h // 2, w // 2, 1]), True).output(0)
                planes = [y, u, v]
        else:
            planes = list(st.values)
        if len(planes) == 2:
            y, uv = planes
            u = ops.slice(uv, i64([0]), i64([1]), i64([1]), i64([3])).output(0)
            v = ops.slice(uv, i64([1]), i64([2]), i64([1]), i64([3])).output(0)
        else:
            y, u, v = planes
        rgb = _yuv_to_rgb(y, _upsample2(u), _upsample2(v), et)
        st.values, st.color, st.layout = [rgb], ColorFormat.RGB, Layout("NHWC")
        if dst == ColorFormat.BGR:
            _convert_color(st, ColorFormat.BGR)
        return
    v = st.value
    if st.layout.empty():
        raise RuntimeError("colour conversion needs the tensor layout (channels axis)")
    axis = st.layout.get_index_by_name("C")
    ax = constant(np.array(axis, dtype=np.int64))
    if src in (ColorFormat.RGBX, ColorFormat.BGRX):
        v = ops.gather(v, constant(np.array([0, 1, 2], dtype=np.int64)), ax).output(0)
        src = ColorFormat.RGB if src == ColorFormat.RGBX else ColorFormat.BGR
    if {src, dst} == {ColorFormat.RGB, ColorFormat.BGR}:
        v = ops.gather(v, constant(np.array([2, 1, 0], dtype=np.int64)), ax).output(0)
    elif dst == ColorFormat.GRAY and src in (ColorFormat.RGB, ColorFormat.BGR):
        et = v.get_element_type()
        f = v if et.is_real() else ops.convert(v, Type.f32).output(0)
        wts = [0.299, 0.587, 0.114] if src == ColorFormat.RGB else [0.114, 0.587, 0.299]
        rank = len(v.get_partial_shape())
        shape = [1] * rank
        shape[axis if axis >= 0 else axis + rank] = 3
        g = ops.reduce_sum(ops.multiply(f, constant(np.array(wts, dtype=np.float32).reshape(shape), f.get_element_type())), ax, True).output(0)
        v = g if et.is_real() else ops.convert(ops.round(g, "half_to_even"), et).output(0)
    elif src != dst:
        raise RuntimeError("colour conversion %s -> %s is not supported" % (src.name, dst.name))
    st.values, st.color = [v], dst


class PreProcessSteps(_Steps):
    pass


class PostProcessSteps(_Steps):
    pass


class InputInfo:
    def __init__(self):
        self._tensor, self._steps, self._model = _TensorInfo(), PreProcessSteps(), _ModelInfo()

    def tensor(self) -> _TensorInfo:
        return self._tensor

    def preprocess(self) -> PreProcessSteps:
        return self._steps

    def model(self) -> _ModelInfo:
        return self._model


class OutputInfo:
    def __init__(self):
        self._tensor, self._steps, self._model = _TensorInfo(), PostProcessSteps(), _ModelInfo()

    def tensor(self) -> _TensorInfo:
        return self._tensor

    def postprocess(self) -> PostProcessSteps:
        return self._steps

    def model(self) -> _ModelInfo:
        return self._model


_PLANES = {ColorFormat.NV12_TWO_PLANES: ("y", "uv"), ColorFormat.I420_THREE_PLANES: ("y", "u", "v")}


class PrePostProcessor:
    def __init__(self, model: Model):
        self._model = model
        self._inputs: Dict[int, InputInfo] = {}
        self._outputs: Dict[int, OutputInfo] = {}

    def input(self, key=None) -> InputInfo:
        idx = self._model.get_parameter_index(self._model.input(key).get_node())
        return self._inputs.setdefault(idx, InputInfo())

    def output(self, key=None) -> OutputInfo:
        port = self._model.output(key)
        idx = self._model.outputs.index(port)
        return self._outputs.setdefault(idx, OutputInfo())

    def build(self) -> Model:
        model = self._model
        params = model.get_parameters()
        new_params: List[Node] = []
        for idx, p in enumerate(params):
            info = self._inputs.get(idx)
            if info is None:
                new_params.append(p)
                continue
            new_params.extend(self._build_input(p, info))
        results = model.get_results()
        for idx, info in self._outputs.items():
            self._build_output(results[idx], info)
        # rebuild in place: swap parameters, keep results/sinks
        for p in params:
            if p not in new_params:
                model.remove_parameter(p)
        model.add_parameters([p for p in new_params if p not in params])
        # keep the user's parameter order
        model._m.params = [p._n for p in new_params]
        model.validate_nodes_and_infer_types()
        return model

    def _build_input(self, p: Node, info: InputInfo) -> List[Node]:
        t, m = info._tensor, info._model
        port = p.output(0)
        model_shape, model_type = port.get_partial_shape(), port.get_element_type()
        model_layout = m.layout or (layout_helpers.get_layout(port) if not layout_helpers.get_layout(port).empty() else None)
        tensor_layout = t.layout or model_layout or Layout()
        tensor_type = t.element_type or model_type
        color = t.color_format
        yuv = color in (ColorFormat.NV12_SINGLE_PLANE, ColorFormat.NV12_TWO_PLANES, ColorFormat.I420_SINGLE_PLANE, ColorFormat.I420_THREE_PLANES)
        if yuv:
            tensor_layout = Layout("NHWC")
        # shape of the new parameter(s): the model shape seen through the tensor layout, with the user's spatial size
        if t.shape is not None:
            shape = PartialShape(t.shape)
        else:
            shape = PartialShape(model_shape)
            if model_layout is not None and not tensor_layout.empty() and tensor_layout != model_layout and shape.rank.is_static:
                order = _permutation(model_layout, tensor_layout, len(shape))
                shape = PartialShape([shape[i] for i in order])
            if not tensor_layout.empty() and shape.rank.is_static and (t.spatial is not None or t.spatial_dynamic):
                h_ax, w_ax = tensor_layout.get_index_by_name("H"), tensor_layout.get_index_by_name("W")
                shape[h_ax] = Dimension(t.spatial[0]) if t.spatial else Dimension()
                shape[w_ax] = Dimension(t.spatial[1]) if t.spatial else Dimension()
        names = port.get_names()
        base = p.get_friendly_name()
        new_params: List[Node] = []
        if yuv:
            n_dim, h, w = shape[0], shape[1], shape[2]
            if color in (ColorFormat.NV12_SINGLE_PLANE, ColorFormat.I420_SINGLE_PLANE):
                hh = Dimension(h.get_length() * 3 // 2) if h.is_static else Dimension()
                planes = [("", PartialShape([n_dim, hh, w, Dimension(1)]))]
            elif color == ColorFormat.NV12_TWO_PLANES:
                half = lambda d: Dimension(d.get_length() // 2) if d.is_static else Dimension()
                planes = [("y", PartialShape([n_dim, h, w, Dimension(1)])), ("uv", PartialShape([n_dim, half(h), half(w), Dimension(2)]))]
            else:
                half = lambda d: Dimension(d.get_length() // 2) if d.is_static else Dimension()
                planes = [("y", PartialShape([n_dim, h, w, Dimension(1)])), ("u", PartialShape([n_dim, half(h), half(w), Dimension(1)])),
                          ("v", PartialShape([n_dim, half(h), half(w), Dimension(1)]))]
            subs = t.sub_names or [s for s, _ in planes]
            for (suffix, ps), sub in zip(planes, subs):
                np_ = parameter(ps, tensor_type, base + ("/" + sub if suffix else ""))
                np_.output(0).set_names({(n + "/" + sub) if suffix else n for n in names} or {np_.get_friendly_name()})
                new_params.append(np_)
        else:
            np_ = parameter(shape, tensor_type, base)
            np_.output(0).set_names(names)
            new_params.append(np_)
        for np_ in new_params:
            if not tensor_layout.empty():
                layout_helpers.set_layout(np_.output(0), tensor_layout)
        st = _State([q.output(0) for q in new_params], Layout(tensor_layout), color)
        ctx = {"model_type": model_type, "model_layout": model_layout, "model_shape": model_shape}
        for step in info._steps._steps:
            step(st, ctx)
        # implicit conversions to what the model expects
        if model_layout is not None and not st.layout.empty() and st.layout != model_layout:
            PreProcessSteps().convert_layout(model_layout)._steps[0](st, ctx)
        v = st.value
        if model_type.is_static() and v.get_element_type() != model_type:
            v = ops.convert(v, model_type).output(0)
        if not model_shape.compatible(v.get_partial_shape()):
            raise RuntimeError("preprocessing of input '%s' gives shape %s, the model expects %s" % (base, v.get_partial_shape(), model_shape))
        port.set_names(set())
        port.replace(v)
        return new_params

    def _build_output(self, res: Node, info: OutputInfo) -> None:
        src = res.input_value(0)
        t, m = info._tensor, info._model
        model_layout = m.layout or Layout()
        st = _State([src], Layout(model_layout), ColorFormat.UNDEFINED)
        ctx = {"model_type": t.element_type or src.get_element_type(), "model_layout": t.layout, "model_shape": src.get_partial_shape()}
        for step in info._steps._steps:
            step(st, ctx)
        if t.layout is not None and not st.layout.empty() and st.layout != t.layout:
            PostProcessSteps().convert_layout(t.layout)._steps[0](st, ctx)
        v = st.value
        if t.element_type is not None and v.get_element_type() != t.element_type:
            v = ops.convert(v, t.element_type).output(0)
        if v != src:
            names = src.get_names()
            src.set_names(set())
            v.set_names(names)
            res.input(0).replace_source_output(v)
        if t.layout is not None:
            layout_helpers.set_layout(res.output(0), t.layout)

    def __repr__(self):
        return "<PrePostProcessor: %d input(s), %d output(s) configured>" % (len(self._inputs), len(self._outputs))
