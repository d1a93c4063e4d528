"""C API: driven through ctypes and through a compiled C program (the hello_classification sample)."""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest

import openvino_b200 as ov
from openvino_b200 import build, opset as ops

PKG = os.path.dirname(os.path.abspath(ov.__file__))


class Shape(C.Structure):
    _fields_ = [("rank", C.c_int64), ("dims", C.POINTER(C.c_int64))]


class Dim(C.Structure):
    _fields_ = [("min", C.c_int64), ("max", C.c_int64)]


class PShape(C.Structure):
    _fields_ = [("rank", Dim), ("dims", C.POINTER(Dim))]


@pytest.fixture(scope="module")
def lib():
    path = build.build_capi()
    l = C.CDLL(str(path))
    l.ov_get_last_err_msg.restype = C.c_char_p
    l.ov_get_error_info.restype = C.c_char_p
    return l


@pytest.fixture(scope="module")
def model_path(tmp_path_factory):
    d = tmp_path_factory.mktemp("capi")
    x = ops.parameter([-1, 3, 8, 8], "f32", "image")
    w = ops.constant(np.random.default_rng(0).standard_normal((4, 3, 3, 3)).astype(np.float32))
    y = ops.relu(ops.convolution(x, w, [1, 1], [1, 1], [1, 1], [1, 1]))
    y = ops.reduce_mean(y, ops.constant(np.array([2, 3], dtype=np.int64)), False)
    y = ops.softmax(y, 1)
    y.output(0).set_names({"prob"})
    m = ov.Model([ops.result(y)], [x], "tiny_classifier")
    path = str(d / "tiny.xml")
    ov.serialize(m, path)
    return path


def check(lib, rc):
    assert rc == 0, (rc, lib.ov_get_error_info(rc), lib.ov_get_last_err_msg())


def test_read_reshape_compile_infer(lib, model_path):
    core, model, cm, req = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
    check(lib, lib.ov_core_create(C.byref(core)))
    check(lib, lib.ov_core_read_model(core, model_path.encode(), None, C.byref(model)))
    n = C.c_size_t()
    check(lib, lib.ov_model_inputs_size(model, C.byref(n)))
    assert n.value == 1 and lib.ov_model_is_dynamic(model)
    port = C.c_void_p()
    check(lib, lib.ov_model_const_input_by_name(model, b"image", C.byref(port)))
    name = C.c_char_p()
    check(lib, lib.ov_port_get_any_name(port, C.byref(name)))
    assert name.value == b"image"
    ps = PShape()
    check(lib, lib.ov_port_get_partial_shape(port, C.byref(ps)))
    assert ps.rank.max == 4 and ps.dims[0].max == -1 and ps.dims[1].min == 3
    # a dynamic port has no static shape
    sh = Shape()
    assert lib.ov_const_port_get_shape(port, C.byref(sh)) != 0
    dims = (C.c_int64 * 4)(2, 3, 8, 8)
    new_shape = PShape()
    check(lib, lib.ov_partial_shape_create_static(4, dims, C.byref(new_shape)))
    check(lib, lib.ov_model_reshape_input_by_name(model, b"image", new_shape))
    assert not lib.ov_model_is_dynamic(model)
    check(lib, lib.ov_core_compile_model(core, model, b"CPU", 2, C.byref(cm), b"PERF_COUNT", b"YES"))
    check(lib, lib.ov_compiled_model_create_infer_request(cm, C.byref(req)))
    x = np.random.default_rng(1).standard_normal((2, 3, 8, 8)).astype(np.float32)
    shape = Shape(4, dims)
    t_in, t_out = C.c_void_p(), C.c_void_p()
    check(lib, lib.ov_tensor_create_from_host_ptr(4, shape, x.ctypes.data_as(C.c_void_p), C.byref(t_in)))
    check(lib, lib.ov_infer_request_set_tensor(req, b"image", t_in))
    check(lib, lib.ov_infer_request_start_async(req))
    check(lib, lib.ov_infer_request_wait(req))
    check(lib, lib.ov_infer_request_get_tensor(req, b"prob", C.byref(t_out)))
    oshape = Shape()
    check(lib, lib.ov_tensor_get_shape(t_out, C.byref(oshape)))
    assert [oshape.dims[i] for i in range(oshape.rank)] == [2, 4]
    data = C.c_void_p()
    check(lib, lib.ov_tensor_data(t_out, C.byref(data)))
    got = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_float)), shape=(2, 4)).copy()
    ref = ov.compile_model(ov.Core().read_model(model_path), "CPU")(x)[0]
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-6)

    class Prof(C.Structure):
        _fields_ = [("infos", C.c_void_p), ("size", C.c_size_t)]
    prof = Prof()
    check(lib, lib.ov_infer_request_get_profiling_info(req, C.byref(prof)))
    assert prof.size > 0
    lib.ov_profiling_info_list_free(C.byref(prof))
    # export / import round trip
    blob = os.path.join(os.path.dirname(model_path), "tiny.blob")
    check(lib, lib.ov_compiled_model_export_model(cm, blob.encode()))
    content = open(blob, "rb").read()
    cm2 = C.c_void_p()
    check(lib, lib.ov_core_import_model(core, content, C.c_size_t(len(content)), b"CPU", C.byref(cm2)))
    # unknown device and wrong tensor type are reported, not crashed on
    bad = C.c_void_p()
    assert lib.ov_core_compile_model(core, model, b"NPU", 0, C.byref(bad)) == -5
    t_i32 = C.c_void_p()
    check(lib, lib.ov_tensor_create(9, shape, C.byref(t_i32)))
    assert lib.ov_infer_request_set_input_tensor(req, t_i32) == -4
    for t in (t_in, t_out, t_i32):
        lib.ov_tensor_free(t)
    lib.ov_infer_request_free(req)
    lib.ov_compiled_model_free(cm)
    lib.ov_compiled_model_free(cm2)
    lib.ov_output_const_port_free(port)
    lib.ov_model_free(model)
    lib.ov_core_free(core)


def test_preprocess_u8_nhwc(lib, model_path):
    core, model, pp, built, cm, req = (C.c_void_p() for _ in range(6))
    check(lib, lib.ov_core_create(C.byref(core)))
    check(lib, lib.ov_core_read_model(core, model_path.encode(), None, C.byref(model)))
    dims = (C.c_int64 * 4)(1, 3, 8, 8)
    s = PShape()
    check(lib, lib.ov_partial_shape_create_static(4, dims, C.byref(s)))
    check(lib, lib.ov_model_reshape_single_input(model, s))
    check(lib, lib.ov_preprocess_prepostprocessor_create(model, C.byref(pp)))
    check(lib, lib.ov_preprocess_prepostprocessor_set_input_element_type(pp, C.c_size_t(0), 16))   # U8
    check(lib, lib.ov_preprocess_prepostprocessor_set_input_nhwc(pp, C.c_size_t(0)))
    mean = (C.c_float * 3)(10, 20, 30)
    scale = (C.c_float * 3)(50, 60, 70)
    check(lib, lib.ov_preprocess_prepostprocessor_set_input_mean_scale(pp, C.c_size_t(0), mean, scale, C.c_size_t(3), C.c_int64(1)))
    check(lib, lib.ov_preprocess_prepostprocessor_build(pp, C.byref(built)))
    check(lib, lib.ov_core_compile_model(core, built, b"AUTO:CPU", 0, C.byref(cm)))
    check(lib, lib.ov_compiled_model_create_infer_request(cm, C.byref(req)))
    img = np.random.default_rng(2).integers(0, 255, (1, 8, 8, 3), dtype=np.uint8)
    hw = (C.c_int64 * 4)(1, 8, 8, 3)
    t_in, t_out = C.c_void_p(), C.c_void_p()
    check(lib, lib.ov_tensor_create_from_host_ptr(16, Shape(4, hw), img.ctypes.data_as(C.c_void_p), C.byref(t_in)))
    check(lib, lib.ov_infer_request_set_input_tensor(req, t_in))
    check(lib, lib.ov_infer_request_infer(req))
    check(lib, lib.ov_infer_request_get_output_tensor(req, C.byref(t_out)))
    data = C.c_void_p()
    check(lib, lib.ov_tensor_data(t_out, C.byref(data)))
    got = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_float)), shape=(1, 4)).copy()
    x = (img.astype(np.float32).transpose(0, 3, 1, 2) - np.array([10, 20, 30], np.float32).reshape(1, 3, 1, 1)) / np.array([50, 60, 70], np.float32).reshape(1, 3, 1, 1)
    ref = ov.compile_model(ov.Core().read_model(model_path), "CPU")(x)[0]
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-6)


def _load_static(lib, model_path):
    core, model = C.c_void_p(), C.c_void_p()
    check(lib, lib.ov_core_create(C.byref(core)))
    check(lib, lib.ov_core_read_model(core, model_path.encode(), None, C.byref(model)))
    dims = (C.c_int64 * 4)(1, 3, 8, 8)
    s = PShape()
    check(lib, lib.ov_partial_shape_create_static(4, dims, C.byref(s)))
    check(lib, lib.ov_model_reshape_single_input(model, s))
    return core, model


def _run_single(lib, core, model, array, et_code):
    cm, req, t_in, t_out, data = (C.c_void_p() for _ in range(5))
    check(lib, lib.ov_core_compile_model(core, model, b"CPU", 0, C.byref(cm)))
    check(lib, lib.ov_compiled_model_create_infer_request(cm, C.byref(req)))
    dims = (C.c_int64 * array.ndim)(*array.shape)
    check(lib, lib.ov_tensor_create_from_host_ptr(et_code, Shape(array.ndim, dims), array.ctypes.data_as(C.c_void_p), C.byref(t_in)))
    check(lib, lib.ov_infer_request_set_input_tensor(req, t_in))
    check(lib, lib.ov_infer_request_infer(req))
    check(lib, lib.ov_infer_request_get_output_tensor(req, C.byref(t_out)))
    check(lib, lib.ov_tensor_data(t_out, C.byref(data)))
    et = C.c_int()
    check(lib, lib.ov_tensor_get_element_type(t_out, C.byref(et)))
    return data, et.value


def test_preprocess_objects_resize_layout_mean_scale(lib, model_path):
    """The object-by-object interface (src/bindings/c/include/openvino/c/ov_prepostprocess.h): u8 NHWC 16x16 image ->
    f32, resize to the model's 8x8, NCHW, per-channel mean / scale; output converted to f16."""
    core, model = _load_static(lib, model_path)
    pp, info, tinfo, steps, minfo, oinfo, otinfo, lay_t, lay_m, built = (C.c_void_p() for _ in range(10))
    check(lib, lib.ov_preprocess_prepostprocessor_create(model, C.byref(pp)))
    check(lib, lib.ov_preprocess_prepostprocessor_get_input_info_by_name(pp, b"image", C.byref(info)))
    check(lib, lib.ov_preprocess_input_info_get_tensor_info(info, C.byref(tinfo)))
    check(lib, lib.ov_layout_create(b"NHWC", C.byref(lay_t)))
    check(lib, lib.ov_layout_create(b"[N,C,H,W]", C.byref(lay_m)))
    lib.ov_layout_to_string.restype = C.c_void_p
    text = lib.ov_layout_to_string(lay_m)
    assert C.string_at(text) == b"[N,C,H,W]"
    lib.ov_free(C.c_void_p(text))
    check(lib, lib.ov_preprocess_input_tensor_info_set_element_type(tinfo, 16))   # U8
    check(lib, lib.ov_preprocess_input_tensor_info_set_layout(tinfo, lay_t))
    check(lib, lib.ov_preprocess_input_tensor_info_set_spatial_static_shape(tinfo, C.c_size_t(16), C.c_size_t(16)))
    check(lib, lib.ov_preprocess_input_info_get_model_info(info, C.byref(minfo)))
    check(lib, lib.ov_preprocess_input_model_info_set_layout(minfo, lay_m))
    check(lib, lib.ov_preprocess_input_info_get_preprocess_steps(info, C.byref(steps)))
    check(lib, lib.ov_preprocess_preprocess_steps_convert_element_type(steps, 4))   # F32
    check(lib, lib.ov_preprocess_preprocess_steps_resize(steps, 2))                 # nearest
    check(lib, lib.ov_preprocess_preprocess_steps_convert_layout(steps, lay_m))
    mean = (C.c_float * 3)(10, 20, 30)
    scale = (C.c_float * 3)(50, 60, 70)
    check(lib, lib.ov_preprocess_preprocess_steps_mean_multi_channels(steps, mean, 3))
    check(lib, lib.ov_preprocess_preprocess_steps_scale_multi_channels(steps, scale, 3))
    check(lib, lib.ov_preprocess_prepostprocessor_get_output_info_by_index(pp, C.c_size_t(0), C.byref(oinfo)))
    check(lib, lib.ov_preprocess_output_info_get_tensor_info(oinfo, C.byref(otinfo)))
    check(lib, lib.ov_preprocess_output_set_element_type(otinfo, 3))                # F16
    check(lib, lib.ov_preprocess_prepostprocessor_build(pp, C.byref(built)))
    img = np.random.default_rng(5).integers(0, 255, (1, 16, 16, 3), dtype=np.uint8)
    data, et = _run_single(lib, core, built, img, 16)
    assert et == 3
    got = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint16)), shape=(1, 4)).copy().view(np.float16)
    x = img[:, ::2, ::2, :].astype(np.float32).transpose(0, 3, 1, 2)
    x = (x - np.array([10, 20, 30], np.float32).reshape(1, 3, 1, 1)) / np.array([50, 60, 70], np.float32).reshape(1, 3, 1, 1)
    ref = ov.compile_model(ov.Core().read_model(model_path), "CPU")(x)[0]
    np.testing.assert_allclose(got.astype(np.float32), ref, rtol=2e-3, atol=2e-3)
    for free, handle in ((lib.ov_preprocess_output_tensor_info_free, otinfo), (lib.ov_preprocess_output_info_free, oinfo),
                         (lib.ov_preprocess_preprocess_steps_free, steps), (lib.ov_preprocess_input_model_info_free, minfo),
                         (lib.ov_preprocess_input_tensor_info_free, tinfo), (lib.ov_preprocess_input_info_free, info),
                         (lib.ov_layout_free, lay_t), (lib.ov_layout_free, lay_m), (lib.ov_preprocess_prepostprocessor_free, pp)):
        free(handle)


def test_preprocess_objects_color_crop_pad_reverse(lib, model_path):
    """BGR input converted to RGB, scalar mean / scale, crop then pad back to 8x8, channels reversed."""
    core, model = _load_static(lib, model_path)
    pp, info, tinfo, steps, lay, built = (C.c_void_p() for _ in range(6))
    check(lib, lib.ov_preprocess_prepostprocessor_create(model, C.byref(pp)))
    check(lib, lib.ov_preprocess_prepostprocessor_get_input_info(pp, C.byref(info)))
    check(lib, lib.ov_preprocess_input_info_get_tensor_info(info, C.byref(tinfo)))
    check(lib, lib.ov_layout_create(b"NCHW", C.byref(lay)))
    check(lib, lib.ov_preprocess_input_tensor_info_set_layout(tinfo, lay))
    check(lib, lib.ov_preprocess_input_tensor_info_set_color_format(tinfo, 6))       # BGR
    assert lib.ov_preprocess_input_tensor_info_set_color_format(tinfo, 2) != 0       # two-plane NV12 is refused
    check(lib, lib.ov_preprocess_input_tensor_info_set_color_format(tinfo, 6))
    check(lib, lib.ov_preprocess_input_info_get_preprocess_steps(info, C.byref(steps)))
    check(lib, lib.ov_preprocess_preprocess_steps_convert_color(steps, 5))           # RGB
    check(lib, lib.ov_preprocess_preprocess_steps_mean(steps, C.c_float(0.5)))
    check(lib, lib.ov_preprocess_preprocess_steps_scale(steps, C.c_float(2.0)))
    begin = (C.c_int32 * 4)(0, 0, 1, 1)
    end = (C.c_int32 * 4)(1, 3, 7, 7)
    check(lib, lib.ov_preprocess_preprocess_steps_crop(steps, begin, 4, end, 4))
    pb = (C.c_int * 4)(0, 0, 1, 1)
    pe = (C.c_int * 4)(0, 0, 1, 1)
    check(lib, lib.ov_preprocess_preprocess_steps_pad(steps, pb, C.c_size_t(4), pe, C.c_size_t(4), C.c_float(0.25), 0))
    check(lib, lib.ov_preprocess_preprocess_steps_reverse_channels(steps))
    check(lib, lib.ov_preprocess_prepostprocessor_build(pp, C.byref(built)))
    img = np.random.default_rng(6).standard_normal((1, 3, 8, 8)).astype(np.float32)
    data, _ = _run_single(lib, core, built, img, 4)
    got = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_float)), shape=(1, 4)).copy()
    x = (img[:, ::-1] - 0.5) / 2.0
    x = np.pad(x[:, :, 1:7, 1:7], ((0, 0), (0, 0), (1, 1), (1, 1)), constant_values=0.25)[:, ::-1]
    ref = ov.compile_model(ov.Core().read_model(model_path), "CPU")(np.ascontiguousarray(x))[0]
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-6)


def test_preprocess_nv12_to_rgb(lib):
    """A single-plane NV12 image feeds a model that wants planar-last RGB."""
    x = ops.parameter([1, 4, 4, 3], "f32", "rgb")
    m = ov.Model([ops.result(ops.multiply(x, ops.constant(np.float32(1.0))))], [x], "copy")
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "copy.xml")
        ov.serialize(m, path)
        core, model = C.c_void_p(), C.c_void_p()
        check(lib, lib.ov_core_create(C.byref(core)))
        check(lib, lib.ov_core_read_model(core, path.encode(), None, C.byref(model)))
    pp, info, tinfo, steps, lay, built = (C.c_void_p() for _ in range(6))
    check(lib, lib.ov_preprocess_prepostprocessor_create(model, C.byref(pp)))
    check(lib, lib.ov_preprocess_prepostprocessor_get_input_info_by_index(pp, C.c_size_t(0), C.byref(info)))
    check(lib, lib.ov_preprocess_input_info_get_tensor_info(info, C.byref(tinfo)))
    check(lib, lib.ov_layout_create(b"NHWC", C.byref(lay)))
    check(lib, lib.ov_preprocess_input_tensor_info_set_layout(tinfo, lay))
    check(lib, lib.ov_preprocess_input_tensor_info_set_element_type(tinfo, 16))
    check(lib, lib.ov_preprocess_input_tensor_info_set_color_format(tinfo, 1))       # NV12, one plane
    check(lib, lib.ov_preprocess_input_info_get_preprocess_steps(info, C.byref(steps)))
    check(lib, lib.ov_preprocess_preprocess_steps_convert_color(steps, 5))
    check(lib, lib.ov_preprocess_prepostprocessor_build(pp, C.byref(built)))
    yuv = np.random.default_rng(7).integers(16, 235, (1, 6, 4, 1), dtype=np.uint8)
    data, _ = _run_single(lib, core, built, yuv, 16)
    got = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_float)), shape=(1, 4, 4, 3)).copy()
    p = ops.parameter([1, 6, 4, 1], "u8")
    ref = ov.compile_model(ov.Model([ops.result(ops.nv12_to_rgb(p))], [p]), "CPU")(yuv)[0]
    np.testing.assert_allclose(got, ref.astype(np.float32), atol=1e-5)


def test_string_tensor_ports_and_unavailable_calls(lib, model_path, tmp_path):
    core, model = _load_static(lib, model_path)
    t = C.c_void_p()
    words = (C.c_char_p * 3)(b"alpha", b"", b"gamma")
    dims = (C.c_int64 * 1)(3)
    check(lib, lib.ov_tensor_create_from_string_array(words, C.c_size_t(3), Shape(1, dims), C.byref(t)))
    et = C.c_int()
    check(lib, lib.ov_tensor_get_element_type(t, C.byref(et)))
    assert et.value == 23
    more = (C.c_char_p * 3)(b"x", b"y", b"z")
    check(lib, lib.ov_tensor_set_string_data(t, more, C.c_size_t(3)))
    assert lib.ov_tensor_set_string_data(t, more, C.c_size_t(2)) != 0
    bad = (C.c_int64 * 1)(2)
    assert lib.ov_tensor_create_from_string_array(words, C.c_size_t(3), Shape(1, bad), C.byref(C.c_void_p())) != 0

    # mutable ports: reshape by port, set / get a request's tensor by port
    port = C.c_void_p()
    check(lib, lib.ov_model_input(model, C.byref(port)))
    d2 = (C.c_int64 * 4)(2, 3, 8, 8)
    s = PShape()
    check(lib, lib.ov_partial_shape_create_static(4, d2, C.byref(s)))
    ports = (C.c_void_p * 1)(port)
    check(lib, lib.ov_model_reshape_by_ports(model, ports, C.byref(s), C.c_size_t(1)))
    cm, req, t_in, t_back = (C.c_void_p() for _ in range(4))
    check(lib, lib.ov_core_compile_model(core, model, b"CPU", 0, C.byref(cm)))
    check(lib, lib.ov_compiled_model_create_infer_request(cm, C.byref(req)))
    img = np.zeros((2, 3, 8, 8), np.float32)
    check(lib, lib.ov_tensor_create_from_host_ptr(4, Shape(4, d2), img.ctypes.data_as(C.c_void_p), C.byref(t_in)))
    check(lib, lib.ov_infer_request_set_tensor_by_port(req, port, t_in))
    check(lib, lib.ov_infer_request_get_tensor_by_port(req, port, C.byref(t_back)))
    shp = Shape()
    check(lib, lib.ov_tensor_get_shape(t_back, C.byref(shp)))
    assert [shp.dims[i] for i in range(shp.rank)] == [2, 3, 8, 8]

    # wide-character path
    lib.ov_core_read_model_unicode.argtypes = [C.c_void_p, C.c_wchar_p, C.c_wchar_p, C.POINTER(C.c_void_p)]
    m2 = C.c_void_p()
    check(lib, lib.ov_core_read_model_unicode(core, model_path, None, C.byref(m2)))
    n = C.c_size_t()
    check(lib, lib.ov_model_inputs_size(m2, C.byref(n)))
    assert n.value == 1

    # what the host device does not have answers with a status and a message, never a crash
    ctx = C.c_void_p()
    assert lib.ov_core_get_default_context(core, b"CPU", C.byref(ctx)) == -2
    assert b"remote context" in lib.ov_get_last_err_msg()
    assert lib.ov_compiled_model_get_context(cm, C.byref(ctx)) == -2
    assert lib.ov_core_add_extension(core, b"libnothing.so") == -2
    lib.ov_remote_context_free(None)
    CB = C.CFUNCTYPE(None, C.c_char_p)
    cb = CB(lambda msg: None)
    lib.ov_util_set_log_callback(cb)
    lib.ov_util_reset_log_callback()


def test_header_covers_reference_function_names(lib):
    """Every function below is named by the reference's C headers (src/bindings/c/include/openvino/c/*.h); the
    library must export each of them."""
    names = """ov_layout_create ov_layout_free ov_layout_to_string ov_core_add_extension ov_core_create_context
    ov_core_get_default_context ov_core_compile_model_with_context ov_compiled_model_get_context ov_remote_context_free
    ov_tensor_create_from_string_array ov_tensor_set_string_data ov_util_set_log_callback ov_util_reset_log_callback
    ov_infer_request_get_tensor_by_port ov_infer_request_set_tensor_by_port ov_model_reshape_by_ports
    ov_core_create_with_config_unicode ov_core_read_model_unicode ov_core_compile_model_from_file_unicode
    ov_preprocess_prepostprocessor_get_input_info ov_preprocess_prepostprocessor_get_output_info
    ov_preprocess_input_tensor_info_set_from ov_preprocess_input_tensor_info_set_memory_type
    ov_preprocess_input_tensor_info_set_color_format_with_subname""".split()
    for name in names:
        assert hasattr(lib, name), name


@pytest.mark.skipif(shutil.which("cc") is None and shutil.which("gcc") is None, reason="no C compiler")
def test_c_sample_builds_and_runs(lib, model_path, tmp_path):
    exe = str(tmp_path / "hello")
    src = os.path.join(os.path.dirname(PKG), "samples", "c", "hello_classification.c")
    cc = shutil.which("cc") or shutil.which("gcc")
    subprocess.check_call([cc, "-std=c99", "-Wall", "-Werror", src, "-I", os.path.join(PKG, "include"), "-L", os.path.join(PKG, "lib"),
                           "-lopenvino_b200_c", "-Wl,-rpath," + os.path.join(PKG, "lib"), "-o", exe])
    # static shape is required by the sample: write a reshaped copy of the model
    m = ov.Core().read_model(model_path)
    m.reshape([1, 3, 8, 8])
    static = str(tmp_path / "static.xml")
    ov.serialize(m, static)
    out = subprocess.run([exe, static], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    assert "top results (of 4)" in out.stdout and out.stdout.count("class ") == 3
