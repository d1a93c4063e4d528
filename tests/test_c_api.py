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
