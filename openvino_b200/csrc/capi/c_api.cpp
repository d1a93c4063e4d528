// C API over the native core (see include/openvino_b200/c/openvino.h for the contract).
//
// Reference counterpart: src/bindings/c/src/*.cpp (ov_core.cpp, ov_model.cpp, ov_compiled_model.cpp,
// ov_infer_request.cpp, ov_tensor.cpp, ov_prepostprocess.cpp), which wrap the C++ API object by object. Here every
// handle owns a shared pointer into the native core; errors are caught at the boundary and turned into status codes,
// the message of the last error of the calling thread is kept for ov_get_last_err_msg.
#include <cstdarg>
#include <cstring>
#include <fstream>

#include "graph.hpp"
#include "ir.hpp"
#include "pass.hpp"
#include "runtime.hpp"
#include "../../include/openvino_b200/c/openvino.h"

using namespace ovc;

struct ov_core {
    std::map<std::string, std::map<std::string, std::string>> props;   // device -> key -> value
};
struct ov_model { ModelPtr m; };
struct ov_output_const_port { Output o; };
struct ov_output_port { Output o; };
struct ov_tensor { Tensor t; };
struct ov_compiled_model {
    ModelPtr m;
    std::map<std::string, std::string> props;
    std::shared_ptr<TaskExecutor> executor;
};
struct ov_infer_request {
    ModelPtr m;
    std::shared_ptr<TaskExecutor> executor;
    std::vector<Tensor> inputs, outputs;
    std::vector<Tensor> preset_outputs;
    std::shared_ptr<AsyncRequest> req;
    VariableStore vars;
    std::vector<std::pair<std::string, double>> prof;
    bool profile = false;
    int threads = 0;
    bool started = false;
};
struct ov_layout { std::string desc; };
// One step of an input's pre-processing, in the order the user asked for them
struct PpStep {
    enum Kind { RESIZE, SCALE, MEAN, CROP, CONVERT_LAYOUT, REVERSE_CHANNELS, CONVERT_ELEMENT_TYPE, CONVERT_COLOR, PAD } kind;
    std::vector<float> values;
    std::vector<int64_t> a, b;
    std::string text;
    int code = 0;
    float fill = 0;
};
struct PpInput {
    ET tensor_et = ET::dynamic;
    std::string tensor_layout, model_layout;
    int color = 0;                  // ov_color_format_e
    int64_t height = -1, width = -1;
    std::vector<PpStep> steps;
};
struct ov_preprocess_prepostprocessor {
    ModelPtr m;
    struct In { ET et = ET::dynamic; std::vector<float> mean, scale; int64_t axis = 1; bool nhwc = false; };
    std::map<size_t, In> ins;
    std::map<size_t, std::shared_ptr<PpInput>> inputs;      // the object-by-object interface of the reference
    std::map<size_t, ET> output_types;
};
struct ov_preprocess_input_info { std::shared_ptr<PpInput> in; };
struct ov_preprocess_input_tensor_info { std::shared_ptr<PpInput> in; };
struct ov_preprocess_preprocess_steps { std::shared_ptr<PpInput> in; };
struct ov_preprocess_input_model_info { std::shared_ptr<PpInput> in; };
struct ov_preprocess_output_info { ov_preprocess_prepostprocessor* pp; size_t index; };
struct ov_preprocess_output_tensor_info { ov_preprocess_prepostprocessor* pp; size_t index; };

namespace {

thread_local std::string g_last_error;

char* dup_str(const std::string& s) {
    char* p = static_cast<char*>(malloc(s.size() + 1));
    memcpy(p, s.c_str(), s.size() + 1);
    return p;
}

template <class F>
ov_status_e guarded(F&& f) {
    try {
        return f();
    } catch (const BusyError& e) {
        g_last_error = e.what();
        return REQUEST_BUSY;
    } catch (const CancelledError& e) {
        g_last_error = e.what();
        return INFER_CANCELLED;
    } catch (const std::out_of_range& e) {
        g_last_error = e.what();
        return OUT_OF_BOUNDS;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return GENERAL_ERROR;
    } catch (...) {
        g_last_error = "unknown exception";
        return UNKNOW_EXCEPTION;
    }
}

#define REQUIRE_PTR(...)                                          \
    do {                                                          \
        const void* ptrs_[] = {__VA_ARGS__};                      \
        for (const void* q_ : ptrs_)                              \
            if (!q_) { g_last_error = "null argument"; return INVALID_C_PARAM; } \
    } while (0)

bool resolves_to_cpu(const std::string& device) {
    // "CPU", "CPU.0", and the policy devices whose candidate list is CPU only (or empty: CPU is the only device here)
    std::string d = device;
    for (const char* pre : {"AUTO", "MULTI", "HETERO", "BATCH"}) {
        const std::string p(pre);
        if (d == p) return true;
        if (d.rfind(p + ":", 0) == 0) { d = d.substr(p.size() + 1); break; }
    }
    size_t start = 0;
    while (start <= d.size()) {
        size_t comma = d.find(',', start);
        std::string one = d.substr(start, comma == std::string::npos ? std::string::npos : comma - start);
        const size_t paren = one.find('(');
        if (paren != std::string::npos) one = one.substr(0, paren);
        if (!(one == "CPU" || one.rfind("CPU.", 0) == 0)) return false;
        if (comma == std::string::npos) break;
        start = comma + 1;
    }
    return true;
}

// Position of an axis letter in a layout string ("NCHW" -> C at 1); -1 when absent
int64_t layout_axis(const std::string& layout, char c) {
    const size_t p = layout.find(c);
    return p == std::string::npos ? -1 : (int64_t)p;
}

// Rebuild input `index` of `m` as: new Parameter (tensor type / layout / colour / spatial shape) -> the user's steps in
// order -> conversion to the model's layout and element type. Mirrors what the reference's PrePostProcessor::build adds.
void apply_input_preprocessing(const ModelPtr& m, size_t index, const PpInput& cfg) {
    NodePtr old = m->params[index];
    const ET model_et = old->outs[0].et;
    const PShape model_shape = old->outs[0].shape;
    OVC_CHECK(model_shape.rank_is_static(), "pre-processing needs an input of known rank");
    const size_t rank = model_shape.rank();
    std::string model_layout = cfg.model_layout, cur_layout = cfg.tensor_layout.empty() ? cfg.model_layout : cfg.tensor_layout;
    // tensor shape: the model's dims permuted into the tensor's layout, spatial extents replaced when given
    PShape tshape = model_shape;
    if (!cur_layout.empty() && !model_layout.empty() && cur_layout != model_layout) {
        OVC_CHECK(cur_layout.size() == rank && model_layout.size() == rank, "layouts must name every axis of the input");
        for (size_t i = 0; i < rank; ++i) {
            const int64_t src = layout_axis(model_layout, cur_layout[i]);
            OVC_CHECK(src >= 0, "tensor layout " << cur_layout << " and model layout " << model_layout << " name different axes");
            tshape.dims[i] = model_shape.dims[(size_t)src];
        }
    }
    const int64_t hp = layout_axis(cur_layout, 'H'), wp = layout_axis(cur_layout, 'W'), cp = layout_axis(cur_layout, 'C');
    if (cfg.height >= 0 && hp >= 0) tshape.dims[(size_t)hp] = Dim(cfg.height);
    if (cfg.width >= 0 && wp >= 0) tshape.dims[(size_t)wp] = Dim(cfg.width);
    const bool yuv = cfg.color == NV12_SINGLE_PLANE || cfg.color == I420_SINGLE_PLANE;
    if (yuv) {
        OVC_CHECK(hp >= 0 && cp >= 0, "a YUV input needs a tensor layout with H and C");
        if (tshape.dims[(size_t)hp].is_static()) tshape.dims[(size_t)hp] = Dim(tshape.dims[(size_t)hp].lo * 3 / 2);
        tshape.dims[(size_t)cp] = Dim(1);
    }
    NodePtr np = make_parameter(cfg.tensor_et == ET::dynamic ? model_et : cfg.tensor_et, tshape, old->name);
    np->outs[0].names = old->outs[0].names;
    Output cur = np->output(0);
    int color = cfg.color;
    auto to_float_first = [&] {
        if (!et_is_real(cur.et())) cur = make_node("Convert", "opset1", {cur}, {{"destination_type", Attr::Type(et_is_real(model_et) ? model_et : ET::f32)}})->output(0);
    };
    auto per_channel = [&](const std::vector<float>& v) {
        if (v.size() == 1) return make_constant_f32(v, Shape{}, cur.et())->output(0);
        const int64_t c = layout_axis(cur_layout, 'C');
        OVC_CHECK(c >= 0, "per-channel values need a layout with a C axis");
        Shape s(rank, 1);
        s[(size_t)c] = (int64_t)v.size();
        return make_constant_f32(v, s, cur.et())->output(0);
    };
    for (const PpStep& st : cfg.steps) {
        switch (st.kind) {
            case PpStep::CONVERT_ELEMENT_TYPE:
                cur = make_node("Convert", "opset1", {cur}, {{"destination_type", Attr::Type(static_cast<ET>(st.code))}})->output(0);
                break;
            case PpStep::CONVERT_COLOR: {
                const bool to_bgr = st.code == BGR;
                OVC_CHECK(st.code == RGB || st.code == BGR, "colour conversion targets RGB or BGR");
                if (color == NV12_SINGLE_PLANE) cur = make_node(to_bgr ? "NV12toBGR" : "NV12toRGB", "opset8", {cur})->output(0);
                else if (color == I420_SINGLE_PLANE) cur = make_node(to_bgr ? "I420toBGR" : "I420toRGB", "opset8", {cur})->output(0);
                else if ((color == RGB && to_bgr) || (color == BGR && !to_bgr)) {
                    const int64_t c = layout_axis(cur_layout, 'C');
                    OVC_CHECK(c >= 0, "RGB <-> BGR needs a layout with a C axis");
                    cur = make_node("Gather", "opset8", {cur, make_constant_i64({2, 1, 0})->output(0), make_constant_i64({c}, ET::i64, true)->output(0)})->output(0);
                } else OVC_CHECK(color == st.code, "this colour conversion is not available");
                color = st.code;
                break;
            }
            case PpStep::RESIZE: {
                const int64_t h = layout_axis(cur_layout, 'H'), w = layout_axis(cur_layout, 'W');
                OVC_CHECK(h >= 0 && w >= 0 && !model_layout.empty(), "resize needs tensor and model layouts with H and W");
                const Dim mh = model_shape.dims[(size_t)layout_axis(model_layout, 'H')], mw = model_shape.dims[(size_t)layout_axis(model_layout, 'W')];
                OVC_CHECK(mh.is_static() && mw.is_static(), "resize needs static spatial extents of the model input");
                to_float_first();
                const char* mode = st.code == RESIZE_LINEAR ? "linear" : (st.code == RESIZE_CUBIC ? "cubic" : "nearest");
                cur = make_node("Interpolate", "opset11", {cur, make_constant_i64({mh.lo, mw.lo})->output(0), make_constant_i64({h, w})->output(0)},
                                {{"mode", Attr::Str(mode)}, {"shape_calculation_mode", Attr::Str("sizes")},
                                 {"coordinate_transformation_mode", Attr::Str(st.code == RESIZE_NEAREST ? "asymmetric" : "half_pixel")},
                                 {"nearest_mode", Attr::Str("floor")}})->output(0);
                break;
            }
            case PpStep::CONVERT_LAYOUT: {
                OVC_CHECK(st.text.size() == rank && cur_layout.size() == rank, "convert_layout needs layouts that name every axis");
                std::vector<int64_t> order;
                for (char c : st.text) { const int64_t a = layout_axis(cur_layout, c); OVC_CHECK(a >= 0, "layout " << st.text << " names an axis the tensor lacks"); order.push_back(a); }
                cur = make_node("Transpose", "opset1", {cur, make_constant_i64(order)->output(0)})->output(0);
                cur_layout = st.text;
                break;
            }
            case PpStep::MEAN:
                to_float_first();
                cur = make_node("Subtract", "opset1", {cur, per_channel(st.values)})->output(0);
                break;
            case PpStep::SCALE:
                to_float_first();
                cur = make_node("Divide", "opset1", {cur, per_channel(st.values)})->output(0);
                break;
            case PpStep::REVERSE_CHANNELS: {
                const int64_t c = layout_axis(cur_layout, 'C');
                OVC_CHECK(c >= 0 && cur.shape().dims[(size_t)c].is_static(), "reverse_channels needs a static C axis");
                std::vector<int64_t> idx;
                for (int64_t k = cur.shape().dims[(size_t)c].lo; k-- > 0;) idx.push_back(k);
                cur = make_node("Gather", "opset8", {cur, make_constant_i64(idx)->output(0), make_constant_i64({c}, ET::i64, true)->output(0)})->output(0);
                break;
            }
            case PpStep::CROP: {
                std::vector<int64_t> step(st.a.size(), 1);
                cur = make_node("Slice", "opset8", {cur, make_constant_i64(st.a)->output(0), make_constant_i64(st.b)->output(0), make_constant_i64(step)->output(0)})->output(0);
                break;
            }
            case PpStep::PAD: {
                static const char* modes[] = {"constant", "edge", "reflect", "symmetric"};
                cur = make_node("Pad", "opset12", {cur, make_constant_i64(st.a)->output(0), make_constant_i64(st.b)->output(0), make_constant_f32({st.fill}, Shape{}, cur.et())->output(0)},
                                {{"pad_mode", Attr::Str(modes[st.code & 3])}})->output(0);
                break;
            }
        }
    }
    // what is left to reach the model's own input: layout, then element type
    if (!model_layout.empty() && !cur_layout.empty() && cur_layout != model_layout) {
        std::vector<int64_t> order;
        for (char c : model_layout) order.push_back(layout_axis(cur_layout, c));
        cur = make_node("Transpose", "opset1", {cur, make_constant_i64(order)->output(0)})->output(0);
    }
    if (cur.et() != model_et) cur = make_node("Convert", "opset1", {cur}, {{"destination_type", Attr::Type(model_et)}})->output(0);
    replace_output(old->output(0), cur);
    m->params[index] = np;
}

std::string port_name(const Output& o) {
    Output src = o;
    if (o.node->is_result()) src = o.node->input(0);
    const auto& names = src.node->outs.at(src.index).names;
    if (!names.empty()) return *names.begin();
    const auto& own = o.node->outs.at(o.index).names;
    if (!own.empty()) return *own.begin();
    return src.node->name;
}

bool port_has_name(const Output& o, const std::string& name) {
    Output src = o.node->is_result() ? o.node->input(0) : o;
    if (src.node->outs.at(src.index).names.count(name)) return true;
    if (o.node->outs.at(o.index).names.count(name)) return true;
    return src.node->name == name || o.node->name == name;
}

int find_port(const std::vector<NodePtr>& nodes, const std::string& name) {
    for (size_t i = 0; i < nodes.size(); ++i)
        if (port_has_name(Output(nodes[i], 0), name)) return (int)i;
    return -1;
}

void fill_shape(const Shape& s, ov_shape_t* out) {
    out->rank = (int64_t)s.size();
    out->dims = static_cast<int64_t*>(malloc(sizeof(int64_t) * (s.empty() ? 1 : s.size())));
    for (size_t i = 0; i < s.size(); ++i) out->dims[i] = s[i];
}

PShape to_pshape(const ov_partial_shape_t& ps) {
    if (ps.rank.min != ps.rank.max || ps.rank.max < 0) return PShape::dynamic();
    std::vector<Dim> dims;
    for (int64_t i = 0; i < ps.rank.max; ++i) {
        const auto& d = ps.dims[i];
        if (d.min == d.max && d.min >= 0) dims.emplace_back(d.min);
        else if (d.max < 0) dims.push_back(d.min > 0 ? Dim(d.min, -1) : Dim::dynamic());
        else dims.emplace_back(d.min < 0 ? 0 : d.min, d.max);
    }
    return PShape(dims);
}

void fill_pshape(const PShape& p, ov_partial_shape_t* out) {
    if (p.rank_dynamic) {
        out->rank = {-1, -1};
        out->dims = nullptr;
        return;
    }
    out->rank = {(int64_t)p.rank(), (int64_t)p.rank()};
    out->dims = static_cast<ov_dimension_t*>(malloc(sizeof(ov_dimension_t) * (p.rank() ? p.rank() : 1)));
    for (size_t i = 0; i < p.rank(); ++i) {
        const Dim& d = p.dims[i];
        if (d.is_static()) out->dims[i] = {d.lo, d.lo};
        else if (d.hi < 0) out->dims[i] = {d.lo > 0 ? d.lo : -1, -1};
        else out->dims[i] = {d.lo, d.hi};
    }
}

std::map<std::string, std::string> read_props(size_t n, va_list ap) {
    std::map<std::string, std::string> out;
    for (size_t i = 0; i + 1 < n; i += 2) {
        const char* k = va_arg(ap, const char*);
        const char* v = va_arg(ap, const char*);
        if (k && v) out[k] = v;
    }
    return out;
}

ov_status_e compile_impl(const ov_core_t* core, const ModelPtr& model, const char* device, const std::map<std::string, std::string>& props,
                         ov_compiled_model_t** out) {
    if (!resolves_to_cpu(device)) {
        g_last_error = std::string("device '") + device + "' is not available through the C API (available: CPU)";
        return NOT_FOUND;
    }
    auto cm = std::make_unique<ov_compiled_model>();
    cm->m = model->clone();
    run_moc_transformations(cm->m, true);
    auto it = core->props.find("CPU");
    if (it != core->props.end()) cm->props = it->second;
    for (auto& kv : props) cm->props[kv.first] = kv.second;
    int streams = 1;
    if (cm->props.count("NUM_STREAMS")) streams = std::max(1, atoi(cm->props["NUM_STREAMS"].c_str()));
    else if (cm->props.count("PERFORMANCE_HINT") && cm->props["PERFORMANCE_HINT"] == "THROUGHPUT") streams = 4;
    cm->props["NUM_STREAMS"] = std::to_string(streams);
    cm->executor = std::make_shared<TaskExecutor>(streams, "cpu_streams");
    *out = cm.release();
    return OK;
}

const char kBlobMagic[8] = {'O', 'V', 'B', '2', '0', '0', 'C', 'B'};

}  // namespace

extern "C" {

const char* ov_get_error_info(ov_status_e status) {
    switch (status) {
        case OK: return "success";
        case GENERAL_ERROR: return "general error";
        case NOT_IMPLEMENTED: return "not implemented";
        case NETWORK_NOT_LOADED: return "network not loaded";
        case PARAMETER_MISMATCH: return "parameter mismatch";
        case NOT_FOUND: return "not found";
        case OUT_OF_BOUNDS: return "out of bounds";
        case UNEXPECTED: return "unexpected";
        case REQUEST_BUSY: return "request busy";
        case RESULT_NOT_READY: return "result not ready";
        case NOT_ALLOCATED: return "not allocated";
        case INFER_NOT_STARTED: return "infer not started";
        case NETWORK_NOT_READ: return "network not read";
        case INFER_CANCELLED: return "infer cancelled";
        case INVALID_C_PARAM: return "invalid c input parameters";
        case UNKNOWN_C_ERROR: return "unknown c error";
        case NOT_IMPLEMENT_C_METHOD: return "not implement c method";
        case UNKNOW_EXCEPTION: return "unknown exception";
    }
    return "unknown status";
}
const char* ov_get_last_err_msg(void) { return dup_str(g_last_error); }
void ov_free(const char* content) { free(const_cast<char*>(content)); }

ov_status_e ov_get_openvino_version(ov_version_t* version) {
    REQUIRE_PTR(version);
    version->buildNumber = dup_str("2026.0.0-openvino_b200");
    version->description = dup_str("openvino_b200 C API");
    return OK;
}
void ov_version_free(ov_version_t* version) {
    if (!version) return;
    free(const_cast<char*>(version->buildNumber));
    free(const_cast<char*>(version->description));
    version->buildNumber = version->description = nullptr;
}
void ov_shutdown(void) {}

// ------------------------------------------------------------------------------------------------ shapes
ov_status_e ov_shape_create(const int64_t rank, const int64_t* dims, ov_shape_t* shape) {
    REQUIRE_PTR(shape);
    if (rank < 0 || (rank > 0 && !dims)) return INVALID_C_PARAM;
    Shape s(dims, dims + rank);
    fill_shape(s, shape);
    return OK;
}
ov_status_e ov_shape_free(ov_shape_t* shape) {
    REQUIRE_PTR(shape);
    free(shape->dims);
    shape->dims = nullptr;
    shape->rank = 0;
    return OK;
}
bool ov_dimension_is_dynamic(const ov_dimension_t dim) { return dim.min != dim.max || dim.max < 0; }
bool ov_rank_is_dynamic(const ov_rank_t rank) { return rank.min != rank.max || rank.max < 0; }
ov_status_e ov_partial_shape_create(const int64_t rank, const ov_dimension_t* dims, ov_partial_shape_t* out) {
    REQUIRE_PTR(out);
    if (rank < 0 || (rank > 0 && !dims)) return INVALID_C_PARAM;
    out->rank = {rank, rank};
    out->dims = static_cast<ov_dimension_t*>(malloc(sizeof(ov_dimension_t) * (rank ? rank : 1)));
    for (int64_t i = 0; i < rank; ++i) out->dims[i] = dims[i];
    return OK;
}
ov_status_e ov_partial_shape_create_dynamic(const ov_rank_t rank, const ov_dimension_t* dims, ov_partial_shape_t* out) {
    REQUIRE_PTR(out);
    if (ov_rank_is_dynamic(rank)) {
        out->rank = {-1, -1};
        out->dims = nullptr;
        return OK;
    }
    return ov_partial_shape_create(rank.max, dims, out);
}
ov_status_e ov_partial_shape_create_static(const int64_t rank, const int64_t* dims, ov_partial_shape_t* out) {
    REQUIRE_PTR(out);
    if (rank < 0 || (rank > 0 && !dims)) return INVALID_C_PARAM;
    out->rank = {rank, rank};
    out->dims = static_cast<ov_dimension_t*>(malloc(sizeof(ov_dimension_t) * (rank ? rank : 1)));
    for (int64_t i = 0; i < rank; ++i) out->dims[i] = {dims[i], dims[i]};
    return OK;
}
void ov_partial_shape_free(ov_partial_shape_t* ps) {
    if (!ps) return;
    free(ps->dims);
    ps->dims = nullptr;
}
ov_status_e ov_partial_shape_to_shape(const ov_partial_shape_t ps, ov_shape_t* shape) {
    REQUIRE_PTR(shape);
    return guarded([&] {
        const PShape p = to_pshape(ps);
        if (!p.is_static()) { g_last_error = "the partial shape is dynamic"; return PARAMETER_MISMATCH; }
        fill_shape(p.to_shape(), shape);
        return OK;
    });
}
ov_status_e ov_shape_to_partial_shape(const ov_shape_t shape, ov_partial_shape_t* ps) {
    return ov_partial_shape_create_static(shape.rank, shape.dims, ps);
}
bool ov_partial_shape_is_dynamic(const ov_partial_shape_t ps) { return to_pshape(ps).is_dynamic(); }
const char* ov_partial_shape_to_string(const ov_partial_shape_t ps) { return dup_str(to_pshape(ps).str()); }

// ------------------------------------------------------------------------------------------------ core
ov_status_e ov_core_create(ov_core_t** core) {
    REQUIRE_PTR(core);
    return guarded([&] {
        register_all_ops();
        *core = new ov_core();
        return OK;
    });
}
ov_status_e ov_core_create_with_config(const char* xml_config_file, ov_core_t** core) {
    (void)xml_config_file;   // the device registry is static: CPU
    return ov_core_create(core);
}
void ov_core_free(ov_core_t* core) { delete core; }

ov_status_e ov_core_read_model(const ov_core_t* core, const char* model_path, const char* bin_path, ov_model_t** model) {
    REQUIRE_PTR(core, model_path, model);
    return guarded([&] {
        auto m = read_model_files(model_path, bin_path ? bin_path : "");
        *model = new ov_model{m};
        return OK;
    });
}
ov_status_e ov_core_read_model_from_memory_buffer(const ov_core_t* core, const char* model_str, const size_t str_len, const ov_tensor_t* weights,
                                                  ov_model_t** model) {
    REQUIRE_PTR(core, model_str, model);
    return guarded([&] {
        BufferPtr w;
        if (weights) w = weights->t.buf;
        auto m = deserialize_model(std::string(model_str, str_len), w);
        *model = new ov_model{m};
        return OK;
    });
}
ov_status_e ov_core_compile_model(const ov_core_t* core, const ov_model_t* model, const char* device_name, const size_t property_args_size,
                                  ov_compiled_model_t** compiled_model, ...) {
    REQUIRE_PTR(core, model, device_name, compiled_model);
    va_list ap;
    va_start(ap, compiled_model);
    auto props = read_props(property_args_size, ap);
    va_end(ap);
    return guarded([&] { return compile_impl(core, model->m, device_name, props, compiled_model); });
}
ov_status_e ov_core_compile_model_from_file(const ov_core_t* core, const char* model_path, const char* device_name, const size_t property_args_size,
                                            ov_compiled_model_t** compiled_model, ...) {
    REQUIRE_PTR(core, model_path, device_name, compiled_model);
    va_list ap;
    va_start(ap, compiled_model);
    auto props = read_props(property_args_size, ap);
    va_end(ap);
    return guarded([&] { return compile_impl(core, read_model_files(model_path, ""), device_name, props, compiled_model); });
}
ov_status_e ov_core_set_property(const ov_core_t* core, const char* device_name, ...) {
    REQUIRE_PTR(core);
    va_list ap;
    va_start(ap, device_name);
    const char* k = va_arg(ap, const char*);
    const char* v = va_arg(ap, const char*);
    va_end(ap);
    if (!k || !v) return INVALID_C_PARAM;
    const_cast<ov_core_t*>(core)->props[device_name && *device_name ? device_name : "CPU"][k] = v;
    return OK;
}
ov_status_e ov_core_get_property(const ov_core_t* core, const char* device_name, const char* key, char** value) {
    REQUIRE_PTR(core, key, value);
    const std::string dev = device_name && *device_name ? device_name : "CPU";
    auto it = core->props.find(dev);
    if (it != core->props.end() && it->second.count(key)) { *value = dup_str(it->second.at(key)); return OK; }
    const std::string k(key);
    if (k == "FULL_DEVICE_NAME") { *value = dup_str("CPU reference executor (openvino_b200 native core)"); return OK; }
    if (k == "AVAILABLE_DEVICES") { *value = dup_str(""); return OK; }
    if (k == "SUPPORTED_PROPERTIES") { *value = dup_str("FULL_DEVICE_NAME AVAILABLE_DEVICES NUM_STREAMS INFERENCE_NUM_THREADS PERFORMANCE_HINT PERF_COUNT"); return OK; }
    if (k == "NUM_STREAMS") { *value = dup_str("1"); return OK; }
    if (k == "PERFORMANCE_HINT") { *value = dup_str("LATENCY"); return OK; }
    if (k == "INFERENCE_NUM_THREADS") { *value = dup_str("0"); return OK; }
    if (k == "PERF_COUNT") { *value = dup_str("NO"); return OK; }
    g_last_error = "unsupported property " + k;
    return NOT_FOUND;
}
ov_status_e ov_core_get_available_devices(const ov_core_t* core, ov_available_devices_t* devices) {
    REQUIRE_PTR(core, devices);
    devices->size = 1;
    devices->devices = static_cast<char**>(malloc(sizeof(char*)));
    devices->devices[0] = dup_str("CPU");
    return OK;
}
void ov_available_devices_free(ov_available_devices_t* devices) {
    if (!devices) return;
    for (size_t i = 0; i < devices->size; ++i) free(devices->devices[i]);
    free(devices->devices);
    devices->devices = nullptr;
    devices->size = 0;
}
ov_status_e ov_core_get_versions_by_device_name(const ov_core_t* core, const char* device_name, ov_core_version_list_t* versions) {
    REQUIRE_PTR(core, device_name, versions);
    if (!resolves_to_cpu(device_name)) return NOT_FOUND;
    versions->size = 1;
    versions->versions = static_cast<ov_core_version_t*>(malloc(sizeof(ov_core_version_t)));
    versions->versions[0].device_name = dup_str("CPU");
    versions->versions[0].version.buildNumber = dup_str("2026.0.0-openvino_b200");
    versions->versions[0].version.description = dup_str("openvino_b200_cpu_plugin");
    return OK;
}
void ov_core_versions_free(ov_core_version_list_t* versions) {
    if (!versions) return;
    for (size_t i = 0; i < versions->size; ++i) {
        free(const_cast<char*>(versions->versions[i].device_name));
        free(const_cast<char*>(versions->versions[i].version.buildNumber));
        free(const_cast<char*>(versions->versions[i].version.description));
    }
    free(versions->versions);
    versions->versions = nullptr;
    versions->size = 0;
}
ov_status_e ov_core_import_model(const ov_core_t* core, const char* content, const size_t content_size, const char* device_name,
                                 ov_compiled_model_t** compiled_model) {
    REQUIRE_PTR(core, content, device_name, compiled_model);
    return guarded([&] {
        if (content_size < 24 || memcmp(content, kBlobMagic, 8) != 0) { g_last_error = "not a compiled-model blob"; return PARAMETER_MISMATCH; }
        uint64_t xl, bl;
        memcpy(&xl, content + 8, 8);
        memcpy(&bl, content + 16, 8);
        if (24 + xl + bl > content_size) { g_last_error = "truncated blob"; return PARAMETER_MISMATCH; }
        auto buf = std::make_shared<Buffer>((size_t)bl);
        memcpy(buf->data, content + 24 + xl, bl);
        auto m = deserialize_model(std::string(content + 24, xl), buf);
        return compile_impl(core, m, device_name, {}, compiled_model);
    });
}

// ------------------------------------------------------------------------------------------------ model
void ov_model_free(ov_model_t* model) { delete model; }

#define PORT_GETTER(fn, PORT_T, list, idx_expr)                                       \
    REQUIRE_PTR(model, port);                                                         \
    return guarded([&] {                                                              \
        const auto& nodes = model->m->list;                                           \
        const long idx = (idx_expr);                                                  \
        if (idx < 0 || (size_t)idx >= nodes.size()) { g_last_error = "no such port"; return NOT_FOUND; } \
        *port = new PORT_T{Output(nodes[idx], 0)};                                    \
        return OK;                                                                    \
    })
#define SINGLE(list) (model->m->list.size() == 1 ? 0 : -1)

ov_status_e ov_model_const_input(const ov_model_t* model, ov_output_const_port_t** port) { PORT_GETTER(0, ov_output_const_port, params, SINGLE(params)); }
ov_status_e ov_model_const_input_by_name(const ov_model_t* model, const char* name, ov_output_const_port_t** port) {
    REQUIRE_PTR(name);
    PORT_GETTER(0, ov_output_const_port, params, find_port(model->m->params, name));
}
ov_status_e ov_model_const_input_by_index(const ov_model_t* model, const size_t index, ov_output_const_port_t** port) {
    PORT_GETTER(0, ov_output_const_port, params, (long)index);
}
ov_status_e ov_model_input(const ov_model_t* model, ov_output_port_t** port) { PORT_GETTER(0, ov_output_port, params, SINGLE(params)); }
ov_status_e ov_model_input_by_name(const ov_model_t* model, const char* name, ov_output_port_t** port) {
    REQUIRE_PTR(name);
    PORT_GETTER(0, ov_output_port, params, find_port(model->m->params, name));
}
ov_status_e ov_model_input_by_index(const ov_model_t* model, const size_t index, ov_output_port_t** port) { PORT_GETTER(0, ov_output_port, params, (long)index); }
ov_status_e ov_model_const_output(const ov_model_t* model, ov_output_const_port_t** port) { PORT_GETTER(0, ov_output_const_port, results, SINGLE(results)); }
ov_status_e ov_model_const_output_by_index(const ov_model_t* model, const size_t index, ov_output_const_port_t** port) {
    PORT_GETTER(0, ov_output_const_port, results, (long)index);
}
ov_status_e ov_model_const_output_by_name(const ov_model_t* model, const char* name, ov_output_const_port_t** port) {
    REQUIRE_PTR(name);
    PORT_GETTER(0, ov_output_const_port, results, find_port(model->m->results, name));
}
ov_status_e ov_model_output(const ov_model_t* model, ov_output_port_t** port) { PORT_GETTER(0, ov_output_port, results, SINGLE(results)); }
ov_status_e ov_model_output_by_index(const ov_model_t* model, const size_t index, ov_output_port_t** port) { PORT_GETTER(0, ov_output_port, results, (long)index); }
ov_status_e ov_model_output_by_name(const ov_model_t* model, const char* name, ov_output_port_t** port) {
    REQUIRE_PTR(name);
    PORT_GETTER(0, ov_output_port, results, find_port(model->m->results, name));
}
ov_status_e ov_model_inputs_size(const ov_model_t* model, size_t* n) {
    REQUIRE_PTR(model, n);
    *n = model->m->params.size();
    return OK;
}
ov_status_e ov_model_outputs_size(const ov_model_t* model, size_t* n) {
    REQUIRE_PTR(model, n);
    *n = model->m->results.size();
    return OK;
}
bool ov_model_is_dynamic(const ov_model_t* model) { return model && model->m->is_dynamic(); }

ov_status_e ov_model_reshape_by_port_indexes(const ov_model_t* model, const size_t* idx, const ov_partial_shape_t* shapes, size_t size) {
    REQUIRE_PTR(model, idx, shapes);
    return guarded([&] {
        std::map<size_t, PShape> m;
        for (size_t i = 0; i < size; ++i) m[idx[i]] = to_pshape(shapes[i]);
        model->m->reshape(m);
        return OK;
    });
}
ov_status_e ov_model_reshape(const ov_model_t* model, const char** names, const ov_partial_shape_t* shapes, size_t size) {
    REQUIRE_PTR(model, names, shapes);
    return guarded([&] {
        std::map<size_t, PShape> m;
        for (size_t i = 0; i < size; ++i) {
            const int k = find_port(model->m->params, names[i]);
            if (k < 0) { g_last_error = std::string("no input named ") + names[i]; return NOT_FOUND; }
            m[(size_t)k] = to_pshape(shapes[i]);
        }
        model->m->reshape(m);
        return OK;
    });
}
ov_status_e ov_model_reshape_input_by_name(const ov_model_t* model, const char* name, const ov_partial_shape_t shape) {
    return ov_model_reshape(model, &name, &shape, 1);
}
ov_status_e ov_model_reshape_single_input(const ov_model_t* model, const ov_partial_shape_t shape) {
    REQUIRE_PTR(model);
    if (model->m->params.size() != 1) { g_last_error = "the model has more than one input"; return PARAMETER_MISMATCH; }
    const size_t zero = 0;
    return ov_model_reshape_by_port_indexes(model, &zero, &shape, 1);
}
ov_status_e ov_model_get_friendly_name(const ov_model_t* model, char** name) {
    REQUIRE_PTR(model, name);
    *name = dup_str(model->m->name);
    return OK;
}
ov_status_e ov_model_save(const ov_model_t* model, const char* xml_path, bool compress_to_fp16) {
    REQUIRE_PTR(model, xml_path);
    return guarded([&] {
        ModelPtr m = model->m;
        if (compress_to_fp16) {
            m = m->clone();
            compress_model_to_f16(m);
        }
        save_model_files(*m, xml_path, "");
        return OK;
    });
}

// ------------------------------------------------------------------------------------------------ ports
ov_status_e ov_const_port_get_shape(const ov_output_const_port_t* port, ov_shape_t* shape) {
    REQUIRE_PTR(port, shape);
    return guarded([&] {
        const PShape& p = port->o.shape();
        if (!p.is_static()) { g_last_error = "the port has a dynamic shape " + p.str(); return PARAMETER_MISMATCH; }
        fill_shape(p.to_shape(), shape);
        return OK;
    });
}
ov_status_e ov_port_get_shape(const ov_output_port_t* port, ov_shape_t* shape) {
    REQUIRE_PTR(port, shape);
    ov_output_const_port c{port->o};
    return ov_const_port_get_shape(&c, shape);
}
ov_status_e ov_port_get_any_name(const ov_output_const_port_t* port, char** name) {
    REQUIRE_PTR(port, name);
    *name = dup_str(port_name(port->o));
    return OK;
}
ov_status_e ov_port_get_partial_shape(const ov_output_const_port_t* port, ov_partial_shape_t* ps) {
    REQUIRE_PTR(port, ps);
    fill_pshape(port->o.shape(), ps);
    return OK;
}
ov_status_e ov_port_get_element_type(const ov_output_const_port_t* port, ov_element_type_e* type) {
    REQUIRE_PTR(port, type);
    *type = static_cast<ov_element_type_e>(port->o.et());
    return OK;
}
void ov_output_port_free(ov_output_port_t* port) { delete port; }
void ov_output_const_port_free(ov_output_const_port_t* port) { delete port; }

// ------------------------------------------------------------------------------------------------ compiled model
#define CM_PORT(list, idx_expr)                                                       \
    REQUIRE_PTR(cm, port);                                                            \
    return guarded([&] {                                                              \
        const auto& nodes = cm->m->list;                                              \
        const long idx = (idx_expr);                                                  \
        if (idx < 0 || (size_t)idx >= nodes.size()) { g_last_error = "no such port"; return NOT_FOUND; } \
        *port = new ov_output_const_port{Output(nodes[idx], 0)};                      \
        return OK;                                                                    \
    })
ov_status_e ov_compiled_model_inputs_size(const ov_compiled_model_t* cm, size_t* n) {
    REQUIRE_PTR(cm, n);
    *n = cm->m->params.size();
    return OK;
}
ov_status_e ov_compiled_model_outputs_size(const ov_compiled_model_t* cm, size_t* n) {
    REQUIRE_PTR(cm, n);
    *n = cm->m->results.size();
    return OK;
}
ov_status_e ov_compiled_model_input(const ov_compiled_model_t* cm, ov_output_const_port_t** port) { CM_PORT(params, cm->m->params.size() == 1 ? 0 : -1); }
ov_status_e ov_compiled_model_input_by_index(const ov_compiled_model_t* cm, const size_t i, ov_output_const_port_t** port) { CM_PORT(params, (long)i); }
ov_status_e ov_compiled_model_input_by_name(const ov_compiled_model_t* cm, const char* name, ov_output_const_port_t** port) {
    REQUIRE_PTR(name);
    CM_PORT(params, find_port(cm->m->params, name));
}
ov_status_e ov_compiled_model_output(const ov_compiled_model_t* cm, ov_output_const_port_t** port) { CM_PORT(results, cm->m->results.size() == 1 ? 0 : -1); }
ov_status_e ov_compiled_model_output_by_index(const ov_compiled_model_t* cm, const size_t i, ov_output_const_port_t** port) { CM_PORT(results, (long)i); }
ov_status_e ov_compiled_model_output_by_name(const ov_compiled_model_t* cm, const char* name, ov_output_const_port_t** port) {
    REQUIRE_PTR(name);
    CM_PORT(results, find_port(cm->m->results, name));
}
ov_status_e ov_compiled_model_get_runtime_model(const ov_compiled_model_t* cm, ov_model_t** model) {
    REQUIRE_PTR(cm, model);
    return guarded([&] {
        *model = new ov_model{cm->m->clone()};
        return OK;
    });
}
ov_status_e ov_compiled_model_set_property(const ov_compiled_model_t* cm, ...) {
    REQUIRE_PTR(cm);
    va_list ap;
    va_start(ap, cm);
    const char* k = va_arg(ap, const char*);
    const char* v = va_arg(ap, const char*);
    va_end(ap);
    if (!k || !v) return INVALID_C_PARAM;
    const_cast<ov_compiled_model_t*>(cm)->props[k] = v;
    return OK;
}
ov_status_e ov_compiled_model_get_property(const ov_compiled_model_t* cm, const char* key, char** value) {
    REQUIRE_PTR(cm, key, value);
    const std::string k(key);
    if (cm->props.count(k)) { *value = dup_str(cm->props.at(k)); return OK; }
    if (k == "NETWORK_NAME") { *value = dup_str(cm->m->name); return OK; }
    if (k == "OPTIMAL_NUMBER_OF_INFER_REQUESTS") { *value = dup_str(std::to_string(cm->executor->num_threads())); return OK; }
    if (k == "EXECUTION_DEVICES") { *value = dup_str("CPU"); return OK; }
    g_last_error = "unsupported property " + k;
    return NOT_FOUND;
}
ov_status_e ov_compiled_model_export_model(const ov_compiled_model_t* cm, const char* path) {
    REQUIRE_PTR(cm, path);
    return guarded([&] {
        std::string xml, bin;
        serialize_model(*cm->m, xml, bin);
        std::ofstream f(path, std::ios::binary);
        if (!f) { g_last_error = std::string("cannot open ") + path; return GENERAL_ERROR; }
        const uint64_t xl = xml.size(), bl = bin.size();
        f.write(kBlobMagic, 8);
        f.write(reinterpret_cast<const char*>(&xl), 8);
        f.write(reinterpret_cast<const char*>(&bl), 8);
        f.write(xml.data(), xl);
        f.write(bin.data(), bl);
        return OK;
    });
}
void ov_compiled_model_free(ov_compiled_model_t* cm) { delete cm; }

ov_status_e ov_compiled_model_create_infer_request(const ov_compiled_model_t* cm, ov_infer_request_t** out) {
    REQUIRE_PTR(cm, out);
    return guarded([&] {
        auto r = std::make_unique<ov_infer_request>();
        r->m = cm->m;
        r->executor = cm->executor;
        r->inputs.resize(cm->m->params.size());
        r->outputs.resize(cm->m->results.size());
        r->preset_outputs.resize(cm->m->results.size());
        for (size_t i = 0; i < cm->m->params.size(); ++i) {
            const Output o(cm->m->params[i], 0);
            if (o.shape().is_static()) r->inputs[i] = Tensor(o.et(), o.shape().to_shape());
        }
        auto pc = cm->props.find("PERF_COUNT");
        r->profile = pc != cm->props.end() && (pc->second == "YES" || pc->second == "true" || pc->second == "1");
        auto nt = cm->props.find("INFERENCE_NUM_THREADS");
        if (nt != cm->props.end()) r->threads = atoi(nt->second.c_str());
        r->req = std::make_shared<AsyncRequest>();
        ov_infer_request* raw = r.get();
        r->req->set_pipeline({{r->executor, [raw] {
            for (size_t i = 0; i < raw->inputs.size(); ++i)
                OVC_CHECK(raw->inputs[i].defined(), "input " << i << " of the request has no tensor");
            EvalContext ctx;
            ctx.variables = &raw->vars;
            ctx.num_threads = raw->threads;
            raw->prof.clear();
            auto outs = evaluate_model(*raw->m, raw->inputs, ctx, raw->profile ? &raw->prof : nullptr);
            for (size_t i = 0; i < outs.size(); ++i) {
                Tensor& user = raw->preset_outputs[i];
                if (user.defined() && user.data() != outs[i].data()) {
                    OVC_CHECK(user.byte_size() == outs[i].byte_size(), "output tensor " << i << " set on the request has the wrong size");
                    memcpy(user.data(), outs[i].data(), outs[i].byte_size());
                    raw->outputs[i] = user;
                } else {
                    raw->outputs[i] = outs[i];
                }
            }
        }}});
        *out = r.release();
        return OK;
    });
}

// ------------------------------------------------------------------------------------------------ infer request
static ov_status_e set_input(ov_infer_request_t* r, long idx, const ov_tensor_t* t) {
    if (idx < 0 || (size_t)idx >= r->inputs.size()) { g_last_error = "no such input"; return NOT_FOUND; }
    const Output port(r->m->params[idx], 0);
    if (port.et() != ET::dynamic && port.et() != t->t.et) {
        g_last_error = std::string("element type of the tensor (") + et_name(t->t.et) + ") does not match the input (" + et_name(port.et()) + ")";
        return PARAMETER_MISMATCH;
    }
    if (!port.shape().compatible(PShape(t->t.shape))) {
        g_last_error = "shape of the tensor does not match the input " + port.shape().str();
        return PARAMETER_MISMATCH;
    }
    r->inputs[idx] = t->t;
    return OK;
}
static ov_status_e set_output(ov_infer_request_t* r, long idx, const ov_tensor_t* t) {
    if (idx < 0 || (size_t)idx >= r->outputs.size()) { g_last_error = "no such output"; return NOT_FOUND; }
    r->preset_outputs[idx] = t->t;
    return OK;
}
ov_status_e ov_infer_request_set_tensor(ov_infer_request_t* r, const char* name, const ov_tensor_t* t) {
    REQUIRE_PTR(r, name, t);
    return guarded([&] {
        const int i = find_port(r->m->params, name);
        if (i >= 0) return set_input(r, i, t);
        return set_output(r, find_port(r->m->results, name), t);
    });
}
ov_status_e ov_infer_request_set_tensor_by_const_port(ov_infer_request_t* r, const ov_output_const_port_t* port, const ov_tensor_t* t) {
    REQUIRE_PTR(r, port, t);
    return guarded([&] {
        for (size_t i = 0; i < r->m->params.size(); ++i)
            if (r->m->params[i] == port->o.node) return set_input(r, (long)i, t);
        for (size_t i = 0; i < r->m->results.size(); ++i)
            if (r->m->results[i] == port->o.node) return set_output(r, (long)i, t);
        g_last_error = "the port does not belong to the request's model";
        return NOT_FOUND;
    });
}
ov_status_e ov_infer_request_set_input_tensor_by_index(ov_infer_request_t* r, const size_t idx, const ov_tensor_t* t) {
    REQUIRE_PTR(r, t);
    return guarded([&] { return set_input(r, (long)idx, t); });
}
ov_status_e ov_infer_request_set_input_tensor(ov_infer_request_t* r, const ov_tensor_t* t) {
    REQUIRE_PTR(r, t);
    return guarded([&] { return set_input(r, r->inputs.size() == 1 ? 0 : -1, t); });
}
ov_status_e ov_infer_request_set_output_tensor_by_index(ov_infer_request_t* r, const size_t idx, const ov_tensor_t* t) {
    REQUIRE_PTR(r, t);
    return guarded([&] { return set_output(r, (long)idx, t); });
}
ov_status_e ov_infer_request_set_output_tensor(ov_infer_request_t* r, const ov_tensor_t* t) {
    REQUIRE_PTR(r, t);
    return guarded([&] { return set_output(r, r->outputs.size() == 1 ? 0 : -1, t); });
}
static ov_status_e get_tensor(const ov_infer_request_t* r, bool input, long idx, ov_tensor_t** out) {
    const auto& list = input ? r->inputs : r->outputs;
    if (idx < 0 || (size_t)idx >= list.size()) { g_last_error = "no such tensor"; return NOT_FOUND; }
    Tensor t = list[idx];
    if (!t.defined() && !input && r->preset_outputs[idx].defined()) t = r->preset_outputs[idx];
    if (!t.defined()) { g_last_error = "the tensor is not allocated yet (dynamic shape before the first inference)"; return NOT_ALLOCATED; }
    *out = new ov_tensor{t};
    return OK;
}
ov_status_e ov_infer_request_get_tensor(const ov_infer_request_t* r, const char* name, ov_tensor_t** t) {
    REQUIRE_PTR(r, name, t);
    return guarded([&] {
        const int i = find_port(r->m->params, name);
        if (i >= 0) return get_tensor(r, true, i, t);
        return get_tensor(r, false, find_port(r->m->results, name), t);
    });
}
ov_status_e ov_infer_request_get_tensor_by_const_port(const ov_infer_request_t* r, const ov_output_const_port_t* port, ov_tensor_t** t) {
    REQUIRE_PTR(r, port, t);
    return guarded([&] {
        for (size_t i = 0; i < r->m->params.size(); ++i)
            if (r->m->params[i] == port->o.node) return get_tensor(r, true, (long)i, t);
        for (size_t i = 0; i < r->m->results.size(); ++i)
            if (r->m->results[i] == port->o.node) return get_tensor(r, false, (long)i, t);
        g_last_error = "the port does not belong to the request's model";
        return NOT_FOUND;
    });
}
ov_status_e ov_infer_request_get_input_tensor_by_index(const ov_infer_request_t* r, const size_t idx, ov_tensor_t** t) {
    REQUIRE_PTR(r, t);
    return guarded([&] { return get_tensor(r, true, (long)idx, t); });
}
ov_status_e ov_infer_request_get_input_tensor(const ov_infer_request_t* r, ov_tensor_t** t) {
    REQUIRE_PTR(r, t);
    return guarded([&] { return get_tensor(r, true, r->inputs.size() == 1 ? 0 : -1, t); });
}
ov_status_e ov_infer_request_get_output_tensor_by_index(const ov_infer_request_t* r, const size_t idx, ov_tensor_t** t) {
    REQUIRE_PTR(r, t);
    return guarded([&] { return get_tensor(r, false, (long)idx, t); });
}
ov_status_e ov_infer_request_get_output_tensor(const ov_infer_request_t* r, ov_tensor_t** t) {
    REQUIRE_PTR(r, t);
    return guarded([&] { return get_tensor(r, false, r->outputs.size() == 1 ? 0 : -1, t); });
}
ov_status_e ov_infer_request_infer(ov_infer_request_t* r) {
    REQUIRE_PTR(r);
    return guarded([&] {
        r->started = true;
        r->req->infer();
        return OK;
    });
}
ov_status_e ov_infer_request_cancel(ov_infer_request_t* r) {
    REQUIRE_PTR(r);
    return guarded([&] {
        r->req->cancel();
        return OK;
    });
}
ov_status_e ov_infer_request_start_async(ov_infer_request_t* r) {
    REQUIRE_PTR(r);
    return guarded([&] {
        r->started = true;
        r->req->start_async();
        return OK;
    });
}
ov_status_e ov_infer_request_wait(ov_infer_request_t* r) {
    REQUIRE_PTR(r);
    return guarded([&] {
        if (!r->started) { g_last_error = "the request was not started"; return INFER_NOT_STARTED; }
        r->req->wait();
        return OK;
    });
}
ov_status_e ov_infer_request_wait_for(ov_infer_request_t* r, const int64_t timeout) {
    REQUIRE_PTR(r);
    return guarded([&] {
        if (!r->started) { g_last_error = "the request was not started"; return INFER_NOT_STARTED; }
        return r->req->wait_for(timeout) ? OK : RESULT_NOT_READY;
    });
}
ov_status_e ov_infer_request_set_callback(ov_infer_request_t* r, const ov_callback_t* cb) {
    REQUIRE_PTR(r, cb);
    const ov_callback_t c = *cb;
    r->req->set_callback([c](std::exception_ptr) { if (c.callback_func) c.callback_func(c.args); });
    return OK;
}
void ov_infer_request_free(ov_infer_request_t* r) {
    if (!r) return;
    try { r->req->stop_and_wait(); } catch (...) {}
    delete r;
}
ov_status_e ov_infer_request_get_profiling_info(const ov_infer_request_t* r, ov_profiling_info_list_t* list) {
    REQUIRE_PTR(r, list);
    list->size = r->prof.size();
    list->profiling_infos = static_cast<ov_profiling_info_t*>(calloc(list->size ? list->size : 1, sizeof(ov_profiling_info_t)));
    for (size_t i = 0; i < r->prof.size(); ++i) {
        auto& p = list->profiling_infos[i];
        p.status = ov_profiling_info_t::EXECUTED;
        p.real_time = p.cpu_time = (int64_t)r->prof[i].second;
        p.node_name = dup_str(r->prof[i].first);
        auto node = r->m->find_node(r->prof[i].first);
        p.node_type = dup_str(node ? node->type : "");
        p.exec_type = dup_str("ref");
    }
    return OK;
}
void ov_profiling_info_list_free(ov_profiling_info_list_t* list) {
    if (!list) return;
    for (size_t i = 0; i < list->size; ++i) {
        free(const_cast<char*>(list->profiling_infos[i].node_name));
        free(const_cast<char*>(list->profiling_infos[i].node_type));
        free(const_cast<char*>(list->profiling_infos[i].exec_type));
    }
    free(list->profiling_infos);
    list->profiling_infos = nullptr;
    list->size = 0;
}
ov_status_e ov_infer_request_reset_state(ov_infer_request_t* r) {
    REQUIRE_PTR(r);
    r->vars.reset();
    return OK;
}

// ------------------------------------------------------------------------------------------------ tensor
ov_status_e ov_tensor_create(const ov_element_type_e type, const ov_shape_t shape, ov_tensor_t** tensor) {
    REQUIRE_PTR(tensor);
    return guarded([&] {
        Tensor t(static_cast<ET>(type), Shape(shape.dims, shape.dims + shape.rank));
        if (t.buf) memset(t.buf->data, 0, t.buf->size);
        *tensor = new ov_tensor{t};
        return OK;
    });
}
ov_status_e ov_tensor_create_from_host_ptr(const ov_element_type_e type, const ov_shape_t shape, void* host_ptr, ov_tensor_t** tensor) {
    REQUIRE_PTR(tensor, host_ptr);
    return guarded([&] {
        const Shape s(shape.dims, shape.dims + shape.rank);
        const size_t bytes = et_byte_size(static_cast<ET>(type), (size_t)shape_size(s));
        auto buf = std::make_shared<Buffer>(static_cast<uint8_t*>(host_ptr), bytes, nullptr);
        *tensor = new ov_tensor{Tensor(static_cast<ET>(type), s, buf)};
        return OK;
    });
}
ov_status_e ov_tensor_set_shape(ov_tensor_t* tensor, const ov_shape_t shape) {
    REQUIRE_PTR(tensor);
    return guarded([&] {
        const Shape s(shape.dims, shape.dims + shape.rank);
        const size_t bytes = et_byte_size(tensor->t.et, (size_t)shape_size(s));
        if (!tensor->t.buf || bytes > tensor->t.buf->size) {
            if (tensor->t.buf && tensor->t.buf->owned.empty() && tensor->t.buf->size) {
                g_last_error = "a tensor over user memory cannot grow";
                return PARAMETER_MISMATCH;
            }
            tensor->t.buf = std::make_shared<Buffer>(bytes);
        }
        tensor->t.shape = s;
        return OK;
    });
}
ov_status_e ov_tensor_get_shape(const ov_tensor_t* tensor, ov_shape_t* shape) {
    REQUIRE_PTR(tensor, shape);
    fill_shape(tensor->t.shape, shape);
    return OK;
}
ov_status_e ov_tensor_get_element_type(const ov_tensor_t* tensor, ov_element_type_e* type) {
    REQUIRE_PTR(tensor, type);
    *type = static_cast<ov_element_type_e>(tensor->t.et);
    return OK;
}
ov_status_e ov_tensor_get_size(const ov_tensor_t* tensor, size_t* n) {
    REQUIRE_PTR(tensor, n);
    *n = (size_t)tensor->t.numel();
    return OK;
}
ov_status_e ov_tensor_get_byte_size(const ov_tensor_t* tensor, size_t* n) {
    REQUIRE_PTR(tensor, n);
    *n = tensor->t.byte_size();
    return OK;
}
ov_status_e ov_tensor_data(const ov_tensor_t* tensor, void** data) {
    REQUIRE_PTR(tensor, data);
    *data = tensor->t.data();
    return OK;
}
void ov_tensor_free(ov_tensor_t* tensor) { delete tensor; }

// ------------------------------------------------------------------------------------------------ pre-processing
ov_status_e ov_preprocess_prepostprocessor_create(const ov_model_t* model, ov_preprocess_prepostprocessor_t** pp) {
    REQUIRE_PTR(model, pp);
    *pp = new ov_preprocess_prepostprocessor{model->m, {}};
    return OK;
}
void ov_preprocess_prepostprocessor_free(ov_preprocess_prepostprocessor_t* pp) { delete pp; }
ov_status_e ov_preprocess_prepostprocessor_set_input_element_type(ov_preprocess_prepostprocessor_t* pp, size_t input, ov_element_type_e type) {
    REQUIRE_PTR(pp);
    pp->ins[input].et = static_cast<ET>(type);
    return OK;
}
ov_status_e ov_preprocess_prepostprocessor_set_input_mean_scale(ov_preprocess_prepostprocessor_t* pp, size_t input, const float* mean, const float* scale,
                                                                size_t channels, int64_t channel_axis) {
    REQUIRE_PTR(pp);
    auto& in = pp->ins[input];
    if (mean) in.mean.assign(mean, mean + channels);
    if (scale) in.scale.assign(scale, scale + channels);
    in.axis = channel_axis;
    return OK;
}
ov_status_e ov_preprocess_prepostprocessor_set_input_nhwc(ov_preprocess_prepostprocessor_t* pp, size_t input) {
    REQUIRE_PTR(pp);
    pp->ins[input].nhwc = true;
    return OK;
}
ov_status_e ov_preprocess_prepostprocessor_build(const ov_preprocess_prepostprocessor_t* pp, ov_model_t** model) {
    REQUIRE_PTR(pp, model);
    return guarded([&] {
        ModelPtr m = pp->m->clone();
        for (auto& kv : pp->ins) {
            if (kv.first >= m->params.size()) { g_last_error = "no such input"; return NOT_FOUND; }
            NodePtr old = m->params[kv.first];
            const auto& cfg = kv.second;
            const ET model_et = old->outs[0].et;
            PShape shape = old->outs[0].shape;
            const size_t rank = shape.rank_is_static() ? shape.rank() : 0;
            if (cfg.nhwc) {
                if (rank != 4) { g_last_error = "NHWC tensor layout needs a rank-4 input"; return PARAMETER_MISMATCH; }
                shape = PShape(std::vector<Dim>{shape.dims[0], shape.dims[2], shape.dims[3], shape.dims[1]});
            }
            NodePtr np = make_parameter(cfg.et == ET::dynamic ? model_et : cfg.et, shape, old->name);
            np->outs[0].names = old->outs[0].names;
            Output cur = np->output(0);
            if (cur.et() != model_et) cur = make_node("Convert", "opset1", {cur}, {{"destination_type", Attr::Type(model_et)}})->output(0);
            if (cfg.nhwc) cur = make_node("Transpose", "opset1", {cur, make_constant_i64({0, 3, 1, 2})->output(0)})->output(0);
            auto per_channel = [&](const std::vector<float>& v) {
                Shape s(rank ? rank : 1, 1);
                const int64_t ax = cfg.axis < 0 ? cfg.axis + (int64_t)s.size() : cfg.axis;
                s.at((size_t)ax) = (int64_t)v.size();
                return make_constant_f32(v, v.size() == 1 ? Shape{} : s, model_et)->output(0);
            };
            if (!cfg.mean.empty()) cur = make_node("Subtract", "opset1", {cur, per_channel(cfg.mean)})->output(0);
            if (!cfg.scale.empty()) cur = make_node("Divide", "opset1", {cur, per_channel(cfg.scale)})->output(0);
            replace_output(old->output(0), cur);
            m->params[kv.first] = np;
        }
        for (auto& kv : pp->inputs) {
            if (kv.first >= m->params.size()) { g_last_error = "no such input"; return NOT_FOUND; }
            apply_input_preprocessing(m, kv.first, *kv.second);
        }
        for (auto& kv : pp->output_types) {
            if (kv.first >= m->results.size()) { g_last_error = "no such output"; return NOT_FOUND; }
            NodePtr r = m->results[kv.first];
            Output src = r->input(0);
            if (src.et() != kv.second) r->set_input(0, make_node("Convert", "opset1", {src}, {{"destination_type", Attr::Type(kv.second)}})->output(0));
        }
        m->validate();
        *model = new ov_model{m};
        return OK;
    });
}

// ---- object-by-object interface: prepostprocessor -> input info -> tensor info / steps / model info; output info
static std::shared_ptr<PpInput> pp_input(const ov_preprocess_prepostprocessor_t* pp, size_t idx) {
    auto* p = const_cast<ov_preprocess_prepostprocessor_t*>(pp);
    auto& slot = p->inputs[idx];
    if (!slot) slot = std::make_shared<PpInput>();
    return slot;
}
ov_status_e ov_preprocess_prepostprocessor_get_input_info_by_index(const ov_preprocess_prepostprocessor_t* pp, const size_t idx, ov_preprocess_input_info_t** info) {
    REQUIRE_PTR(pp, info);
    if (idx >= pp->m->params.size()) { g_last_error = "no such input"; return NOT_FOUND; }
    *info = new ov_preprocess_input_info{pp_input(pp, idx)};
    return OK;
}
ov_status_e ov_preprocess_prepostprocessor_get_input_info(const ov_preprocess_prepostprocessor_t* pp, ov_preprocess_input_info_t** info) {
    REQUIRE_PTR(pp, info);
    if (pp->m->params.size() != 1) { g_last_error = "the model has more than one input: name it or give its index"; return PARAMETER_MISMATCH; }
    return ov_preprocess_prepostprocessor_get_input_info_by_index(pp, 0, info);
}
ov_status_e ov_preprocess_prepostprocessor_get_input_info_by_name(const ov_preprocess_prepostprocessor_t* pp, const char* name, ov_preprocess_input_info_t** info) {
    REQUIRE_PTR(pp, name, info);
    const int k = find_port(pp->m->params, name);
    if (k < 0) { g_last_error = std::string("no input named ") + name; return NOT_FOUND; }
    return ov_preprocess_prepostprocessor_get_input_info_by_index(pp, (size_t)k, info);
}
void ov_preprocess_input_info_free(ov_preprocess_input_info_t* p) { delete p; }
ov_status_e ov_preprocess_input_info_get_tensor_info(const ov_preprocess_input_info_t* info, ov_preprocess_input_tensor_info_t** t) {
    REQUIRE_PTR(info, t);
    *t = new ov_preprocess_input_tensor_info{info->in};
    return OK;
}
void ov_preprocess_input_tensor_info_free(ov_preprocess_input_tensor_info_t* p) { delete p; }
ov_status_e ov_preprocess_input_info_get_preprocess_steps(const ov_preprocess_input_info_t* info, ov_preprocess_preprocess_steps_t** steps) {
    REQUIRE_PTR(info, steps);
    *steps = new ov_preprocess_preprocess_steps{info->in};
    return OK;
}
void ov_preprocess_preprocess_steps_free(ov_preprocess_preprocess_steps_t* p) { delete p; }
ov_status_e ov_preprocess_input_info_get_model_info(const ov_preprocess_input_info_t* info, ov_preprocess_input_model_info_t** mi) {
    REQUIRE_PTR(info, mi);
    *mi = new ov_preprocess_input_model_info{info->in};
    return OK;
}
void ov_preprocess_input_model_info_free(ov_preprocess_input_model_info_t* p) { delete p; }
ov_status_e ov_preprocess_input_model_info_set_layout(ov_preprocess_input_model_info_t* mi, ov_layout_t* layout) {
    REQUIRE_PTR(mi, layout);
    mi->in->model_layout = layout->desc;
    return OK;
}
ov_status_e ov_preprocess_input_tensor_info_set_element_type(ov_preprocess_input_tensor_info_t* t, const ov_element_type_e type) {
    REQUIRE_PTR(t);
    t->in->tensor_et = static_cast<ET>(type);
    return OK;
}
ov_status_e ov_preprocess_input_tensor_info_set_layout(ov_preprocess_input_tensor_info_t* t, ov_layout_t* layout) {
    REQUIRE_PTR(t, layout);
    t->in->tensor_layout = layout->desc;
    return OK;
}
ov_status_e ov_preprocess_input_tensor_info_set_color_format(ov_preprocess_input_tensor_info_t* t, const ov_color_format_e fmt) {
    REQUIRE_PTR(t);
    if (fmt == NV12_TWO_PLANES || fmt == I420_THREE_PLANES) { g_last_error = "multi-plane colour formats are served through the single-plane forms here"; return NOT_IMPLEMENTED; }
    t->in->color = (int)fmt;
    return OK;
}
ov_status_e ov_preprocess_input_tensor_info_set_color_format_with_subname(ov_preprocess_input_tensor_info_t* t, const ov_color_format_e fmt, const size_t, ...) {
    return ov_preprocess_input_tensor_info_set_color_format(t, fmt);
}
ov_status_e ov_preprocess_input_tensor_info_set_spatial_static_shape(ov_preprocess_input_tensor_info_t* t, const size_t h, const size_t w) {
    REQUIRE_PTR(t);
    t->in->height = (int64_t)h;
    t->in->width = (int64_t)w;
    return OK;
}
ov_status_e ov_preprocess_input_tensor_info_set_memory_type(ov_preprocess_input_tensor_info_t* t, const char* mem_type) {
    REQUIRE_PTR(t, mem_type);
    return OK;             // host memory is the only kind of this library
}
ov_status_e ov_preprocess_input_tensor_info_set_from(ov_preprocess_input_tensor_info_t* t, const ov_tensor_t* tensor) {
    REQUIRE_PTR(t, tensor);
    t->in->tensor_et = tensor->t.et;
    // spatial extents follow the tensor's layout when one is set ('H' and 'W' positions), else NHWC is assumed for rank 4
    const Shape& s = tensor->t.shape;
    const std::string& lay = t->in->tensor_layout;
    const size_t hp = lay.find('H'), wp = lay.find('W');
    if (hp != std::string::npos && wp != std::string::npos && hp < s.size() && wp < s.size()) { t->in->height = s[hp]; t->in->width = s[wp]; }
    else if (s.size() == 4) { t->in->height = s[1]; t->in->width = s[2]; }
    return OK;
}
static ov_status_e add_step(ov_preprocess_preprocess_steps_t* st, PpStep step) {
    if (!st) { g_last_error = "null argument"; return INVALID_C_PARAM; }
    st->in->steps.push_back(std::move(step));
    return OK;
}
ov_status_e ov_preprocess_preprocess_steps_resize(ov_preprocess_preprocess_steps_t* st, const ov_preprocess_resize_algorithm_e alg) {
    PpStep s{PpStep::RESIZE};
    s.code = (int)alg;
    return add_step(st, s);
}
ov_status_e ov_preprocess_preprocess_steps_scale(ov_preprocess_preprocess_steps_t* st, float v) { PpStep s{PpStep::SCALE}; s.values = {v}; return add_step(st, s); }
ov_status_e ov_preprocess_preprocess_steps_scale_multi_channels(ov_preprocess_preprocess_steps_t* st, const float* v, const int32_t n) {
    REQUIRE_PTR(v);
    PpStep s{PpStep::SCALE};
    s.values.assign(v, v + n);
    return add_step(st, s);
}
ov_status_e ov_preprocess_preprocess_steps_mean(ov_preprocess_preprocess_steps_t* st, float v) { PpStep s{PpStep::MEAN}; s.values = {v}; return add_step(st, s); }
ov_status_e ov_preprocess_preprocess_steps_mean_multi_channels(ov_preprocess_preprocess_steps_t* st, const float* v, const int32_t n) {
    REQUIRE_PTR(v);
    PpStep s{PpStep::MEAN};
    s.values.assign(v, v + n);
    return add_step(st, s);
}
ov_status_e ov_preprocess_preprocess_steps_crop(ov_preprocess_preprocess_steps_t* st, int32_t* begin, int32_t bn, int32_t* end, int32_t en) {
    REQUIRE_PTR(begin, end);
    PpStep s{PpStep::CROP};
    s.a.assign(begin, begin + bn);
    s.b.assign(end, end + en);
    return add_step(st, s);
}
ov_status_e ov_preprocess_preprocess_steps_convert_layout(ov_preprocess_preprocess_steps_t* st, ov_layout_t* layout) {
    REQUIRE_PTR(layout);
    PpStep s{PpStep::CONVERT_LAYOUT};
    s.text = layout->desc;
    return add_step(st, s);
}
ov_status_e ov_preprocess_preprocess_steps_reverse_channels(ov_preprocess_preprocess_steps_t* st) { return add_step(st, PpStep{PpStep::REVERSE_CHANNELS}); }
ov_status_e ov_preprocess_preprocess_steps_convert_element_type(ov_preprocess_preprocess_steps_t* st, const ov_element_type_e type) {
    PpStep s{PpStep::CONVERT_ELEMENT_TYPE};
    s.code = (int)type;
    return add_step(st, s);
}
ov_status_e ov_preprocess_preprocess_steps_convert_color(ov_preprocess_preprocess_steps_t* st, const ov_color_format_e fmt) {
    PpStep s{PpStep::CONVERT_COLOR};
    s.code = (int)fmt;
    return add_step(st, s);
}
ov_status_e ov_preprocess_preprocess_steps_pad(const ov_preprocess_preprocess_steps_t* st, const int* const pb, size_t pbn, const int* const pe, size_t pen, float value,
                                               ov_padding_mode_e mode) {
    REQUIRE_PTR(pb, pe);
    PpStep s{PpStep::PAD};
    s.a.assign(pb, pb + pbn);
    s.b.assign(pe, pe + pen);
    s.fill = value;
    s.code = (int)mode;
    return add_step(const_cast<ov_preprocess_preprocess_steps_t*>(st), s);
}
ov_status_e ov_preprocess_prepostprocessor_get_output_info_by_index(const ov_preprocess_prepostprocessor_t* pp, const size_t idx, ov_preprocess_output_info_t** info) {
    REQUIRE_PTR(pp, info);
    if (idx >= pp->m->results.size()) { g_last_error = "no such output"; return NOT_FOUND; }
    *info = new ov_preprocess_output_info{const_cast<ov_preprocess_prepostprocessor_t*>(pp), idx};
    return OK;
}
ov_status_e ov_preprocess_prepostprocessor_get_output_info(const ov_preprocess_prepostprocessor_t* pp, ov_preprocess_output_info_t** info) {
    REQUIRE_PTR(pp, info);
    if (pp->m->results.size() != 1) { g_last_error = "the model has more than one output: name it or give its index"; return PARAMETER_MISMATCH; }
    return ov_preprocess_prepostprocessor_get_output_info_by_index(pp, 0, info);
}
ov_status_e ov_preprocess_prepostprocessor_get_output_info_by_name(const ov_preprocess_prepostprocessor_t* pp, const char* name, ov_preprocess_output_info_t** info) {
    REQUIRE_PTR(pp, name, info);
    const int k = find_port(pp->m->results, name);
    if (k < 0) { g_last_error = std::string("no output named ") + name; return NOT_FOUND; }
    return ov_preprocess_prepostprocessor_get_output_info_by_index(pp, (size_t)k, info);
}
void ov_preprocess_output_info_free(ov_preprocess_output_info_t* p) { delete p; }
ov_status_e ov_preprocess_output_info_get_tensor_info(const ov_preprocess_output_info_t* info, ov_preprocess_output_tensor_info_t** t) {
    REQUIRE_PTR(info, t);
    *t = new ov_preprocess_output_tensor_info{info->pp, info->index};
    return OK;
}
void ov_preprocess_output_tensor_info_free(ov_preprocess_output_tensor_info_t* p) { delete p; }
ov_status_e ov_preprocess_output_set_element_type(ov_preprocess_output_tensor_info_t* t, const ov_element_type_e type) {
    REQUIRE_PTR(t);
    t->pp->output_types[t->index] = static_cast<ET>(type);
    return OK;
}

// ---- layouts
ov_status_e ov_layout_create(const char* desc, ov_layout_t** layout) {
    REQUIRE_PTR(desc, layout);
    std::string d;
    for (const char* c = desc; *c; ++c)
        if (*c != '[' && *c != ']' && *c != ',' && *c != ' ') d.push_back((char)std::toupper((unsigned char)*c));
    if (d.empty()) { g_last_error = "empty layout"; return INVALID_C_PARAM; }
    *layout = new ov_layout{d};
    return OK;
}
void ov_layout_free(ov_layout_t* layout) { delete layout; }
const char* ov_layout_to_string(const ov_layout_t* layout) {
    if (!layout) return nullptr;
    std::string s = "[";
    for (size_t i = 0; i < layout->desc.size(); ++i) { if (i) s += ","; s.push_back(layout->desc[i]); }
    return dup_str(s + "]");
}

// ---- the remaining names of the reference headers
ov_status_e ov_tensor_create_from_string_array(const char** strings, const size_t n, const ov_shape_t shape, ov_tensor_t** tensor) {
    REQUIRE_PTR(strings, tensor);
    return guarded([&] {
        Shape s(shape.dims, shape.dims + shape.rank);
        Tensor t(ET::string, s);
        if ((size_t)t.numel() != n) { g_last_error = "the shape does not hold that many strings"; return PARAMETER_MISMATCH; }
        for (size_t i = 0; i < n; ++i) t.strings[i] = strings[i] ? strings[i] : "";
        *tensor = new ov_tensor{t};
        return OK;
    });
}
ov_status_e ov_tensor_set_string_data(ov_tensor_t* tensor, const char** strings, const size_t n) {
    REQUIRE_PTR(tensor, strings);
    if (tensor->t.et != ET::string || tensor->t.strings.size() != n) { g_last_error = "not a string tensor of that size"; return PARAMETER_MISMATCH; }
    for (size_t i = 0; i < n; ++i) tensor->t.strings[i] = strings[i] ? strings[i] : "";
    return OK;
}
ov_status_e ov_model_reshape_by_ports(const ov_model_t* model, const ov_output_port_t** ports, const ov_partial_shape_t* shapes, size_t size) {
    REQUIRE_PTR(model, ports, shapes);
    return guarded([&] {
        std::map<size_t, PShape> m;
        for (size_t i = 0; i < size; ++i) {
            bool found = false;
            for (size_t k = 0; k < model->m->params.size(); ++k)
                if (ports[i] && model->m->params[k] == ports[i]->o.node) { m[k] = to_pshape(shapes[i]); found = true; }
            if (!found) { g_last_error = "a port does not belong to the model's inputs"; return NOT_FOUND; }
        }
        model->m->reshape(m);
        return OK;
    });
}
ov_status_e ov_infer_request_set_tensor_by_port(ov_infer_request_t* r, const ov_output_port_t* port, const ov_tensor_t* t) {
    REQUIRE_PTR(r, port, t);
    // a port of the model the request was compiled from is matched by its tensor name, as the compiled copy has its own nodes
    ov_output_const_port cp{port->o};
    if (ov_infer_request_set_tensor_by_const_port(r, &cp, t) == OK) return OK;
    return ov_infer_request_set_tensor(r, port_name(port->o).c_str(), t);
}
ov_status_e ov_infer_request_get_tensor_by_port(const ov_infer_request_t* r, const ov_output_port_t* port, ov_tensor_t** t) {
    REQUIRE_PTR(r, port, t);
    ov_output_const_port cp{port->o};
    if (ov_infer_request_get_tensor_by_const_port(r, &cp, t) == OK) return OK;
    return ov_infer_request_get_tensor(r, port_name(port->o).c_str(), t);
}
// wide-character paths: converted to UTF-8 and handed to the narrow entry points
static std::string narrow(const wchar_t* w) {
    std::string out;
    for (; w && *w; ++w) {
        uint32_t c = (uint32_t)*w;
        if (c < 0x80) out.push_back((char)c);
        else if (c < 0x800) { out.push_back((char)(0xC0 | (c >> 6))); out.push_back((char)(0x80 | (c & 0x3F))); }
        else if (c < 0x10000) { out.push_back((char)(0xE0 | (c >> 12))); out.push_back((char)(0x80 | ((c >> 6) & 0x3F))); out.push_back((char)(0x80 | (c & 0x3F))); }
        else { out.push_back((char)(0xF0 | (c >> 18))); out.push_back((char)(0x80 | ((c >> 12) & 0x3F))); out.push_back((char)(0x80 | ((c >> 6) & 0x3F))); out.push_back((char)(0x80 | (c & 0x3F))); }
    }
    return out;
}
ov_status_e ov_core_create_with_config_unicode(const wchar_t* xml_config_file, ov_core_t** core) {
    return ov_core_create_with_config(xml_config_file ? narrow(xml_config_file).c_str() : nullptr, core);
}
ov_status_e ov_core_read_model_unicode(const ov_core_t* core, const wchar_t* model_path, const wchar_t* bin_path, ov_model_t** model) {
    REQUIRE_PTR(core, model_path, model);
    const std::string mp = narrow(model_path), bp = narrow(bin_path);
    return ov_core_read_model(core, mp.c_str(), bin_path ? bp.c_str() : nullptr, model);
}
ov_status_e ov_core_compile_model_from_file_unicode(const ov_core_t* core, const wchar_t* model_path, const char* device_name, const size_t property_args_size,
                                                    ov_compiled_model_t** compiled_model, ...) {
    REQUIRE_PTR(core, model_path, device_name, compiled_model);
    va_list ap;
    va_start(ap, compiled_model);
    auto props = read_props(property_args_size, ap);
    va_end(ap);
    return guarded([&] { return compile_impl(core, read_model_files(narrow(model_path), ""), device_name, props, compiled_model); });
}
ov_status_e ov_core_add_extension(const ov_core_t* core, const char* path) {
    REQUIRE_PTR(core, path);
    g_last_error = std::string("extension libraries are not loaded by this runtime: ") + path;
    return NOT_IMPLEMENTED;
}
// device memory contexts belong to devices with their own memory; the host device of this library has none
ov_status_e ov_core_create_context(const ov_core_t* core, const char* device, const size_t, ov_remote_context_t** ctx, ...) {
    REQUIRE_PTR(core, device, ctx);
    g_last_error = std::string("device ") + device + " has no remote context";
    return NOT_IMPLEMENTED;
}
ov_status_e ov_core_get_default_context(const ov_core_t* core, const char* device, ov_remote_context_t** ctx) {
    REQUIRE_PTR(core, device, ctx);
    g_last_error = std::string("device ") + device + " has no remote context";
    return NOT_IMPLEMENTED;
}
ov_status_e ov_compiled_model_get_context(const ov_compiled_model_t* cm, ov_remote_context_t** ctx) {
    REQUIRE_PTR(cm, ctx);
    g_last_error = "the host device has no remote context";
    return NOT_IMPLEMENTED;
}
ov_status_e ov_core_compile_model_with_context(const ov_core_t* core, const ov_model_t* model, const ov_remote_context_t* ctx, const size_t, ov_compiled_model_t** cm, ...) {
    REQUIRE_PTR(core, model, cm);
    (void)ctx;
    g_last_error = "the host device has no remote context";
    return NOT_IMPLEMENTED;
}
void ov_remote_context_free(ov_remote_context_t*) {}
static ov_status_e no_remote() { g_last_error = "the host device has no remote context"; return NOT_IMPLEMENTED; }
ov_status_e ov_remote_context_get_device_name(const ov_remote_context_t*, char**) { return no_remote(); }
ov_status_e ov_remote_context_get_params(const ov_remote_context_t*, size_t*, char**) { return no_remote(); }
ov_status_e ov_remote_context_create_tensor(const ov_remote_context_t*, const ov_element_type_e, const ov_shape_t, const size_t, ov_tensor_t**, ...) { return no_remote(); }
ov_status_e ov_remote_context_create_host_tensor(const ov_remote_context_t*, const ov_element_type_e, const ov_shape_t, ov_tensor_t**) { return no_remote(); }
ov_status_e ov_remote_tensor_get_params(ov_tensor_t*, size_t*, char**) { return no_remote(); }
ov_status_e ov_remote_tensor_get_device_name(ov_tensor_t*, char**) { return no_remote(); }
static void (*g_log_callback)(const char*) = nullptr;
void ov_util_set_log_callback(void (*callback)(const char*)) { g_log_callback = callback; }
void ov_util_reset_log_callback() { g_log_callback = nullptr; }

}  // extern "C"
