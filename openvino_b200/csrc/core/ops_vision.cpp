// Image / detection helpers of the operation set: colour conversion from NV12 and I420, prior boxes for clustered
// anchors, position-sensitive ROI pooling, emulated fp8 conversion and the sparse "fill empty rows" helper: attribute
// schemas (reference visit_attributes order), shape / type inference, reference evaluation.
//
// Reference counterparts: src/core/src/op/{nv12_to_rgb,nv12_to_bgr,i420_to_rgb,i420_to_bgr,prior_box_clustered,
// psroi_pooling,fake_convert,sparse_fill_empty_rows}.cpp and the kernels of the same names under
// src/core/reference/include/openvino/reference/ (convert_color_nv12.hpp holds both colour conversions).
#include <algorithm>
#include <cmath>
#include <limits>

#include "graph.hpp"

namespace ovc {

namespace {

using K = Attr::Kind;
using N = const Node&;
using Ins = const std::vector<Tensor>&;
using Outs = std::vector<Tensor>&;
using C = EvalContext&;

AttrSpec A(const char* name, K kind, Attr def) {
    AttrSpec s;
    s.name = name;
    s.kind = kind;
    s.def = std::move(def);
    return s;
}
AttrSpec Ai(const char* n, int64_t d = 0) { return A(n, K::INT, Attr::Int(d)); }
AttrSpec Ab(const char* n, bool d = false) { return A(n, K::BOOL, Attr::Bool(d)); }
AttrSpec Af(const char* n, double d = 0, bool f32 = true) { AttrSpec s = A(n, K::FLOAT, Attr::Float(d)); s.f32 = f32; return s; }
AttrSpec As(const char* n, const char* d = "") { return A(n, K::STR, Attr::Str(d)); }
AttrSpec Afs(const char* n, std::vector<double> d = {}) { return A(n, K::FLOATS, Attr::Floats(std::move(d))); }

void reg(const char* type, const char* version, std::vector<AttrSpec> attrs, InferFn infer, EvalFn eval, int min_in, int max_in) {
    OpSchema s;
    s.type = type;
    s.version = version;
    s.attrs = std::move(attrs);
    s.infer = std::move(infer);
    s.eval = std::move(eval);
    s.min_inputs = min_in;
    s.max_inputs = max_in;
    OpRegistry::get().add(std::move(s));
}

// BT.601 limited range: the coefficients that the reference's plugins agree on
void yuv_to_rgb(float y, float u, float v, bool integral, float* rgb) {
    const float c = y - 16.f, d = u - 128.f, e = v - 128.f;
    auto clip = [&](float a) { return std::min(std::max(integral ? std::round(a) : a, 0.f), 255.f); };
    rgb[0] = clip(1.164f * c + 1.596f * e);
    rgb[1] = clip(1.164f * c - 0.391f * d - 0.813f * e);
    rgb[2] = clip(1.164f * c + 2.018f * d);
}

// planes: 1 (whole frame in one tensor of height 3H/2), 2 (NV12: Y + interleaved UV) or 3 (I420: Y, U, V)
void infer_color(Node& n, int max_planes) {
    const PShape& y = n.in_shape(0);
    if (y.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic(4)); return; }
    OVC_CHECK(y.dims.size() == 4, n.description() << ": [N, H, W, C] input expected");
    PShape o = y;
    o.dims[3] = Dim(3);
    if (n.num_inputs() == 1) {
        if (y.dims[1].is_static()) {
            OVC_CHECK(y.dims[1].lo % 3 == 0, n.description() << ": the height of a single-plane frame must be a multiple of 3");
            o.dims[1] = Dim(y.dims[1].lo * 2 / 3);
        }
    } else {
        OVC_CHECK((int)n.num_inputs() == max_planes, n.description() << ": " << max_planes << " planes or one expected");
    }
    n.set_output(0, n.in_et(0), o);
}

bool eval_color(const Node& n, Ins in, Outs out, bool nv12, bool bgr) {
    const Tensor& Y = in[0];
    const bool single = in.size() == 1;
    const int64_t B = Y.shape[0], W = Y.shape[2], H = single ? Y.shape[1] * 2 / 3 : Y.shape[1];
    OVC_CHECK(H % 2 == 0 && W % 2 == 0, n.description() << ": image height and width must be even");
    const auto y = to_f32(Y);
    std::vector<float> p1, p2;
    if (!single) {
        p1 = to_f32(in[1]);
        if (!nv12) p2 = to_f32(in[2]);
    }
    const bool integral = Y.et == ET::u8;
    std::vector<float> o((size_t)(B * H * W * 3));
    const int64_t frame = single ? H * 3 / 2 * W : H * W;
    for (int64_t b = 0; b < B; ++b)
        for (int64_t h = 0; h < H; ++h)
            for (int64_t w = 0; w < W; ++w) {
                const float yv = y[(size_t)(b * frame + h * W + w)];
                float u, v;
                if (nv12) {
                    const int64_t uv = (h / 2) * W + (w / 2) * 2;
                    const float* src = single ? y.data() + b * frame + H * W : p1.data() + b * (H / 2) * W;
                    u = src[uv];
                    v = src[uv + 1];
                } else {
                    const int64_t q = (h / 2) * (W / 2) + w / 2;
                    const float* us = single ? y.data() + b * frame + H * W : p1.data() + b * (H / 2) * (W / 2);
                    const float* vs = single ? y.data() + b * frame + H * W + (H / 2) * (W / 2) : p2.data() + b * (H / 2) * (W / 2);
                    u = us[q];
                    v = vs[q];
                }
                float rgb[3];
                yuv_to_rgb(yv, u, v, integral, rgb);
                float* dst = o.data() + ((b * H + h) * W + w) * 3;
                dst[0] = bgr ? rgb[2] : rgb[0];
                dst[1] = rgb[1];
                dst[2] = bgr ? rgb[0] : rgb[2];
            }
    out[0] = from_f32(Y.et, {B, H, W, 3}, o);
    return true;
}

}  // namespace

void register_vision_ops() {
    for (const char* t : {"NV12toRGB", "NV12toBGR"}) {
        const bool bgr = std::string(t) == "NV12toBGR";
        reg(t, "opset8", {}, [](Node& n) { infer_color(n, 2); }, [bgr](N n, Ins in, Outs out, C) { return eval_color(n, in, out, true, bgr); }, 1, 2);
    }
    for (const char* t : {"I420toRGB", "I420toBGR"}) {
        const bool bgr = std::string(t) == "I420toBGR";
        reg(t, "opset8", {}, [](Node& n) { infer_color(n, 3); }, [bgr](N n, Ins in, Outs out, C) { return eval_color(n, in, out, false, bgr); }, 1, 3);
    }

    // ---- PriorBoxClustered: boxes of the given (width, height) pairs around every cell of the feature map, then the variances
    reg("PriorBoxClustered", "opset1",
        {Af("step", 0), Af("step_w", 0), Af("step_h", 0), Afs("width", {1.0}), Afs("height", {1.0}), Ab("clip", true), Af("offset", 0), Afs("variance")},
        [](Node& n) {
            std::vector<int64_t> layer;
            PShape o = PShape::dynamic(2);
            o.dims[0] = Dim(2);
            if (get_constant_ints(n.input(0), layer) && layer.size() == 2)
                o.dims[1] = Dim(4 * layer[0] * layer[1] * (int64_t)n.attr("width").fs.size());
            n.set_output(0, ET::f32, o);
        },
        [](N n, Ins in, Outs out, C) {
            const auto layer = to_i64(in[0]), img = to_i64(in[1]);
            const auto &ws = n.attr("width").fs, &hs = n.attr("height").fs;
            OVC_CHECK(ws.size() == hs.size() && layer.size() == 2 && img.size() == 2, n.description() << ": widths and heights must pair up; sizes are [h, w]");
            std::vector<double> var = n.attr("variance").fs;
            OVC_CHECK(var.empty() || var.size() == 1 || var.size() == 4, n.description() << ": 0, 1 or 4 variances expected");
            if (var.empty()) var.push_back(0.1);
            const int64_t LH = layer[0], LW = layer[1], IH = img[0], IW = img[1], P = (int64_t)ws.size();
            float step_w = (float)(n.attr_float("step_w") == 0 ? n.attr_float("step") : n.attr_float("step_w"));
            float step_h = (float)(n.attr_float("step_h") == 0 ? n.attr_float("step") : n.attr_float("step_h"));
            if (step_w == 0 && step_h == 0) {
                step_w = (float)IW / LW;
                step_h = (float)IH / LH;
            }
            const float off = (float)n.attr_float("offset");
            const bool clip = n.attr_bool("clip");
            const int64_t row = 4 * LH * LW * P;
            std::vector<float> o((size_t)(2 * row));
            for (int64_t h = 0; h < LH; ++h)
                for (int64_t w = 0; w < LW; ++w) {
                    const float cx = (w + off) * step_w, cy = (h + off) * step_h;
                    for (int64_t s = 0; s < P; ++s) {
                        float box[4] = {(cx - (float)ws[(size_t)s] / 2.f) / IW, (cy - (float)hs[(size_t)s] / 2.f) / IH,
                                        (cx + (float)ws[(size_t)s] / 2.f) / IW, (cy + (float)hs[(size_t)s] / 2.f) / IH};
                        const int64_t at = ((h * LW + w) * P + s) * 4;
                        for (int k = 0; k < 4; ++k) {
                            o[(size_t)(at + k)] = clip ? std::min(std::max(box[k], 0.f), 1.f) : box[k];
                            o[(size_t)(row + at + k)] = (float)var[var.size() == 1 ? 0 : (size_t)k];
                        }
                    }
                }
            out[0] = from_f32(ET::f32, {2, row}, o);
            return true;
        }, 2, 2);

    // ---- PSROIPooling (average mode): output channel c, bin (ph, pw) reads input channel (c * PH + ph) * PW + pw
    reg("PSROIPooling", "opset1", {Ai("output_dim", 0), Ai("group_size", 1), Af("spatial_scale", 1), As("mode", "average"), Ai("spatial_bins_x", 1), Ai("spatial_bins_y", 1)},
        [](Node& n) {
            const PShape& r = n.in_shape(1);
            PShape o = PShape::dynamic(4);
            if (!r.rank_dynamic && !r.dims.empty()) o.dims[0] = r.dims[0];
            o.dims[1] = Dim(n.attr_int("output_dim"));
            o.dims[2] = o.dims[3] = Dim(n.attr_int("group_size"));
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            OVC_CHECK(n.attr_str("mode") == "average", n.description() << ": the reference executor serves the average mode");
            const Tensor& X = in[0];
            const auto x = to_f32(X), rois = to_f32(in[1]);
            const int64_t Cin = X.shape[1], H = X.shape[2], W = X.shape[3], R = in[1].shape[0];
            const int64_t Cout = n.attr_int("output_dim"), G = n.attr_int("group_size");
            OVC_CHECK(Cin == Cout * G * G, n.description() << ": " << Cin << " input channels do not equal output_dim * group_size^2");
            const float scale = (float)n.attr_float("spatial_scale");
            std::vector<float> o((size_t)(R * Cout * G * G), 0.f);
            for (int64_t r = 0; r < R; ++r) {
                const float* box = rois.data() + r * 5;
                const int64_t b = (int64_t)box[0];
                const float sw = std::round(box[1]) * scale, sh = std::round(box[2]) * scale;
                const float ew = (std::round(box[3]) + 1.f) * scale, eh = (std::round(box[4]) + 1.f) * scale;
                const float bw = (ew - sw) / G, bh = (eh - sh) / G;
                for (int64_t c = 0; c < Cout; ++c)
                    for (int64_t ph = 0; ph < G; ++ph)
                        for (int64_t pw = 0; pw < G; ++pw) {
                            const int64_t cin = (c * G + ph) * G + pw;
                            const int64_t w0 = std::min<int64_t>((int64_t)std::floor(sw + pw * bw), W - 1), h0 = std::min<int64_t>((int64_t)std::floor(sh + ph * bh), H - 1);
                            const int64_t w1 = std::min<int64_t>((int64_t)std::ceil(sw + (pw + 1) * bw), W), h1 = std::min<int64_t>((int64_t)std::ceil(sh + (ph + 1) * bh), H);
                            if (w0 < 0 || h0 < 0 || w1 <= w0 || h1 <= h0) continue;
                            float sum = 0;
                            for (int64_t h = h0; h < h1; ++h)
                                for (int64_t w = w0; w < w1; ++w) sum += x[(size_t)(((b * Cin + cin) * H + h) * W + w)];
                            o[(size_t)(((r * Cout + c) * G + ph) * G + pw)] = sum / (float)((w1 - w0) * (h1 - h0));
                        }
            }
            out[0] = from_f32(X.et, {R, Cout, G, G}, o);
            return true;
        }, 2, 2);

    // ---- FakeConvert: what the data would be after a round trip through fp8 with a scale (and shift)
    reg("FakeConvert", "opset13", {As("destination_type", "f8e4m3")},
        [](Node& n) { n.set_output(0, n.in_et(0), n.in_shape(0)); },
        [](N n, Ins in, Outs out, C) {
            const Tensor& X = in[0];
            auto x = to_f32(X);
            const auto scale = to_f32(in[1]);
            std::vector<float> shift;
            if (in.size() > 2) shift = to_f32(in[2]);
            const bool e4m3 = n.attr_str("destination_type") == "f8e4m3";
            OVC_CHECK(e4m3 || n.attr_str("destination_type") == "f8e5m2", n.description() << ": destination_type must be f8e4m3 or f8e5m2");
            // scale / shift broadcast over the trailing axes: one value per leading index (per tensor or per channel)
            const size_t ns = std::max<size_t>(scale.size(), 1);
            OVC_CHECK(x.size() % ns == 0 && (shift.empty() || shift.size() == scale.size()), n.description() << ": scale / shift do not broadcast to the data");
            size_t inner = 1, lead = 1;
            if (ns > 1) {
                // locate the axis that the scale runs along (the only axis of its shape that is not 1)
                const Shape& ss = in[1].shape;
                size_t ax = 0;
                for (size_t i = 0; i < ss.size(); ++i) if (ss[i] != 1) ax = i + (X.shape.size() - ss.size());
                for (size_t i = ax + 1; i < X.shape.size(); ++i) inner *= (size_t)X.shape[i];
                lead = ns;
            }
            for (size_t i = 0; i < x.size(); ++i) {
                const size_t g = ns == 1 ? 0 : (i / inner) % lead;
                const float sh = shift.empty() ? 0.f : shift[g];
                const float t = x[i] * scale[g] - sh;
                const float q = e4m3 ? f8e4m3_to_f32(f32_to_f8e4m3(t)) : f8e5m2_to_f32(f32_to_f8e5m2(t));
                x[i] = (q + sh) / scale[g];
            }
            out[0] = from_f32(X.et, X.shape, x);
            return true;
        }, 2, 3);

    // ---- SparseFillEmptyRows: rows of a sparse matrix that hold no value get one entry (row, 0) with the default value
    reg("SparseFillEmptyRows", "opset16", {},
        [](Node& n) {
            n.set_num_outputs(3);
            PShape idx = PShape::dynamic(2);
            idx.dims[1] = Dim(2);
            n.set_output(0, n.in_et(2), idx);
            n.set_output(1, n.in_et(0), PShape::dynamic(1));
            PShape ind = PShape::dynamic(1);
            std::vector<int64_t> ds;
            if (get_constant_ints(n.input(1), ds) && ds.size() == 2) ind.dims[0] = Dim(ds[0]);
            n.set_output(2, ET::boolean, ind);
        },
        [](N n, Ins in, Outs out, C) {
            const auto vals = to_f32(in[0]);
            const auto dense = to_i64(in[1]), idx = to_i64(in[2]);
            const float dflt = to_f32(in[3]).at(0);
            OVC_CHECK(dense.size() == 2 && idx.size() == 2 * vals.size(), n.description() << ": a 2-D sparse matrix is expected");
            const int64_t rows = dense[0];
            std::vector<int64_t> per_row((size_t)rows, 0);
            for (size_t i = 0; i < vals.size(); ++i) {
                OVC_CHECK(idx[2 * i] >= 0 && idx[2 * i] < rows, n.description() << ": row index " << idx[2 * i] << " out of range");
                ++per_row[(size_t)idx[2 * i]];
            }
            // output in row order; entries of a row keep their input order
            std::vector<int64_t> start((size_t)rows + 1, 0);
            for (int64_t r = 0; r < rows; ++r) start[(size_t)r + 1] = start[(size_t)r] + std::max<int64_t>(per_row[(size_t)r], 1);
            const int64_t M = start[(size_t)rows];
            std::vector<int64_t> oi((size_t)(2 * M)), fill = start;
            std::vector<float> ov((size_t)M);
            std::vector<int64_t> empty((size_t)rows);
            for (int64_t r = 0; r < rows; ++r) {
                empty[(size_t)r] = per_row[(size_t)r] == 0;
                if (per_row[(size_t)r] == 0) {
                    oi[(size_t)(2 * start[(size_t)r])] = r;
                    oi[(size_t)(2 * start[(size_t)r] + 1)] = 0;
                    ov[(size_t)start[(size_t)r]] = dflt;
                }
            }
            for (size_t i = 0; i < vals.size(); ++i) {
                const int64_t at = fill[(size_t)idx[2 * i]]++;
                oi[(size_t)(2 * at)] = idx[2 * i];
                oi[(size_t)(2 * at + 1)] = idx[2 * i + 1];
                ov[(size_t)at] = vals[i];
            }
            out[0] = from_i64(in[2].et, {M, 2}, oi);
            out[1] = from_f32(in[0].et, {M}, ov);
            out[2] = from_i64(ET::boolean, {rows}, empty);
            return true;
        }, 4, 4);
}

}  // namespace ovc
