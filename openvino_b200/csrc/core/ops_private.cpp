// Transformation-private operations that passes of the reference leave in a model for the plugins: expert-gathered
// matrix products (plain and weight-compressed), the weight-compressed grouped product, the quantised fully-connected
// forms and the segment-wise attention of vision encoders: shape / type inference and reference evaluation.
//
// Reference counterparts: src/common/transformations/include/ov_ops/{gather_matmul,gather_matmul_compressed,
// grouped_matmul_compressed,fully_connected_quantized,fully_connected_quantized_legacy,vl_sdpa}.hpp.
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
AttrSpec At(const char* n, ET d) { return A(n, K::TYPE, Attr::Type(d)); }
AttrSpec Ais(const char* n) { return A(n, K::INTS, Attr::Ints({})); }

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

Dim dim_of(const PShape& s, size_t i) { return (!s.rank_dynamic && i < s.dims.size()) ? s.dims[i] : Dim::dynamic(); }

// Weights [E, N, K] or [E, N, G, gs] with scales (and zero points) [E, N, G or 1, 1 or absent] -> fp32 [E, N, K]
std::vector<float> expand_weights(const Node& n, const Tensor& w, const Tensor* scales, const Tensor* zp, int64_t& E, int64_t& Nn, int64_t& Kk) {
    OVC_CHECK(w.shape.size() == 3 || w.shape.size() == 4, n.description() << ": weights are [experts, N, K] or [experts, N, groups, group_size]");
    E = w.shape[0];
    Nn = w.shape[1];
    Kk = w.numel() / std::max<int64_t>(E * Nn, 1);
    std::vector<float> out((size_t)w.numel());
    for (int64_t i = 0; i < w.numel(); ++i) out[(size_t)i] = (float)get_elem_f64(w, i);
    if (!scales || scales->numel() == 0) return out;
    const auto sc = to_f32(*scales);
    std::vector<float> z;
    if (zp && zp->numel() > 0) z = to_f32(*zp);
    const int64_t per_row = std::max<int64_t>(1, (int64_t)sc.size() / std::max<int64_t>(E * Nn, 1));      // groups along K
    OVC_CHECK(sc.size() == 1 || (int64_t)sc.size() == E * Nn * per_row, n.description() << ": scales do not match the weight rows");
    const int64_t gs = Kk / per_row;
    for (int64_t r = 0; r < E * Nn; ++r)
        for (int64_t k = 0; k < Kk; ++k) {
            const size_t g = sc.size() == 1 ? 0 : (size_t)(r * per_row + k / gs);
            const float zero = z.empty() ? 0.f : z[z.size() == 1 ? 0 : g];
            out[(size_t)(r * Kk + k)] = (out[(size_t)(r * Kk + k)] - zero) * sc[g];
        }
    return out;
}

void infer_gather_matmul(Node& n) {
    const PShape &a = n.in_shape(0), &b = n.in_shape(1), &idx = n.in_shape(2);
    n.set_output(0, n.in_et(0), PShape({dim_of(idx, 1), dim_of(a, 1), dim_of(b, 1)}));
}

// A [top_k or 1, tokens, K]; indices [tokens, top_k] name the expert of every (token, slot); out [top_k, tokens, N]
bool eval_gather_matmul(N n, Ins in, Outs out, C) {
    const Tensor& At_ = in[0];
    const auto a = to_f32(At_);
    const auto idx = to_i64(in[2]);
    int64_t E, Nn, Kk;
    const bool compressed = n.type == "GatherMatmulCompressed";
    const auto w = expand_weights(n, in[1], compressed ? &in[4] : nullptr, compressed && in.size() > 5 ? &in[5] : nullptr, E, Nn, Kk);
    const int64_t A0 = At_.shape[0], T = At_.shape[1], top = in[2].shape[1];
    OVC_CHECK(At_.shape[2] == Kk && in[2].shape[0] == T && (A0 == 1 || A0 == top), n.description() << ": A is [top_k or 1, tokens, K] and indices [tokens, top_k]");
    std::vector<float> bias;
    if (in.size() > 3 && in[3].numel() > 0) bias = to_f32(in[3]);
    std::vector<float> o((size_t)(top * T * Nn));
    for (int64_t s = 0; s < top; ++s)
        for (int64_t t = 0; t < T; ++t) {
            const int64_t e = idx[(size_t)(t * top + s)];
            OVC_CHECK(e >= 0 && e < E, n.description() << ": expert index " << e << " outside [0, " << E << ")");
            const float* x = a.data() + ((A0 == 1 ? 0 : s) * T + t) * Kk;
            for (int64_t j = 0; j < Nn; ++j) {
                float acc = 0;
                const float* wr = w.data() + (e * Nn + j) * Kk;
                for (int64_t k = 0; k < Kk; ++k) acc += x[k] * wr[k];
                if (!bias.empty()) acc += bias.size() == 1 ? bias[0] : ((int64_t)bias.size() == Nn ? bias[(size_t)j] : bias[(size_t)((e * Nn + j) % (int64_t)bias.size())]);
                o[(size_t)((s * T + t) * Nn + j)] = acc;
            }
        }
    out[0] = from_f32(At_.et, {top, T, Nn}, o);
    return true;
}

// out = quantise(dequantise(X) x dequantise(W)^T + bias); absent parameters are empty tensors
bool eval_fc_quantized(N n, Ins in, Outs out, C) {
    const Tensor &X = in[0], &W = in[1];
    const int64_t Nn = W.shape[0], Kk = W.numel() / Nn, rows = X.numel() / Kk;
    OVC_CHECK(X.shape.back() == Kk, n.description() << ": the innermost extent of X must equal K = " << Kk);
    auto get = [&](size_t i) { return (in.size() > i && in[i].numel() > 0) ? to_f32(in[i]) : std::vector<float>(); };
    const bool legacy = n.type == "FullyConnectedQuantizedLegacy";
    const auto bias = get(2);
    const auto w_scale = legacy ? std::vector<float>() : get(3), w_zp = legacy ? std::vector<float>() : get(4);
    const auto x_scale = legacy ? std::vector<float>() : get(5), x_zp = legacy ? std::vector<float>() : get(6);
    const auto o_scale = legacy ? get(3) : get(7), o_zp = legacy ? get(4) : get(8);
    auto pick = [](const std::vector<float>& v, int64_t i, float dflt) { return v.empty() ? dflt : v[(size_t)(v.size() == 1 ? 0 : i)]; };
    std::vector<float> o((size_t)(rows * Nn));
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t j = 0; j < Nn; ++j) {
            double acc = 0;
            for (int64_t k = 0; k < Kk; ++k) {
                const double xv = (get_elem_f64(X, r * Kk + k) - pick(x_zp, k, 0.f)) * pick(x_scale, k, 1.f);
                const double wv = (get_elem_f64(W, j * Kk + k) - pick(w_zp, j, 0.f)) * pick(w_scale, j, 1.f);
                acc += xv * wv;
            }
            float v = (float)acc;
            if (legacy) {
                // the integer accumulator is scaled back to real values, then the bias is added
                v = (v - pick(o_zp, j, 0.f)) * pick(o_scale, j, 1.f) + pick(bias, j, 0.f);
            } else {
                v += pick(bias, j, 0.f);
                if (!o_scale.empty()) v = v / pick(o_scale, j, 1.f) + pick(o_zp, j, 0.f);
            }
            o[(size_t)(r * Nn + j)] = v;
        }
    Shape os = X.shape;
    os.back() = Nn;
    const ET want = n.attr("output_type").et;
    ET et = want != ET::dynamic ? want : (et_is_real(X.et) ? X.et : ET::f32);
    if (!et_is_real(et)) for (auto& v : o) v = std::round(v);
    out[0] = from_f32(et, os, o);
    return true;
}


// ---- static-shape forms of the suppression / proposal operations: the dynamic operation of the public set does the
// work on a detached node with the same attributes; the rows are then padded to the upper bound that inference gave
std::vector<Tensor> run_public(const char* type, const char* version, Ins in, const std::vector<std::pair<std::string, Attr>>& attrs, C ctx) {
    std::vector<Output> ports;
    for (const Tensor& t : in) ports.push_back(make_parameter(t.et, PShape(t.shape))->output(0));
    NodePtr node = make_node(type, version, ports, attrs, false);
    const OpSchema* schema = OpRegistry::get().find(type, version);
    OVC_CHECK(schema && schema->eval, type << " has no evaluation");
    node->set_num_outputs(3);
    std::vector<Tensor> out(3);
    OVC_CHECK(schema->eval(*node, in, out, ctx), type << ": evaluation refused the inputs");
    return out;
}

Tensor pad_rows(const Tensor& t, int64_t rows, double fill) {
    Shape s = t.shape;
    const int64_t have = s.empty() ? 0 : s[0];
    s[0] = rows;
    Tensor o(t.et, s);
    const int64_t width = have > 0 ? t.numel() / have : (rows > 0 ? o.numel() / rows : 0);
    for (int64_t i = 0; i < o.numel(); ++i) {
        if (i < std::min(have, rows) * width) {
            if (et_is_real(t.et)) set_elem_f64(o, i, get_elem_f64(t, i)); else set_elem_i64(o, i, get_elem_i64(t, i));
        } else {
            if (et_is_real(t.et)) set_elem_f64(o, i, fill); else set_elem_i64(o, i, (int64_t)fill);
        }
    }
    return o;
}

// The operation a TypeRelaxed node wraps, built over stand-in inputs that carry the overriding element types (and the
// shapes of the node's inputs, or of the tensors of an evaluation) so that the wrapped operation's own rules run.
NodePtr relaxed_base(const Node& n, const std::vector<Tensor>* tensors) {
    const std::string type = n.attr_str("base_type"), version = n.attr_str("base_version");
    const OpSchema* schema = version.empty() ? OpRegistry::get().find_latest(type) : OpRegistry::get().find(type, version);
    OVC_CHECK(schema, n.description() << ": no operation " << type << " in " << (version.empty() ? "any opset" : version));
    const auto& its = n.attr("input_data_types").ss;
    std::vector<Output> ports;
    for (size_t i = 0; i < n.num_inputs(); ++i) {
        const ET et = i < its.size() && its[i] != "dynamic" && !its[i].empty() ? et_from_name(its[i]) : n.in_et(i);
        std::vector<int64_t> values;
        // constant inputs keep their values: shape arguments (Reshape pattern, axes) drive the wrapped operation's inference
        if (!tensors && n.input(i).node->type == "Constant" && et == n.in_et(i)) { ports.push_back(n.input(i)); continue; }
        ports.push_back(make_parameter(et, tensors ? PShape((*tensors)[i].shape) : n.in_shape(i))->output(0));
    }
    std::vector<std::pair<std::string, Attr>> attrs;
    for (const auto& kv : n.attrs)
        if (kv.first != "base_type" && kv.first != "base_version" && kv.first != "input_data_types" && kv.first != "output_data_types") attrs.push_back(kv);
    // a model read back from a file carries the wrapped operation's attributes as text: give each the kind its schema names
    for (auto& kv : attrs)
        for (const AttrSpec& spec : schema->attrs)
            if (spec.name == kv.first && kv.second.kind == Attr::STR && spec.kind != Attr::STR) kv.second = Attr::from_string(spec.kind, kv.second.s);
    return make_node(schema->type, schema->version, ports, attrs, true);
}

}  // namespace

void register_private_ops() {
    reg("GatherMatmul", "ie_internal_opset", {}, infer_gather_matmul, eval_gather_matmul, 3, 4);
    reg("GatherMatmulCompressed", "ie_internal_opset", {}, infer_gather_matmul, eval_gather_matmul, 5, 6);

    // mat_a [rows, K] x compressed mat_b [G, N, K] with offsets (rows up to offsets[g] use group g), or [G, M, K] x [G, N, K]
    reg("GroupedMatMulCompressed", "ie_internal_opset", {},
        [](Node& n) {
            const PShape &a = n.in_shape(0), &b = n.in_shape(1);
            const bool with_offsets = !a.rank_dynamic && a.dims.size() == 2;
            if (with_offsets) n.set_output(0, n.in_et(0), PShape({dim_of(a, 0), dim_of(b, 1)}));
            else n.set_output(0, n.in_et(0), PShape({dim_of(a, 0), dim_of(a, 1), dim_of(b, 1)}));
        },
        [](N n, Ins in, Outs out, C) {
            const bool with_offsets = in[0].shape.size() == 2;
            const size_t sc = with_offsets ? 3 : 2;
            int64_t G, Nn, Kk;
            const auto w = expand_weights(n, in[1], &in[sc], in.size() > sc + 1 ? &in[sc + 1] : nullptr, G, Nn, Kk);
            const auto a = to_f32(in[0]);
            if (with_offsets) {
                const auto offs = to_i64(in[2]);
                const int64_t rows = in[0].shape[0];
                std::vector<float> o((size_t)(rows * Nn), 0.f);
                int64_t begin = 0;
                for (int64_t g = 0; g < G; ++g) {
                    const int64_t end = std::min<int64_t>(offs[(size_t)g], rows);
                    for (int64_t r = begin; r < end; ++r)
                        for (int64_t j = 0; j < Nn; ++j) {
                            float acc = 0;
                            for (int64_t k = 0; k < Kk; ++k) acc += a[(size_t)(r * Kk + k)] * w[(size_t)((g * Nn + j) * Kk + k)];
                            o[(size_t)(r * Nn + j)] = acc;
                        }
                    begin = std::max(begin, end);
                }
                out[0] = from_f32(in[0].et, {rows, Nn}, o);
            } else {
                const int64_t M = in[0].shape[1];
                std::vector<float> o((size_t)(G * M * Nn));
                for (int64_t g = 0; g < G; ++g)
                    for (int64_t r = 0; r < M; ++r)
                        for (int64_t j = 0; j < Nn; ++j) {
                            float acc = 0;
                            for (int64_t k = 0; k < Kk; ++k) acc += a[(size_t)((g * M + r) * Kk + k)] * w[(size_t)((g * Nn + j) * Kk + k)];
                            o[(size_t)((g * M + r) * Nn + j)] = acc;
                        }
                out[0] = from_f32(in[0].et, {G, M, Nn}, o);
            }
            return true;
        }, 3, 5);

    auto infer_fcq = [](Node& n) {
        PShape o = n.in_shape(0);
        if (!o.rank_dynamic && !o.dims.empty()) o.dims.back() = dim_of(n.in_shape(1), 0);
        const ET want = n.attr("output_type").et;
        n.set_output(0, want != ET::dynamic ? want : (et_is_real(n.in_et(0)) ? n.in_et(0) : ET::f32), o);
    };
    reg("FullyConnectedQuantized", "ie_internal_opset", {At("output_type", ET::dynamic)}, infer_fcq, eval_fc_quantized, 9, 9);
    reg("FullyConnectedQuantizedLegacy", "ie_internal_opset", {At("output_type", ET::dynamic)}, infer_fcq, eval_fc_quantized, 4, 5);

    // VLSDPA: full (non-causal) attention inside the segments given by cumulative lengths; q / k / v are [L, H, S] with the
    // order {1, 0, 2} (heads moved in front by the operation itself) or [H, L, S] without orders
    reg("VLSDPA", "ie_internal_opset", {Ais("order_q"), Ais("order_k"), Ais("order_v"), Ais("order_out")},
        [](Node& n) {
            OVC_CHECK(n.attr_ints("order_q") == n.attr_ints("order_k") && n.attr_ints("order_q") == n.attr_ints("order_v") && n.attr_ints("order_q") == n.attr_ints("order_out"),
                      n.description() << ": the four orders must be equal");
            OVC_CHECK(n.attr_ints("order_q").empty() || n.attr_ints("order_q") == std::vector<int64_t>({1, 0, 2}), n.description() << ": order must be {1, 0, 2} or empty");
            PShape o = n.in_shape(0);
            if (!o.rank_dynamic && o.dims.size() == 3) o.dims[2] = dim_of(n.in_shape(2), 2);
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            const bool lhs = !n.attr_ints("order_q").empty();          // data is [L, H, S]
            const Tensor& Q = in[0];
            const auto q = to_f32(Q), k = to_f32(in[1]), v = to_f32(in[2]);
            const auto cu = to_i64(in[3]);
            const int64_t L = Q.shape[lhs ? 0 : 1], H = Q.shape[lhs ? 1 : 0], S = Q.shape[2], Sv = in[2].shape[2];
            auto at = [&](int64_t l, int64_t h, int64_t width) { return lhs ? (l * H + h) * width : (h * L + l) * width; };
            const float scale = 1.f / std::sqrt((float)S);
            std::vector<float> o((size_t)(L * H * Sv), 0.f), p;
            for (size_t s = 0; s + 1 < cu.size(); ++s) {
                const int64_t b = cu[s], e = cu[s + 1];
                OVC_CHECK(0 <= b && b <= e && e <= L, n.description() << ": cumulative lengths must rise from 0 to at most " << L);
                p.resize((size_t)(e - b));
                for (int64_t h = 0; h < H; ++h)
                    for (int64_t i = b; i < e; ++i) {
                        float mx = -std::numeric_limits<float>::infinity();
                        for (int64_t j = b; j < e; ++j) {
                            float acc = 0;
                            for (int64_t d = 0; d < S; ++d) acc += q[(size_t)(at(i, h, S) + d)] * k[(size_t)(at(j, h, S) + d)];
                            p[(size_t)(j - b)] = acc * scale;
                            mx = std::max(mx, acc * scale);
                        }
                        double sum = 0;
                        for (auto& x : p) { x = std::exp(x - mx); sum += x; }
                        for (int64_t j = b; j < e; ++j) {
                            const float w = (float)(p[(size_t)(j - b)] / sum);
                            for (int64_t d = 0; d < Sv; ++d) o[(size_t)(at(i, h, Sv) + d)] += w * v[(size_t)(at(j, h, Sv) + d)];
                        }
                    }
            }
            Shape os = Q.shape;
            os[2] = Sv;
            out[0] = from_f32(Q.et, os, o);
            return true;
        }, 4, 4);

    // ---- NonMaxSuppressionIEInternal: [B * C * min(boxes, max per class), 3] rows, unused rows filled with -1
    reg("NonMaxSuppressionIEInternal", "ie_internal_opset", {A("center_point_box", K::INT, Attr::Int(0)), A("sort_result_descending", K::BOOL, Attr::Bool(true)),
                                                             At("output_type", ET::i64), At("score_output_type", ET::f32), A("rotation", K::INT, Attr::Int(0))},
        [](Node& n) {
            n.set_num_outputs(3);
            PShape o = PShape::dynamic(2);
            o.dims[1] = Dim(3);
            std::vector<int64_t> mx;
            const PShape &b = n.in_shape(0), &s = n.in_shape(1);
            if (n.num_inputs() > 2 && get_constant_ints(n.input(2), mx) && !mx.empty() && dim_of(b, 1).is_static() && dim_of(s, 0).is_static() && dim_of(s, 1).is_static())
                o.dims[0] = Dim(std::min(dim_of(b, 1).lo, mx[0]) * dim_of(s, 0).lo * dim_of(s, 1).lo);
            n.set_output(0, n.attr("output_type").et, o);
            n.set_output(1, n.attr("score_output_type").et, o);
            n.set_output(2, n.attr("output_type").et, PShape({Dim(1)}));
        },
        [](N n, Ins in, Outs out, C c) {
            const int64_t rot = n.attr_int("rotation");
            std::vector<Tensor> res;
            if (rot == 0) {
                res = run_public("NonMaxSuppression", "opset9", in, {{"box_encoding", Attr::Str(n.attr_int("center_point_box") ? "center" : "corner")},
                                 {"sort_result_descending", Attr::Bool(n.attr_bool("sort_result_descending", true))}, {"output_type", Attr::Type(n.attr("output_type").et)}}, c);
            } else {
                std::vector<Tensor> five(in.begin(), in.begin() + std::min<size_t>(in.size(), 5));
                res = run_public("NMSRotated", "opset13", five, {{"sort_result_descending", Attr::Bool(n.attr_bool("sort_result_descending", true))},
                                 {"output_type", Attr::Type(n.attr("output_type").et)}, {"clockwise", Attr::Bool(rot == 1)}}, c);
            }
            const int64_t mx = in.size() > 2 ? get_elem_i64(in[2], 0) : 0;
            const int64_t rows = std::min<int64_t>(in[0].shape[1], mx) * in[1].shape[0] * in[1].shape[1];
            out[0] = pad_rows(res[0], rows, -1);
            out[1] = pad_rows(convert_tensor(res[1], n.attr("score_output_type").et), rows, -1);
            out[2] = res[2];
            return true;
        }, 2, 6);

    // ---- MulticlassNmsIEInternal / MatrixNms static form: rows padded with -1 up to the bound per image
    auto infer_static_nms = [](Node& n) {
        n.set_num_outputs(3);
        const ET it = n.attr("output_type").et;
        const PShape &b = n.in_shape(0), &s = n.in_shape(1);
        PShape sel = PShape::dynamic(2), idx = PShape::dynamic(2);
        sel.dims[1] = Dim(6);
        idx.dims[1] = Dim(1);
        const Dim batch = dim_of(b, 0), classes = dim_of(s, 1), boxes = dim_of(b, 1);
        if (batch.is_static() && classes.is_static() && boxes.is_static()) {
            int64_t per_class = boxes.lo;
            if (n.attr_int("nms_top_k", -1) >= 0) per_class = std::min(per_class, n.attr_int("nms_top_k", -1));
            int64_t per_batch = per_class * classes.lo;
            if (n.attr_int("keep_top_k", -1) >= 0) per_batch = std::min(per_batch, n.attr_int("keep_top_k", -1));
            sel.dims[0] = idx.dims[0] = Dim(per_batch * batch.lo);
        }
        n.set_output(0, n.in_et(0), sel);
        n.set_output(1, it, idx);
        n.set_output(2, it, PShape({batch}));
    };
    auto static_nms_eval = [](const char* type, const char* version) {
        return [type, version](N n, Ins in, Outs out, C c) {
            auto res = run_public(type, version, in, n.attrs, c);
            const int64_t rows = n.outs[0].shape.dims[0].is_static() ? n.outs[0].shape.dims[0].lo : res[0].shape[0];
            out[0] = pad_rows(res[0], rows, -1);
            out[1] = pad_rows(res[1], rows, -1);
            out[2] = res[2];
            return true;
        };
    };
    const std::vector<AttrSpec> mc = {A("sort_result_type", K::STR, Attr::Str("none")), At("output_type", ET::i64), A("nms_top_k", K::INT, Attr::Int(-1)),
                                      A("keep_top_k", K::INT, Attr::Int(-1)), A("sort_result_across_batch", K::BOOL, Attr::Bool(false)),
                                      A("iou_threshold", K::FLOAT, Attr::Float(0)), A("score_threshold", K::FLOAT, Attr::Float(0)),
                                      A("background_class", K::INT, Attr::Int(-1)), A("nms_eta", K::FLOAT, Attr::Float(1)), A("normalized", K::BOOL, Attr::Bool(true))};
    reg("MulticlassNmsIEInternal", "ie_internal_opset", mc, infer_static_nms, static_nms_eval("MulticlassNms", "opset9"), 2, 3);
    const std::vector<AttrSpec> mx = {A("sort_result_type", K::STR, Attr::Str("none")), At("output_type", ET::i64), A("nms_top_k", K::INT, Attr::Int(-1)),
                                      A("keep_top_k", K::INT, Attr::Int(-1)), A("sort_result_across_batch", K::BOOL, Attr::Bool(false)),
                                      A("score_threshold", K::FLOAT, Attr::Float(0)), A("background_class", K::INT, Attr::Int(-1)),
                                      A("decay_function", K::STR, Attr::Str("linear")), A("gaussian_sigma", K::FLOAT, Attr::Float(2)),
                                      A("post_threshold", K::FLOAT, Attr::Float(0)), A("normalized", K::BOOL, Attr::Bool(true))};
    reg("NmsStaticShapeIE", "ie_internal_opset", mx, infer_static_nms, static_nms_eval("MatrixNms", "opset8"), 2, 2);

    // ---- GenerateProposalsIEInternal: [B * post_nms_count] rows, zero filled
    reg("GenerateProposalsIEInternal", "ie_internal_opset", {A("min_size", K::FLOAT, Attr::Float(0)), A("nms_threshold", K::FLOAT, Attr::Float(0)), A("post_nms_count", K::INT, Attr::Int(0)),
                                                             A("pre_nms_count", K::INT, Attr::Int(0)), A("normalized", K::BOOL, Attr::Bool(true)), A("nms_eta", K::FLOAT, Attr::Float(1)),
                                                             At("roi_num_type", ET::i64)},
        [](Node& n) {
            n.set_num_outputs(3);
            const Dim batch = dim_of(n.in_shape(0), 0);
            const Dim rows = batch.is_static() ? Dim(batch.lo * n.attr_int("post_nms_count")) : Dim::dynamic();
            n.set_output(0, n.in_et(0), PShape({rows, Dim(4)}));
            n.set_output(1, n.in_et(0), PShape({rows}));
            n.set_output(2, n.attr("roi_num_type").et, PShape({batch}));
        },
        [](N n, Ins in, Outs out, C c) {
            auto res = run_public("GenerateProposals", "opset9", in, n.attrs, c);
            const int64_t rows = in[3].shape[0] * n.attr_int("post_nms_count");
            out[0] = pad_rows(res[0], rows, 0);
            out[1] = pad_rows(res[1], rows, 0);
            out[2] = res[2];
            return true;
        }, 4, 4);

    // ---- GroupQueryAttention (src/core/dev_api/openvino/op/group_query_attention.hpp): q [B, N, S, H], k / v
    // [B, Nkv, S, H], past k / v [B, Nkv, P, H], seqlens_k = (past + current) - 1, total_sequence_length, then optional
    // cos / sin caches [positions, H / 2], position ids [B, S], attention bias [B or 1, N or 1, S, total], head sink [N].
    // Outputs: attention [B, S, N * H], present k / v [B, Nkv, past + S, H]. An empty tensor stands for an absent input.
    reg("GroupQueryAttention", "ie_internal_opset",
        {A("num_heads", K::INT, Attr::Int(0)), A("kv_num_heads", K::INT, Attr::Int(0)), A("scale", K::FLOAT, Attr::Float(0)), A("do_rotary", K::BOOL, Attr::Bool(false)),
         A("rotary_interleaved", K::BOOL, Attr::Bool(false)), A("local_window_size", K::INT, Attr::Int(-1)), A("smooth_softmax", K::BOOL, Attr::Bool(false))},
        [](Node& n) {
            n.set_num_outputs(3);
            const PShape &q = n.in_shape(0), &k = n.in_shape(1), &pk = n.in_shape(3);
            const Dim heads = dim_of(q, 1), width = dim_of(q, 3);
            n.set_output(0, n.in_et(0), PShape({dim_of(q, 0), dim_of(q, 2), heads.is_static() && width.is_static() ? Dim(heads.lo * width.lo) : Dim::dynamic()}));
            PShape present({dim_of(k, 0), dim_of(k, 1), Dim::dynamic(), dim_of(k, 3)});
            std::vector<int64_t> lens;
            if (get_constant_ints(n.input(5), lens) && !lens.empty()) present.dims[2] = Dim(lens[0] + 1);
            (void)pk;
            n.set_output(1, n.in_et(1), present);
            n.set_output(2, n.in_et(2), present);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& Q = in[0];
            OVC_CHECK(Q.shape.size() == 4 && in[1].shape.size() == 4 && in[3].shape.size() == 4, n.description() << ": q, k, v and the past are rank-4 [batch, heads, length, width]");
            const int64_t B = Q.shape[0], Nq = Q.shape[1], S = Q.shape[2], H = Q.shape[3], Nkv = in[1].shape[1], Pmax = in[3].shape[2];
            OVC_CHECK(Nkv > 0 && Nq % Nkv == 0, n.description() << ": " << Nq << " query heads do not divide into " << Nkv << " key / value heads");
            const int64_t total = to_i64(in[5])[0] + 1, P = total - S, group = Nq / Nkv;
            OVC_CHECK(P >= 0 && P <= Pmax, n.description() << ": seqlens_k names a past of " << P << " positions, the past tensors hold " << Pmax);
            auto q = to_f32(Q), kn = to_f32(in[1]);
            const auto vn = to_f32(in[2]), pk = to_f32(in[3]), pv = to_f32(in[4]);
            auto present = [&](size_t i) { return i < in.size() && in[i].numel() > 0; };
            if (n.attr_bool("do_rotary")) {
                OVC_CHECK(present(7) && present(8), n.description() << ": do_rotary needs the cos and sin caches");
                const auto cs = to_f32(in[7]), sn = to_f32(in[8]);
                const int64_t half = in[7].shape.back(), rows = in[7].numel() / half;
                std::vector<int64_t> pos;
                if (present(9)) pos = to_i64(in[9]);
                const bool inter = n.attr_bool("rotary_interleaved");
                auto rotate = [&](std::vector<float>& x, int64_t heads) {
                    for (int64_t b = 0; b < B; ++b)
                        for (int64_t h = 0; h < heads; ++h)
                            for (int64_t s_ = 0; s_ < S; ++s_) {
                                const int64_t p_ = pos.empty() ? P + s_ : pos[(size_t)((b * S + s_) % (int64_t)pos.size())];
                                OVC_CHECK(p_ >= 0 && p_ < rows, n.description() << ": position " << p_ << " outside the rotary caches of " << rows << " rows");
                                float* r = x.data() + ((b * heads + h) * S + s_) * H;
                                for (int64_t d = 0; d < half; ++d) {
                                    const int64_t i0 = inter ? 2 * d : d, i1 = inter ? 2 * d + 1 : d + half;
                                    const float c = cs[(size_t)(p_ * half + d)], s2 = sn[(size_t)(p_ * half + d)], a = r[i0], b2 = r[i1];
                                    r[i0] = a * c - b2 * s2;
                                    r[i1] = a * s2 + b2 * c;
                                }
                            }
                };
                rotate(q, Nq);
                rotate(kn, Nkv);
            }
            // present = past[:P] ++ new
            std::vector<float> K_((size_t)(B * Nkv * total * H)), V_((size_t)(B * Nkv * total * H));
            for (int64_t b = 0; b < B; ++b)
                for (int64_t h = 0; h < Nkv; ++h)
                    for (int64_t t = 0; t < total; ++t) {
                        float* kd = K_.data() + ((b * Nkv + h) * total + t) * H;
                        float* vd = V_.data() + ((b * Nkv + h) * total + t) * H;
                        const float* ks = t < P ? pk.data() + ((b * Nkv + h) * Pmax + t) * H : kn.data() + ((b * Nkv + h) * S + (t - P)) * H;
                        const float* vs = t < P ? pv.data() + ((b * Nkv + h) * Pmax + t) * H : vn.data() + ((b * Nkv + h) * S + (t - P)) * H;
                        std::copy(ks, ks + H, kd);
                        std::copy(vs, vs + H, vd);
                    }
            const float scale = n.attr_float("scale") != 0 ? (float)n.attr_float("scale") : 1.f / std::sqrt((float)H);
            const int64_t window = n.attr_int("local_window_size", -1);
            std::vector<float> bias, sink;
            Shape bs;
            if (present(10)) { bias = to_f32(in[10]); bs = in[10].shape; OVC_CHECK(bs.size() == 4 && bs[3] >= total && bs[2] == S, n.description() << ": attention bias is [B or 1, N or 1, S, >= total]"); }
            if (present(11)) sink = to_f32(in[11]);
            const bool smooth = n.attr_bool("smooth_softmax") || !sink.empty();
            std::vector<float> o((size_t)(B * S * Nq * H), 0.f), p((size_t)total);
            for (int64_t b = 0; b < B; ++b)
                for (int64_t h = 0; h < Nq; ++h)
                    for (int64_t i = 0; i < S; ++i) {
                        const float* qr = q.data() + ((b * Nq + h) * S + i) * H;
                        const int64_t last = P + i, first = window > 0 ? std::max<int64_t>(0, last - window + 1) : 0;
                        float mx = smooth ? (sink.empty() ? 0.f : sink[(size_t)(h % (int64_t)sink.size())]) : -std::numeric_limits<float>::infinity();
                        for (int64_t j = first; j <= last; ++j) {
                            const float* kr = K_.data() + ((b * Nkv + h / group) * total + j) * H;
                            float acc = 0;
                            for (int64_t d = 0; d < H; ++d) acc += qr[d] * kr[d];
                            acc *= scale;
                            if (!bias.empty()) acc += bias[(size_t)((((bs[0] == 1 ? 0 : b) * bs[1] + (bs[1] == 1 ? 0 : h)) * S + i) * bs[3] + j)];
                            p[(size_t)j] = acc;
                            mx = std::max(mx, acc);
                        }
                        double sum = smooth ? std::exp((sink.empty() ? 0.f : sink[(size_t)(h % (int64_t)sink.size())]) - mx) : 0.0;
                        for (int64_t j = first; j <= last; ++j) { p[(size_t)j] = std::exp(p[(size_t)j] - mx); sum += p[(size_t)j]; }
                        float* orow = o.data() + ((b * S + i) * Nq + h) * H;
                        for (int64_t j = first; j <= last; ++j) {
                            const float w = (float)(p[(size_t)j] / sum);
                            const float* vr = V_.data() + ((b * Nkv + h / group) * total + j) * H;
                            for (int64_t d = 0; d < H; ++d) orow[d] += w * vr[d];
                        }
                    }
            out[0] = from_f32(Q.et, {B, S, Nq * H}, o);
            out[1] = from_f32(in[1].et, {B, Nkv, total, H}, K_);
            out[2] = from_f32(in[2].et, {B, Nkv, total, H}, V_);
            return true;
        }, 7, 14);

    // ---- TypeRelaxed (src/core/dev_api/openvino/op/util/type_relaxed... ov_ops/type_relaxed.hpp): an operation whose inputs
    // are seen by its own type rules as `input_data_types` whatever feeds it, and whose outputs are declared as
    // `output_data_types`. The wrapped operation is named by base_type / base_version; every other attribute is the
    // wrapped operation's own.
    reg("TypeRelaxed", "type_relaxed_opset",
        {A("base_type", K::STR, Attr::Str("")), A("base_version", K::STR, Attr::Str("")), A("input_data_types", K::STRS, Attr::Strs({})),
         A("output_data_types", K::STRS, Attr::Strs({}))},
        [](Node& n) {
            NodePtr base = relaxed_base(n, nullptr);
            n.set_num_outputs(base->outs.size());
            const auto& outs = n.attr("output_data_types").ss;
            for (size_t i = 0; i < base->outs.size(); ++i) {
                const ET et = i < outs.size() && outs[i] != "dynamic" && !outs[i].empty() ? et_from_name(outs[i]) : base->outs[i].et;
                n.set_output(i, et, base->outs[i].shape);
            }
        },
        [](N n, Ins in, Outs out, C c) {
            std::vector<Tensor> seen;
            NodePtr base = relaxed_base(n, &in);
            const auto& its = n.attr("input_data_types").ss;
            for (size_t i = 0; i < in.size(); ++i)
                seen.push_back(i < its.size() && its[i] != "dynamic" && !its[i].empty() && in[i].et != et_from_name(its[i]) ? convert_tensor(in[i], et_from_name(its[i])) : in[i]);
            OVC_CHECK(base->schema && base->schema->eval, n.description() << ": " << base->type << " has no evaluation");
            std::vector<Tensor> res(base->outs.size());
            if (!base->schema->eval(*base, seen, res, c)) return false;
            for (size_t i = 0; i < res.size(); ++i) out[i] = res[i].et == n.outs[i].et ? res[i] : convert_tensor(res[i], n.outs[i].et);
            return true;
        }, 0, -1);
}

}  // namespace ovc
