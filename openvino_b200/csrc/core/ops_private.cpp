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
}

}  // namespace ovc
