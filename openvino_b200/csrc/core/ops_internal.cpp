// Operations of the plugins' internal opset (compressed gather, dynamic activation quantisation, experts with compressed
// weights) and a further batch of the public operation set (ExtractImagePatches, RegionYolo, CTCLoss, STFT): attribute
// schemas in the reference's visit_attributes order, shape / type inference and reference evaluation.
//
// Reference counterparts: src/common/transformations/include/ov_ops/{gather_compressed,dynamic_quantize,moe_compressed}.hpp
// (and their .cpp files), src/core/src/op/{extractimagepatches,region_yolo,ctc_loss,stft}.cpp and the kernels
// src/core/reference/include/openvino/reference/{extract_image_patches,region_yolo,ctc_loss,stft}.hpp.
#include <algorithm>
#include <cmath>
#include <limits>
#include <numeric>

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
AttrSpec Ais(const char* n, std::vector<int64_t> d = {}) { return A(n, K::INTS, Attr::Ints(std::move(d))); }
AttrSpec Afs(const char* n, std::vector<double> d = {}) { return A(n, K::FLOATS, Attr::Floats(std::move(d))); }
AttrSpec At(const char* n, ET d = ET::dynamic) { return A(n, K::TYPE, Attr::Type(d)); }

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

// (q - zp) * scale over [rows, groups, group_size] (scale / zp hold one value per (row, group), or per row, or one in all)
std::vector<float> dequantise(const Tensor& q, const Tensor& scale, const Tensor* zp) {
    auto v = to_f32(q);
    const auto s = to_f32(scale);
    std::vector<float> z;
    if (zp != nullptr && zp->numel() > 0) z = to_f32(*zp);
    const size_t n = v.size(), ns = std::max<size_t>(s.size(), 1);
    OVC_CHECK(n % ns == 0, "compressed weight of " << n << " elements does not divide into " << ns << " scale groups");
    const size_t per = n / ns;
    for (size_t i = 0; i < n; ++i) {
        const size_t g = i / per;
        const float zv = z.empty() ? 0.f : z[z.size() == 1 ? 0 : g];
        v[i] = (v[i] - zv) * s[g];
    }
    return v;
}

}  // namespace

void register_internal_ops() {
    // ---- GatherCompressed: Gather over a compressed table, rows dequantised on the way out
    reg("GatherCompressed", "ie_internal_opset", {Ai("batch_dims", 0)},
        [](Node& n) {
            const PShape& d = n.in_shape(0);
            const PShape& idx = n.in_shape(1);
            const ET out_et = n.in_et(3);
            std::vector<int64_t> ax;
            if (d.rank_dynamic || idx.rank_dynamic || !get_constant_ints(n.input(2), ax) || ax.empty()) {
                n.set_output(0, out_et, PShape::dynamic());
                return;
            }
            // the compressed table may carry its groups as an extra axis ([rows, groups, group_size]): gathered rows are flat
            PShape data = d;
            const PShape& sc = n.in_shape(3);
            if (!sc.rank_dynamic && sc.dims.size() == d.dims.size() && d.dims.size() == 3) {
                data.dims = {d.dims[0], (d.dims[1].is_static() && d.dims[2].is_static()) ? Dim(d.dims[1].lo * d.dims[2].lo) : Dim::dynamic()};
            }
            const int64_t rank = (int64_t)data.dims.size();
            const int64_t axis = ax[0] < 0 ? ax[0] + rank : ax[0];
            const int64_t bd = n.attr_int("batch_dims") < 0 ? n.attr_int("batch_dims") + (int64_t)idx.dims.size() : n.attr_int("batch_dims");
            OVC_CHECK(axis >= 0 && axis < rank && bd >= 0 && bd <= axis, n.description() << ": bad axis / batch_dims");
            PShape o;
            o.rank_dynamic = false;
            for (int64_t i = 0; i < axis; ++i) o.dims.push_back(data.dims[(size_t)i]);
            for (size_t i = (size_t)bd; i < idx.dims.size(); ++i) o.dims.push_back(idx.dims[i]);
            for (int64_t i = axis + 1; i < rank; ++i) o.dims.push_back(data.dims[(size_t)i]);
            n.set_output(0, out_et, o);
        },
        [](N n, Ins in, Outs out, C) {
            const auto table = dequantise(in[0], in[3], in.size() > 4 ? &in[4] : nullptr);
            const auto idx = to_i64(in[1]);
            const int64_t axis0 = to_i64(in[2]).at(0);
            OVC_CHECK(n.attr_int("batch_dims") == 0, n.description() << ": the reference executor gathers with batch_dims = 0");
            Shape ds = in[0].shape;
            if (ds.size() == 3 && in[3].shape.size() == 3) ds = {ds[0], ds[1] * ds[2]};
            const int64_t rank = (int64_t)ds.size(), axis = axis0 < 0 ? axis0 + rank : axis0;
            int64_t outer = 1, inner = 1;
            for (int64_t i = 0; i < axis; ++i) outer *= ds[(size_t)i];
            for (int64_t i = axis + 1; i < rank; ++i) inner *= ds[(size_t)i];
            const int64_t A_ = ds[(size_t)axis];
            std::vector<float> o((size_t)(outer * (int64_t)idx.size() * inner));
            for (int64_t a = 0; a < outer; ++a)
                for (size_t j = 0; j < idx.size(); ++j) {
                    int64_t r = idx[j] < 0 ? idx[j] + A_ : idx[j];
                    OVC_CHECK(r >= 0 && r < A_, n.description() << ": index " << idx[j] << " out of range");
                    std::copy_n(table.begin() + (a * A_ + r) * inner, inner, o.begin() + ((a * (int64_t)idx.size() + (int64_t)j) * inner));
                }
            Shape os;
            for (int64_t i = 0; i < axis; ++i) os.push_back(ds[(size_t)i]);
            for (auto d : in[1].shape) os.push_back(d);
            for (int64_t i = axis + 1; i < rank; ++i) os.push_back(ds[(size_t)i]);
            out[0] = from_f32(in[3].et, os, o);
            return true;
        }, 4, 5);

    // ---- DynamicQuantize: per-group activation quantisation at run time (planar scales / zero points)
    reg("DynamicQuantize", "ie_internal_opset",
        {As("quantization_type", "Symmetric"), At("quantization_dt", ET::i8), At("scale_dt", ET::f16), At("zp_dt", ET::dynamic),
         At("precomputed_reduction_dt", ET::dynamic), Ab("precomputed_reduction", false), Ais("group_sizes"), Ais("scales_zp_output_order"),
         As("output_storage_type", "Planar")},
        [](Node& n) {
            const PShape& x = n.in_shape(0);
            const bool asym = n.attr_str("quantization_type") == "Asymmetric";
            n.set_num_outputs(asym ? 3 : 2);
            n.set_output(0, n.attr("quantization_dt").et, x);
            PShape sc = x;
            const auto& gs = n.attr_ints("group_sizes");
            if (!x.rank_dynamic) {
                OVC_CHECK(gs.size() == x.dims.size(), n.description() << ": group_sizes must have one entry per input axis");
                for (size_t i = 0; i < sc.dims.size(); ++i) {
                    if (!sc.dims[i].is_static() || sc.dims[i].lo == 0) continue;
                    // -1 (all bits set): one group spans the axis
                    sc.dims[i] = gs[i] < 0 ? Dim(1) : Dim((sc.dims[i].lo + gs[i] - 1) / std::max<int64_t>(gs[i], 1));
                }
                const auto& order = n.attr_ints("scales_zp_output_order");
                if (!order.empty()) {
                    PShape t = sc;
                    for (size_t i = 0; i < order.size() && i < t.dims.size(); ++i) t.dims[i] = sc.dims[(size_t)order[i]];
                    sc = t;
                }
            }
            n.set_output(1, n.attr("scale_dt").et, sc);
            if (asym) n.set_output(2, n.attr("zp_dt").et == ET::dynamic ? n.attr("quantization_dt").et : n.attr("zp_dt").et, sc);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& X = in[0];
            const auto order = n.attr_ints("scales_zp_output_order");
            OVC_CHECK(n.attr_str("output_storage_type") == "Planar" && (order.empty() || std::is_sorted(order.begin(), order.end())),
                      n.description() << ": the reference executor writes planar scales in the input's axis order");
            const auto x = to_f32(X);
            const auto& gs = n.attr_ints("group_sizes");
            const size_t rank = X.shape.size();
            OVC_CHECK(gs.size() == rank, n.description() << ": group_sizes must have one entry per input axis");
            Shape gshape(rank), gsize(rank);
            for (size_t i = 0; i < rank; ++i) {
                gsize[i] = gs[i] < 0 ? std::max<int64_t>(X.shape[i], 1) : std::max<int64_t>(gs[i], 1);
                gshape[i] = (X.shape[i] + gsize[i] - 1) / gsize[i];
            }
            const int64_t ngroups = shape_size(gshape);
            const bool asym = n.attr_str("quantization_type") == "Asymmetric";
            const ET qt = n.attr("quantization_dt").et;
            const bool is_unsigned = qt == ET::u8;
            std::vector<float> mn((size_t)ngroups, std::numeric_limits<float>::infinity()), mx((size_t)ngroups, -std::numeric_limits<float>::infinity());
            std::vector<int64_t> group_of(x.size());
            std::vector<int64_t> coord(rank, 0);
            for (size_t i = 0; i < x.size(); ++i) {
                int64_t g = 0;
                for (size_t d = 0; d < rank; ++d) g = g * gshape[d] + coord[d] / gsize[d];
                group_of[i] = g;
                mn[(size_t)g] = std::min(mn[(size_t)g], x[i]);
                mx[(size_t)g] = std::max(mx[(size_t)g], x[i]);
                for (int64_t d = (int64_t)rank - 1; d >= 0; --d) {
                    if (++coord[(size_t)d] < X.shape[(size_t)d]) break;
                    coord[(size_t)d] = 0;
                }
            }
            std::vector<float> scale((size_t)ngroups), zp((size_t)ngroups, 0.f);
            const float qmax = is_unsigned ? 255.f : 127.f, qmin = is_unsigned ? 0.f : (asym ? -128.f : -127.f);
            for (int64_t g = 0; g < ngroups; ++g) {
                if (asym) {
                    const float range = std::max(mx[(size_t)g] - mn[(size_t)g], 1e-8f);
                    scale[(size_t)g] = range / (qmax - qmin);
                    zp[(size_t)g] = std::nearbyint(qmin - mn[(size_t)g] / scale[(size_t)g]);
                } else {
                    const float amax = std::max(std::max(std::fabs(mn[(size_t)g]), std::fabs(mx[(size_t)g])), 1e-8f);
                    scale[(size_t)g] = amax / 127.f;
                }
            }
            std::vector<float> q(x.size());
            for (size_t i = 0; i < x.size(); ++i) {
                const size_t g = (size_t)group_of[i];
                q[i] = std::min(std::max(std::nearbyint(x[i] / scale[g] + zp[g]), qmin), qmax);
            }
            out[0] = from_f32(qt, X.shape, q);
            out[1] = from_f32(n.attr("scale_dt").et, gshape, scale);
            if (asym) out[2] = from_f32(n.attr("zp_dt").et == ET::dynamic ? qt : n.attr("zp_dt").et, gshape, zp);
            return true;
        }, 1, 1);

    // ---- MOECompressed: the MOE operation with group-quantised expert weights (weight, scale, zero point per projection)
    reg("MOECompressed", "",
        {As("expert_type", "GEMM3_SWIGLU"), Af("expert_alpha", 0, false), Af("expert_beta", 1, false), Ai("gate_idx", 0), As("activation_type", "SWISH"),
         Ai("hidden_size", 0), Ai("inter_size", 0), Ai("num_expert", 0), Ai("num_shared_expert", 0), Ai("top_k", 0), Ai("group_size", 0),
         Ab("has_batch_dim", false), Ab("has_zp", false), At("out_type", ET::dynamic)},
        [](Node& n) {
            const ET t = n.attr("out_type").et;
            n.set_output(0, t == ET::dynamic ? n.in_et(0) : t, n.in_shape(0));
        },
        [](N n, Ins in, Outs out, C ctx) {
            OVC_CHECK(n.attr_str("expert_type") == "GEMM3_SWIGLU" && in.size() == 12,
                      n.description() << ": the reference executor serves GEMM3_SWIGLU experts with (weight, scale, zero point) triples");
            const OpSchema* moe = OpRegistry::get().find("MOE", "internal");
            OVC_CHECK(moe != nullptr && moe->eval, "the MOE operation is not registered");
            std::vector<Tensor> ins = {in[0], in[1], in[2]};
            for (int p = 0; p < 3; ++p) {
                const Tensor& w = in[(size_t)(3 + 3 * p)];
                const auto deq = dequantise(w, in[(size_t)(4 + 3 * p)], &in[(size_t)(5 + 3 * p)]);
                Shape s = {w.shape[0], w.shape[1], (int64_t)(deq.size() / (size_t)(w.shape[0] * w.shape[1]))};
                ins.push_back(from_f32(ET::f32, s, deq));
            }
            return moe->eval(n, ins, out, ctx);
        }, 12, 12);

    // ---- LoraSubgraph (flat form): main_flow + ((x @ A^T) * alpha) @ B^T; A [r, in], alpha [1, r] or scalar, B [out, r]
    reg("LoraSubgraph", "ie_internal_opset", {},
        [](Node& n) { n.set_output(0, n.in_et(0), n.in_shape(0)); },
        [](N n, Ins in, Outs out, C) {
            const Tensor &M = in[0], &X = in[1], &Aw = in[2], &Al = in[3], &Bw = in[4];
            OVC_CHECK(Aw.shape.size() == 2 && Bw.shape.size() == 2, n.description() << ": the adapter matrices are 2-D");
            const int64_t r = Aw.shape[0], din = Aw.shape[1], dout = Bw.shape[0];
            OVC_CHECK(X.shape.back() == din && Bw.shape[1] == r && M.shape.back() == dout, n.description() << ": adapter shapes do not fit the projection");
            const int64_t rows = X.numel() / std::max<int64_t>(din, 1);
            auto o = to_f32(M);
            const auto x = to_f32(X), a = to_f32(Aw), al = to_f32(Al), b = to_f32(Bw);
            std::vector<float> t((size_t)r);
            for (int64_t i = 0; i < rows; ++i) {
                for (int64_t k = 0; k < r; ++k) {
                    float acc = 0;
                    for (int64_t d = 0; d < din; ++d) acc += x[(size_t)(i * din + d)] * a[(size_t)(k * din + d)];
                    t[(size_t)k] = acc * (al.size() == 1 ? al[0] : al[(size_t)(k % (int64_t)al.size())]);
                }
                for (int64_t j = 0; j < dout; ++j) {
                    float acc = 0;
                    for (int64_t k = 0; k < r; ++k) acc += t[(size_t)k] * b[(size_t)(j * r + k)];
                    o[(size_t)(i * dout + j)] += acc;
                }
            }
            out[0] = from_f32(M.et, M.shape, o);
            return true;
        }, 5, 5);

    // ---- ExtractImagePatches: [B, C, H, W] -> [B, C * kh * kw, OH, OW], channel = (kh * KW + kw) * C + c
    reg("ExtractImagePatches", "opset3", {Ais("sizes"), Ais("strides"), Ais("rates"), As("auto_pad", "valid")},
        [](Node& n) {
            const PShape& x = n.in_shape(0);
            if (x.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic(4)); return; }
            const auto &k = n.attr_ints("sizes"), &s = n.attr_ints("strides"), &r = n.attr_ints("rates");
            OVC_CHECK(x.dims.size() == 4 && k.size() == 2 && s.size() == 2 && r.size() == 2, n.description() << ": 4-D input and 2-D sizes / strides / rates expected");
            PShape o = x;
            o.dims[1] = x.dims[1].is_static() ? Dim(x.dims[1].lo * k[0] * k[1]) : Dim::dynamic();
            const bool valid = n.attr_str("auto_pad") == "valid";
            for (int i = 0; i < 2; ++i) {
                const Dim& d = x.dims[(size_t)(2 + i)];
                if (!d.is_static()) { o.dims[(size_t)(2 + i)] = Dim::dynamic(); continue; }
                const int64_t span = k[(size_t)i] + (r[(size_t)i] - 1) * (k[(size_t)i] - 1);
                o.dims[(size_t)(2 + i)] = valid ? Dim(d.lo < span ? 0 : (d.lo - span) / s[(size_t)i] + 1) : Dim((d.lo + s[(size_t)i] - 1) / s[(size_t)i]);
            }
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& X = in[0];
            const auto x = to_f32(X);
            const auto &k = n.attr_ints("sizes"), &s = n.attr_ints("strides"), &r = n.attr_ints("rates");
            const std::string pad = n.attr_str("auto_pad");
            const int64_t B = X.shape[0], Cc = X.shape[1], H = X.shape[2], W = X.shape[3];
            const int64_t span_h = k[0] + (r[0] - 1) * (k[0] - 1), span_w = k[1] + (r[1] - 1) * (k[1] - 1);
            const bool valid = pad == "valid";
            const int64_t OH = valid ? (H < span_h ? 0 : (H - span_h) / s[0] + 1) : (H + s[0] - 1) / s[0];
            const int64_t OW = valid ? (W < span_w ? 0 : (W - span_w) / s[1] + 1) : (W + s[1] - 1) / s[1];
            int64_t pt = 0, pl = 0;
            if (!valid) {
                // total padding so that ceil(size / stride) windows fit; an odd total puts the extra cell first for same_lower
                const int64_t ph = (OH - 1) * s[0] + span_h - H, pw = (OW - 1) * s[1] + span_w - W;
                if (ph > 0 && ph < span_h) pt = (ph % 2 == 1) ? (pad == "same_lower" ? (ph + 1) / 2 : (ph - 1) / 2) : ph / 2;
                if (pw > 0 && pw < span_w) pl = (pw % 2 == 1) ? (pad == "same_lower" ? (pw + 1) / 2 : (pw - 1) / 2) : pw / 2;
            }
            const int64_t OC = Cc * k[0] * k[1];
            std::vector<float> o((size_t)(B * OC * OH * OW), 0.f);
            for (int64_t b = 0; b < B; ++b)
                for (int64_t kh = 0; kh < k[0]; ++kh)
                    for (int64_t kw = 0; kw < k[1]; ++kw)
                        for (int64_t c = 0; c < Cc; ++c) {
                            const int64_t oc = (kh * k[1] + kw) * Cc + c;
                            for (int64_t oh = 0; oh < OH; ++oh) {
                                const int64_t ih = oh * s[0] - pt + kh * r[0];
                                if (ih < 0 || ih >= H) continue;
                                for (int64_t ow = 0; ow < OW; ++ow) {
                                    const int64_t iw = ow * s[1] - pl + kw * r[1];
                                    if (iw < 0 || iw >= W) continue;
                                    o[(size_t)(((b * OC + oc) * OH + oh) * OW + ow)] = x[(size_t)(((b * Cc + c) * H + ih) * W + iw)];
                                }
                            }
                        }
            out[0] = from_f32(X.et, {B, OC, OH, OW}, o);
            return true;
        }, 1, 1);

    // ---- RegionYolo
    reg("RegionYolo", "opset1",
        {Afs("anchors"), Ai("axis", 1), Ai("coords", 4), Ai("classes", 20), Ai("end_axis", 3), Ai("num", 1), Ab("do_softmax", true), Ais("mask")},
        [](Node& n) {
            const PShape& x = n.in_shape(0);
            if (x.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
            PShape o;
            o.rank_dynamic = false;
            const int64_t rank = (int64_t)x.dims.size();
            if (n.attr_bool("do_softmax")) {
                // axes [axis, end_axis] are flattened into one
                int64_t a = n.attr_int("axis"), e = n.attr_int("end_axis");
                a = a < 0 ? a + rank : a;
                e = e < 0 ? e + rank : e;
                OVC_CHECK(a >= 0 && e >= a && e < rank, n.description() << ": bad axis / end_axis");
                for (int64_t i = 0; i < a; ++i) o.dims.push_back(x.dims[(size_t)i]);
                Dim flat(1);
                for (int64_t i = a; i <= e; ++i) flat = (flat.is_static() && x.dims[(size_t)i].is_static()) ? Dim(flat.lo * x.dims[(size_t)i].lo) : Dim::dynamic();
                o.dims.push_back(flat);
                for (int64_t i = e + 1; i < rank; ++i) o.dims.push_back(x.dims[(size_t)i]);
            } else {
                OVC_CHECK(rank == 4, n.description() << ": 4-D input expected");
                o = x;
                o.dims[1] = Dim((n.attr_int("classes") + n.attr_int("coords") + 1) * (int64_t)n.attr_ints("mask").size());
            }
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& X = in[0];
            auto v = to_f32(X);
            const int64_t B = X.shape[0], Cc = X.shape[1], HW = X.numel() / std::max<int64_t>(B * Cc, 1);
            const int64_t coords = n.attr_int("coords"), classes = n.attr_int("classes");
            const bool sm = n.attr_bool("do_softmax");
            const int64_t regions = sm ? n.attr_int("num") : (int64_t)n.attr_ints("mask").size();
            const int64_t per = coords + classes + 1;
            OVC_CHECK(regions * per <= Cc, n.description() << ": " << regions << " regions of " << per << " channels do not fit " << Cc << " channels");
            auto logistic = [](float t) { return 1.f / (1.f + std::exp(-t)); };
            const int64_t out_c = sm ? Cc : regions * per;
            std::vector<float> o((size_t)(B * out_c * HW));
            for (int64_t b = 0; b < B; ++b) {
                const float* src = v.data() + b * Cc * HW;
                float* dst = o.data() + b * out_c * HW;
                std::copy_n(src, out_c * HW, dst);
                for (int64_t r = 0; r < regions; ++r) {
                    float* reg_ = dst + r * per * HW;
                    for (int64_t i = 0; i < 2 * HW; ++i) reg_[i] = logistic(reg_[i]);                  // x, y
                    for (int64_t i = 0; i < HW; ++i) reg_[coords * HW + i] = logistic(reg_[coords * HW + i]);   // objectness
                    float* cls = reg_ + (coords + 1) * HW;
                    if (sm) {
                        for (int64_t i = 0; i < HW; ++i) {
                            float m = -std::numeric_limits<float>::infinity(), sum = 0.f;
                            for (int64_t c = 0; c < classes; ++c) m = std::max(m, cls[c * HW + i]);
                            for (int64_t c = 0; c < classes; ++c) { cls[c * HW + i] = std::exp(cls[c * HW + i] - m); sum += cls[c * HW + i]; }
                            for (int64_t c = 0; c < classes; ++c) cls[c * HW + i] /= sum;
                        }
                    } else {
                        for (int64_t i = 0; i < classes * HW; ++i) cls[i] = logistic(cls[i]);
                    }
                }
            }
            Shape os;
            if (sm) {
                const int64_t rank = (int64_t)X.shape.size();
                int64_t a = n.attr_int("axis"), e = n.attr_int("end_axis");
                a = a < 0 ? a + rank : a;
                e = e < 0 ? e + rank : e;
                for (int64_t i = 0; i < a; ++i) os.push_back(X.shape[(size_t)i]);
                int64_t flat = 1;
                for (int64_t i = a; i <= e; ++i) flat *= X.shape[(size_t)i];
                os.push_back(flat);
                for (int64_t i = e + 1; i < rank; ++i) os.push_back(X.shape[(size_t)i]);
            } else {
                os = {B, out_c, X.shape[2], X.shape[3]};
            }
            out[0] = from_f32(X.et, os, o);
            return true;
        }, 1, 1);

    // ---- CTCLoss: negative log-likelihood of the label sequence under the connectionist temporal classification model
    reg("CTCLoss", "opset4", {Ab("preprocess_collapse_repeated", false), Ab("ctc_merge_repeated", true), Ab("unique", false)},
        [](Node& n) {
            const PShape& l = n.in_shape(0);
            PShape o = PShape::dynamic(1);
            if (!l.rank_dynamic && !l.dims.empty()) o.dims[0] = l.dims[0];
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& L = in[0];
            const auto logits = to_f32(L);
            const auto logit_len = to_i64(in[1]), labels = to_i64(in[2]), label_len = to_i64(in[3]);
            const int64_t B = L.shape[0], T = L.shape[1], Cc = L.shape[2];
            const int64_t blank = in.size() > 4 ? to_i64(in[4]).at(0) : Cc - 1;
            const bool collapse = n.attr_bool("preprocess_collapse_repeated"), merge = n.attr_bool("ctc_merge_repeated"), uniq = n.attr_bool("unique");
            const double ninf = -std::numeric_limits<double>::infinity();
            auto lse = [&](double a, double b) {
                if (a == ninf) return b;
                if (b == ninf) return a;
                return std::max(a, b) + std::log1p(std::exp(-std::fabs(a - b)));
            };
            std::vector<float> loss((size_t)B);
            for (int64_t b = 0; b < B; ++b) {
                const int64_t tl = logit_len[(size_t)b], ll = label_len[(size_t)b];
                OVC_CHECK(tl >= 0 && tl <= T && ll >= 0 && ll <= T && ll <= tl, n.description() << ": bad lengths for batch " << b);
                std::vector<int64_t> tgt;
                for (int64_t i = 0; i < ll; ++i) {
                    const int64_t c = labels[(size_t)(b * T + i)];
                    if (uniq && std::find(tgt.begin(), tgt.end(), c) != tgt.end()) continue;
                    if (collapse && !tgt.empty() && tgt.back() == c) continue;
                    tgt.push_back(c);
                }
                // extended sequence: blank, l1, blank, l2, ..., blank
                const int64_t S = 2 * (int64_t)tgt.size() + 1;
                std::vector<int64_t> ext((size_t)S, blank);
                for (size_t i = 0; i < tgt.size(); ++i) ext[2 * i + 1] = tgt[i];
                std::vector<double> alpha((size_t)S, ninf), next((size_t)S);
                auto logp = [&](int64_t t, int64_t c) {
                    const float* row = logits.data() + (b * T + t) * Cc;
                    double m = row[0];
                    for (int64_t k = 1; k < Cc; ++k) m = std::max<double>(m, row[k]);
                    double sum = 0;
                    for (int64_t k = 0; k < Cc; ++k) sum += std::exp(row[k] - m);
                    return row[c] - m - std::log(sum);
                };
                if (tl == 0) { loss[(size_t)b] = tgt.empty() ? 0.f : std::numeric_limits<float>::infinity(); continue; }
                alpha[0] = logp(0, ext[0]);
                if (S > 1) alpha[1] = logp(0, ext[1]);
                for (int64_t t = 1; t < tl; ++t) {
                    for (int64_t s = 0; s < S; ++s) {
                        double a = alpha[(size_t)s];
                        if (s >= 1) a = lse(a, alpha[(size_t)(s - 1)]);
                        // skipping the blank between two labels: always for different labels; for equal labels only when
                        // repeated labels are NOT merged (then "aa" may be emitted without a blank in between)
                        if (s >= 2 && ext[(size_t)s] != blank && (ext[(size_t)s] != ext[(size_t)(s - 2)] || !merge)) a = lse(a, alpha[(size_t)(s - 2)]);
                        next[(size_t)s] = a == ninf ? ninf : a + logp(t, ext[(size_t)s]);
                    }
                    alpha.swap(next);
                }
                double total = alpha[(size_t)(S - 1)];
                if (S > 1) total = lse(total, alpha[(size_t)(S - 2)]);
                loss[(size_t)b] = (float)-total;
            }
            out[0] = from_f32(L.et, {B}, loss);
            return true;
        }, 4, 5);

    // ---- STFT: short-time Fourier transform of real signals; frames of frame_size samples every frame_step samples
    reg("STFT", "opset15", {Ab("transpose_frames", false)},
        [](Node& n) {
            const PShape& sig = n.in_shape(0);
            std::vector<int64_t> fs, st;
            PShape o = PShape::dynamic(sig.rank_dynamic ? 4 : (int64_t)sig.dims.size() + 2);
            if (!sig.rank_dynamic && get_constant_ints(n.input(2), fs) && get_constant_ints(n.input(3), st) && !fs.empty() && !st.empty()) {
                const size_t r = sig.dims.size();
                OVC_CHECK(r == 1 || r == 2, n.description() << ": the signal is [length] or [batch, length]");
                const Dim& len = sig.dims[r - 1];
                const Dim frames = len.is_static() ? Dim(len.lo < fs[0] ? 0 : (len.lo - fs[0]) / st[0] + 1) : Dim::dynamic();
                const Dim bins(fs[0] / 2 + 1);
                o.dims.clear();
                if (r == 2) o.dims.push_back(sig.dims[0]);
                if (n.attr_bool("transpose_frames")) { o.dims.push_back(bins); o.dims.push_back(frames); }
                else { o.dims.push_back(frames); o.dims.push_back(bins); }
                o.dims.push_back(Dim(2));
            }
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& S = in[0];
            const auto sig = to_f32(S), win = to_f32(in[1]);
            const int64_t fs = to_i64(in[2]).at(0), step = to_i64(in[3]).at(0);
            OVC_CHECK(fs > 0 && step > 0 && (int64_t)win.size() <= fs, n.description() << ": frame_size / frame_step must be positive and the window no longer than a frame");
            const bool batched = S.shape.size() == 2;
            const int64_t B = batched ? S.shape[0] : 1, Len = S.shape.back();
            const int64_t frames = Len < fs ? 0 : (Len - fs) / step + 1, bins = fs / 2 + 1;
            // the window is centred in the frame and zero-padded
            std::vector<double> w((size_t)fs, 0.0);
            const int64_t off = (fs - (int64_t)win.size()) / 2;
            for (size_t i = 0; i < win.size(); ++i) w[(size_t)off + i] = win[i];
            const bool tr = n.attr_bool("transpose_frames");
            std::vector<float> o((size_t)(B * frames * bins * 2));
            std::vector<double> cs((size_t)fs), sn((size_t)fs);
            for (int64_t i = 0; i < fs; ++i) { cs[(size_t)i] = std::cos(2.0 * M_PI * i / fs); sn[(size_t)i] = std::sin(2.0 * M_PI * i / fs); }
            for (int64_t b = 0; b < B; ++b)
                for (int64_t f = 0; f < frames; ++f)
                    for (int64_t k = 0; k < bins; ++k) {
                        double re = 0, im = 0;
                        for (int64_t t = 0; t < fs; ++t) {
                            const double v = sig[(size_t)(b * Len + f * step + t)] * w[(size_t)t];
                            const int64_t ph = (k * t) % fs;
                            re += v * cs[(size_t)ph];
                            im -= v * sn[(size_t)ph];
                        }
                        const int64_t at = tr ? ((b * bins + k) * frames + f) : ((b * frames + f) * bins + k);
                        o[(size_t)(2 * at)] = (float)re;
                        o[(size_t)(2 * at + 1)] = (float)im;
                    }
            Shape os;
            if (batched) os.push_back(B);
            if (tr) { os.push_back(bins); os.push_back(frames); } else { os.push_back(frames); os.push_back(bins); }
            os.push_back(2);
            out[0] = from_f32(S.et, os, o);
            return true;
        }, 4, 4);
}

}  // namespace ovc
