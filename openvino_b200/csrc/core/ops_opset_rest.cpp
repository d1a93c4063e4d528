// The remaining operations of the public operation sets: deformable convolution and deformable position-sensitive ROI
// pooling, binary (xnor-popcount) convolution, string tensor pack / unpack, Reverse, inverse STFT, the opset1 Xor and
// the RGB / BGR -> NV12 colour conversions: attribute schemas (reference visit_attributes order), shape / type
// inference, reference evaluation.
//
// Reference counterparts: src/core/src/op/{deformable_convolution,deformable_psroi_pooling,binary_convolution,
// string_tensor_pack,string_tensor_unpack,reverse,istft,xor,rgb_to_nv12,bgr_to_nv12}.cpp and the kernels of the same
// names under src/core/reference/include/openvino/reference/.
#include <algorithm>
#include <cmath>
#include <limits>
#include <map>

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
AttrSpec Ais(const char* n, std::vector<int64_t> d = {}) { return A(n, K::INTS, Attr::Ints(std::move(d))); }
AttrSpec Ab(const char* n, bool d = false) { return A(n, K::BOOL, Attr::Bool(d)); }
AttrSpec Af(const char* n, double d = 0) { AttrSpec s = A(n, K::FLOAT, Attr::Float(d)); s.f32 = true; return s; }
AttrSpec As(const char* n, const char* d = "") { return A(n, K::STR, Attr::Str(d)); }

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

// ---- 2-D window geometry shared by the convolutions of this file
struct Win {
    int64_t sh = 1, sw = 1, dh = 1, dw = 1, pt = 0, pl = 0, pb = 0, pr = 0;
};

int64_t or1(const std::vector<int64_t>& v, size_t i) { return i < v.size() ? v[i] : 1; }
int64_t or0(const std::vector<int64_t>& v, size_t i) { return i < v.size() ? v[i] : 0; }

// strides / dilations / pads of a node with the auto_pad rule applied for a static input extent
Win window_of(const Node& n, int64_t H, int64_t W, int64_t KH, int64_t KW) {
    Win w;
    const auto st = n.attr_ints("strides"), dl = n.attr_ints("dilations"), pb = n.attr_ints("pads_begin"), pe = n.attr_ints("pads_end");
    w.sh = or1(st, 0); w.sw = or1(st, 1); w.dh = or1(dl, 0); w.dw = or1(dl, 1);
    w.pt = or0(pb, 0); w.pl = or0(pb, 1); w.pb = or0(pe, 0); w.pr = or0(pe, 1);
    const std::string ap = n.attr_str("auto_pad", "explicit");
    if (ap == "valid") w.pt = w.pl = w.pb = w.pr = 0;
    if (ap == "same_upper" || ap == "same_lower") {
        auto split = [&](int64_t in, int64_t k, int64_t s, int64_t d, int64_t& lo, int64_t& hi) {
            const int64_t out = (in + s - 1) / s, total = std::max<int64_t>(0, (out - 1) * s + d * (k - 1) + 1 - in), half = total / 2;
            if (ap == "same_upper") { lo = half; hi = total - half; } else { hi = half; lo = total - half; }
        };
        split(H, KH, w.sh, w.dh, w.pt, w.pb);
        split(W, KW, w.sw, w.dw, w.pl, w.pr);
    }
    return w;
}

Dim out_extent(const Dim& in, int64_t k, int64_t s, int64_t d, int64_t p0, int64_t p1, const std::string& ap) {
    if (!in.is_static()) return Dim::dynamic();
    if (ap == "same_upper" || ap == "same_lower") return Dim((in.lo + s - 1) / s);
    const int64_t padded = in.lo + (ap == "valid" ? 0 : p0 + p1), eff = d * (k - 1) + 1;
    return Dim(padded < eff ? 0 : (padded - eff) / s + 1);
}

void infer_conv_like(Node& n, size_t filt_input) {
    const PShape &x = n.in_shape(0), &f = n.in_shape(filt_input);
    PShape o = PShape::dynamic(4);
    o.dims[0] = dim_of(x, 0);
    o.dims[1] = dim_of(f, 0);
    const Dim kh = dim_of(f, 2), kw = dim_of(f, 3);
    if (kh.is_static() && kw.is_static()) {
        const auto st = n.attr_ints("strides"), dl = n.attr_ints("dilations"), pb = n.attr_ints("pads_begin"), pe = n.attr_ints("pads_end");
        const std::string ap = n.attr_str("auto_pad", "explicit");
        o.dims[2] = out_extent(dim_of(x, 2), kh.lo, or1(st, 0), or1(dl, 0), or0(pb, 0), or0(pe, 0), ap);
        o.dims[3] = out_extent(dim_of(x, 3), kw.lo, or1(st, 1), or1(dl, 1), or0(pb, 1), or0(pe, 1), ap);
    }
    n.set_output(0, n.in_et(0), o);
}

// value of a plane at a fractional position. `padded`: positions up to one pixel outside blend with zeros; otherwise
// only positions inside the plane count and the far neighbours are clamped to the last row / column.
float sample(const float* p, int64_t H, int64_t W, float y, float x, bool padded) {
    if (padded) {
        if (y <= -1.f || y >= (float)H || x <= -1.f || x >= (float)W) return 0.f;
        const int64_t y0 = (int64_t)std::floor(y), x0 = (int64_t)std::floor(x);
        const float ly = y - y0, lx = x - x0;
        auto at = [&](int64_t yy, int64_t xx) { return (yy < 0 || yy >= H || xx < 0 || xx >= W) ? 0.f : p[yy * W + xx]; };
        return (1 - ly) * (1 - lx) * at(y0, x0) + (1 - ly) * lx * at(y0, x0 + 1) + ly * (1 - lx) * at(y0 + 1, x0) + ly * lx * at(y0 + 1, x0 + 1);
    }
    if (y < 0.f || y >= (float)H || x < 0.f || x >= (float)W) return 0.f;
    const int64_t y0 = (int64_t)std::floor(y), x0 = (int64_t)std::floor(x), y1 = std::min(y0 + 1, H - 1), x1 = std::min(x0 + 1, W - 1);
    const float ly = y - y0, lx = x - x0;
    return (1 - ly) * (1 - lx) * p[y0 * W + x0] + (1 - ly) * lx * p[y0 * W + x1] + ly * (1 - lx) * p[y1 * W + x0] + ly * lx * p[y1 * W + x1];
}

bool eval_deformable_conv(N n, Ins in, Outs out, C) {
    const Tensor &X = in[0], &O = in[1], &F = in[2];
    const auto x = to_f32(X), off = to_f32(O), f = to_f32(F);
    std::vector<float> mask;
    if (in.size() > 3) mask = to_f32(in[3]);
    const int64_t B = X.shape[0], Cin = X.shape[1], H = X.shape[2], W = X.shape[3];
    const int64_t OC = F.shape[0], Cg = F.shape[1], KH = F.shape[2], KW = F.shape[3];
    const int64_t G = n.attr_int("group", 1), DG = n.attr_int("deformable_group", 1);
    OVC_CHECK(Cin == Cg * G && OC % G == 0 && Cin % DG == 0, n.description() << ": channels do not divide into " << G << " groups / " << DG << " deformable groups");
    const Win w = window_of(n, H, W, KH, KW);
    const int64_t OH = O.shape[2], OW = O.shape[3];
    OVC_CHECK(O.shape[1] == DG * KH * KW * 2, n.description() << ": the offsets input needs deformable_group * kh * kw * 2 channels");
    const bool padded = n.has_attr("bilinear_interpolation_pad") && n.attr_bool("bilinear_interpolation_pad");
    std::vector<float> o((size_t)(B * OC * OH * OW), 0.f);
    const int64_t oc_per_g = OC / G, c_per_dg = Cin / DG;
    for (int64_t b = 0; b < B; ++b)
        for (int64_t oc = 0; oc < OC; ++oc) {
            const int64_t g = oc / oc_per_g;
            for (int64_t oh = 0; oh < OH; ++oh)
                for (int64_t ow = 0; ow < OW; ++ow) {
                    float acc = 0;
                    for (int64_t ci = 0; ci < Cg; ++ci) {
                        const int64_t c = g * Cg + ci, dg = c / c_per_dg;
                        const float* plane = x.data() + (b * Cin + c) * H * W;
                        for (int64_t kh = 0; kh < KH; ++kh)
                            for (int64_t kw = 0; kw < KW; ++kw) {
                                const int64_t kpos = kh * KW + kw;
                                const float dy = off[(size_t)(((b * DG * KH * KW * 2 + (dg * KH * KW + kpos) * 2) * OH + oh) * OW + ow)];
                                const float dx = off[(size_t)(((b * DG * KH * KW * 2 + (dg * KH * KW + kpos) * 2 + 1) * OH + oh) * OW + ow)];
                                float v = sample(plane, H, W, (float)(oh * w.sh - w.pt + kh * w.dh) + dy, (float)(ow * w.sw - w.pl + kw * w.dw) + dx, padded);
                                if (!mask.empty()) v *= mask[(size_t)(((b * DG * KH * KW + dg * KH * KW + kpos) * OH + oh) * OW + ow)];
                                acc += v * f[(size_t)(((oc * Cg + ci) * KH + kh) * KW + kw)];
                            }
                    }
                    o[(size_t)(((b * OC + oc) * OH + oh) * OW + ow)] = acc;
                }
        }
    out[0] = from_f32(X.et, {B, OC, OH, OW}, o);
    return true;
}

// ---- string tensors
void infer_string_unpack(Node& n) {
    n.set_num_outputs(3);
    n.set_output(0, ET::i32, n.in_shape(0));
    n.set_output(1, ET::i32, n.in_shape(0));
    n.set_output(2, ET::u8, PShape::dynamic(1));
}

// ---- RGB / BGR -> NV12 (BT.601 limited range, the inverse of the NV12 -> RGB operations)
void infer_to_nv12(Node& n) {
    const PShape& x = n.in_shape(0);
    const bool single = n.attr_bool("single_plane", true);
    if (x.rank_dynamic) {
        n.set_num_outputs(single ? 1 : 2);
        n.set_output(0, n.in_et(0), PShape::dynamic(4));
        if (!single) n.set_output(1, n.in_et(0), PShape::dynamic(4));
        return;
    }
    OVC_CHECK(x.dims.size() == 4, n.description() << ": [N, H, W, 3] input expected");
    const Dim H = x.dims[1], W = x.dims[2];
    if (H.is_static()) OVC_CHECK(H.lo % 2 == 0, n.description() << ": the image height must be even");
    if (W.is_static()) OVC_CHECK(W.lo % 2 == 0, n.description() << ": the image width must be even");
    if (single) {
        n.set_output(0, n.in_et(0), PShape({x.dims[0], H.is_static() ? Dim(H.lo * 3 / 2) : Dim::dynamic(), W, Dim(1)}));
    } else {
        n.set_num_outputs(2);
        n.set_output(0, n.in_et(0), PShape({x.dims[0], H, W, Dim(1)}));
        n.set_output(1, n.in_et(0), PShape({x.dims[0], H.is_static() ? Dim(H.lo / 2) : Dim::dynamic(), W.is_static() ? Dim(W.lo / 2) : Dim::dynamic(), Dim(2)}));
    }
}

bool eval_to_nv12(N n, Ins in, Outs out, bool bgr) {
    const Tensor& X = in[0];
    const auto x = to_f32(X);
    const int64_t B = X.shape[0], H = X.shape[1], W = X.shape[2];
    OVC_CHECK(X.shape.size() == 4 && X.shape[3] == 3 && H % 2 == 0 && W % 2 == 0, n.description() << ": [N, even H, even W, 3] input expected");
    const bool integral = !et_is_real(X.et);
    auto clip = [&](double a) { return (float)std::min(std::max(integral ? std::round(a) : a, 0.0), 255.0); };
    std::vector<float> y((size_t)(B * H * W)), uv((size_t)(B * (H / 2) * (W / 2) * 2));
    std::vector<float> u((size_t)(H * W)), v((size_t)(H * W));
    for (int64_t b = 0; b < B; ++b) {
        for (int64_t i = 0; i < H * W; ++i) {
            const float* p = x.data() + (b * H * W + i) * 3;
            const double r = bgr ? p[2] : p[0], g = p[1], bl = bgr ? p[0] : p[2];
            y[(size_t)(b * H * W + i)] = clip(0.257 * r + 0.504 * g + 0.098 * bl + 16.0);
            u[(size_t)i] = clip(-0.148 * r - 0.291 * g + 0.439 * bl + 128.0);
            v[(size_t)i] = clip(0.439 * r - 0.368 * g - 0.071 * bl + 128.0);
        }
        // chroma: mean of each 2 x 2 block
        for (int64_t h = 0; h < H / 2; ++h)
            for (int64_t w = 0; w < W / 2; ++w) {
                auto mean4 = [&](const std::vector<float>& pl) {
                    const double s = (double)pl[(size_t)(2 * h * W + 2 * w)] + pl[(size_t)(2 * h * W + 2 * w + 1)] + pl[(size_t)((2 * h + 1) * W + 2 * w)] + pl[(size_t)((2 * h + 1) * W + 2 * w + 1)];
                    return (float)(integral ? std::round(s / 4.0) : s / 4.0);
                };
                const int64_t at = ((b * (H / 2) + h) * (W / 2) + w) * 2;
                uv[(size_t)at] = mean4(u);
                uv[(size_t)at + 1] = mean4(v);
            }
    }
    if (n.attr_bool("single_plane", true)) {
        // the UV plane follows the Y plane: H/2 rows of W interleaved bytes
        std::vector<float> o((size_t)(B * (H * 3 / 2) * W));
        for (int64_t b = 0; b < B; ++b) {
            std::copy(y.begin() + b * H * W, y.begin() + (b + 1) * H * W, o.begin() + b * (H * 3 / 2) * W);
            std::copy(uv.begin() + b * (H / 2) * W, uv.begin() + (b + 1) * (H / 2) * W, o.begin() + b * (H * 3 / 2) * W + H * W);
        }
        out[0] = from_f32(X.et, {B, H * 3 / 2, W, 1}, o);
    } else {
        out[0] = from_f32(X.et, {B, H, W, 1}, y);
        out[1] = from_f32(X.et, {B, H / 2, W / 2, 2}, uv);
    }
    return true;
}


// ---- Einsum: every output element is the sum over the contracted labels of the product of the operands
bool eval_einsum(N n, Ins in, Outs out, C) {
    std::string eq = n.attr_str("equation");
    eq.erase(std::remove(eq.begin(), eq.end(), ' '), eq.end());
    const size_t arrow = eq.find("->");
    std::string lhs = arrow == std::string::npos ? eq : eq.substr(0, arrow);
    std::vector<std::string> terms;
    for (size_t p = 0;;) {
        const size_t c = lhs.find(',', p);
        terms.push_back(lhs.substr(p, c == std::string::npos ? std::string::npos : c - p));
        if (c == std::string::npos) break;
        p = c + 1;
    }
    OVC_CHECK(terms.size() == in.size(), n.description() << ": the equation names " << terms.size() << " operands, " << in.size() << " are given");
    // labels: letters, plus one synthetic label per broadcast axis that an ellipsis stands for (aligned from the right)
    size_t ell_rank = 0;
    for (size_t t = 0; t < terms.size(); ++t) {
        const size_t e = terms[t].find("...");
        if (e != std::string::npos) ell_rank = std::max(ell_rank, in[t].shape.size() - (terms[t].size() - 3));
    }
    auto expand = [&](const std::string& term, size_t rank_of_operand, bool is_output) {
        std::vector<int> labels;
        const size_t e = term.find("...");
        for (size_t k = 0; k < term.size(); ++k) {
            if (e != std::string::npos && k == e) {
                const size_t here = is_output ? ell_rank : rank_of_operand - (term.size() - 3);
                for (size_t a = 0; a < here; ++a) labels.push_back(256 + (int)(ell_rank - here + a));
                k += 2;
                continue;
            }
            labels.push_back((int)(unsigned char)term[k]);
        }
        return labels;
    };
    std::vector<std::vector<int>> tl;
    for (size_t t = 0; t < terms.size(); ++t) {
        tl.push_back(expand(terms[t], in[t].shape.size(), false));
        OVC_CHECK(tl.back().size() == in[t].shape.size(), n.description() << ": term '" << terms[t] << "' does not match an operand of rank " << in[t].shape.size());
    }
    std::map<int, int64_t> extent;
    for (size_t t = 0; t < tl.size(); ++t)
        for (size_t a = 0; a < tl[t].size(); ++a) {
            const int64_t d = in[t].shape[a];
            auto it = extent.find(tl[t][a]);
            if (it == extent.end() || it->second == 1) extent[tl[t][a]] = d;
            else OVC_CHECK(d == 1 || d == it->second, n.description() << ": label extents " << it->second << " and " << d << " do not agree");
        }
    std::vector<int> ol;
    if (arrow != std::string::npos) {
        ol = expand(eq.substr(arrow + 2), 0, true);
    } else {                                     // implicit output: ellipsis axes, then the letters that occur once, sorted
        for (size_t a = 0; a < ell_rank; ++a) ol.push_back(256 + (int)a);
        std::map<int, int> count;
        for (auto& t : tl) for (int l : t) if (l < 256) ++count[l];
        for (auto& kv : count) if (kv.second == 1) ol.push_back(kv.first);
    }
    std::vector<int> all = ol;                    // output labels first, then the contracted ones
    for (auto& kv : extent) if (std::find(all.begin(), all.end(), kv.first) == all.end()) all.push_back(kv.first);
    std::vector<int64_t> ext;
    for (int l : all) { OVC_CHECK(extent.count(l), n.description() << ": output label without an operand"); ext.push_back(extent[l]); }
    Shape os(ext.begin(), ext.begin() + (long)ol.size());
    int64_t out_total = 1, red_total = 1;
    for (size_t k = 0; k < all.size(); ++k) (k < ol.size() ? out_total : red_total) *= ext[k];
    std::vector<std::vector<float>> data;
    for (auto& t : in) data.push_back(to_f32(t));
    // stride of every label in every operand (0 where the operand lacks the label or broadcasts it)
    std::vector<std::vector<int64_t>> stride(in.size(), std::vector<int64_t>(all.size(), 0));
    for (size_t t = 0; t < in.size(); ++t) {
        int64_t st = 1;
        for (size_t a = tl[t].size(); a-- > 0;) {
            if (in[t].shape[a] != 1) {
                const size_t pos = std::find(all.begin(), all.end(), tl[t][a]) - all.begin();
                stride[t][pos] += st;            // a label used twice in one term walks the diagonal
            }
            st *= in[t].shape[a];
        }
    }
    std::vector<float> o((size_t)out_total);
    std::vector<int64_t> idx(all.size(), 0);
    for (int64_t oi = 0; oi < out_total; ++oi) {
        int64_t rem = oi;
        for (size_t k = ol.size(); k-- > 0;) { idx[k] = rem % ext[k]; rem /= ext[k]; }
        double acc = 0;
        for (int64_t ri = 0; ri < red_total; ++ri) {
            int64_t r2 = ri;
            for (size_t k = all.size(); k-- > ol.size();) { idx[k] = r2 % ext[k]; r2 /= ext[k]; }
            double prod = 1;
            for (size_t t = 0; t < in.size(); ++t) {
                int64_t off = 0;
                for (size_t k = 0; k < all.size(); ++k) off += idx[k] * stride[t][k];
                prod *= data[t][(size_t)off];
            }
            acc += prod;
        }
        o[(size_t)oi] = (float)acc;
    }
    out[0] = from_f32(in[0].et, os, o);
    return true;
}

}  // namespace

void register_rest_ops() {
    if (auto* es = const_cast<OpSchema*>(OpRegistry::get().find("Einsum", "opset7")); es && !es->eval) es->eval = eval_einsum;
    // ---- DeformableConvolution: every kernel tap reads the input at its own learned offset
    const std::vector<AttrSpec> dc1 = {Ais("strides"), Ais("dilations"), Ais("pads_begin"), Ais("pads_end"), As("auto_pad", "explicit"), Ai("group", 1), Ai("deformable_group", 1)};
    std::vector<AttrSpec> dc8 = {Ab("bilinear_interpolation_pad")};
    dc8.insert(dc8.end(), dc1.begin(), dc1.end());
    auto infer_dc = [](Node& n) {
        // the output extent equals the spatial extent of the offsets
        infer_conv_like(n, 2);
    };
    reg("DeformableConvolution", "opset1", dc1, infer_dc, eval_deformable_conv, 3, 3);
    reg("DeformableConvolution", "opset8", dc8, infer_dc, eval_deformable_conv, 3, 4);

    // ---- DeformablePSROIPooling
    reg("DeformablePSROIPooling", "opset1", {Ai("output_dim", 0), Af("spatial_scale", 1), Ai("group_size", 1), As("mode", "bilinear_deformable"), Ai("spatial_bins_x", 1),
                                             Ai("spatial_bins_y", 1), Af("trans_std", 1), Ai("part_size", 1)},
        [](Node& n) {
            const int64_t G = n.attr_int("group_size", 1);
            n.set_output(0, n.in_et(0), PShape({dim_of(n.in_shape(1), 0), Dim(n.attr_int("output_dim")), Dim(G), Dim(G)}));
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& X = in[0];
            const auto x = to_f32(X), rois = to_f32(in[1]);
            const bool no_trans = in.size() < 3;
            std::vector<float> tr;
            if (!no_trans) tr = to_f32(in[2]);
            const int64_t Cin = X.shape[1], H = X.shape[2], W = X.shape[3], R = in[1].shape[0];
            const int64_t OD = n.attr_int("output_dim"), G = n.attr_int("group_size", 1), SBX = n.attr_int("spatial_bins_x", 1), SBY = n.attr_int("spatial_bins_y", 1);
            const int64_t part = n.attr_int("part_size", 1) > 0 ? n.attr_int("part_size", 1) : G;
            const float scale = (float)n.attr_float("spatial_scale"), tstd = (float)n.attr_float("trans_std", 1);
            const int64_t n_cls = no_trans ? 1 : in[2].shape[1] / 2, ch_per_cls = OD / n_cls;
            OVC_CHECK(Cin >= OD * G * G, n.description() << ": the input needs output_dim * group_size^2 channels");
            std::vector<float> o((size_t)(R * OD * G * G), 0.f);
            for (int64_t r = 0; r < R; ++r) {
                const float* box = rois.data() + r * 5;
                const int64_t b = (int64_t)box[0];
                const float x0 = std::round(box[1]) * scale - 0.5f, y0 = std::round(box[2]) * scale - 0.5f;
                const float x1 = (std::round(box[3]) + 1.f) * scale - 0.5f, y1 = (std::round(box[4]) + 1.f) * scale - 0.5f;
                const float rw = std::max(x1 - x0, 0.1f), rh = std::max(y1 - y0, 0.1f), bw = rw / G, bh = rh / G;
                for (int64_t c = 0; c < OD; ++c)
                    for (int64_t ph = 0; ph < G; ++ph)
                        for (int64_t pw = 0; pw < G; ++pw) {
                            float tx = 0, ty = 0;
                            if (!no_trans) {
                                const int64_t cls = c / ch_per_cls, py = ph * part / G, px = pw * part / G;
                                tx = tr[(size_t)((((r * n_cls + cls) * 2) * part + py) * part + px)] * tstd;
                                ty = tr[(size_t)((((r * n_cls + cls) * 2 + 1) * part + py) * part + px)] * tstd;
                            }
                            const float ws = pw * bw + x0 + tx * rw, hs = ph * bh + y0 + ty * rh;
                            const float* plane = x.data() + (b * Cin + (c * G + ph) * G + pw) * H * W;     // group cell == output bin
                            float sum = 0;
                            int64_t cnt = 0;
                            for (int64_t iy = 0; iy < SBY; ++iy)
                                for (int64_t ix = 0; ix < SBX; ++ix) {
                                    float sx = ws + ix * bw / SBX, sy = hs + iy * bh / SBY;
                                    if (sx < -0.5f || sx > W - 0.5f || sy < -0.5f || sy > H - 0.5f) continue;
                                    sx = std::min(std::max(sx, 0.f), (float)W - 1.f);
                                    sy = std::min(std::max(sy, 0.f), (float)H - 1.f);
                                    sum += sample(plane, H, W, sy, sx, false);
                                    ++cnt;
                                }
                            o[(size_t)(((r * OD + c) * G + ph) * G + pw)] = cnt ? sum / cnt : 0.f;
                        }
            }
            out[0] = from_f32(X.et, {R, OD, G, G}, o);
            return true;
        }, 2, 3);

    // ---- BinaryConvolution (xnor-popcount): input and 1-bit filters both read as -1 / +1
    reg("BinaryConvolution", "opset1", {Ais("strides"), Ais("pads_begin"), Ais("pads_end"), Ais("dilations"), As("mode", "xnor-popcount"), Af("pad_value", 0), As("auto_pad", "explicit")},
        [](Node& n) { infer_conv_like(n, 1); },
        [](N n, Ins in, Outs out, C) {
            OVC_CHECK(n.attr_str("mode", "xnor-popcount") == "xnor-popcount", n.description() << ": mode must be xnor-popcount");
            const Tensor &X = in[0], &F = in[1];
            const auto x = to_f32(X), f = to_f32(F);                 // 1-bit filters unpack to 0 / 1
            const int64_t B = X.shape[0], Cin = X.shape[1], H = X.shape[2], W = X.shape[3], OC = F.shape[0], KH = F.shape[2], KW = F.shape[3];
            OVC_CHECK(F.shape[1] == Cin, n.description() << ": filter channels differ from the input's");
            const Win w = window_of(n, H, W, KH, KW);
            const int64_t OH = (H + w.pt + w.pb - (w.dh * (KH - 1) + 1)) / w.sh + 1, OW = (W + w.pl + w.pr - (w.dw * (KW - 1) + 1)) / w.sw + 1;
            const bool pad_bit = n.attr_float("pad_value") > 0;
            std::vector<float> o((size_t)(B * OC * OH * OW));
            for (int64_t b = 0; b < B; ++b)
                for (int64_t oc = 0; oc < OC; ++oc)
                    for (int64_t oh = 0; oh < OH; ++oh)
                        for (int64_t ow = 0; ow < OW; ++ow) {
                            int64_t same = 0;
                            for (int64_t c = 0; c < Cin; ++c)
                                for (int64_t kh = 0; kh < KH; ++kh)
                                    for (int64_t kw = 0; kw < KW; ++kw) {
                                        const int64_t ih = oh * w.sh - w.pt + kh * w.dh, iw = ow * w.sw - w.pl + kw * w.dw;
                                        const bool xb = (ih < 0 || ih >= H || iw < 0 || iw >= W) ? pad_bit : x[(size_t)(((b * Cin + c) * H + ih) * W + iw)] > 0;
                                        same += xb == (f[(size_t)(((oc * Cin + c) * KH + kh) * KW + kw)] > 0);
                                    }
                            o[(size_t)(((b * OC + oc) * OH + oh) * OW + ow)] = (float)(2 * same - Cin * KH * KW);
                        }
            out[0] = from_f32(X.et, {B, OC, OH, OW}, o);
            return true;
        }, 2, 2);

    // ---- StringTensorUnpack: strings -> begin / end offsets into one byte array;  StringTensorPack: the inverse
    reg("StringTensorUnpack", "opset15", {}, infer_string_unpack,
        [](N n, Ins in, Outs out, C) {
            OVC_CHECK(in[0].et == ET::string, n.description() << ": a string tensor is expected");
            const auto& s = in[0].strings;
            std::vector<int64_t> b, e, sym;
            int64_t at = 0;
            for (const std::string& v : s) {
                b.push_back(at);
                at += (int64_t)v.size();
                e.push_back(at);
                for (unsigned char ch : v) sym.push_back(ch);
            }
            out[0] = from_i64(ET::i32, in[0].shape, b);
            out[1] = from_i64(ET::i32, in[0].shape, e);
            out[2] = from_i64(ET::u8, {at}, sym);
            return true;
        }, 1, 1);
    reg("StringTensorPack", "opset15", {},
        [](Node& n) { n.set_output(0, ET::string, n.in_shape(0)); },
        [](N n, Ins in, Outs out, C) {
            const auto b = to_i64(in[0]), e = to_i64(in[1]), sym = to_i64(in[2]);
            OVC_CHECK(b.size() == e.size(), n.description() << ": begins and ends differ in size");
            Tensor t(ET::string, in[0].shape);
            for (size_t i = 0; i < b.size(); ++i) {
                OVC_CHECK(0 <= b[i] && b[i] <= e[i] && e[i] <= (int64_t)sym.size(), n.description() << ": string " << i << " spans [" << b[i] << ", " << e[i] << ") outside the symbols");
                std::string s;
                for (int64_t k = b[i]; k < e[i]; ++k) s.push_back((char)sym[(size_t)k]);
                t.strings[i] = std::move(s);
            }
            out[0] = std::move(t);
            return true;
        }, 3, 3);

    // ---- Reverse: flip along the axes given as indices or as a boolean mask
    reg("Reverse", "opset1", {As("mode", "index")},
        [](Node& n) { n.set_output(0, n.in_et(0), n.in_shape(0)); },
        [](N n, Ins in, Outs out, C) {
            const Tensor& X = in[0];
            const auto ax = to_i64(in[1]);
            const size_t r = X.shape.size();
            std::vector<bool> flip(r, false);
            if (n.attr_str("mode", "index") == "mask") {
                OVC_CHECK(ax.size() == r, n.description() << ": the mask needs one flag per axis");
                for (size_t i = 0; i < r; ++i) flip[i] = ax[i] != 0;
            } else {
                for (int64_t a : ax) {
                    OVC_CHECK(a >= -(int64_t)r && a < (int64_t)r, n.description() << ": axis " << a << " out of range");
                    flip[(size_t)(a < 0 ? a + (int64_t)r : a)] = true;
                }
            }
            Tensor o(X.et, X.shape);
            const size_t esz = et_byte_size(X.et, 1);
            OVC_CHECK(X.et != ET::string && esz * (size_t)X.numel() == X.byte_size(), n.description() << ": whole-byte element types only");
            const int64_t total = X.numel();
            std::vector<int64_t> idx(r, 0);
            for (int64_t i = 0; i < total; ++i) {
                int64_t rem = i, src = 0, stride = 1;
                for (size_t d = r; d-- > 0;) {
                    const int64_t c = rem % X.shape[d];
                    rem /= X.shape[d];
                    src += (flip[d] ? X.shape[d] - 1 - c : c) * stride;
                    stride *= X.shape[d];
                }
                std::copy(X.data() + (size_t)src * esz, X.data() + (size_t)(src + 1) * esz, o.data() + (size_t)i * esz);
            }
            out[0] = std::move(o);
            return true;
        }, 2, 2);

    // ---- ISTFT: inverse real FFT of every frame, windowed overlap-add, division by the summed squared window
    reg("ISTFT", "opset16", {Ab("center"), Ab("normalized")},
        [](Node& n) {
            const PShape& d = n.in_shape(0);
            PShape o = PShape::dynamic(d.rank_dynamic ? 1 : d.dims.size() - 2);
            if (!d.rank_dynamic) {
                OVC_CHECK(d.dims.size() == 3 || d.dims.size() == 4, n.description() << ": data is [bins, frames, 2] or [batch, bins, frames, 2]");
                const bool batched = d.dims.size() == 4;
                if (batched) o.dims[0] = d.dims[0];
                std::vector<int64_t> len, fs, st;
                const Dim frames = d.dims[batched ? 2 : 1];
                if (n.num_inputs() > 4 && get_constant_ints(n.input(4), len) && !len.empty()) o.dims.back() = Dim(len[0]);
                else if (n.num_inputs() <= 4 && frames.is_static() && get_constant_ints(n.input(2), fs) && get_constant_ints(n.input(3), st) && !fs.empty() && !st.empty())
                    o.dims.back() = Dim((frames.lo - 1) * st[0] + (n.attr_bool("center") ? 0 : fs[0]));
            }
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& D = in[0];
            const auto d = to_f32(D), win = to_f32(in[1]);
            const int64_t fs = to_i64(in[2]).at(0), step = to_i64(in[3]).at(0);
            const bool batched = D.shape.size() == 4, center = n.attr_bool("center");
            const int64_t B = batched ? D.shape[0] : 1, bins = D.shape[batched ? 1 : 0], frames = D.shape[batched ? 2 : 1];
            OVC_CHECK(fs > 0 && step > 0 && bins == fs / 2 + 1 && (int64_t)win.size() <= fs, n.description() << ": " << bins << " bins do not belong to frame_size " << fs << " (or the window is longer than a frame)");
            std::vector<double> w((size_t)fs, 0.0);
            const int64_t woff = (fs - (int64_t)win.size()) / 2;
            for (size_t i = 0; i < win.size(); ++i) w[(size_t)woff + i] = win[i];
            const int64_t full = (frames - 1) * step + fs, trim = center ? fs / 2 : 0;
            const int64_t dflt = center ? (frames - 1) * step : full;
            const int64_t len = in.size() > 4 ? to_i64(in[4]).at(0) : dflt;
            const double norm = n.attr_bool("normalized") ? std::sqrt((double)fs) : 1.0;
            std::vector<double> cs((size_t)fs), sn((size_t)fs);
            for (int64_t i = 0; i < fs; ++i) { cs[(size_t)i] = std::cos(2.0 * M_PI * i / fs); sn[(size_t)i] = std::sin(2.0 * M_PI * i / fs); }
            std::vector<float> o((size_t)(B * len), 0.f);
            for (int64_t b = 0; b < B; ++b) {
                std::vector<double> sig((size_t)full, 0.0), env((size_t)full, 0.0);
                for (int64_t f = 0; f < frames; ++f)
                    for (int64_t t = 0; t < fs; ++t) {
                        // inverse of a real FFT: bins above fs/2 are the conjugates of the stored ones
                        double acc = 0;
                        for (int64_t k = 0; k < fs; ++k) {
                            const int64_t kk = k < bins ? k : fs - k;
                            const size_t at = (size_t)((((b * bins + kk) * frames) + f) * 2);
                            const double re = d[at], im = k < bins ? d[at + 1] : -d[at + 1];
                            const int64_t ph = (k * t) % fs;
                            acc += re * cs[(size_t)ph] - im * sn[(size_t)ph];
                        }
                        sig[(size_t)(f * step + t)] += acc / fs * norm * w[(size_t)t];
                        env[(size_t)(f * step + t)] += w[(size_t)t] * w[(size_t)t];
                    }
                for (int64_t i = 0; i < len; ++i) {
                    const int64_t src = i + trim;
                    if (src >= full) break;
                    o[(size_t)(b * len + i)] = env[(size_t)src] > 1e-11 ? (float)(sig[(size_t)src] / env[(size_t)src]) : (float)sig[(size_t)src];
                }
            }
            out[0] = from_f32(D.et, batched ? Shape{B, len} : Shape{len}, o);
            return true;
        }, 4, 5);

    // ---- colour conversion to NV12
    for (const bool bgr : {false, true})
        reg(bgr ? "BGRtoNV12" : "RGBtoNV12", "opset17", {Ab("single_plane", true)}, infer_to_nv12,
            [bgr](N n, Ins in, Outs out, C) { return eval_to_nv12(n, in, out, bgr); }, 1, 1);
}

}  // namespace ovc
