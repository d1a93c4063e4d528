// Object-detection operations of the operation set: prior boxes, SSD detection output, region proposals (Faster R-CNN,
// Detectron, the batched opset9 form), Detectron helpers (prior grid, top-k ROIs, ROI feature extractor, detection
// output), matrix / multiclass / rotated non-maximum suppression and rotated ROI align: attribute schemas (reference
// visit_attributes order), shape / type inference, reference evaluation.
//
// Reference counterparts: src/core/src/op/{prior_box,detection_output,proposal,generate_proposals,matrix_nms,
// multiclass_nms,nms_rotated,roi_align_rotated,experimental_detectron_*}.cpp and the kernels of the same names under
// src/core/reference/include/openvino/reference/.
#include <algorithm>
#include <array>
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
AttrSpec Ais(const char* n, std::vector<int64_t> d = {}) { return A(n, K::INTS, Attr::Ints(std::move(d))); }
AttrSpec Ab(const char* n, bool d = false) { return A(n, K::BOOL, Attr::Bool(d)); }
AttrSpec Af(const char* n, double d = 0) { AttrSpec s = A(n, K::FLOAT, Attr::Float(d)); s.f32 = true; return s; }
AttrSpec As(const char* n, const char* d = "") { return A(n, K::STR, Attr::Str(d)); }
AttrSpec Afs(const char* n, std::vector<double> d = {}) { return A(n, K::FLOATS, Attr::Floats(std::move(d))); }
AttrSpec At(const char* n, ET d) { return A(n, K::TYPE, Attr::Type(d)); }

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

std::vector<float> floats_of(const Node& n, const char* k) {
    const auto& d = n.attr(k).fs;
    return std::vector<float>(d.begin(), d.end());
}

Dim dim_of(const PShape& s, size_t i) { return (!s.rank_dynamic && i < s.dims.size()) ? s.dims[i] : Dim::dynamic(); }

// ------------------------------------------------------------------------------------------------ boxes
struct Box { float x0, y0, x1, y1; };

// `off` is 1 for pixel-inclusive boxes (integer image coordinates), 0 for normalised ones
float box_area(const Box& b, float off) {
    const float w = b.x1 - b.x0 + off, h = b.y1 - b.y0 + off;
    return (w <= 0 || h <= 0) ? 0.f : w * h;
}
float box_iou(const Box& a, const Box& b, float off) {
    const float ix = std::min(a.x1, b.x1) - std::max(a.x0, b.x0) + off, iy = std::min(a.y1, b.y1) - std::max(a.y0, b.y0) + off;
    if (ix <= 0 || iy <= 0) return 0.f;
    const float inter = ix * iy, uni = box_area(a, off) + box_area(b, off) - inter;
    return uni <= 0 ? 0.f : inter / uni;
}

// Greedy suppression over candidates already sorted by falling score: returns the kept positions. With eta < 1 the
// threshold shrinks after every kept box while it is above 0.5 (adaptive NMS).
std::vector<size_t> greedy_nms(const std::vector<Box>& boxes, float thr, float off, int64_t limit, float eta = 1.f) {
    std::vector<size_t> keep;
    for (size_t i = 0; i < boxes.size(); ++i) {
        if (limit >= 0 && (int64_t)keep.size() >= limit) break;
        bool ok = true;
        for (size_t k : keep)
            if (box_iou(boxes[i], boxes[k], off) > thr) { ok = false; break; }
        if (ok) {
            keep.push_back(i);
            if (eta < 1.f && thr > 0.5f) thr *= eta;
        }
    }
    return keep;
}

// positions 0..n-1 ordered by falling score; equal scores keep the lower position first
std::vector<size_t> order_by_score(const float* s, size_t n) {
    std::vector<size_t> o(n);
    std::iota(o.begin(), o.end(), 0);
    std::stable_sort(o.begin(), o.end(), [&](size_t a, size_t b) { return s[a] > s[b]; });
    return o;
}

// ------------------------------------------------------------------------------------------------ PriorBox
std::vector<float> distinct_ratios(const Node& n) {
    // 1 first, then every new ratio (and its reciprocal with flip) in the order given
    std::vector<float> r = {1.f};
    const bool flip = n.attr_bool("flip");
    for (float a : floats_of(n, "aspect_ratio")) {
        if (std::any_of(r.begin(), r.end(), [&](float e) { return std::fabs(a - e) < 1e-6f; })) continue;
        r.push_back(a);
        if (flip) r.push_back(1.f / a);
    }
    return r;
}

int64_t priors_per_cell(const Node& n) {
    // the count follows the set of ratios rounded to 1e-6 (1 always included)
    std::vector<float> uniq = {1.f};
    auto add = [&](float v) {
        v = std::round(v * 1e6f) / 1e6f;
        if (std::find(uniq.begin(), uniq.end(), v) == uniq.end()) uniq.push_back(v);
    };
    for (float a : floats_of(n, "aspect_ratio")) {
        add(a);
        if (n.attr_bool("flip")) add(1.f / a);
    }
    const int64_t ratios = (int64_t)uniq.size();
    const int64_t mins = (int64_t)n.attr("min_size").fs.size(), maxs = (int64_t)n.attr("max_size").fs.size();
    int64_t count = n.attr_bool("scale_all_sizes", true) ? ratios * mins + maxs : ratios + mins - 1;
    if (!n.attr("fixed_size").fs.empty()) count = ratios * (int64_t)n.attr("fixed_size").fs.size();
    const int64_t fixed_ratios = (int64_t)n.attr("fixed_ratio").fs.size();
    for (double d : n.attr("density").fs) {
        const int64_t extra = (int64_t)d * (int64_t)d - 1;
        count += (fixed_ratios ? fixed_ratios : ratios) * extra;
    }
    return count;
}

void infer_prior_box(Node& n) {
    PShape o = PShape::dynamic(2);
    o.dims[0] = Dim(2);
    std::vector<int64_t> layer;
    if (get_constant_ints(n.input(0), layer) && layer.size() == 2) o.dims[1] = Dim(4 * layer[0] * layer[1] * priors_per_cell(n));
    n.set_output(0, ET::f32, o);
}

bool eval_prior_box(N n, Ins in, Outs out, C) {
    const auto layer = to_i64(in[0]), img = to_i64(in[1]);
    OVC_CHECK(layer.size() == 2 && img.size() == 2, n.description() << ": sizes are [height, width]");
    const int64_t LH = layer[0], LW = layer[1];
    const float IH = (float)img[0], IW = (float)img[1];
    const auto ratios = distinct_ratios(n);
    auto mins = floats_of(n, "min_size");
    const auto maxs = floats_of(n, "max_size"), fixed = floats_of(n, "fixed_size"), fixed_ratio = floats_of(n, "fixed_ratio"), density = floats_of(n, "density");
    std::vector<float> var = floats_of(n, "variance");
    OVC_CHECK(var.empty() || var.size() == 1 || var.size() == 4, n.description() << ": 0, 1 or 4 variances expected");
    if (var.empty()) var.push_back(0.1f);
    const bool scale_all = n.attr_bool("scale_all_sizes", true), minmax_first = n.attr_bool("min_max_aspect_ratios_order", true);
    const float offset = (float)n.attr_float("offset");
    float step = (float)n.attr_float("step");
    if (!scale_all) {                       // sizes and step are fractions of the image height in this mode
        step = step == -1.f ? IH / LH : step * IH;
        for (auto& m : mins) m *= IH;
    }
    const float sx = step == 0 ? IW / LW : step, sy = step == 0 ? IH / LH : step;
    const int64_t P = priors_per_cell(n), row = 4 * LH * LW * P;
    std::vector<float> o((size_t)(2 * row), 0.f);
    size_t at = 0;
    auto emit = [&](float cx, float cy, float hw, float hh, bool clamp) {
        OVC_CHECK(at + 4 <= (size_t)row, n.description() << ": the attributes describe more boxes per cell than their count (" << P << ")");
        float b[4] = {(cx - hw) / IW, (cy - hh) / IH, (cx + hw) / IW, (cy + hh) / IH};
        if (clamp) { b[0] = std::max(b[0], 0.f); b[1] = std::max(b[1], 0.f); b[2] = std::min(b[2], 1.f); b[3] = std::min(b[3], 1.f); }
        for (float v : b) o[at++] = v;
    };
    // a density x density grid of centres inside the cell of a fixed-size box
    auto dense = [&](float cx, float cy, size_t s, float hw, float hh) {
        const int64_t d = (int64_t)density.at(s), fs = (int64_t)fixed[s];
        const int64_t shift = (int64_t)(fixed[s] / d);
        for (int64_t r = 0; r < d; ++r)
            for (int64_t c = 0; c < d; ++c)
                emit(cx - fs / 2 + shift / 2.f + c * shift, cy - fs / 2 + shift / 2.f + r * shift, hw, hh, true);
    };
    for (int64_t h = 0; h < LH; ++h)
        for (int64_t w = 0; w < LW; ++w) {
            const float cx = step == 0 ? (w + 0.5f) * sx : (offset + w) * step, cy = step == 0 ? (h + 0.5f) * sy : (offset + h) * step;
            for (size_t s = 0; s < fixed.size(); ++s) {
                const float half = (float)(size_t)fixed[s] * 0.5f;
                if (!fixed_ratio.empty()) {
                    for (float ar : fixed_ratio) dense(cx, cy, s, fixed[s] * 0.5f * std::sqrt(ar), fixed[s] * 0.5f / std::sqrt(ar));
                    continue;
                }
                if (!density.empty()) dense(cx, cy, s, half, half);
                for (float ar : ratios)
                    if (std::fabs(ar - 1.f) >= 1e-6f) dense(cx, cy, s, fixed[s] * 0.5f * std::sqrt(ar), fixed[s] * 0.5f / std::sqrt(ar));
            }
            for (size_t m = 0; m < mins.size(); ++m) {
                emit(cx, cy, mins[m] * 0.5f, mins[m] * 0.5f, false);
                auto with_max = [&] {
                    if (m < maxs.size()) { const float e = std::sqrt(mins[m] * maxs[m]) * 0.5f; emit(cx, cy, e, e, false); }
                };
                auto with_ratios = [&] {
                    if (!scale_all && m + 1 != mins.size()) return;
                    const float base = mins[scale_all ? m : 0];
                    for (float ar : ratios)
                        if (std::fabs(ar - 1.f) >= 1e-6f) emit(cx, cy, base * 0.5f * std::sqrt(ar), base * 0.5f / std::sqrt(ar), false);
                };
                if (minmax_first) { with_max(); with_ratios(); } else { with_ratios(); with_max(); }
            }
        }
    if (n.attr_bool("clip"))
        for (int64_t i = 0; i < row; ++i) o[(size_t)i] = std::min(std::max(o[(size_t)i], 0.f), 1.f);
    for (int64_t i = 0; i < row; ++i) o[(size_t)(row + i)] = var[var.size() == 1 ? 0 : (size_t)(i % 4)];
    out[0] = from_f32(ET::f32, {2, row}, o);
    return true;
}

// ------------------------------------------------------------------------------------------------ DetectionOutput
void infer_detection_output(Node& n) {
    PShape o = PShape::dynamic(4);
    o.dims[0] = o.dims[1] = Dim(1);
    o.dims[3] = Dim(7);
    const PShape &loc = n.in_shape(0), &conf = n.in_shape(1), &pri = n.in_shape(2);
    const Dim batch = dim_of(loc, 0).is_static() ? dim_of(loc, 0) : dim_of(conf, 0);
    const auto keep = n.attr_ints("keep_top_k");
    const int64_t top_k = n.attr_int("top_k", -1);
    const int64_t prior_size = n.attr_bool("normalized") ? 4 : 5;
    Dim priors = Dim::dynamic();
    if (dim_of(pri, 2).is_static()) priors = Dim(dim_of(pri, 2).lo / prior_size);
    int64_t classes = n.has_attr("num_classes") ? n.attr_int("num_classes") : -1;     // opset8 derives it from the inputs
    if (classes <= 0 && priors.is_static() && dim_of(conf, 1).is_static() && priors.lo > 0) classes = dim_of(conf, 1).lo / priors.lo;
    if (batch.is_static()) {
        if (!keep.empty() && keep[0] > 0) o.dims[2] = Dim(batch.lo * keep[0]);
        else if (top_k > 0 && classes > 0) o.dims[2] = Dim(batch.lo * top_k * classes);
        else if (classes > 0 && priors.is_static()) o.dims[2] = Dim(batch.lo * classes * priors.lo);
    }
    n.set_output(0, n.in_et(0) == ET::dynamic ? ET::f32 : n.in_et(0), o);
}

bool eval_detection_output(N n, Ins in, Outs out, C) {
    const bool normalized = n.attr_bool("normalized"), share = n.attr_bool("share_location", true);
    const bool var_in_target = n.attr_bool("variance_encoded_in_target"), mx_style = n.attr_bool("decrease_label_id");
    const bool clip_before = n.attr_bool("clip_before_nms"), clip_after = n.attr_bool("clip_after_nms");
    const int64_t prior_size = normalized ? 4 : 5, skip = normalized ? 0 : 1;
    const auto loc = to_f32(in[0]), conf = to_f32(in[1]), pri = to_f32(in[2]);
    const int64_t B = in[0].shape[0];
    const int64_t P = in[2].shape[2] / prior_size;
    int64_t Cn = n.has_attr("num_classes") ? n.attr_int("num_classes") : 0;
    if (Cn <= 0) Cn = in[1].shape[1] / P;
    const int64_t loc_classes = share ? 1 : Cn;
    OVC_CHECK(in[0].shape[1] == P * loc_classes * 4 && in[1].shape[1] == P * Cn, n.description() << ": location / confidence widths do not match " << P << " priors");
    const int64_t bg = n.attr_int("background_label_id");
    const int64_t top_k = n.attr_int("top_k", -1);
    const auto keep_attr = n.attr_ints("keep_top_k");
    const int64_t keep_top_k = keep_attr.empty() ? -1 : keep_attr[0];
    const float nms_thr = (float)n.attr_float("nms_threshold"), conf_thr = (float)n.attr_float("confidence_threshold", -std::numeric_limits<float>::max());
    const float obj_thr = (float)n.attr_float("objectness_score");
    const std::string code = n.attr_str("code_type", "caffe.PriorBoxParameter.CORNER");
    const bool center = code.find("CENTER_SIZE") != std::string::npos;
    const float in_h = normalized ? 1.f : (float)n.attr_int("input_height", 1), in_w = normalized ? 1.f : (float)n.attr_int("input_width", 1);
    const bool with_arm = in.size() == 5;
    std::vector<float> arm_conf, arm_loc;
    if (with_arm) { arm_conf = to_f32(in[3]); arm_loc = to_f32(in[4]); }
    const int64_t pri_batch = in[2].shape[0], pri_rows = in[2].shape[1];

    auto decode = [&](const float* pb, const float* pv, const float* d) {
        float v[4] = {1, 1, 1, 1};
        if (!var_in_target) for (int k = 0; k < 4; ++k) v[k] = pv[k];
        Box p{pb[0] / in_w, pb[1] / in_h, pb[2] / in_w, pb[3] / in_h}, r;
        if (!center) {
            r = {p.x0 + v[0] * d[0], p.y0 + v[1] * d[1], p.x1 + v[2] * d[2], p.y1 + v[3] * d[3]};
        } else {
            const float pw = p.x1 - p.x0, ph = p.y1 - p.y0, pcx = (p.x0 + p.x1) / 2, pcy = (p.y0 + p.y1) / 2;
            const float cx = v[0] * d[0] * pw + pcx, cy = v[1] * d[1] * ph + pcy;
            const float w = std::exp(v[2] * d[2]) * pw, h = std::exp(v[3] * d[3]) * ph;
            r = {cx - w / 2, cy - h / 2, cx + w / 2, cy + h / 2};
        }
        return r;
    };
    auto clamp01 = [](Box& b) {
        b.x0 = std::min(std::max(b.x0, 0.f), 1.f); b.y0 = std::min(std::max(b.y0, 0.f), 1.f);
        b.x1 = std::min(std::max(b.x1, 0.f), 1.f); b.y1 = std::min(std::max(b.y1, 0.f), 1.f);
    };

    int64_t rows_out;
    if (keep_top_k > 0) rows_out = B * keep_top_k;
    else if (top_k > 0) rows_out = B * top_k * Cn;
    else rows_out = B * Cn * P;
    std::vector<float> o((size_t)(rows_out * 7), 0.f);
    int64_t written = 0;
    struct Det { int64_t label; float score; Box box; int64_t prior; };
    for (int64_t b = 0; b < B; ++b) {
        const float* pbase = pri.data() + (pri_batch > 1 ? b : 0) * pri_rows * P * prior_size;
        const float* pvar = pri_rows > 1 ? pbase + P * prior_size : nullptr;
        const float unit_var[4] = {1, 1, 1, 1};
        // boxes per location class
        std::vector<std::vector<Box>> boxes((size_t)loc_classes, std::vector<Box>((size_t)P));
        for (int64_t p = 0; p < P; ++p)
            for (int64_t c = 0; c < loc_classes; ++c) {
                const float* pb = pbase + p * prior_size + skip;
                const float* pv = (pvar && !var_in_target) ? pvar + p * 4 : unit_var;   // variances are stored four per prior
                Box prior_box{pb[0], pb[1], pb[2], pb[3]};
                if (with_arm) {         // the refinement head moves the prior first
                    const float* ad = arm_loc.data() + (b * P + p) * 4;
                    const Box r = decode(pb, pv, ad);
                    prior_box = {r.x0 * in_w, r.y0 * in_h, r.x1 * in_w, r.y1 * in_h};
                }
                const float pbv[4] = {prior_box.x0, prior_box.y0, prior_box.x1, prior_box.y1};
                Box r = decode(pbv, pv, loc.data() + ((b * P + p) * loc_classes + c) * 4);
                if (clip_before) clamp01(r);
                boxes[(size_t)c][(size_t)p] = r;
            }
        auto score_of = [&](int64_t p, int64_t c) {
            if (with_arm && arm_conf[(size_t)((b * P + p) * 2 + 1)] < obj_thr) return c == bg ? 1.f : 0.f;
            return conf[(size_t)((b * P + p) * Cn + c)];
        };
        std::vector<Det> dets;
        if (!mx_style) {
            for (int64_t c = 0; c < Cn; ++c) {
                if (c == bg) continue;
                std::vector<std::pair<float, int64_t>> cand;
                for (int64_t p = 0; p < P; ++p) {
                    const float s = score_of(p, c);
                    if (s > conf_thr) cand.emplace_back(s, p);
                }
                std::stable_sort(cand.begin(), cand.end(), [](const auto& x, const auto& y) { return x.first > y.first; });
                if (top_k > -1 && (int64_t)cand.size() > top_k) cand.resize((size_t)top_k);
                const auto& bx = boxes[(size_t)(share ? 0 : c)];
                std::vector<Box> sorted;
                for (auto& e : cand) sorted.push_back(bx[(size_t)e.second]);
                for (size_t k : greedy_nms(sorted, nms_thr, 0.f, -1)) dets.push_back({c, cand[k].first, sorted[k], cand[k].second});
            }
        } else {
            // every prior votes for its best foreground class; one suppression pass over all priors, boxes of different
            // classes do not suppress one another
            std::vector<Det> cand;
            for (int64_t p = 0; p < P; ++p) {
                int64_t best = -1;
                float bs = -1;
                for (int64_t c = 1; c < Cn; ++c) {
                    const float s = score_of(p, c);
                    if (s > bs) { bs = s; best = c; }
                }
                if (best > 0 && bs > conf_thr) cand.push_back({best - 1, bs, boxes[0][(size_t)p], p});
            }
            std::stable_sort(cand.begin(), cand.end(), [](const Det& x, const Det& y) { return x.score > y.score || (x.score == y.score && x.prior < y.prior); });
            if (top_k > -1 && (int64_t)cand.size() > top_k) cand.resize((size_t)top_k);
            for (const Det& d : cand) {
                bool ok = true;
                for (const Det& k : dets)
                    if (k.label == d.label && box_iou(d.box, k.box, 0.f) > nms_thr) { ok = false; break; }
                if (ok) dets.push_back(d);
            }
        }
        if (keep_top_k > -1 && (int64_t)dets.size() > keep_top_k) {
            std::stable_sort(dets.begin(), dets.end(), [](const Det& x, const Det& y) { return x.score > y.score; });
            dets.resize((size_t)keep_top_k);
            std::stable_sort(dets.begin(), dets.end(), [](const Det& x, const Det& y) { return x.label < y.label; });   // rows stay grouped by class
        }
        for (Det& d : dets) {
            if (written >= rows_out) break;
            if (clip_after) clamp01(d.box);
            float* r = o.data() + written * 7;
            r[0] = (float)b; r[1] = (float)d.label; r[2] = d.score;
            r[3] = d.box.x0; r[4] = d.box.y0; r[5] = d.box.x1; r[6] = d.box.y1;
            ++written;
        }
    }
    if (written < rows_out) o[(size_t)(written * 7)] = -1.f;       // end-of-list marker
    out[0] = from_f32(in[0].et, {1, 1, rows_out, 7}, o);
    return true;
}

// ------------------------------------------------------------------------------------------------ proposals
// Anchors around a base_size square for every (ratio, scale): the py-faster-rcnn enumeration. `rounded` follows the
// Caffe convention (pixel-inclusive corners, rounded ratio widths); otherwise continuous coordinates.
std::vector<Box> make_anchors(float base, const std::vector<float>& ratios, const std::vector<float>& scales, bool rounded, bool shift_to_centre) {
    const float off = rounded ? 1.f : 0.f;
    const float ctr = 0.5f * (base - off), area = base * base;
    std::vector<Box> a;
    for (float r : ratios) {
        float w = std::sqrt(area / r), h;
        if (rounded) { w = std::round(w); h = std::round(w * r); } else { h = w * r; }
        for (float s : scales) {
            const float ws = 0.5f * (w * s - off), hs = 0.5f * (h * s - off);
            Box b{ctr - ws, ctr - hs, ctr + ws, ctr + hs};
            if (shift_to_centre) { b.x0 -= base * 0.5f; b.y0 -= base * 0.5f; b.x1 -= base * 0.5f; b.y1 -= base * 0.5f; }
            a.push_back(b);
        }
    }
    return a;
}

// anchor + regression deltas -> box; widths count `off` extra pixels
Box apply_deltas(const Box& a, float dx, float dy, float dw, float dh, float off, float max_log = std::numeric_limits<float>::max()) {
    const float w = a.x1 - a.x0 + off, h = a.y1 - a.y0 + off;
    const float cx = a.x0 + 0.5f * w, cy = a.y0 + 0.5f * h;
    const float pcx = dx * w + cx, pcy = dy * h + cy;
    const float pw = std::exp(std::min(dw, max_log)) * w, ph = std::exp(std::min(dh, max_log)) * h;
    return {pcx - 0.5f * pw, pcy - 0.5f * ph, pcx + 0.5f * pw - off, pcy + 0.5f * ph - off};
}

void infer_proposal(Node& n) {
    const Dim batch = dim_of(n.in_shape(0), 0);
    const int64_t post = n.attr_int("post_nms_topn");
    PShape rois = PShape::dynamic(2);
    rois.dims[1] = Dim(5);
    PShape probs = PShape::dynamic(1);
    if (batch.is_static()) rois.dims[0] = probs.dims[0] = Dim(batch.lo * post);
    n.set_output(0, n.in_et(0), rois);
    if (n.version != "opset1") {
        n.set_num_outputs(2);
        n.set_output(1, n.in_et(0), probs);
    }
}

bool eval_proposal(N n, Ins in, Outs out, C) {
    const auto probs = to_f32(in[0]), deltas = to_f32(in[1]), info = to_f32(in[2]);
    const int64_t B = in[0].shape[0], A2 = in[0].shape[1], H = in[0].shape[2], W = in[0].shape[3], An = A2 / 2;
    OVC_CHECK(info.size() == 3 || info.size() == 4, n.description() << ": image_shape has 3 or 4 values");
    const float img_h = info[0], img_w = info[1], scale_h = info.size() == 4 ? info[2] : info[2], scale_w = info.size() == 4 ? info[3] : info[2];
    const bool tf = n.attr_str("framework") == "tensorflow";
    const float off = tf ? 0.f : 1.f;
    const auto anchors = make_anchors((float)n.attr_int("base_size"), floats_of(n, "ratio"), floats_of(n, "scale"), !tf, tf);
    OVC_CHECK((int64_t)anchors.size() == An, n.description() << ": " << anchors.size() << " anchors from ratio x scale, " << An << " in the class scores");
    const float stride = (float)n.attr_int("feat_stride"), min_size = (float)n.attr_int("min_size");
    const float bcs = (float)n.attr_float("box_coordinate_scale", 1), bss = (float)n.attr_float("box_size_scale", 1);
    const bool clip_before = n.attr_bool("clip_before_nms", true), clip_after = n.attr_bool("clip_after_nms"), normalize = n.attr_bool("normalize");
    const int64_t pre = n.attr_int("pre_nms_topn"), post = n.attr_int("post_nms_topn");
    const float thr = (float)n.attr_float("nms_thresh");
    std::vector<float> rois((size_t)(B * post * 5), 0.f), scores((size_t)(B * post), 0.f);
    for (int64_t b = 0; b < B; ++b) {
        std::vector<Box> boxes;
        std::vector<float> sc;
        for (int64_t h = 0; h < H; ++h)
            for (int64_t w = 0; w < W; ++w)
                for (int64_t a = 0; a < An; ++a) {
                    auto d = [&](int64_t k) { return deltas[(size_t)(((b * An * 4 + a * 4 + k) * H + h) * W + w)]; };
                    Box anc = anchors[(size_t)a];
                    anc.x0 += w * stride; anc.x1 += w * stride; anc.y0 += h * stride; anc.y1 += h * stride;
                    Box r = apply_deltas(anc, d(0) / bcs, d(1) / bcs, d(2) / bss, d(3) / bss, off);
                    if (clip_before) {
                        r.x0 = std::min(std::max(r.x0, 0.f), img_w - off); r.x1 = std::min(std::max(r.x1, 0.f), img_w - off);
                        r.y0 = std::min(std::max(r.y0, 0.f), img_h - off); r.y1 = std::min(std::max(r.y1, 0.f), img_h - off);
                    }
                    const float bw = r.x1 - r.x0 + off, bh = r.y1 - r.y0 + off;
                    const float s = probs[(size_t)(((b * A2 + An + a) * H + h) * W + w)];
                    boxes.push_back(r);
                    sc.push_back((bw >= min_size * scale_w && bh >= min_size * scale_h) ? s : 0.f);
                }
        auto order = order_by_score(sc.data(), sc.size());
        if (pre > 0 && (int64_t)order.size() > pre) order.resize((size_t)pre);
        std::vector<Box> sorted;
        for (size_t i : order) sorted.push_back(boxes[i]);
        const auto keep = greedy_nms(sorted, thr, off, post);
        for (size_t k = 0; k < keep.size(); ++k) {
            Box r = sorted[keep[k]];
            if (clip_after) {
                r.x0 = std::min(std::max(r.x0, 0.f), img_w - off); r.x1 = std::min(std::max(r.x1, 0.f), img_w - off);
                r.y0 = std::min(std::max(r.y0, 0.f), img_h - off); r.y1 = std::min(std::max(r.y1, 0.f), img_h - off);
            }
            if (normalize) { r.x0 /= img_w; r.x1 /= img_w; r.y0 /= img_h; r.y1 /= img_h; }
            float* o = rois.data() + (b * post + (int64_t)k) * 5;
            o[0] = (float)b; o[1] = r.x0; o[2] = r.y0; o[3] = r.x1; o[4] = r.y1;
            scores[(size_t)(b * post + (int64_t)k)] = sc[order[keep[k]]];
        }
    }
    out[0] = from_f32(in[0].et, {B * post, 5}, rois);
    if (out.size() > 1) out[1] = from_f32(in[0].et, {B * post}, scores);
    return true;
}

// One image of the Detectron / opset9 proposal generators: anchors are given, scores [A, H, W], deltas [A*4, H, W].
// Returns (box, score) pairs after the size filter, the pre-NMS cut, suppression and the post-NMS cut.
std::vector<std::pair<Box, float>> proposals_one_image(const float* anchors, const float* deltas, const float* scores, int64_t An, int64_t H, int64_t W,
                                                       float img_h, float img_w, float min_size, float thr, int64_t pre, int64_t post, float off, float eta) {
    const float max_log = std::log(1000.f / 16.f);
    min_size = std::max(min_size, 1.f);
    std::vector<Box> boxes;
    std::vector<float> sc;
    for (int64_t h = 0; h < H; ++h)
        for (int64_t w = 0; w < W; ++w)
            for (int64_t a = 0; a < An; ++a) {
                const float* an = anchors + ((h * W + w) * An + a) * 4;
                auto d = [&](int64_t k) { return deltas[((a * 4 + k) * H + h) * W + w]; };
                Box r = apply_deltas(Box{an[0], an[1], an[2], an[3]}, d(0), d(1), d(2), d(3), off, max_log);
                r.x0 = std::min(std::max(r.x0, 0.f), img_w - off); r.x1 = std::min(std::max(r.x1, 0.f), img_w - off);
                r.y0 = std::min(std::max(r.y0, 0.f), img_h - off); r.y1 = std::min(std::max(r.y1, 0.f), img_h - off);
                if (r.x1 - r.x0 + off >= min_size && r.y1 - r.y0 + off >= min_size) {
                    boxes.push_back(r);
                    sc.push_back(scores[(a * H + h) * W + w]);
                }
            }
    auto order = order_by_score(sc.data(), sc.size());
    if (pre > 0 && (int64_t)order.size() > pre) order.resize((size_t)pre);
    std::vector<Box> sorted;
    for (size_t i : order) sorted.push_back(boxes[i]);
    std::vector<std::pair<Box, float>> res;
    for (size_t k : greedy_nms(sorted, thr, off, post, eta)) res.emplace_back(sorted[k], sc[order[k]]);
    return res;
}

// ------------------------------------------------------------------------------------------------ ROI align helpers
float bilinear_at(const float* plane, int64_t H, int64_t W, float y, float x) {
    if (y < -1.f || y > (float)H || x < -1.f || x > (float)W) return 0.f;
    y = std::max(y, 0.f);
    x = std::max(x, 0.f);
    int64_t y0 = (int64_t)y, x0 = (int64_t)x, y1, x1;
    if (y0 >= H - 1) { y0 = y1 = H - 1; y = (float)y0; } else y1 = y0 + 1;
    if (x0 >= W - 1) { x0 = x1 = W - 1; x = (float)x0; } else x1 = x0 + 1;
    const float ly = y - y0, lx = x - x0, hy = 1.f - ly, hx = 1.f - lx;
    return hy * hx * plane[y0 * W + x0] + hy * lx * plane[y0 * W + x1] + ly * hx * plane[y1 * W + x0] + ly * lx * plane[y1 * W + x1];
}

// average ROI align of one box on one feature map [C, H, W] -> [C, P, P]
void roi_align_avg(const float* feat, int64_t Cn, int64_t H, int64_t W, const Box& roi, float scale, int64_t P, int64_t sampling, bool aligned, float* dst) {
    const float shift = aligned ? 0.5f : 0.f;
    const float x0 = roi.x0 * scale - shift, y0 = roi.y0 * scale - shift, x1 = roi.x1 * scale - shift, y1 = roi.y1 * scale - shift;
    float rw = x1 - x0, rh = y1 - y0;
    if (!aligned) { rw = std::max(rw, 1.f); rh = std::max(rh, 1.f); }
    const float bw = rw / P, bh = rh / P;
    const int64_t gy = sampling > 0 ? sampling : (int64_t)std::ceil(rh / P), gx = sampling > 0 ? sampling : (int64_t)std::ceil(rw / P);
    const float count = (float)std::max<int64_t>(gy * gx, 1);
    for (int64_t c = 0; c < Cn; ++c)
        for (int64_t ph = 0; ph < P; ++ph)
            for (int64_t pw = 0; pw < P; ++pw) {
                float sum = 0;
                for (int64_t iy = 0; iy < gy; ++iy)
                    for (int64_t ix = 0; ix < gx; ++ix)
                        sum += bilinear_at(feat + c * H * W, H, W, y0 + ph * bh + (iy + 0.5f) * bh / gy, x0 + pw * bw + (ix + 0.5f) * bw / gx);
                dst[(c * P + ph) * P + pw] = sum / count;
            }
}

// ------------------------------------------------------------------------------------------------ rotated boxes
struct Pt { double x, y; };
struct RBox { double cx, cy, w, h, a; };

std::array<Pt, 4> corners(const RBox& b) {
    const double c = std::cos(b.a) * 0.5, s = std::sin(b.a) * 0.5;
    return {Pt{b.cx - s * b.h - c * b.w, b.cy + c * b.h - s * b.w}, Pt{b.cx + s * b.h - c * b.w, b.cy - c * b.h - s * b.w},
            Pt{b.cx + s * b.h + c * b.w, b.cy - c * b.h + s * b.w}, Pt{b.cx - s * b.h + c * b.w, b.cy + c * b.h + s * b.w}};
}

double polygon_area(const std::vector<Pt>& p) {
    double a = 0;
    for (size_t i = 0; i < p.size(); ++i) {
        const Pt &u = p[i], &v = p[(i + 1) % p.size()];
        a += u.x * v.y - v.x * u.y;
    }
    return std::fabs(a) * 0.5;
}

// convex clip of `subject` by the half planes of `clip` (both convex)
std::vector<Pt> clip_polygon(std::vector<Pt> subject, const std::array<Pt, 4>& clip) {
    // orientation of the clip polygon decides which side is inside
    double orient = 0;
    for (size_t i = 0; i < 4; ++i) orient += clip[i].x * clip[(i + 1) % 4].y - clip[(i + 1) % 4].x * clip[i].y;
    const double sgn = orient >= 0 ? 1.0 : -1.0;
    for (size_t e = 0; e < 4 && !subject.empty(); ++e) {
        const Pt a = clip[e], b = clip[(e + 1) % 4];
        auto side = [&](const Pt& p) { return sgn * ((b.x - a.x) * (p.y - a.y) - (b.y - a.y) * (p.x - a.x)); };
        std::vector<Pt> next;
        for (size_t i = 0; i < subject.size(); ++i) {
            const Pt &p = subject[i], &q = subject[(i + 1) % subject.size()];
            const double sp = side(p), sq = side(q);
            if (sp >= 0) next.push_back(p);
            if ((sp >= 0) != (sq >= 0)) {
                const double t = sp / (sp - sq);
                next.push_back({p.x + t * (q.x - p.x), p.y + t * (q.y - p.y)});
            }
        }
        subject = std::move(next);
    }
    return subject;
}

double rotated_iou(RBox a, RBox b) {
    const double area_a = a.w * a.h, area_b = b.w * b.h;
    if (area_a < 1e-14 || area_b < 1e-14) return 0.0;
    // shift both boxes to their common centre: keeps the products small
    const double mx = (a.cx + b.cx) * 0.5, my = (a.cy + b.cy) * 0.5;
    a.cx -= mx; a.cy -= my; b.cx -= mx; b.cy -= my;
    const auto ca = corners(a);
    const auto inter = clip_polygon(std::vector<Pt>(ca.begin(), ca.end()), corners(b));
    const double ia = inter.size() < 3 ? 0.0 : polygon_area(inter);
    return ia / (area_a + area_b - ia);
}

// ------------------------------------------------------------------------------------------------ matrix / multiclass NMS
struct Sel { int64_t batch, cls, box; float score; };

void order_selection(std::vector<Sel>& s, const std::string& how, bool across_batch) {
    auto by_score = [](const Sel& a, const Sel& b) {
        if (a.score != b.score) return a.score > b.score;
        if (a.cls != b.cls) return a.cls < b.cls;
        return a.box < b.box;
    };
    auto by_class = [](const Sel& a, const Sel& b) {
        if (a.cls != b.cls) return a.cls < b.cls;
        if (a.score != b.score) return a.score > b.score;
        return a.box < b.box;
    };
    if (how == "none") return;
    auto cmp = [&](const Sel& a, const Sel& b) {
        if (!across_batch && a.batch != b.batch) return a.batch < b.batch;
        return how == "classid" ? by_class(a, b) : by_score(a, b);
    };
    std::stable_sort(s.begin(), s.end(), cmp);
}

void infer_class_nms(Node& n) {
    n.set_num_outputs(3);
    const ET it = n.attr("output_type").et;
    PShape sel = PShape::dynamic(2), idx = PShape::dynamic(2), valid = PShape::dynamic(1);
    sel.dims[1] = Dim(6);
    idx.dims[1] = Dim(1);
    const bool shared = n.num_inputs() == 3;                // boxes [C, M, 4], scores [C, M], roisnum [N]
    valid.dims[0] = shared ? dim_of(n.in_shape(2), 0) : dim_of(n.in_shape(0), 0);
    // an upper bound for the rows when everything is static
    const Dim batch = valid.dims[0], classes = shared ? dim_of(n.in_shape(0), 0) : dim_of(n.in_shape(1), 1), boxes = dim_of(n.in_shape(0), 1);
    if (batch.is_static() && classes.is_static() && boxes.is_static()) {
        int64_t per_class = boxes.lo;
        const int64_t nms_top = n.attr_int("nms_top_k", -1), keep = n.attr_int("keep_top_k", -1);
        if (nms_top >= 0) per_class = std::min(per_class, nms_top);
        int64_t per_batch = per_class * classes.lo;
        if (keep >= 0) per_batch = std::min(per_batch, keep);
        sel.dims[0] = idx.dims[0] = Dim(0, per_batch * batch.lo);
    }
    n.set_output(0, n.in_et(0), sel);
    n.set_output(1, it, idx);
    n.set_output(2, it, valid);
}

void write_class_nms(N n, const Tensor& boxes_t, const std::vector<float>& boxes, int64_t M, int64_t B, std::vector<Sel>& all, Outs out, bool shared) {
    order_selection(all, n.attr_str("sort_result_type", "none"), n.attr_bool("sort_result_across_batch"));
    const ET it = n.attr("output_type").et;
    const int64_t K = (int64_t)all.size();
    std::vector<float> sel((size_t)(K * 6));
    std::vector<int64_t> idx((size_t)K), valid((size_t)B, 0);
    for (int64_t i = 0; i < K; ++i) {
        const Sel& s = all[(size_t)i];
        const float* bx = boxes.data() + (shared ? (s.cls * M + s.box) : (s.batch * M + s.box)) * 4;
        float* r = sel.data() + i * 6;
        r[0] = (float)s.cls; r[1] = s.score; r[2] = bx[0]; r[3] = bx[1]; r[4] = bx[2]; r[5] = bx[3];
        idx[(size_t)i] = shared ? s.box : s.batch * M + s.box;
        ++valid[(size_t)s.batch];
    }
    out[0] = from_f32(boxes_t.et, {K, 6}, sel);
    out[1] = from_i64(it, {K, 1}, idx);
    out[2] = from_i64(it, {B}, valid);
}

bool eval_matrix_nms(N n, Ins in, Outs out, C) {
    const auto boxes = to_f32(in[0]), scores = to_f32(in[1]);
    const int64_t B = in[0].shape[0], M = in[0].shape[1], Cn = in[1].shape[1];
    const float off = n.attr_bool("normalized", true) ? 0.f : 1.f;
    const float score_thr = (float)n.attr_float("score_threshold"), post_thr = (float)n.attr_float("post_threshold"), sigma = (float)n.attr_float("gaussian_sigma", 2.0);
    const bool gaussian = n.attr_str("decay_function", "linear") == "gaussian";
    const int64_t nms_top = n.attr_int("nms_top_k", -1), keep_top = n.attr_int("keep_top_k", -1), bg = n.attr_int("background_class", -1);
    std::vector<Sel> all;
    for (int64_t b = 0; b < B; ++b) {
        std::vector<Sel> img;
        for (int64_t c = 0; c < Cn; ++c) {
            if (c == bg) continue;
            const float* sc = scores.data() + (b * Cn + c) * M;
            std::vector<size_t> cand;
            for (size_t i : order_by_score(sc, (size_t)M))
                if (sc[i] > score_thr) cand.push_back(i);
            if (nms_top >= 0 && (int64_t)cand.size() > nms_top) cand.resize((size_t)nms_top);
            const size_t Kc = cand.size();
            auto bx = [&](size_t i) { const float* p = boxes.data() + (b * M + (int64_t)cand[i]) * 4; return Box{p[0], p[1], p[2], p[3]}; };
            // iou[i][j] for j < i; max_iou[j] = largest overlap of j with any better-scored box
            std::vector<float> iou(Kc * Kc, 0.f), max_iou(Kc, 0.f);
            for (size_t i = 1; i < Kc; ++i)
                for (size_t j = 0; j < i; ++j) {
                    iou[i * Kc + j] = box_iou(bx(i), bx(j), off);
                    max_iou[i] = std::max(max_iou[i], iou[i * Kc + j]);
                }
            for (size_t i = 0; i < Kc; ++i) {
                float decay = 1.f;
                for (size_t j = 0; j < i; ++j) {
                    const float v = iou[i * Kc + j], m = max_iou[j];
                    decay = std::min(decay, gaussian ? std::exp((m * m - v * v) * sigma) : (1.f - v) / (1.f - m));
                }
                const float s = sc[cand[i]] * decay;
                if (s >= post_thr) img.push_back({b, c, (int64_t)cand[i], s});
            }
        }
        std::stable_sort(img.begin(), img.end(), [](const Sel& a, const Sel& b2) { return a.score > b2.score; });
        if (keep_top >= 0 && (int64_t)img.size() > keep_top) img.resize((size_t)keep_top);
        all.insert(all.end(), img.begin(), img.end());
    }
    write_class_nms(n, in[0], boxes, M, B, all, out, false);
    return true;
}

bool eval_multiclass_nms(N n, Ins in, Outs out, C) {
    const auto boxes = to_f32(in[0]), scores = to_f32(in[1]);
    const bool shared = in.size() == 3;
    std::vector<int64_t> roisnum;
    if (shared) roisnum = to_i64(in[2]);
    const int64_t B = shared ? (int64_t)roisnum.size() : in[0].shape[0], M = in[0].shape[1], Cn = shared ? in[0].shape[0] : in[1].shape[1];
    const float off = n.attr_bool("normalized", true) ? 0.f : 1.f;
    const float iou_thr = (float)n.attr_float("iou_threshold"), score_thr = (float)n.attr_float("score_threshold"), eta = (float)n.attr_float("nms_eta", 1.0);
    const int64_t nms_top = n.attr_int("nms_top_k", -1), keep_top = n.attr_int("keep_top_k", -1), bg = n.attr_int("background_class", -1);
    std::vector<Sel> all;
    int64_t first = 0;                 // shared form: the boxes of image b are [first, first + roisnum[b]) in every class
    for (int64_t b = 0; b < B; ++b) {
        const int64_t cnt = shared ? roisnum[(size_t)b] : M;
        std::vector<Sel> img;
        for (int64_t c = 0; c < Cn; ++c) {
            if (c == bg) continue;
            const float* sc = shared ? scores.data() + c * M + first : scores.data() + (b * Cn + c) * M;
            std::vector<size_t> cand;
            for (size_t i : order_by_score(sc, (size_t)cnt))
                if (sc[i] > score_thr) cand.push_back(i);
            if (nms_top >= 0 && (int64_t)cand.size() > nms_top) cand.resize((size_t)nms_top);
            std::vector<Box> sorted;
            for (size_t i : cand) {
                const float* p = boxes.data() + (shared ? (c * M + first + (int64_t)i) : (b * M + (int64_t)i)) * 4;
                sorted.push_back({p[0], p[1], p[2], p[3]});
            }
            for (size_t k : greedy_nms(sorted, iou_thr, off, -1, eta)) img.push_back({b, c, (shared ? first : 0) + (int64_t)cand[k], sc[cand[k]]});
        }
        if (keep_top >= 0 && (int64_t)img.size() > keep_top) {
            std::stable_sort(img.begin(), img.end(), [](const Sel& a, const Sel& b2) { return a.score > b2.score; });
            img.resize((size_t)keep_top);
        }
        all.insert(all.end(), img.begin(), img.end());
        first += cnt;
    }
    write_class_nms(n, in[0], boxes, M, B, all, out, shared);
    return true;
}

}  // namespace

void register_detection_ops() {
    // ---- PriorBox
    const std::vector<AttrSpec> pb0 = {Afs("min_size"), Afs("max_size"), Afs("aspect_ratio"), Afs("density"), Afs("fixed_ratio"), Afs("fixed_size"), Ab("clip"), Ab("flip"),
                                       Af("step", 0), Af("offset", 0), Afs("variance"), Ab("scale_all_sizes", true)};
    std::vector<AttrSpec> pb8 = pb0;
    pb8.push_back(Ab("min_max_aspect_ratios_order", true));
    reg("PriorBox", "opset1", pb0, infer_prior_box, eval_prior_box, 2, 2);
    reg("PriorBox", "opset8", pb8, infer_prior_box, eval_prior_box, 2, 2);

    // ---- DetectionOutput (opset8 drops num_classes: it follows from the inputs)
    const std::vector<AttrSpec> do8 = {Ai("background_label_id", 0), Ai("top_k", -1), Ab("variance_encoded_in_target"), Ais("keep_top_k", {1}),
                                       As("code_type", "caffe.PriorBoxParameter.CORNER"), Ab("share_location", true), Af("nms_threshold", 0),
                                       Af("confidence_threshold", 0), Ab("clip_after_nms"), Ab("clip_before_nms"), Ab("decrease_label_id"), Ab("normalized"),
                                       Ai("input_height", 1), Ai("input_width", 1), Af("objectness_score", 0)};
    std::vector<AttrSpec> do1 = {Ai("num_classes", 0)};
    do1.insert(do1.end(), do8.begin(), do8.end());
    reg("DetectionOutput", "opset1", do1, infer_detection_output, eval_detection_output, 3, 5);
    reg("DetectionOutput", "opset8", do8, infer_detection_output, eval_detection_output, 3, 5);

    // ---- Proposal
    const std::vector<AttrSpec> prop = {Ai("base_size", 0), Ai("pre_nms_topn", 0), Ai("post_nms_topn", 0), Af("nms_thresh", 0), Ai("feat_stride", 1), Ai("min_size", 1),
                                        Afs("ratio"), Afs("scale"), Ab("clip_before_nms", true), Ab("clip_after_nms"), Ab("normalize"), Af("box_size_scale", 1),
                                        Af("box_coordinate_scale", 1), As("framework", "")};
    reg("Proposal", "opset1", prop, infer_proposal, eval_proposal, 3, 3);
    reg("Proposal", "opset4", prop, infer_proposal, eval_proposal, 3, 3);

    // ---- ExperimentalDetectronGenerateProposalsSingleImage: im_info [3], anchors [H*W*A, 4], deltas [A*4, H, W], scores [A, H, W]
    reg("ExperimentalDetectronGenerateProposalsSingleImage", "opset6", {Af("min_size", 0), Af("nms_threshold", 0), Ai("post_nms_count", 0), Ai("pre_nms_count", 0)},
        [](Node& n) {
            n.set_num_outputs(2);
            const int64_t post = n.attr_int("post_nms_count");
            n.set_output(0, n.in_et(0), PShape({Dim(post), Dim(4)}));
            n.set_output(1, n.in_et(0), PShape({Dim(post)}));
        },
        [](N n, Ins in, Outs out, C) {
            const auto info = to_f32(in[0]), anchors = to_f32(in[1]), deltas = to_f32(in[2]), scores = to_f32(in[3]);
            const int64_t An = in[3].shape[0], H = in[3].shape[1], W = in[3].shape[2], post = n.attr_int("post_nms_count");
            OVC_CHECK((int64_t)anchors.size() == H * W * An * 4, n.description() << ": one anchor per (cell, score channel) expected");
            const auto got = proposals_one_image(anchors.data(), deltas.data(), scores.data(), An, H, W, info[0], info[1], (float)n.attr_float("min_size"),
                                                 (float)n.attr_float("nms_threshold"), n.attr_int("pre_nms_count"), post, 1.f, 1.f);
            std::vector<float> rois((size_t)(post * 4), 0.f), sc((size_t)post, 0.f);
            for (size_t i = 0; i < got.size(); ++i) {
                const Box& b = got[i].first;
                rois[i * 4] = b.x0; rois[i * 4 + 1] = b.y0; rois[i * 4 + 2] = b.x1; rois[i * 4 + 3] = b.y1;
                sc[i] = got[i].second;
            }
            out[0] = from_f32(in[0].et, {post, 4}, rois);
            out[1] = from_f32(in[0].et, {post}, sc);
            return true;
        }, 4, 4);

    // ---- GenerateProposals: the batched form with a data-dependent number of rows
    reg("GenerateProposals", "opset9", {Af("min_size", 0), Af("nms_threshold", 0), Ai("post_nms_count", 0), Ai("pre_nms_count", 0), Ab("normalized", true), Af("nms_eta", 1),
                                        At("roi_num_type", ET::i64)},
        [](Node& n) {
            n.set_num_outputs(3);
            PShape rois = PShape::dynamic(2), sc = PShape::dynamic(1), num = PShape::dynamic(1);
            rois.dims[1] = Dim(4);
            const Dim batch = dim_of(n.in_shape(0), 0);
            num.dims[0] = batch;
            if (batch.is_static()) rois.dims[0] = sc.dims[0] = Dim(0, batch.lo * n.attr_int("post_nms_count"));
            n.set_output(0, n.in_et(0), rois);
            n.set_output(1, n.in_et(0), sc);
            n.set_output(2, n.attr("roi_num_type").et, num);
        },
        [](N n, Ins in, Outs out, C) {
            const auto info = to_f32(in[0]), anchors = to_f32(in[1]), deltas = to_f32(in[2]), scores = to_f32(in[3]);
            const int64_t B = in[3].shape[0], An = in[3].shape[1], H = in[3].shape[2], W = in[3].shape[3], info_w = in[0].shape[1];
            const float off = n.attr_bool("normalized", true) ? 0.f : 1.f;
            std::vector<float> rois, sc;
            std::vector<int64_t> num;
            for (int64_t b = 0; b < B; ++b) {
                const auto got = proposals_one_image(anchors.data(), deltas.data() + b * An * 4 * H * W, scores.data() + b * An * H * W, An, H, W, info[(size_t)(b * info_w)],
                                                     info[(size_t)(b * info_w + 1)], (float)n.attr_float("min_size"), (float)n.attr_float("nms_threshold"),
                                                     n.attr_int("pre_nms_count"), n.attr_int("post_nms_count"), off, (float)n.attr_float("nms_eta", 1));
                for (const auto& g : got) {
                    rois.insert(rois.end(), {g.first.x0, g.first.y0, g.first.x1, g.first.y1});
                    sc.push_back(g.second);
                }
                num.push_back((int64_t)got.size());
            }
            out[0] = from_f32(in[0].et, {(int64_t)sc.size(), 4}, rois);
            out[1] = from_f32(in[0].et, {(int64_t)sc.size()}, sc);
            out[2] = from_i64(n.attr("roi_num_type").et, {B}, num);
            return true;
        }, 4, 4);

    // ---- ExperimentalDetectronPriorGridGenerator: the priors repeated at the centre of every feature-map cell
    reg("ExperimentalDetectronPriorGridGenerator", "opset6", {Ab("flatten", true), Ai("h", 0), Ai("w", 0), Af("stride_x", 0), Af("stride_y", 0)},
        [](Node& n) {
            const Dim P = dim_of(n.in_shape(0), 0), H = n.attr_int("h") ? Dim(n.attr_int("h")) : dim_of(n.in_shape(1), 2), W = n.attr_int("w") ? Dim(n.attr_int("w")) : dim_of(n.in_shape(1), 3);
            if (n.attr_bool("flatten", true)) {
                PShape o = PShape::dynamic(2);
                o.dims[1] = Dim(4);
                if (P.is_static() && H.is_static() && W.is_static()) o.dims[0] = Dim(P.lo * H.lo * W.lo);
                n.set_output(0, n.in_et(0), o);
            } else {
                n.set_output(0, n.in_et(0), PShape({H, W, P, Dim(4)}));
            }
        },
        [](N n, Ins in, Outs out, C) {
            const auto pri = to_f32(in[0]);
            const int64_t P = in[0].shape[0];
            const int64_t H = n.attr_int("h") ? n.attr_int("h") : in[1].shape[2], W = n.attr_int("w") ? n.attr_int("w") : in[1].shape[3];
            float sx = (float)n.attr_float("stride_x"), sy = (float)n.attr_float("stride_y");
            if (sx == 0) sx = (float)in[2].shape[3] / W;
            if (sy == 0) sy = (float)in[2].shape[2] / H;
            std::vector<float> o((size_t)(H * W * P * 4));
            size_t at = 0;
            for (int64_t h = 0; h < H; ++h)
                for (int64_t w = 0; w < W; ++w)
                    for (int64_t p = 0; p < P; ++p) {
                        o[at++] = pri[(size_t)(p * 4)] + (w + 0.5f) * sx;
                        o[at++] = pri[(size_t)(p * 4 + 1)] + (h + 0.5f) * sy;
                        o[at++] = pri[(size_t)(p * 4 + 2)] + (w + 0.5f) * sx;
                        o[at++] = pri[(size_t)(p * 4 + 3)] + (h + 0.5f) * sy;
                    }
            out[0] = from_f32(in[0].et, n.attr_bool("flatten", true) ? Shape{H * W * P, 4} : Shape{H, W, P, 4}, o);
            return true;
        }, 3, 3);

    // ---- ExperimentalDetectronTopKROIs: the max_rois boxes of highest probability
    reg("ExperimentalDetectronTopKROIs", "opset6", {Ai("max_rois", 0)},
        [](Node& n) { n.set_output(0, n.in_et(0), PShape({Dim(n.attr_int("max_rois")), Dim(4)})); },
        [](N n, Ins in, Outs out, C) {
            const auto rois = to_f32(in[0]), probs = to_f32(in[1]);
            const int64_t R = n.attr_int("max_rois");
            const auto order = order_by_score(probs.data(), probs.size());
            std::vector<float> o((size_t)(R * 4), 0.f);
            for (int64_t i = 0; i < std::min<int64_t>(R, (int64_t)order.size()); ++i)
                for (int k = 0; k < 4; ++k) o[(size_t)(i * 4 + k)] = rois[order[(size_t)i] * 4 + (size_t)k];
            out[0] = from_f32(in[0].et, {R, 4}, o);
            return true;
        }, 2, 2);

    // ---- ExperimentalDetectronROIFeatureExtractor: every ROI is pooled from the pyramid level that suits its size
    reg("ExperimentalDetectronROIFeatureExtractor", "opset6", {Ai("output_size", 7), Ai("sampling_ratio", 2), Ais("pyramid_scales"), Ab("aligned")},
        [](Node& n) {
            n.set_num_outputs(2);
            const int64_t P = n.attr_int("output_size");
            n.set_output(0, n.in_et(0), PShape({dim_of(n.in_shape(0), 0), dim_of(n.in_shape(1), 1), Dim(P), Dim(P)}));
            n.set_output(1, n.in_et(0), PShape({dim_of(n.in_shape(0), 0), Dim(4)}));
        },
        [](N n, Ins in, Outs out, C) {
            const auto rois = to_f32(in[0]);
            const int64_t R = in[0].shape[0], L = (int64_t)in.size() - 1, Cn = in[1].shape[1], P = n.attr_int("output_size");
            const auto scales = n.attr_ints("pyramid_scales");
            OVC_CHECK((int64_t)scales.size() == L, n.description() << ": one pyramid scale per feature map expected");
            std::vector<std::vector<float>> feats;
            for (int64_t l = 0; l < L; ++l) feats.push_back(to_f32(in[(size_t)l + 1]));
            std::vector<float> o((size_t)(R * Cn * P * P), 0.f);
            for (int64_t r = 0; r < R; ++r) {
                const Box b{rois[(size_t)(r * 4)], rois[(size_t)(r * 4 + 1)], rois[(size_t)(r * 4 + 2)], rois[(size_t)(r * 4 + 3)]};
                // a 224-pixel box belongs to level 2 of the pyramid (stride 4 is level 0 of the inputs when the scales start at 4)
                const float area = std::max(b.x1 - b.x0, 0.f) * std::max(b.y1 - b.y0, 0.f);
                int64_t level = (int64_t)std::floor(2.0 + std::log2(std::sqrt((double)area) / 224.0 + 1e-6));
                level = std::min<int64_t>(std::max<int64_t>(level, 2), 2 + L - 1) - 2;
                const Tensor& F = in[(size_t)level + 1];
                roi_align_avg(feats[(size_t)level].data(), Cn, F.shape[2], F.shape[3], b, 1.f / (float)scales[(size_t)level], P, n.attr_int("sampling_ratio"),
                              n.attr_bool("aligned"), o.data() + r * Cn * P * P);
            }
            out[0] = from_f32(in[0].et, {R, Cn, P, P}, o);
            out[1] = from_f32(in[0].et, {R, 4}, rois);
            return true;
        }, 2, -1);

    // ---- ExperimentalDetectronDetectionOutput: per-class box refinement, suppression per class, best detections of the image
    reg("ExperimentalDetectronDetectionOutput", "opset6", {Af("score_threshold", 0), Af("nms_threshold", 0), Af("max_delta_log_wh", 0), Ai("num_classes", 0), Ai("post_nms_count", 0),
                                                           Ai("max_detections_per_image", 0), Ab("class_agnostic_box_regression"), Afs("deltas_weights")},
        [](Node& n) {
            n.set_num_outputs(3);
            const int64_t D = n.attr_int("max_detections_per_image");
            n.set_output(0, n.in_et(0), PShape({Dim(D), Dim(4)}));
            n.set_output(1, ET::i32, PShape({Dim(D)}));
            n.set_output(2, n.in_et(0), PShape({Dim(D)}));
        },
        [](N n, Ins in, Outs out, C) {
            const auto rois = to_f32(in[0]), deltas = to_f32(in[1]), scores = to_f32(in[2]), info = to_f32(in[3]);
            const int64_t R = in[0].shape[0], Cn = n.attr_int("num_classes"), D = n.attr_int("max_detections_per_image");
            const auto wts = floats_of(n, "deltas_weights");
            OVC_CHECK(wts.size() == 4, n.description() << ": four deltas_weights expected");
            const bool agnostic = n.attr_bool("class_agnostic_box_regression");
            const float img_h = info[0], img_w = info[1], max_log = (float)n.attr_float("max_delta_log_wh");
            const float score_thr = (float)n.attr_float("score_threshold"), thr = (float)n.attr_float("nms_threshold");
            struct Det { Box box; int64_t cls; float score; };
            std::vector<Det> dets;
            for (int64_t c = 1; c < Cn; ++c) {
                std::vector<Box> boxes;
                std::vector<float> sc;
                for (int64_t r = 0; r < R; ++r) {
                    const float s = scores[(size_t)(r * Cn + c)];
                    if (s <= score_thr) continue;
                    const float* d = deltas.data() + (r * (in[1].shape[1] / 4) + (agnostic ? 0 : c)) * 4;
                    const float* rb = rois.data() + r * 4;
                    Box b = apply_deltas(Box{rb[0], rb[1], rb[2], rb[3]}, d[0] / wts[0], d[1] / wts[1], d[2] / wts[2], d[3] / wts[3], 1.f, max_log);
                    b.x0 = std::min(std::max(b.x0, 0.f), img_w - 1.f); b.x1 = std::min(std::max(b.x1, 0.f), img_w - 1.f);
                    b.y0 = std::min(std::max(b.y0, 0.f), img_h - 1.f); b.y1 = std::min(std::max(b.y1, 0.f), img_h - 1.f);
                    boxes.push_back(b);
                    sc.push_back(s);
                }
                const auto order = order_by_score(sc.data(), sc.size());
                std::vector<Box> sorted;
                for (size_t i : order) sorted.push_back(boxes[i]);
                for (size_t k : greedy_nms(sorted, thr, 1.f, n.attr_int("post_nms_count"))) dets.push_back({sorted[k], c, sc[order[k]]});
            }
            std::stable_sort(dets.begin(), dets.end(), [](const Det& a, const Det& b) { return a.score > b.score; });
            if ((int64_t)dets.size() > D) dets.resize((size_t)D);
            std::vector<float> ob((size_t)(D * 4), 0.f), os((size_t)D, 0.f);
            std::vector<int64_t> oc((size_t)D, 0);
            for (size_t i = 0; i < dets.size(); ++i) {
                ob[i * 4] = dets[i].box.x0; ob[i * 4 + 1] = dets[i].box.y0; ob[i * 4 + 2] = dets[i].box.x1; ob[i * 4 + 3] = dets[i].box.y1;
                oc[i] = dets[i].cls;
                os[i] = dets[i].score;
            }
            out[0] = from_f32(in[0].et, {D, 4}, ob);
            out[1] = from_i64(ET::i32, {D}, oc);
            out[2] = from_f32(in[0].et, {D}, os);
            return true;
        }, 4, 4);

    // ---- MatrixNms / MulticlassNms
    reg("MatrixNms", "opset8", {As("sort_result_type", "none"), At("output_type", ET::i64), Ai("nms_top_k", -1), Ai("keep_top_k", -1), Ab("sort_result_across_batch"),
                                Af("score_threshold", 0), Ai("background_class", -1), As("decay_function", "linear"), Af("gaussian_sigma", 2), Af("post_threshold", 0),
                                Ab("normalized", true)},
        infer_class_nms, eval_matrix_nms, 2, 2);
    const std::vector<AttrSpec> mc = {As("sort_result_type", "none"), At("output_type", ET::i64), Ai("nms_top_k", -1), Ai("keep_top_k", -1), Ab("sort_result_across_batch"),
                                      Af("iou_threshold", 0), Af("score_threshold", 0), Ai("background_class", -1), Af("nms_eta", 1), Ab("normalized", true)};
    reg("MulticlassNms", "opset8", mc, infer_class_nms, eval_multiclass_nms, 2, 2);
    reg("MulticlassNms", "opset9", mc, infer_class_nms, eval_multiclass_nms, 2, 3);

    // ---- NMSRotated: boxes (cx, cy, w, h, angle in radians); overlap from the intersection polygon
    reg("NMSRotated", "opset13", {Ab("sort_result_descending", true), At("output_type", ET::i64), Ab("clockwise", true)},
        [](Node& n) {
            n.set_num_outputs(3);
            PShape sel = PShape::dynamic(2);
            sel.dims[1] = Dim(3);
            const ET it = n.attr("output_type").et;
            n.set_output(0, it, sel);
            n.set_output(1, n.in_et(0), sel);
            n.set_output(2, it, PShape({Dim(1)}));
        },
        [](N n, Ins in, Outs out, C) {
            const auto boxes = to_f32(in[0]), scores = to_f32(in[1]);
            const int64_t B = in[0].shape[0], M = in[0].shape[1], Cn = in[1].shape[1];
            const int64_t max_out = to_i64(in[2]).at(0);
            const float iou_thr = to_f32(in[3]).at(0), score_thr = in.size() > 4 ? to_f32(in[4]).at(0) : 0.f;
            const double sign = n.attr_bool("clockwise", true) ? 1.0 : -1.0;   // only the relative rotation of two boxes matters; one convention is used for both
            struct Pick { int64_t b, c, i; float s; };
            std::vector<Pick> picks;
            for (int64_t b = 0; b < B; ++b)
                for (int64_t c = 0; c < Cn; ++c) {
                    const float* sc = scores.data() + (b * Cn + c) * M;
                    std::vector<size_t> kept;
                    for (size_t i : order_by_score(sc, (size_t)M)) {
                        if ((int64_t)kept.size() >= max_out) break;
                        if (sc[i] <= score_thr) break;
                        const float* p = boxes.data() + (b * M + (int64_t)i) * 5;
                        const RBox cand{p[0], p[1], p[2], p[3], sign * p[4]};
                        bool ok = true;
                        for (size_t k : kept) {
                            const float* q = boxes.data() + (b * M + (int64_t)k) * 5;
                            if (rotated_iou(cand, RBox{q[0], q[1], q[2], q[3], sign * q[4]}) > iou_thr) { ok = false; break; }
                        }
                        if (ok) { kept.push_back(i); picks.push_back({b, c, (int64_t)i, sc[i]}); }
                    }
                }
            if (n.attr_bool("sort_result_descending", true))
                std::stable_sort(picks.begin(), picks.end(), [](const Pick& a, const Pick& b) { return a.s > b.s; });
            const int64_t Kn = (int64_t)picks.size();
            std::vector<int64_t> idx((size_t)(Kn * 3));
            std::vector<float> ss((size_t)(Kn * 3));
            for (int64_t i = 0; i < Kn; ++i) {
                const Pick& p = picks[(size_t)i];
                idx[(size_t)(i * 3)] = p.b; idx[(size_t)(i * 3 + 1)] = p.c; idx[(size_t)(i * 3 + 2)] = p.i;
                ss[(size_t)(i * 3)] = (float)p.b; ss[(size_t)(i * 3 + 1)] = (float)p.c; ss[(size_t)(i * 3 + 2)] = p.s;
            }
            const ET it = n.attr("output_type").et;
            out[0] = from_i64(it, {Kn, 3}, idx);
            out[1] = from_f32(in[0].et, {Kn, 3}, ss);
            out[2] = from_i64(it, {1}, {Kn});
            return true;
        }, 4, 5);

    // ---- ROIAlignRotated: average pooling on a sampling grid rotated around the box centre
    reg("ROIAlignRotated", "opset15", {Ai("pooled_h", 1), Ai("pooled_w", 1), Ai("sampling_ratio", 0), Af("spatial_scale", 1), Ab("clockwise_mode")},
        [](Node& n) {
            n.set_output(0, n.in_et(0), PShape({dim_of(n.in_shape(1), 0), dim_of(n.in_shape(0), 1), Dim(n.attr_int("pooled_h")), Dim(n.attr_int("pooled_w"))}));
        },
        [](N n, Ins in, Outs out, C) {
            const auto x = to_f32(in[0]), rois = to_f32(in[1]);
            const auto bidx = to_i64(in[2]);
            const int64_t Cn = in[0].shape[1], H = in[0].shape[2], W = in[0].shape[3], R = in[1].shape[0];
            const int64_t PH = n.attr_int("pooled_h"), PW = n.attr_int("pooled_w"), sampling = n.attr_int("sampling_ratio");
            const float scale = (float)n.attr_float("spatial_scale");
            std::vector<float> o((size_t)(R * Cn * PH * PW));
            for (int64_t r = 0; r < R; ++r) {
                const float* b = rois.data() + r * 5;
                const float cx = b[0] * scale - 0.5f, cy = b[1] * scale - 0.5f, rw = b[2] * scale, rh = b[3] * scale;
                const float ang = n.attr_bool("clockwise_mode") ? -b[4] : b[4];
                const float ca = std::cos(ang), sa = std::sin(ang);
                const float bw = rw / PW, bh = rh / PH;
                const int64_t gy = sampling > 0 ? sampling : (int64_t)std::ceil(rh / PH), gx = sampling > 0 ? sampling : (int64_t)std::ceil(rw / PW);
                const float count = (float)std::max<int64_t>(gy * gx, 1);
                OVC_CHECK(bidx[(size_t)r] >= 0 && bidx[(size_t)r] < in[0].shape[0], n.description() << ": batch index " << bidx[(size_t)r] << " out of range");
                for (int64_t c = 0; c < Cn; ++c) {
                    const float* plane = x.data() + (bidx[(size_t)r] * Cn + c) * H * W;
                    for (int64_t ph = 0; ph < PH; ++ph)
                        for (int64_t pw = 0; pw < PW; ++pw) {
                            float sum = 0;
                            for (int64_t iy = 0; iy < gy; ++iy)
                                for (int64_t ix = 0; ix < gx; ++ix) {
                                    const float yy = -rh / 2 + ph * bh + (iy + 0.5f) * bh / gy, xx = -rw / 2 + pw * bw + (ix + 0.5f) * bw / gx;
                                    sum += bilinear_at(plane, H, W, yy * ca - xx * sa + cy, yy * sa + xx * ca + cx);
                                }
                            o[(size_t)(((r * Cn + c) * PH + ph) * PW + pw)] = sum / count;
                        }
                }
            }
            out[0] = from_f32(in[0].et, {R, Cn, PH, PW}, o);
            return true;
        }, 3, 3);
}

}  // namespace ovc
