// Operation table: attribute schemas (in the reference's visit_attributes order, which is the order of
// the <data> attributes in IR xml) and shape / type inference for every supported operation.
//
// Reference counterparts: src/core/src/op/*.cpp (validate_and_infer_types / visit_attributes),
// src/core/shape_inference/include/*_shape_inference.hpp, the internal ops under
// src/core/dev_api/openvino/op/ and src/common/transformations/include/ov_ops/.
#include <numeric>

#include "graph.hpp"

namespace ovc {

// Reference evaluation functions live in eval.cpp
void register_eval_functions();
// More operations, registered together with their reference evaluation (ops_ext.cpp)
void register_ext_ops();
void register_internal_ops();
void register_vision_ops();
void register_detection_ops();
void register_rest_ops();
void register_recurrent_ops();
void register_private_ops();

namespace {

using K = Attr::Kind;

AttrSpec A(const char* name, K kind, Attr def = Attr(), bool required = false, bool f32 = false) {
    AttrSpec s;
    s.name = name;
    s.kind = kind;
    s.def = std::move(def);
    s.required = required;
    s.f32 = f32;
    return s;
}
AttrSpec Ai(const char* n, int64_t d = 0) { return A(n, K::INT, Attr::Int(d)); }
AttrSpec Ab(const char* n, bool d = false) { return A(n, K::BOOL, Attr::Bool(d)); }
AttrSpec Af(const char* n, double d = 0, bool f32 = true) { return A(n, K::FLOAT, Attr::Float(d), false, f32); }
AttrSpec As(const char* n, const char* d = "") { return A(n, K::STR, Attr::Str(d)); }
AttrSpec Ais(const char* n, std::vector<int64_t> d = {}) { return A(n, K::INTS, Attr::Ints(std::move(d))); }
AttrSpec At(const char* n, ET d = ET::dynamic) { return A(n, K::TYPE, Attr::Type(d)); }

void reg(const char* type, const char* version, std::vector<AttrSpec> attrs, InferFn infer, int min_in, int max_in,
         bool commutative = false, bool side_effects = false) {
    OpSchema s;
    s.type = type;
    s.version = version;
    s.attrs = std::move(attrs);
    s.infer = std::move(infer);
    s.min_inputs = min_in;
    s.max_inputs = max_in;
    s.commutative = commutative;
    s.has_side_effects = side_effects;
    OpRegistry::get().add(std::move(s));
}

// ------------------------------------------------------------------------------------ helpers
int64_t norm_axis(int64_t a, int64_t rank, const Node& n) {
    OVC_CHECK(a >= -rank && a < std::max<int64_t>(rank, 1), n.description() << ": axis " << a << " out of range for rank " << rank);
    return a < 0 ? a + rank : a;
}

PShape broadcast_numpy(const PShape& a, const PShape& b, const Node& n) {
    if (a.rank_dynamic || b.rank_dynamic) return PShape::dynamic();
    const size_t r = std::max(a.rank(), b.rank());
    PShape out = PShape::dynamic(r);
    for (size_t i = 0; i < r; ++i) {
        const Dim da = i < r - a.rank() ? Dim(1) : a.dims[i - (r - a.rank())];
        const Dim db = i < r - b.rank() ? Dim(1) : b.dims[i - (r - b.rank())];
        Dim d;
        if (da.is_static() && da.lo == 1) d = db;
        else if (db.is_static() && db.lo == 1) d = da;
        else if (da.is_static() && db.is_static()) {
            OVC_CHECK(da.lo == db.lo, n.description() << ": shapes " << a.str() << " and " << b.str() << " do not broadcast");
            d = da;
        } else if (da.is_static()) {
            d = (db.lo <= 1 && (db.hi < 0 || db.hi >= da.lo)) ? da : da;
        } else if (db.is_static()) {
            d = db;
        } else {
            // both dynamic: the result is at least the larger lower bound; 1 may broadcast
            Dim m;
            if (symbols_equal(da.sym, db.sym)) d = da;       // known to be the same value: nothing broadcasts
            else if (Dim::merge(m, da, db) && da.lo > 1 && db.lo > 1) d = m;
            else d = Dim(std::max<int64_t>(std::min(da.lo, db.lo), 0), (da.hi < 0 || db.hi < 0) ? -1 : std::max(da.hi, db.hi));
        }
        out.dims[i] = d;
    }
    return out;
}

PShape broadcast_by_attr(const Node& n, const PShape& a, const PShape& b) {
    const std::string ab = n.attr_str("auto_broadcast", "numpy");
    if (ab == "none" || ab == "NONE") {
        PShape m;
        OVC_CHECK(PShape::merge(m, a, b), n.description() << ": shapes " << a.str() << " and " << b.str() << " differ");
        return m;
    }
    return broadcast_numpy(a, b, n);
}

ET merge_types(const Node& n, ET a, ET b) {
    if (a == ET::dynamic) return b;
    if (b == ET::dynamic) return a;
    OVC_CHECK(a == b, n.description() << ": argument element types " << et_name(a) << " and " << et_name(b) << " do not match");
    return a;
}

// ---- partial value propagation for shape arithmetic (the role of bound evaluation in the reference,
//      src/core/src/bound_evaluate.cpp): values of small integer tensors as intervals.
bool partial_ints(const Output& o, std::vector<Dim>& out, int depth = 0) {
    if (depth > 32) return false;
    Node& n = *o.node;
    const PShape& os = o.shape();
    if (os.rank_dynamic || os.rank() > 1) {
        if (!(os.rank_is_static() && os.rank() == 0)) return false;
    }
    if (n.is_constant()) {
        if (n.constant.et == ET::string || n.constant.numel() > 4096) return false;
        out.clear();
        for (auto v : to_i64(n.constant)) out.emplace_back(Dim(v, v));
        return true;
    }
    const std::string& t = n.type;
    if (t == "ShapeOf") {
        const PShape& s = n.in_shape(0);
        if (s.rank_dynamic) return false;
        out = s.dims;
        return true;
    }
    if (t == "Convert" || t == "Squeeze" || t == "Unsqueeze" || t == "Reshape") {
        if (t == "Reshape") {
            const PShape& is = n.in_shape(0);
            if (is.rank_dynamic || is.rank() > 1) return false;
        }
        return partial_ints(n.input(0), out, depth + 1);
    }
    if (t == "Gather") {
        std::vector<Dim> data;
        std::vector<int64_t> idx, axis;
        if (!partial_ints(n.input(0), data, depth + 1) || !get_constant_ints(n.input(1), idx) ||
            !get_constant_ints(n.input(2), axis))
            return false;
        out.clear();
        for (auto i : idx) {
            if (i < 0) i += (int64_t)data.size();
            if (i < 0 || i >= (int64_t)data.size()) return false;
            out.push_back(data[(size_t)i]);
        }
        return true;
    }
    if (t == "Concat") {
        out.clear();
        for (auto& in : n.inputs()) {
            std::vector<Dim> p;
            if (!partial_ints(in, p, depth + 1)) return false;
            out.insert(out.end(), p.begin(), p.end());
        }
        return true;
    }
    if (t == "Add" || t == "Multiply" || t == "Subtract" || t == "Divide" || t == "Maximum" || t == "Minimum") {
        std::vector<Dim> a, b;
        if (!partial_ints(n.input(0), a, depth + 1) || !partial_ints(n.input(1), b, depth + 1)) return false;
        if (a.size() != b.size()) {
            if (a.size() == 1) a.assign(b.size(), a[0]);
            else if (b.size() == 1) b.assign(a.size(), b[0]);
            else return false;
        }
        out.resize(a.size());
        for (size_t i = 0; i < a.size(); ++i) {
            const Dim &x = a[i], &y = b[i];
            const bool stat = x.is_static() && y.is_static();
            if (t == "Add") out[i] = Dim(x.lo + y.lo, (x.hi < 0 || y.hi < 0) ? -1 : x.hi + y.hi);
            else if (t == "Multiply") {
                if (x.lo < 0 || y.lo < 0) { if (!stat) return false; out[i] = Dim(x.lo * y.lo, x.lo * y.lo); }
                else out[i] = x * y;
            } else if (t == "Subtract") {
                if (!stat) { if (!y.is_static()) return false; out[i] = Dim(x.lo - y.lo, x.hi < 0 ? -1 : x.hi - y.lo); }
                else out[i] = Dim(x.lo - y.lo, x.lo - y.lo);
            } else if (t == "Divide") {
                if (!y.is_static() || y.lo <= 0) return false;
                out[i] = Dim(x.lo / y.lo, x.hi < 0 ? -1 : x.hi / y.lo);
            } else if (t == "Maximum") {
                out[i] = Dim(std::max(x.lo, y.lo), (x.hi < 0 || y.hi < 0) ? -1 : std::max(x.hi, y.hi));
            } else {
                out[i] = Dim(std::min(x.lo, y.lo), x.hi < 0 ? y.hi : (y.hi < 0 ? x.hi : std::min(x.hi, y.hi)));
            }
        }
        return true;
    }
    if (t == "Slice" || t == "StridedSlice") {
        std::vector<Dim> data;
        std::vector<int64_t> b, e, st;
        if (!partial_ints(n.input(0), data, depth + 1) || !get_constant_ints(n.input(1), b) || !get_constant_ints(n.input(2), e))
            return false;
        if (n.num_inputs() > 3) { if (!get_constant_ints(n.input(3), st)) return false; } else st = {1};
        if (b.size() != 1 || e.size() != 1 || st.size() != 1 || st[0] != 1) return false;
        if (t == "StridedSlice") {
            auto bm = n.attr_ints("begin_mask"), em = n.attr_ints("end_mask");
            if (!bm.empty() && bm[0]) b[0] = 0;
            if (!em.empty() && em[0]) e[0] = (int64_t)data.size();
            for (auto k : {"new_axis_mask", "shrink_axis_mask", "ellipsis_mask"})
                for (auto v : n.attr_ints(k)) if (v) return false;
        }
        const int64_t sz = (int64_t)data.size();
        int64_t bb = b[0] < 0 ? b[0] + sz : b[0], ee = e[0] < 0 ? e[0] + sz : e[0];
        bb = std::max<int64_t>(0, std::min(bb, sz));
        ee = std::max<int64_t>(0, std::min(ee, sz));
        out.assign(data.begin() + bb, data.begin() + std::max(bb, ee));
        return true;
    }
    Tensor c;
    if (try_constant_value(o, c) && c.et != ET::string && c.numel() <= 4096) {
        out.clear();
        for (auto v : to_i64(c)) out.emplace_back(Dim(v, v));
        return true;
    }
    return false;
}

// ---- inference functions ---------------------------------------------------------------------
void infer_same(Node& n) { n.set_output(0, n.in_et(0), n.in_shape(0)); }

void infer_binary_arith(Node& n) {
    n.set_output(0, merge_types(n, n.in_et(0), n.in_et(1)), broadcast_by_attr(n, n.in_shape(0), n.in_shape(1)));
}
void infer_binary_cmp(Node& n) {
    merge_types(n, n.in_et(0), n.in_et(1));
    n.set_output(0, ET::boolean, broadcast_by_attr(n, n.in_shape(0), n.in_shape(1)));
}

void infer_reduce(Node& n) {
    const PShape& in = n.in_shape(0);
    const bool keep = n.attr_bool("keep_dims");
    std::vector<int64_t> axes;
    if (in.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
    if (!get_constant_ints(n.input(1), axes)) {
        n.set_output(0, n.in_et(0), keep ? PShape::dynamic(in.rank()) : PShape::dynamic());
        return;
    }
    std::set<int64_t> ax;
    for (auto a : axes) ax.insert(norm_axis(a, (int64_t)in.rank(), n));
    PShape out;
    for (size_t i = 0; i < in.rank(); ++i) {
        if (ax.count((int64_t)i)) { if (keep) out.dims.emplace_back(1); }
        else out.dims.push_back(in.dims[i]);
    }
    n.set_output(0, n.type.rfind("ReduceLogical", 0) == 0 ? ET::boolean : n.in_et(0), out);
}

// spatial output size of conv / pool windows
Dim window_out(const Dim& in, int64_t k, int64_t stride, int64_t dil, int64_t pb, int64_t pe, bool ceil_mode,
               const std::string& auto_pad) {
    auto f = [&](int64_t v) -> int64_t {
        if (auto_pad == "same_upper" || auto_pad == "same_lower") return (v + stride - 1) / stride;
        const int64_t eff = dil * (k - 1) + 1;
        const int64_t padded = v + (auto_pad == "valid" ? 0 : pb + pe);
        if (padded < eff) return 0;
        const int64_t num = padded - eff;
        int64_t o = (ceil_mode ? (num + stride - 1) / stride : num / stride) + 1;
        if (ceil_mode && (o - 1) * stride >= v + pb) --o;   // the last window must start inside the (left-padded) input
        return o;
    };
    if (in.is_static()) return Dim(f(in.lo));
    return Dim(f(in.lo), in.hi < 0 ? -1 : f(in.hi));
}

void same_pads(const Node& n, const PShape& in, const std::vector<int64_t>& k, const std::vector<int64_t>& st,
               const std::vector<int64_t>& dil, std::vector<int64_t>& pb, std::vector<int64_t>& pe) {
    const std::string ap = n.attr_str("auto_pad", "explicit");
    const size_t sp = k.size();
    if (ap == "same_upper" || ap == "same_lower") {
        pb.assign(sp, 0);
        pe.assign(sp, 0);
        for (size_t i = 0; i < sp; ++i) {
            const Dim& d = in.dims[2 + i];
            if (!d.is_static()) continue;
            const int64_t out = (d.lo + st[i] - 1) / st[i];
            const int64_t total = std::max<int64_t>(0, (out - 1) * st[i] + dil[i] * (k[i] - 1) + 1 - d.lo);
            const int64_t half = total / 2;
            if (ap == "same_upper") { pb[i] = half; pe[i] = total - half; } else { pe[i] = half; pb[i] = total - half; }
        }
    } else if (ap == "valid") {
        pb.assign(sp, 0);
        pe.assign(sp, 0);
    }
}

void infer_conv(Node& n, bool group) {
    const PShape& x = n.in_shape(0);
    const PShape& w = n.in_shape(1);
    const ET et = merge_types(n, n.in_et(0), n.in_et(1));
    if (x.rank_dynamic || w.rank_dynamic) { n.set_output(0, et, PShape::dynamic()); return; }
    const size_t sp = x.rank() - 2;
    OVC_CHECK(w.rank() == x.rank() + (group ? 1 : 0), n.description() << ": filter rank " << w.rank() << " does not fit data rank " << x.rank());
    auto st = n.attr_ints("strides"), dil = n.attr_ints("dilations"), pb = n.attr_ints("pads_begin"), pe = n.attr_ints("pads_end");
    if (st.empty()) st.assign(sp, 1);
    if (dil.empty()) dil.assign(sp, 1);
    if (pb.empty()) pb.assign(sp, 0);
    if (pe.empty()) pe.assign(sp, 0);
    OVC_CHECK(st.size() == sp && dil.size() == sp && pb.size() == sp && pe.size() == sp, n.description() << ": attribute ranks do not match " << sp << " spatial dims");
    const size_t wo = group ? 1 : 0;
    PShape out = PShape::dynamic(x.rank());
    out.dims[0] = x.dims[0];
    if (group) out.dims[1] = w.dims[0] * w.dims[1]; else out.dims[1] = w.dims[0];
    if (x.dims[1].is_static() && w.dims[wo + 1].is_static()) {
        const int64_t cin = group ? (w.dims[0].is_static() ? w.dims[0].lo * w.dims[2].lo : -1) : w.dims[1].lo;
        OVC_CHECK(cin < 0 || cin == x.dims[1].lo, n.description() << ": data channels " << x.dims[1].lo << " do not match filter input channels " << cin);
    }
    const std::string ap = n.attr_str("auto_pad", "explicit");
    for (size_t i = 0; i < sp; ++i) {
        const Dim& kd = w.dims[wo + 2 + i];
        if (!kd.is_static()) { out.dims[2 + i] = Dim::dynamic(); continue; }
        out.dims[2 + i] = window_out(x.dims[2 + i], kd.lo, st[i], dil[i], pb[i], pe[i], false, ap);
    }
    n.set_output(0, et, out);
}

void infer_pool(Node& n, bool maxpool) {
    const PShape& x = n.in_shape(0);
    if (x.rank_dynamic) {
        n.set_output(0, n.in_et(0), PShape::dynamic());
        if (maxpool && n.version != "opset1") n.set_output(1, n.attr("index_element_type").et, PShape::dynamic());
        return;
    }
    const size_t sp = x.rank() - 2;
    auto k = n.attr_ints("kernel"), st = n.attr_ints("strides"), pb = n.attr_ints("pads_begin"), pe = n.attr_ints("pads_end");
    auto dil = n.has_attr("dilations") ? n.attr_ints("dilations") : std::vector<int64_t>();
    if (dil.empty()) dil.assign(sp, 1);
    if (st.empty()) st.assign(sp, 1);
    if (pb.empty()) pb.assign(sp, 0);
    if (pe.empty()) pe.assign(sp, 0);
    OVC_CHECK(k.size() == sp, n.description() << ": kernel rank " << k.size() << " does not match " << sp << " spatial dims");
    const std::string rt = n.attr_str("rounding_type", "floor");
    const bool ceil_mode = rt == "ceil" || rt == "ceil_torch";
    const std::string ap = n.attr_str("auto_pad", "explicit");
    PShape out = x;
    for (size_t i = 0; i < sp; ++i) out.dims[2 + i] = window_out(x.dims[2 + i], k[i], st[i], dil[i], pb[i], pe[i], ceil_mode, ap);
    n.set_output(0, n.in_et(0), out);
    if (maxpool && n.version != "opset1") n.set_output(1, n.attr("index_element_type").et, out);
}

void infer_matmul_like(Node& n, bool ta, bool tb, ET out_et) {
    PShape a = n.in_shape(0), b = n.in_shape(1);
    if (a.rank_dynamic || b.rank_dynamic) { n.set_output(0, out_et, PShape::dynamic()); return; }
    OVC_CHECK(a.rank() >= 1 && b.rank() >= 1, n.description() << ": scalar arguments are not allowed");
    const bool a1 = a.rank() == 1, b1 = b.rank() == 1;
    if (a1) { a.dims.insert(a.dims.begin(), Dim(1)); ta = false; }
    if (b1) { b.dims.push_back(Dim(1)); tb = false; }
    if (ta) std::swap(a.dims[a.rank() - 1], a.dims[a.rank() - 2]);
    if (tb) std::swap(b.dims[b.rank() - 1], b.dims[b.rank() - 2]);
    const Dim ka = a.dims[a.rank() - 1], kb = b.dims[b.rank() - 2];
    OVC_CHECK(ka.compatible(kb), n.description() << ": incompatible inner dimensions " << ka.str() << " and " << kb.str()
              << " (shapes " << n.in_shape(0).str() << ", " << n.in_shape(1).str() << ")");
    PShape ba(std::vector<Dim>(a.dims.begin(), a.dims.end() - 2)), bb(std::vector<Dim>(b.dims.begin(), b.dims.end() - 2));
    PShape out = broadcast_numpy(ba, bb, n);
    if (!a1) out.dims.push_back(a.dims[a.rank() - 2]);
    if (!b1) out.dims.push_back(b.dims[b.rank() - 1]);
    n.set_output(0, out_et, out);
}

void infer_reshape(Node& n) {
    const PShape& in = n.in_shape(0);
    const bool special_zero = n.attr_bool("special_zero");
    std::vector<Dim> pat;
    if (!partial_ints(n.input(1), pat)) {
        const PShape& ps = n.in_shape(1);
        if (ps.rank_is_static() && ps.rank() == 1 && ps.dims[0].is_static()) n.set_output(0, n.in_et(0), PShape::dynamic((size_t)ps.dims[0].lo));
        else n.set_output(0, n.in_et(0), PShape::dynamic());
        return;
    }
    PShape out = PShape::dynamic(pat.size());
    int minus_one = -1;
    bool all_known = true;
    int64_t known_prod = 1;
    for (size_t i = 0; i < pat.size(); ++i) {
        const Dim& p = pat[i];
        if (p.is_static() && p.lo == -1) {
            OVC_CHECK(minus_one < 0, n.description() << ": more than one -1 in the pattern");
            minus_one = (int)i;
            out.dims[i] = Dim::dynamic();
        } else if (p.is_static() && p.lo == 0 && special_zero) {
            OVC_CHECK(in.rank_dynamic || i < in.rank(), n.description() << ": '0' in the pattern refers to a missing input dimension");
            out.dims[i] = in.rank_dynamic ? Dim::dynamic() : in.dims[i];
        } else if (p.is_static()) {
            OVC_CHECK(p.lo >= 0, n.description() << ": negative dimension " << p.lo << " in the pattern");
            out.dims[i] = p;
        } else {
            out.dims[i] = Dim(std::max<int64_t>(p.lo, 0), p.hi);   // may also be -1 at run time: stays an interval
        }
    }
    if (minus_one >= 0) {
        out.dims[(size_t)minus_one] = Dim::dynamic();
        if (in.is_static()) {
            for (size_t i = 0; i < out.dims.size(); ++i) {
                if ((int)i == minus_one) continue;
                if (!out.dims[i].is_static()) { all_known = false; break; }
                known_prod *= out.dims[i].lo;
            }
            if (all_known) {
                const int64_t total = shape_size(in.to_shape());
                if (known_prod == 0) out.dims[(size_t)minus_one] = Dim(0);
                else {
                    OVC_CHECK(total % known_prod == 0, n.description() << ": cannot reshape " << in.str() << " with pattern product " << known_prod);
                    out.dims[(size_t)minus_one] = Dim(total / known_prod);
                }
            }
        } else if (!in.rank_dynamic) {
            // dynamic input: cancel equal dynamic dims (e.g. [?,S,H] -> [0,0,heads,-1])
            int64_t in_static = 1, out_static = 1;
            std::vector<Dim> in_dyn, out_dyn;
            for (auto& d : in.dims) { if (d.is_static()) in_static *= d.lo; else in_dyn.push_back(d); }
            for (size_t i = 0; i < out.dims.size(); ++i) {
                if ((int)i == minus_one) continue;
                if (out.dims[i].is_static()) out_static *= out.dims[i].lo; else out_dyn.push_back(out.dims[i]);
            }
            if (in_dyn.size() == out_dyn.size() && out_static > 0 && in_static % out_static == 0) {
                bool same = true;
                for (size_t i = 0; i < in_dyn.size(); ++i) same = same && (in_dyn[i] == out_dyn[i]);
                if (same && special_zero) out.dims[(size_t)minus_one] = Dim(in_static / out_static);
            }
        }
    } else if (in.is_static() && out.is_static()) {
        OVC_CHECK(shape_size(in.to_shape()) == shape_size(out.to_shape()),
                  n.description() << ": cannot reshape " << in.str() << " to " << out.str());
    }
    n.set_output(0, n.in_et(0), out);
}

void infer_concat(Node& n) {
    int64_t axis = n.attr_int("axis");
    PShape out = PShape::dynamic();
    ET et = ET::dynamic;
    for (auto& i : n.inputs()) {
        et = merge_types(n, et, i.et());
        if (!i.shape().rank_dynamic && out.rank_dynamic) out = PShape::dynamic(i.shape().rank());
    }
    if (out.rank_dynamic) { n.set_output(0, et, out); return; }
    axis = norm_axis(axis, (int64_t)out.rank(), n);
    Dim sum(0);
    for (auto& i : n.inputs()) {
        const PShape& s = i.shape();
        if (s.rank_dynamic) { sum = sum + Dim::dynamic(); continue; }
        OVC_CHECK(s.rank() == out.rank(), n.description() << ": inputs have different ranks");
        for (size_t d = 0; d < s.rank(); ++d) {
            if ((int64_t)d == axis) continue;
            OVC_CHECK(Dim::merge(out.dims[d], out.dims[d], s.dims[d]), n.description() << ": dimension " << d << " differs between inputs ("
                      << out.dims[d].str() << " vs " << s.dims[d].str() << ")");
        }
        sum = sum + s.dims[(size_t)axis];
    }
    out.dims[(size_t)axis] = sum;
    n.set_output(0, et, out);
    // value propagation for shape arithmetic
}

void infer_gather(Node& n) {
    const PShape& d = n.in_shape(0);
    const PShape& idx = n.in_shape(1);
    std::vector<int64_t> ax;
    int64_t batch_dims = n.attr_int("batch_dims");
    if (d.rank_dynamic || idx.rank_dynamic || !get_constant_ints(n.input(2), ax) || ax.empty()) {
        n.set_output(0, n.in_et(0), PShape::dynamic());
        return;
    }
    if (batch_dims < 0) batch_dims += (int64_t)idx.rank();
    const int64_t axis = norm_axis(ax[0], (int64_t)d.rank(), n);
    OVC_CHECK(batch_dims <= axis, n.description() << ": batch_dims " << batch_dims << " exceeds axis " << axis);
    PShape out;
    for (int64_t i = 0; i < axis; ++i) out.dims.push_back(d.dims[(size_t)i]);
    for (size_t i = (size_t)batch_dims; i < idx.rank(); ++i) out.dims.push_back(idx.dims[i]);
    for (size_t i = (size_t)axis + 1; i < d.rank(); ++i) out.dims.push_back(d.dims[i]);
    n.set_output(0, n.in_et(0), out);
}

void infer_slice_v8(Node& n) {
    const PShape& in = n.in_shape(0);
    if (in.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
    std::vector<int64_t> step, axes;
    std::vector<Dim> start, stop;
    PShape out = in;
    const bool have_vals = partial_ints(n.input(1), start) && partial_ints(n.input(2), stop) && get_constant_ints(n.input(3), step);
    if (n.num_inputs() > 4) {
        if (!get_constant_ints(n.input(4), axes)) { n.set_output(0, n.in_et(0), PShape::dynamic(in.rank())); return; }
    } else if (have_vals) {
        axes.resize(start.size());
        std::iota(axes.begin(), axes.end(), 0);
    }
    if (!have_vals) {
        if (axes.empty()) { n.set_output(0, n.in_et(0), PShape::dynamic(in.rank())); return; }
        for (auto a : axes) out.dims[(size_t)norm_axis(a, (int64_t)in.rank(), n)] = Dim(0, in.dims[(size_t)norm_axis(a, (int64_t)in.rank(), n)].hi);
        n.set_output(0, n.in_et(0), out);
        return;
    }
    for (size_t k = 0; k < axes.size(); ++k) {
        const size_t a = (size_t)norm_axis(axes[k], (int64_t)in.rank(), n);
        const Dim& d = in.dims[a];
        const int64_t st = step[k];
        OVC_CHECK(st != 0, n.description() << ": step must not be 0");
        if (!d.is_static() || !start[k].is_static() || !stop[k].is_static()) {
            // common dynamic cases: start >= 0 and a huge stop keep "dim - start"; otherwise unknown up to dim
            if (start[k].is_static() && stop[k].is_static() && st == 1 && start[k].lo >= 0 && stop[k].lo >= 0) {
                const int64_t b = start[k].lo, e = stop[k].lo;
                const int64_t lo = std::max<int64_t>(0, std::min(d.lo, e) - b);
                const int64_t hi = d.hi < 0 ? (e >= (int64_t(1) << 40) ? -1 : std::max<int64_t>(0, e - b)) : std::max<int64_t>(0, std::min(d.hi, e) - b);
                out.dims[a] = Dim(lo, hi);
            } else {
                out.dims[a] = Dim(0, d.hi);
            }
            continue;
        }
        const int64_t dim = d.lo;
        int64_t b = start[k].lo, e = stop[k].lo;
        // values written as negative numbers arrive clamped by Dim; read the raw constants when available
        std::vector<int64_t> rb, re;
        if (get_constant_ints(n.input(1), rb) && get_constant_ints(n.input(2), re)) { b = rb[k]; e = re[k]; }
        if (b < 0) b += dim;
        if (e < 0) e += dim;
        int64_t cnt;
        if (st > 0) {
            b = std::max<int64_t>(0, std::min(b, dim));
            e = std::max<int64_t>(0, std::min(e, dim));
            cnt = e > b ? (e - b + st - 1) / st : 0;
        } else {
            b = std::max<int64_t>(-1, std::min(b, dim - 1));
            e = std::max<int64_t>(-1, std::min(e, dim - 1));
            cnt = b > e ? (b - e + (-st) - 1) / (-st) : 0;
        }
        out.dims[a] = Dim(cnt);
    }
    n.set_output(0, n.in_et(0), out);
}

void infer_strided_slice(Node& n) {
    const PShape& in = n.in_shape(0);
    std::vector<int64_t> b, e, st;
    if (in.rank_dynamic || !get_constant_ints(n.input(1), b) || !get_constant_ints(n.input(2), e)) {
        n.set_output(0, n.in_et(0), PShape::dynamic());
        return;
    }
    if (n.num_inputs() > 3) { if (!get_constant_ints(n.input(3), st)) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; } }
    else st.assign(b.size(), 1);
    auto mask = [&](const char* k, size_t i) { auto v = n.attr_ints(k); return i < v.size() && v[i] != 0; };
    PShape out;
    size_t in_d = 0;
    const size_t nspec = b.size();
    size_t num_new = 0;
    for (size_t i = 0; i < nspec; ++i) if (mask("new_axis_mask", i)) ++num_new;
    for (size_t i = 0; i < nspec; ++i) {
        if (mask("ellipsis_mask", i)) {
            const size_t remaining_spec = nspec - i - 1;
            size_t rem_new = 0;
            for (size_t j = i + 1; j < nspec; ++j) if (mask("new_axis_mask", j)) ++rem_new;
            const size_t take = in.rank() - in_d - (remaining_spec - rem_new);
            for (size_t k = 0; k < take; ++k) out.dims.push_back(in.dims[in_d++]);
            continue;
        }
        if (mask("new_axis_mask", i)) { out.dims.emplace_back(1); continue; }
        OVC_CHECK(in_d < in.rank(), n.description() << ": more slice specs than input dimensions");
        const Dim& d = in.dims[in_d++];
        if (mask("shrink_axis_mask", i)) continue;
        const int64_t s = st[i];
        OVC_CHECK(s != 0, n.description() << ": stride must not be 0");
        if (!d.is_static()) {
            const bool bm = mask("begin_mask", i), em = mask("end_mask", i);
            if (bm && em && s == 1) out.dims.push_back(d);
            else if (s == 1 && em && !bm && b[i] >= 0) out.dims.emplace_back(Dim(std::max<int64_t>(0, d.lo - b[i]), d.hi < 0 ? -1 : std::max<int64_t>(0, d.hi - b[i])));
            else if (s == 1 && !em && e[i] >= 0 && (bm || b[i] >= 0)) {
                const int64_t bb = bm ? 0 : b[i];
                out.dims.emplace_back(Dim(std::max<int64_t>(0, std::min(d.lo, e[i]) - bb), std::max<int64_t>(0, (d.hi < 0 ? e[i] : std::min(d.hi, e[i])) - bb)));
            } else out.dims.emplace_back(Dim(0, d.hi));
            continue;
        }
        const int64_t dim = d.lo;
        int64_t bb = b[i], ee = e[i];
        if (bb < 0) bb += dim;
        if (ee < 0) ee += dim;
        int64_t cnt;
        if (s > 0) {
            if (mask("begin_mask", i)) bb = 0;
            if (mask("end_mask", i)) ee = dim;
            bb = std::max<int64_t>(0, std::min(bb, dim));
            ee = std::max<int64_t>(0, std::min(ee, dim));
            cnt = ee > bb ? (ee - bb + s - 1) / s : 0;
        } else {
            if (mask("begin_mask", i)) bb = dim - 1;
            if (mask("end_mask", i)) ee = -1;
            else ee = std::max<int64_t>(-1, std::min(ee, dim - 1));
            bb = std::max<int64_t>(-1, std::min(bb, dim - 1));
            cnt = bb > ee ? (bb - ee + (-s) - 1) / (-s) : 0;
        }
        out.dims.emplace_back(cnt);
    }
    while (in_d < in.rank()) out.dims.push_back(in.dims[in_d++]);
    n.set_output(0, n.in_et(0), out);
}

void infer_split(Node& n) {
    const PShape& in = n.in_shape(0);
    const int64_t parts = n.attr_int("num_splits");
    std::vector<int64_t> ax;
    n.set_num_outputs((size_t)parts);
    if (in.rank_dynamic || !get_constant_ints(n.input(1), ax)) {
        for (int64_t i = 0; i < parts; ++i) n.set_output((size_t)i, n.in_et(0), in.rank_dynamic ? PShape::dynamic() : PShape::dynamic(in.rank()));
        return;
    }
    const size_t a = (size_t)norm_axis(ax[0], (int64_t)in.rank(), n);
    PShape out = in;
    if (in.dims[a].is_static()) {
        OVC_CHECK(in.dims[a].lo % parts == 0, n.description() << ": dimension " << in.dims[a].lo << " is not divisible by " << parts);
        out.dims[a] = Dim(in.dims[a].lo / parts);
    } else {
        out.dims[a] = Dim(in.dims[a].lo / parts, in.dims[a].hi < 0 ? -1 : in.dims[a].hi / parts);
    }
    for (int64_t i = 0; i < parts; ++i) n.set_output((size_t)i, n.in_et(0), out);
}

void infer_variadic_split(Node& n) {
    const PShape& in = n.in_shape(0);
    std::vector<int64_t> ax, lens;
    const PShape& ls = n.in_shape(2);
    if (!get_constant_ints(n.input(2), lens)) {
        OVC_CHECK(ls.is_static() && ls.rank() == 1, n.description() << ": split_lengths must have a static 1-D shape");
        n.set_num_outputs((size_t)ls.dims[0].lo);
        for (int64_t i = 0; i < ls.dims[0].lo; ++i) n.set_output((size_t)i, n.in_et(0), in.rank_dynamic ? PShape::dynamic() : PShape::dynamic(in.rank()));
        return;
    }
    n.set_num_outputs(lens.size());
    if (in.rank_dynamic || !get_constant_ints(n.input(1), ax)) {
        for (size_t i = 0; i < lens.size(); ++i) n.set_output(i, n.in_et(0), in.rank_dynamic ? PShape::dynamic() : PShape::dynamic(in.rank()));
        return;
    }
    const size_t a = (size_t)norm_axis(ax[0], (int64_t)in.rank(), n);
    int64_t known = 0, neg = -1;
    for (size_t i = 0; i < lens.size(); ++i) { if (lens[i] == -1) neg = (int64_t)i; else known += lens[i]; }
    for (size_t i = 0; i < lens.size(); ++i) {
        PShape out = in;
        if ((int64_t)i == neg) {
            out.dims[a] = in.dims[a].is_static() ? Dim(in.dims[a].lo - known) : Dim(std::max<int64_t>(0, in.dims[a].lo - known), in.dims[a].hi < 0 ? -1 : in.dims[a].hi - known);
        } else out.dims[a] = Dim(lens[i]);
        n.set_output(i, n.in_et(0), out);
    }
    if (neg < 0 && in.dims[a].is_static())
        OVC_CHECK(known == in.dims[a].lo, n.description() << ": split lengths sum to " << known << ", dimension is " << in.dims[a].lo);
}

void infer_broadcast(Node& n) {
    std::vector<Dim> target;
    const PShape& in = n.in_shape(0);
    const std::string mode = n.attr_str("mode", "numpy");
    if (!partial_ints(n.input(1), target)) {
        const PShape& ts = n.in_shape(1);
        if (ts.is_static() && ts.rank() == 1) {
            const size_t r = (mode == "bidirectional" && !in.rank_dynamic) ? std::max(in.rank(), (size_t)ts.dims[0].lo) : (size_t)ts.dims[0].lo;
            n.set_output(0, n.in_et(0), PShape::dynamic(r));
        } else n.set_output(0, n.in_et(0), PShape::dynamic());
        return;
    }
    PShape t(target);
    if (mode == "bidirectional") { n.set_output(0, n.in_et(0), broadcast_numpy(in, t, n)); return; }
    if (mode == "explicit") { n.set_output(0, n.in_et(0), t); return; }
    // numpy: the target shape wins; input dims must be 1 or equal
    if (!in.rank_dynamic) {
        OVC_CHECK(in.rank() <= t.rank(), n.description() << ": input rank " << in.rank() << " exceeds target rank " << t.rank());
        for (size_t i = 0; i < in.rank(); ++i) {
            const Dim& di = in.dims[in.rank() - 1 - i];
            Dim& dt = t.dims[t.rank() - 1 - i];
            if (di.is_static() && di.lo != 1 && dt.is_static())
                OVC_CHECK(di.lo == dt.lo, n.description() << ": cannot broadcast " << in.str() << " to " << t.str());
            if (!dt.is_static() && di.is_static() && di.lo != 1) dt = di;
        }
    }
    n.set_output(0, n.in_et(0), t);
}

void infer_unsqueeze(Node& n) {
    const PShape& in = n.in_shape(0);
    std::vector<int64_t> axes;
    if (in.rank_dynamic || !get_constant_ints(n.input(1), axes)) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
    const int64_t r = (int64_t)in.rank() + (int64_t)axes.size();
    std::set<int64_t> ax;
    for (auto a : axes) ax.insert(norm_axis(a, r, n));
    PShape out;
    size_t k = 0;
    for (int64_t i = 0; i < (int64_t)in.rank() + (int64_t)ax.size(); ++i) {
        if (ax.count(i)) out.dims.emplace_back(1); else out.dims.push_back(in.dims[k++]);
    }
    n.set_output(0, n.in_et(0), out);
}

void infer_squeeze(Node& n) {
    const PShape& in = n.in_shape(0);
    if (in.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
    PShape out;
    if (n.num_inputs() < 2) {
        for (auto& d : in.dims) {
            if (d.is_static() && d.lo == 1) continue;
            if (!d.is_static() && d.lo <= 1 && (d.hi < 0 || d.hi >= 1)) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
            out.dims.push_back(d);
        }
        n.set_output(0, n.in_et(0), out);
        return;
    }
    std::vector<int64_t> axes;
    if (!get_constant_ints(n.input(1), axes)) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
    std::set<int64_t> ax;
    for (auto a : axes) ax.insert(norm_axis(a, (int64_t)in.rank(), n));
    for (size_t i = 0; i < in.rank(); ++i) {
        if (ax.count((int64_t)i)) {
            const Dim& d = in.dims[i];
            if (d.is_static() && d.lo != 1) { out.dims.push_back(d); continue; }   // non-unit axes are kept (torch semantics)
            continue;
        }
        out.dims.push_back(in.dims[i]);
    }
    n.set_output(0, n.in_et(0), out);
}

void infer_transpose(Node& n) {
    const PShape& in = n.in_shape(0);
    std::vector<int64_t> order;
    if (in.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
    if (!get_constant_ints(n.input(1), order)) { n.set_output(0, n.in_et(0), PShape::dynamic(in.rank())); return; }
    if (order.empty()) { for (int64_t i = (int64_t)in.rank() - 1; i >= 0; --i) order.push_back(i); }
    OVC_CHECK(order.size() == in.rank(), n.description() << ": order has " << order.size() << " entries for rank " << in.rank());
    PShape out = PShape::dynamic(in.rank());
    std::vector<bool> seen(in.rank(), false);
    for (size_t i = 0; i < order.size(); ++i) {
        const int64_t a = norm_axis(order[i], (int64_t)in.rank(), n);
        OVC_CHECK(!seen[(size_t)a], n.description() << ": order is not a permutation");
        seen[(size_t)a] = true;
        out.dims[i] = in.dims[(size_t)a];
    }
    n.set_output(0, n.in_et(0), out);
}

void infer_topk(Node& n) {
    const PShape& in = n.in_shape(0);
    const ET iet = n.attr("index_element_type").et;
    if (in.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); n.set_output(1, iet, PShape::dynamic()); return; }
    const size_t a = (size_t)norm_axis(n.attr_int("axis"), (int64_t)in.rank(), n);
    PShape out = in;
    std::vector<Dim> k;
    if (partial_ints(n.input(1), k) && k.size() == 1) out.dims[a] = k[0]; else out.dims[a] = Dim(0, in.dims[a].hi);
    n.set_output(0, n.in_et(0), out);
    n.set_output(1, iet, out);
}

void infer_sdpa(Node& n) {
    const PShape& q = n.in_shape(0);
    const PShape& v = n.in_shape(2);
    if (q.rank_dynamic || v.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
    PShape out = q;
    out.dims[out.rank() - 1] = v.dims[v.rank() - 1];
    // batch dims broadcast between q and k/v
    const PShape& k = n.in_shape(1);
    if (!k.rank_dynamic && k.rank() == q.rank()) {
        for (size_t i = 0; i + 2 < q.rank(); ++i) {
            if (q.dims[i].is_static() && q.dims[i].lo == 1) out.dims[i] = k.dims[i];
        }
    }
    n.set_output(0, n.in_et(0), out);
}

void infer_interpolate(Node& n) {
    const PShape& in = n.in_shape(0);
    if (in.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
    std::vector<int64_t> axes;
    const bool v11 = n.version == "opset11";
    const size_t axes_port = v11 ? 2 : 3;
    if (n.num_inputs() > axes_port) { if (!get_constant_ints(n.input(axes_port), axes)) { n.set_output(0, n.in_et(0), PShape::dynamic(in.rank())); return; } }
    else { axes.resize(in.rank()); std::iota(axes.begin(), axes.end(), 0); }
    PShape out = in;
    const std::string scm = n.attr_str("shape_calculation_mode", "sizes");
    auto pb = n.attr_ints("pads_begin"), pe = n.attr_ints("pads_end");
    if (scm == "sizes") {
        std::vector<Dim> sizes;
        if (!partial_ints(n.input(1), sizes)) { for (auto a : axes) out.dims[(size_t)norm_axis(a, (int64_t)in.rank(), n)] = Dim::dynamic(); }
        else for (size_t i = 0; i < axes.size() && i < sizes.size(); ++i) out.dims[(size_t)norm_axis(axes[i], (int64_t)in.rank(), n)] = sizes[i];
    } else {
        Tensor sc;
        const size_t scales_port = v11 ? 1 : 2;
        if (!try_constant_value(n.input(scales_port), sc)) { for (auto a : axes) out.dims[(size_t)norm_axis(a, (int64_t)in.rank(), n)] = Dim::dynamic(); }
        else {
            auto s = to_f32(sc);
            for (size_t i = 0; i < axes.size() && i < s.size(); ++i) {
                const size_t a = (size_t)norm_axis(axes[i], (int64_t)in.rank(), n);
                const int64_t pad = (a < pb.size() ? pb[a] : 0) + (a < pe.size() ? pe[a] : 0);
                if (in.dims[a].is_static()) out.dims[a] = Dim(int64_t(std::floor((in.dims[a].lo + pad) * double(s[i]) + 1e-5)));
                else out.dims[a] = Dim::dynamic();
            }
        }
    }
    n.set_output(0, n.in_et(0), out);
}

void infer_body_op(Node& n) {
    // If: outputs follow the then-body results; Loop/TensorIterator: follow the body with the iteration axis unknown
    OVC_CHECK(!n.bodies.empty() && n.bodies[0], n.description() << ": missing body");
    const auto out_map = n.attr_ints("output_map");   // pairs (body result index, concat axis or -1) per node output, body 0
    const size_t nout = out_map.size() / 2;
    n.set_num_outputs(std::max<size_t>(nout, 1));
    for (size_t i = 0; i < nout; ++i) {
        const auto& res = n.bodies[0]->results.at((size_t)out_map[2 * i]);
        PShape s = res->outs[0].shape;
        ET et = res->outs[0].et;
        if (n.type == "If" && n.bodies.size() > 1 && n.bodies[1]) {
            const auto em = n.attr_ints("else_output_map");
            if (2 * i < em.size()) {
                const auto& r2 = n.bodies[1]->results.at((size_t)em[2 * i]);
                PShape m;
                if (!PShape::merge(m, s, r2->outs[0].shape) || s != r2->outs[0].shape) {
                    if (!s.rank_dynamic && !r2->outs[0].shape.rank_dynamic && s.rank() == r2->outs[0].shape.rank()) {
                        for (size_t d = 0; d < s.rank(); ++d) if (s.dims[d] != r2->outs[0].shape.dims[d]) s.dims[d] = Dim::dynamic();
                    } else s = PShape::dynamic();
                }
            }
        } else if (out_map[2 * i + 1] >= 0 && !s.rank_dynamic) {
            s.dims[(size_t)out_map[2 * i + 1]] = Dim::dynamic();
        }
        n.set_output(i, et, s);
    }
}

}  // namespace

// ------------------------------------------------------------------------------------ registration
void register_all_ops() {
    static std::once_flag once;
    std::call_once(once, [] {
        const auto AB = [] { return As("auto_broadcast", "numpy"); };

        // ---- graph plumbing
        reg("Parameter", "opset1", {A("shape", K::PSHAPE, Attr::Shape_(PShape::dynamic())), At("element_type", ET::f32)},
            [](Node& n) { n.set_output(0, n.attr("element_type").et, n.attr("shape").ps); }, 0, 0, false, true);
        reg("Result", "opset1", {}, [](Node& n) { n.set_output(0, n.in_et(0), n.in_shape(0)); }, 1, 1, false, true);
        reg("Constant", "opset1", {At("element_type", ET::f32), A("shape", K::PSHAPE, Attr::Shape_(PShape()))},
            [](Node& n) {
                if (n.constant.defined()) {
                    n.set_attr("element_type", Attr::Type(n.constant.et));
                    n.set_attr("shape", Attr::Shape_(PShape(n.constant.shape)));
                }
                n.set_output(0, n.attr("element_type").et, n.attr("shape").ps);
            }, 0, 0);
        reg("Convert", "opset1", {At("destination_type", ET::f32)},
            [](Node& n) { n.set_output(0, n.attr("destination_type").et, n.in_shape(0)); }, 1, 1);
        reg("ConvertLike", "opset1", {}, [](Node& n) { n.set_output(0, n.in_et(1), n.in_shape(0)); }, 2, 2);

        // ---- unary elementwise
        for (const char* t : {"Abs", "Acos", "Asin", "Atan", "Ceiling", "Cos", "Cosh", "Erf", "Exp", "Floor", "Log", "Negative",
                              "Relu", "Sigmoid", "Sign", "Sin", "Sinh", "Sqrt", "Tan", "Tanh"})
            reg(t, "opset1", {}, infer_same, 1, 1);
        for (const char* t : {"Asinh", "Acosh", "Atanh"}) reg(t, "opset4", {}, infer_same, 1, 1);
        reg("LogicalNot", "opset1", {}, [](Node& n) { n.set_output(0, ET::boolean, n.in_shape(0)); }, 1, 1);
        reg("Gelu", "opset7", {As("approximation_mode", "ERF")}, infer_same, 1, 1);
        reg("Gelu", "opset2", {}, infer_same, 1, 1);
        reg("Swish", "opset4", {}, infer_same, 1, 2);
        reg("Mish", "opset4", {}, infer_same, 1, 1);
        reg("HSwish", "opset4", {}, infer_same, 1, 1);
        reg("HSigmoid", "opset5", {}, infer_same, 1, 1);
        reg("SoftPlus", "opset4", {}, infer_same, 1, 1);
        reg("SoftSign", "opset9", {}, infer_same, 1, 1);
        reg("Elu", "opset1", {Af("alpha", 1.0, false)}, infer_same, 1, 1);
        reg("Selu", "opset1", {}, infer_same, 3, 3);
        reg("Clamp", "opset1", {Af("min", 0, false), Af("max", 0, false)}, infer_same, 1, 1);
        reg("Round", "opset5", {As("mode", "half_to_even")}, infer_same, 1, 1);
        reg("IsNaN", "opset10", {}, [](Node& n) { n.set_output(0, ET::boolean, n.in_shape(0)); }, 1, 1);
        reg("IsFinite", "opset10", {}, [](Node& n) { n.set_output(0, ET::boolean, n.in_shape(0)); }, 1, 1);
        reg("IsInf", "opset10", {Ab("detect_negative", true), Ab("detect_positive", true)},
            [](Node& n) { n.set_output(0, ET::boolean, n.in_shape(0)); }, 1, 1);
        reg("HardSigmoid", "opset1", {}, infer_same, 3, 3);
        reg("LogSoftmax", "opset5", {Ai("axis", 1)}, infer_same, 1, 1);
        reg("Softmax", "opset1", {Ai("axis", 1)}, infer_same, 1, 1);
        reg("Softmax", "opset8", {Ai("axis", 1)}, infer_same, 1, 1);
        reg("PRelu", "opset1", {}, infer_same, 2, 2);

        // ---- binary elementwise
        for (const char* t : {"Add", "Multiply", "Maximum", "Minimum"}) reg(t, "opset1", {AB()}, infer_binary_arith, 2, 2, true);
        for (const char* t : {"Subtract", "Power", "Mod", "FloorMod", "SquaredDifference"}) reg(t, "opset1", {AB()}, infer_binary_arith, 2, 2);
        reg("Divide", "opset1", {AB(), Ab("m_pythondiv", true)}, infer_binary_arith, 2, 2);
        for (const char* t : {"Equal", "NotEqual"}) reg(t, "opset1", {AB()}, infer_binary_cmp, 2, 2, true);
        for (const char* t : {"Less", "LessEqual", "Greater", "GreaterEqual"}) reg(t, "opset1", {AB()}, infer_binary_cmp, 2, 2);
        for (const char* t : {"LogicalAnd", "LogicalOr", "LogicalXor", "Xor"}) reg(t, "opset1", {AB()}, infer_binary_cmp, 2, 2, true);
        for (const char* t : {"BitwiseAnd", "BitwiseOr", "BitwiseXor"}) reg(t, "opset13", {AB()}, infer_binary_arith, 2, 2, true);
        reg("BitwiseNot", "opset13", {}, infer_same, 1, 1);
        reg("Select", "opset1", {AB()},
            [](Node& n) {
                const ET et = merge_types(n, n.in_et(1), n.in_et(2));
                n.set_output(0, et, broadcast_by_attr(n, n.in_shape(0), broadcast_by_attr(n, n.in_shape(1), n.in_shape(2))));
            }, 3, 3);

        // ---- reductions
        for (const char* t : {"ReduceSum", "ReduceMean", "ReduceMax", "ReduceMin", "ReduceProd", "ReduceLogicalAnd", "ReduceLogicalOr"})
            reg(t, "opset1", {Ab("keep_dims", false)}, infer_reduce, 2, 2);
        for (const char* t : {"ReduceL1", "ReduceL2"}) reg(t, "opset4", {Ab("keep_dims", false)}, infer_reduce, 2, 2);

        // ---- linear algebra / NN
        reg("MatMul", "opset1", {Ab("transpose_a", false), Ab("transpose_b", false)},
            [](Node& n) { infer_matmul_like(n, n.attr_bool("transpose_a"), n.attr_bool("transpose_b"), merge_types(n, n.in_et(0), n.in_et(1))); }, 2, 2);
        const std::vector<AttrSpec> conv_attrs = {Ais("strides"), Ais("dilations"), Ais("pads_begin"), Ais("pads_end"), As("auto_pad", "explicit")};
        reg("Convolution", "opset1", conv_attrs, [](Node& n) { infer_conv(n, false); }, 2, 2);
        reg("GroupConvolution", "opset1", {Ais("strides"), Ais("pads_begin"), Ais("pads_end"), Ais("dilations"), As("auto_pad", "explicit")},
            [](Node& n) { infer_conv(n, true); }, 2, 2);
        reg("MaxPool", "opset1", {Ais("strides"), Ais("pads_begin"), Ais("pads_end"), Ais("kernel"), As("rounding_type", "floor"), As("auto_pad", "explicit")},
            [](Node& n) { infer_pool(n, true); }, 1, 1);
        const std::vector<AttrSpec> mp8 = {Ais("strides"), Ais("dilations"), Ais("pads_begin"), Ais("pads_end"), Ais("kernel"),
                                           As("rounding_type", "floor"), As("auto_pad", "explicit"), At("index_element_type", ET::i64), Ai("axis", 0)};
        reg("MaxPool", "opset8", mp8, [](Node& n) { n.set_num_outputs(2); infer_pool(n, true); }, 1, 1);
        reg("MaxPool", "opset14", mp8, [](Node& n) { n.set_num_outputs(2); infer_pool(n, true); }, 1, 1);
        const std::vector<AttrSpec> ap1 = {Ais("kernel"), Ais("strides"), Ais("pads_begin"), Ais("pads_end"), Ab("exclude-pad", false),
                                           As("auto_pad", "explicit"), As("rounding_type", "floor")};
        reg("AvgPool", "opset1", ap1, [](Node& n) { infer_pool(n, false); }, 1, 1);
        reg("AvgPool", "opset14", ap1, [](Node& n) { infer_pool(n, false); }, 1, 1);
        reg("AdaptiveAvgPool", "opset8", {},
            [](Node& n) {
                const PShape& in = n.in_shape(0);
                if (in.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
                PShape out = in;
                std::vector<Dim> sz;
                if (partial_ints(n.input(1), sz)) for (size_t i = 0; i < sz.size() && 2 + i < out.rank(); ++i) out.dims[2 + i] = sz[i];
                else for (size_t i = 2; i < out.rank(); ++i) out.dims[i] = Dim::dynamic();
                n.set_output(0, n.in_et(0), out);
            }, 2, 2);
        reg("BatchNormInference", "opset5", {Af("epsilon", 1e-5, false)}, infer_same, 5, 5);
        reg("MVN", "opset6", {Af("eps", 1e-9), Ab("normalize_variance", true), As("eps_mode", "inside_sqrt")}, infer_same, 2, 2);
        reg("NormalizeL2", "opset1", {Af("eps", 1e-12), As("eps_mode", "add")}, infer_same, 2, 2);
        reg("GroupNormalization", "opset12", {Ai("num_groups", 1), Af("epsilon", 1e-5, false)}, infer_same, 3, 3);
        reg("ScaledDotProductAttention", "opset13", {Ab("causal", false)}, infer_sdpa, 3, 6);
        reg("FakeQuantize", "opset1", {Ai("levels", 256), AB()}, infer_same, 5, 5);
        const std::vector<AttrSpec> interp = {As("mode", "nearest"), As("shape_calculation_mode", "sizes"),
                                              As("coordinate_transformation_mode", "half_pixel"), As("nearest_mode", "round_prefer_floor"),
                                              Ab("antialias", false), Ais("pads_begin"), Ais("pads_end"), Af("cube_coeff", -0.75, false)};
        reg("Interpolate", "opset4", interp, infer_interpolate, 3, 4);
        reg("Interpolate", "opset11", interp, infer_interpolate, 2, 3);
        reg("Einsum", "opset7", {As("equation", "")}, [](Node& n) { n.set_output(0, n.in_et(0), PShape::dynamic()); }, 1, -1);

        // ---- data movement
        reg("Reshape", "opset1", {Ab("special_zero", false)}, infer_reshape, 2, 2);
        reg("Transpose", "opset1", {}, infer_transpose, 2, 2);
        reg("Concat", "opset1", {Ai("axis", 0)}, infer_concat, 1, -1);
        reg("Split", "opset1", {Ai("num_splits", 1)}, infer_split, 2, 2);
        reg("VariadicSplit", "opset1", {}, infer_variadic_split, 3, 3);
        reg("Slice", "opset8", {}, infer_slice_v8, 4, 5);
        reg("StridedSlice", "opset1", {Ais("begin_mask"), Ais("end_mask"), Ais("new_axis_mask"), Ais("shrink_axis_mask"), Ais("ellipsis_mask")},
            infer_strided_slice, 3, 4);
        reg("Gather", "opset1", {}, infer_gather, 3, 3);
        reg("Gather", "opset7", {Ai("batch_dims", 0)}, infer_gather, 3, 3);
        reg("Gather", "opset8", {Ai("batch_dims", 0)}, infer_gather, 3, 3);
        reg("GatherElements", "opset6", {Ai("axis", 0)}, [](Node& n) { n.set_output(0, n.in_et(0), n.in_shape(1)); }, 2, 2);
        reg("GatherND", "opset8", {Ai("batch_dims", 0)},
            [](Node& n) {
                const PShape &d = n.in_shape(0), &i = n.in_shape(1);
                if (d.rank_dynamic || i.rank_dynamic || !i.dims.back().is_static()) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
                const size_t bd = (size_t)n.attr_int("batch_dims"), k = (size_t)i.dims.back().lo;
                PShape out;
                for (size_t a = 0; a + 1 < i.rank(); ++a) out.dims.push_back(i.dims[a]);
                for (size_t a = bd + k; a < d.rank(); ++a) out.dims.push_back(d.dims[a]);
                n.set_output(0, n.in_et(0), out);
            }, 2, 2);
        reg("ScatterUpdate", "opset3", {}, infer_same, 4, 4);
        reg("ScatterNDUpdate", "opset3", {}, infer_same, 3, 3);
        reg("ScatterNDUpdate", "opset15", {As("reduction", "none")}, infer_same, 3, 3);
        reg("ScatterElementsUpdate", "opset3", {}, infer_same, 4, 4);
        reg("ScatterElementsUpdate", "opset12", {As("reduction", "none"), Ab("use_init_val", true)}, infer_same, 4, 4);
        reg("ShapeOf", "opset1", {},
            [](Node& n) { n.set_output(0, ET::i64, n.in_shape(0).rank_dynamic ? PShape::dynamic(1) : PShape(Shape{(int64_t)n.in_shape(0).rank()})); }, 1, 1);
        reg("ShapeOf", "opset3", {At("output_type", ET::i64)},
            [](Node& n) { n.set_output(0, n.attr("output_type").et, n.in_shape(0).rank_dynamic ? PShape::dynamic(1) : PShape(Shape{(int64_t)n.in_shape(0).rank()})); }, 1, 1);
        reg("Broadcast", "opset3", {As("mode", "numpy")}, infer_broadcast, 2, 3);
        reg("Broadcast", "opset1", {As("mode", "numpy")}, infer_broadcast, 2, 3);
        reg("Unsqueeze", "opset1", {}, infer_unsqueeze, 2, 2);
        reg("Squeeze", "opset1", {}, infer_squeeze, 1, 2);
        reg("Squeeze", "opset15", {Ab("allow_axis_skip", false)}, infer_squeeze, 1, 2);
        reg("Tile", "opset1", {},
            [](Node& n) {
                const PShape& in = n.in_shape(0);
                std::vector<int64_t> rep;
                if (in.rank_dynamic || !get_constant_ints(n.input(1), rep)) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
                const size_t r = std::max(in.rank(), rep.size());
                PShape out = PShape::dynamic(r);
                for (size_t i = 0; i < r; ++i) {
                    const Dim d = i < r - in.rank() ? Dim(1) : in.dims[i - (r - in.rank())];
                    const int64_t m = i < r - rep.size() ? 1 : rep[i - (r - rep.size())];
                    out.dims[i] = d * Dim(m);
                }
                n.set_output(0, n.in_et(0), out);
            }, 2, 2);
        auto infer_pad = [](Node& n) {
            const PShape& in = n.in_shape(0);
            std::vector<int64_t> pb, pe;
            if (in.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
            if (!get_constant_ints(n.input(1), pb) || !get_constant_ints(n.input(2), pe)) { n.set_output(0, n.in_et(0), PShape::dynamic(in.rank())); return; }
            PShape out = in;
            for (size_t i = 0; i < in.rank() && i < pb.size(); ++i) {
                const int64_t add = pb[i] + pe[i];
                out.dims[i] = Dim(std::max<int64_t>(0, in.dims[i].lo + add), in.dims[i].hi < 0 ? -1 : std::max<int64_t>(0, in.dims[i].hi + add));
            }
            n.set_output(0, n.in_et(0), out);
        };
        reg("Pad", "opset1", {As("pad_mode", "constant")}, infer_pad, 3, 4);
        reg("Pad", "opset12", {As("pad_mode", "constant")}, infer_pad, 3, 4);
        reg("Range", "opset4", {At("output_type", ET::i64)},
            [](Node& n) {
                Tensor a, b, c;
                if (try_constant_value(n.input(0), a) && try_constant_value(n.input(1), b) && try_constant_value(n.input(2), c)) {
                    const double s = get_elem_f64(a, 0), e = get_elem_f64(b, 0), st = get_elem_f64(c, 0);
                    OVC_CHECK(st != 0, n.description() << ": step must not be 0");
                    const int64_t cnt = std::max<int64_t>(0, (int64_t)std::ceil((e - s) / st));
                    n.set_output(0, n.attr("output_type").et, PShape(Shape{cnt}));
                } else n.set_output(0, n.attr("output_type").et, PShape::dynamic(1));
            }, 3, 3);
        reg("OneHot", "opset1", {Ai("axis", -1)},
            [](Node& n) {
                const PShape& in = n.in_shape(0);
                if (in.rank_dynamic) { n.set_output(0, n.in_et(2), PShape::dynamic()); return; }
                std::vector<Dim> depth;
                Dim dd = Dim::dynamic();
                if (partial_ints(n.input(1), depth) && depth.size() == 1) dd = depth[0];
                int64_t axis = n.attr_int("axis");
                if (axis < 0) axis += (int64_t)in.rank() + 1;
                PShape out = in;
                out.dims.insert(out.dims.begin() + axis, dd);
                n.set_output(0, n.in_et(2), out);
            }, 4, 4);
        reg("CumSum", "opset3", {Ab("exclusive", false), Ab("reverse", false)}, infer_same, 1, 2);
        reg("TopK", "opset11", {Ai("axis", 0), As("mode", "max"), As("sort", "value"), At("index_element_type", ET::i32), Ab("stable", false)},
            [](Node& n) { n.set_num_outputs(2); infer_topk(n); }, 2, 2);
        reg("TopK", "opset3", {Ai("axis", 0), As("mode", "max"), As("sort", "value"), At("index_element_type", ET::i32)},
            [](Node& n) { n.set_num_outputs(2); infer_topk(n); }, 2, 2);
        reg("NonZero", "opset3", {At("output_type", ET::i64)},
            [](Node& n) {
                const PShape& in = n.in_shape(0);
                PShape out = PShape::dynamic(2);
                if (!in.rank_dynamic) out.dims[0] = Dim((int64_t)in.rank());
                if (in.is_static()) out.dims[1] = Dim(0, shape_size(in.to_shape()));
                n.set_output(0, n.attr("output_type").et, out);
            }, 1, 1);
        reg("Roll", "opset7", {}, infer_same, 3, 3);
        reg("DepthToSpace", "opset1", {Ai("block_size", 1), As("mode", "blocks_first")},
            [](Node& n) {
                const PShape& in = n.in_shape(0);
                if (in.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
                const int64_t b = n.attr_int("block_size");
                PShape out = in;
                int64_t div = 1;
                for (size_t i = 2; i < in.rank(); ++i) { out.dims[i] = in.dims[i] * Dim(b); div *= b; }
                out.dims[1] = in.dims[1].is_static() ? Dim(in.dims[1].lo / div) : Dim::dynamic();
                n.set_output(0, n.in_et(0), out);
            }, 1, 1);
        reg("ArgMaxMin_internal", "ie_internal_opset", {Ai("axis", 0), Ab("keep_dims", false), As("mode", "max"), At("index_element_type", ET::i64)},
            [](Node& n) {
                const PShape& in = n.in_shape(0);
                if (in.rank_dynamic) { n.set_output(0, n.attr("index_element_type").et, PShape::dynamic()); return; }
                const size_t a = (size_t)norm_axis(n.attr_int("axis"), (int64_t)in.rank(), n);
                PShape out;
                for (size_t i = 0; i < in.rank(); ++i) { if (i == a) { if (n.attr_bool("keep_dims")) out.dims.emplace_back(1); } else out.dims.push_back(in.dims[i]); }
                n.set_output(0, n.attr("index_element_type").et, out);
            }, 1, 1);

        // ---- stateful
        reg("ReadValue", "opset6", {As("variable_id", ""), At("variable_type", ET::dynamic), A("variable_shape", K::PSHAPE, Attr::Shape_(PShape::dynamic()))},
            [](Node& n) {
                if (n.num_inputs() > 0) {
                    ET et = n.attr("variable_type").et;
                    PShape s = n.attr("variable_shape").ps;
                    if (et == ET::dynamic) et = n.in_et(0);
                    if (s.rank_dynamic) s = n.in_shape(0);
                    n.set_output(0, et, s);
                } else n.set_output(0, n.attr("variable_type").et, n.attr("variable_shape").ps);
            }, 0, 1, false, true);
        reg("ReadValue", "opset3", {As("variable_id", "")}, [](Node& n) { n.set_output(0, n.in_et(0), n.in_shape(0)); }, 1, 1, false, true);
        reg("Assign", "opset6", {As("variable_id", "")}, [](Node& n) { n.set_output(0, n.in_et(0), n.in_shape(0)); }, 1, 1, false, true);
        reg("Assign", "opset3", {As("variable_id", "")}, [](Node& n) { n.set_output(0, n.in_et(0), n.in_shape(0)); }, 1, 1, false, true);

        // ---- control flow (bodies are Models; port maps are stored as integer lists)
        //   input_map / else_input_map : triples (node input, body parameter, slice axis or -1 [, merged: back-edge result])
        //   output_map / else_output_map: pairs (body result, concat axis or -1)
        const std::vector<AttrSpec> body_attrs = {Ais("input_map"), Ais("output_map"), Ais("else_input_map"), Ais("else_output_map"),
                                                  Ais("back_edges"), Ai("current_iteration_input", -1), Ai("body_condition_output", -1)};
        reg("If", "opset8", body_attrs, infer_body_op, 1, -1);
        reg("Loop", "opset5", body_attrs, infer_body_op, 2, -1);
        reg("TensorIterator", "opset1", body_attrs, infer_body_op, 0, -1);

        // ---- LLM / internal operations
        reg("RMS", "ie_internal_opset", {Af("epsilon", 1e-6, false), At("output_type", ET::dynamic), Ab("elementwise_affine", true)},
            [](Node& n) { const ET t = n.attr("output_type").et; n.set_output(0, t == ET::dynamic ? n.in_et(0) : t, n.in_shape(0)); }, 1, 2);
        reg("RMSNorm", "internal", {Af("epsilon", 1e-6, false), At("compute_type", ET::dynamic)}, infer_same, 2, 3);
        reg("RoPE", "ie_internal_opset",
            {Ai("slice_start", 0), Ai("slice_stop", 0), Ab("input_trans0213", false), Ab("output_trans0213", false), Ab("is_interleaved", false),
             Ai("rotary_ndims", 0), Ab("is_chatglm", false), Ab("support_2d_rope", false), Ab("support_3d_rope", false), Ab("is_qwen", false),
             Ab("use_rope_cache", false), Ab("is_ltx_video", false), Ai("head_cnt", 0), Ai("head_size", 0), Ai("gather_position_arg_id", 0)},
            [](Node& n) {
                PShape s = n.in_shape(0);
                if (n.attr_bool("is_qwen") || n.attr_bool("is_chatglm")) {      // fused QKV [a, b, W] -> [a, b, heads, head size]
                    const bool r3 = !s.rank_dynamic && s.rank() == 3;
                    n.set_output(0, n.in_et(0), PShape({r3 ? s.dims[0] : Dim::dynamic(), r3 ? s.dims[1] : Dim::dynamic(), Dim(n.attr_int("head_cnt")), Dim(n.attr_int("head_size"))}));
                    return;
                }
                if (!s.rank_dynamic && s.rank() == 4 && (n.attr_bool("input_trans0213") != n.attr_bool("output_trans0213"))) std::swap(s.dims[1], s.dims[2]);
                if (!s.rank_dynamic && n.attr_int("slice_stop") > n.attr_int("slice_start")) s.dims.back() = Dim(n.attr_int("slice_stop") - n.attr_int("slice_start"));
                n.set_output(0, n.in_et(0), s);
            }, 3, 4);
        reg("FullyConnected", "ie_internal_opset", {At("output_type", ET::dynamic)},
            [](Node& n) { const ET t = n.attr("output_type").et; infer_matmul_like(n, false, true, t == ET::dynamic ? n.in_et(0) : t); }, 2, 3);
        reg("FullyConnectedCompressed", "ie_internal_opset", {At("output_type", ET::dynamic)},
            [](Node& n) { const ET t = n.attr("output_type").et; infer_matmul_like(n, false, true, t == ET::dynamic ? n.in_et(0) : t); }, 4, 5);
        reg("GLU", "ie_internal_opset", {Ai("axis", -1), Ai("split_lengths", 0), As("glu_type", "Swish"), Ai("split_to_glu_idx", 0), At("output_type", ET::dynamic)},
            [](Node& n) {
                PShape s = n.in_shape(0);
                if (!s.rank_dynamic) s.dims[(size_t)norm_axis(n.attr_int("axis"), (int64_t)s.rank(), n)] = Dim(n.attr_int("split_lengths"));
                const ET t = n.attr("output_type").et;
                n.set_output(0, t == ET::dynamic ? n.in_et(0) : t, s);
            }, 1, 1);
        reg("PagedAttentionExtension", "extension", {Ab("write_kv_cache", true)},
            [](Node& n) {
                n.set_num_outputs(3);
                PShape out = n.in_shape(0);
                // value head size may differ from the key head size: [T, Hq * Sv]
                auto it = n.rt_info.find("num_k_heads");
                (void)it;
                n.set_output(0, n.in_et(0), out);
                n.set_output(1, n.in_et(0), PShape::dynamic(1));
                n.set_output(2, n.in_et(0), PShape::dynamic(1));
            }, 13, 28);
        reg("MOE", "internal", {As("expert_type", "GEMM3_SWIGLU"), Af("expert_alpha", 0, false), Af("expert_beta", 1, false), Ai("gate_idx", 0), As("activation_type", "SWISH")},
            infer_same, 6, 9);
        reg("SwiGLU_internal", "ie_internal_opset", {}, [](Node& n) {
                PShape s = n.in_shape(0);
                if (!s.rank_dynamic && s.dims.back().is_static()) s.dims.back() = Dim(s.dims.back().lo / 2);
                n.set_output(0, n.in_et(0), s);
            }, 1, 1);

        // aliases: the same implementation serves older/newer opset spellings found in IR files
        auto& r = OpRegistry::get();
        r.alias("Convert", "opset1", "opset16");
        r.alias("ShapeOf", "opset3", "opset17");
        r.alias("Gather", "opset8", "opset17");

        register_eval_functions();
        register_ext_ops();
        register_internal_ops();
        register_vision_ops();
        register_detection_ops();
        register_rest_ops();
        register_recurrent_ops();
        register_private_ops();
    });
}

}  // namespace ovc
