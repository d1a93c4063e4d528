// General-purpose transformations: ConstantFolding, NopElimination, BatchNorm folding, fp16
// compression of constants, weight compression to int4/int8, stateful <-> stateless conversion,
// FusedNames bookkeeping and the MOC-style pipeline that runs them in order.
//
// Reference counterparts: src/core/src/pass/constant_folding.cpp:105, src/common/transformations/src/
// transformations/common_optimizations/{nop_elimination,moc_transformations}.cpp,
// fp16_compression/compress_float_constants.cpp (:37-92 the keep-in-f32 rule),
// src/core/src/pass/{make_stateful,stateful_to_stateless}.cpp; the weight-compression algorithm itself
// lives outside the reference tree (NNCF) - this file emits the IR pattern that
// pattern_blocks/compressed_weights_block.cpp:17-75 recognises.

#include "pass.hpp"

namespace ovc {

using namespace pattern;

static NodePtr op(const std::string& type, const std::vector<Output>& in, const std::vector<std::pair<std::string, Attr>>& attrs = {},
                  const std::string& version = "") {
    return make_node(type, version, in, attrs);
}
static Output c_i64(const std::vector<int64_t>& v, bool scalar = false) { return make_constant_i64(v, ET::i64, scalar)->output(0); }

static bool is_low_precision(ET t) {
    return t == ET::u4 || t == ET::i4 || t == ET::nf4 || t == ET::f4e2m1 || t == ET::f8e4m3 || t == ET::f8e5m2 || t == ET::u8 || t == ET::i8 ||
           t == ET::u2 || t == ET::u3 || t == ET::u6 || t == ET::f8e8m0;
}

// A node belongs to a weight-decompression subgraph when it only consumes constants and starts at a
// low-precision (or f16-compressed, marked) constant: such subgraphs are kept so that plugins can fuse them.
static bool in_decompression_subgraph(const NodePtr& n, int depth = 0) {
    if (depth > 6) return false;
    if (n->rt_info.count("decompression_0")) return true;
    if (n->type == "Convert" && n->input_node(0)->is_constant()) {
        const Tensor& c = n->input_node(0)->constant;
        if (is_low_precision(c.et) && c.numel() >= 64) return true;
        if (n->input_node(0)->rt_info.count("keep_const_precision_0")) return true;
    }
    if (n->type == "Convert" || n->type == "Subtract" || n->type == "Multiply" || n->type == "Reshape" || n->type == "Transpose") {
        for (auto& i : n->inputs()) if (!i.node->is_constant() && in_decompression_subgraph(i.node, depth + 1)) return true;
        if (n->type == "Convert" && !n->input_node(0)->is_constant()) return in_decompression_subgraph(n->input_node(0), depth + 1);
    }
    return false;
}

// ------------------------------------------------------------------------------------ ConstantFolding
static bool constant_folding(const ModelPtr& m) {
    bool changed = false;
    for (auto& n : m->ordered_ops()) {
        if (n->is_constant() || n->is_parameter() || n->is_result() || !n->schema || !n->schema->eval || n->schema->has_side_effects) continue;
        if (!n->bodies.empty()) continue;
        if (n->rt_info.count("disable_constant_folding")) continue;
        bool used = false;
        for (auto& o : n->outs) if (!o.uses.empty()) used = true;
        if (!used) continue;
        // ShapeOf of a static shape folds even when its producer is not constant
        if (n->type == "ShapeOf" && n->in_shape(0).is_static()) {
            auto c = make_constant(from_i64(n->outs[0].et, Shape{(int64_t)n->in_shape(0).rank()}, n->in_shape(0).to_shape()));
            copy_runtime_info({n}, {c});
            replace_node(n, c);
            changed = true;
            continue;
        }
        if (n->num_inputs() == 0) continue;
        bool all_const = true;
        for (auto& i : n->inputs()) if (!i.node->is_constant()) { all_const = false; break; }
        if (!all_const) continue;
        if (in_decompression_subgraph(n)) continue;
        std::vector<Tensor> ins, outs(n->num_outputs());
        for (auto& i : n->inputs()) ins.push_back(i.node->constant);
        EvalContext ctx;
        try {
            if (!n->schema->eval(*n, ins, outs, ctx)) continue;
        } catch (const Error&) {
            continue;
        }
        for (size_t i = 0; i < outs.size(); ++i) {
            if (n->outs[i].uses.empty()) continue;
            // detach views from their source buffers so that the folded constant owns exactly its bytes
            Tensor t = outs[i];
            if (t.buf && t.et != ET::string && t.buf->size != t.byte_size()) {
                Tensor own(t.et, t.shape);
                std::memcpy(own.data(), t.data(), own.byte_size());
                t = own;
            }
            auto c = make_constant(t);
            c->name = n->num_outputs() == 1 ? n->name : n->name + "." + std::to_string(i);
            copy_runtime_info({n}, {c});
            replace_output(Output(n, i), c->output(0));
        }
        changed = true;
    }
    return changed;
}

// ------------------------------------------------------------------------------------ NopElimination
static bool nop_elimination(const ModelPtr& m) {
    bool changed = false;
    for (auto& n : m->ordered_ops()) {
        Output repl;
        if (n->type == "Convert" && n->in_et(0) == n->outs[0].et) repl = n->input(0);
        else if ((n->type == "Reshape" || n->type == "Squeeze" || n->type == "Unsqueeze" || n->type == "Broadcast") && n->in_shape(0).is_static() &&
                 n->outs[0].shape.is_static() && n->in_shape(0) == n->outs[0].shape)
            repl = n->input(0);
        else if (n->type == "Transpose") {
            std::vector<int64_t> order;
            if (get_constant_ints(n->input(1), order) && !order.empty()) {
                bool ident = true;
                for (size_t i = 0; i < order.size(); ++i) ident = ident && order[i] == (int64_t)i;
                if (ident) repl = n->input(0);
            }
        } else if (n->type == "Concat" && n->num_inputs() == 1) repl = n->input(0);
        else if ((n->type == "Add" || n->type == "Subtract") && n->input_node(1)->is_constant() && n->input_node(1)->constant.numel() == 1 &&
                 et_is_real(n->outs[0].et) && get_elem_f64(n->input_node(1)->constant, 0) == 0.0 && n->in_shape(0) == n->outs[0].shape)
            repl = n->input(0);
        else if ((n->type == "Multiply" || n->type == "Divide") && n->input_node(1)->is_constant() && n->input_node(1)->constant.numel() == 1 &&
                 get_elem_f64(n->input_node(1)->constant, 0) == 1.0 && n->in_shape(0) == n->outs[0].shape)
            repl = n->input(0);
        // Reshape(Reshape(x)) -> Reshape(x)
        if (!repl && n->type == "Reshape" && n->input_node(0)->type == "Reshape" && n->input_node(0)->outs[0].uses.size() == 1 && !n->attr_bool("special_zero")) {
            n->set_input(0, n->input_node(0)->input(0));
            n->validate_and_infer();
            changed = true;
            continue;
        }
        if (repl) {
            // a Result keeps its producer's tensor names
            if (repl.node->is_parameter() && !n->outs[0].uses.empty() && n->outs[0].uses[0].node->is_result() && repl.node->outs[0].uses.size() == 1) continue;
            replace_output(n->output(0), repl);
            changed = true;
        }
    }
    return changed;
}

// ------------------------------------------------------------------------------------ BatchNorm -> scale/shift, Conv+BN
static bool batch_norm_decomposition(const ModelPtr& m) {
    bool changed = false;
    for (auto& n : m->ordered_ops()) {
        if (n->type != "BatchNormInference") continue;
        bool all_const = true;
        for (size_t i = 1; i < 5; ++i) all_const = all_const && n->input_node(i)->is_constant();
        if (!all_const || n->in_shape(0).rank_dynamic) continue;
        auto g = to_f32(n->input_node(1)->constant), b = to_f32(n->input_node(2)->constant), mean = to_f32(n->input_node(3)->constant), var = to_f32(n->input_node(4)->constant);
        const float eps = float(n->attr_float("epsilon"));
        const size_t C = g.size();
        std::vector<float> scale(C), shift(C);
        for (size_t c = 0; c < C; ++c) { scale[c] = g[c] / std::sqrt(var[c] + eps); shift[c] = b[c] - mean[c] * scale[c]; }
        Shape bs(n->in_shape(0).rank(), 1);
        bs[1] = (int64_t)C;
        const ET et = n->outs[0].et;
        NodePtr prod = n->input_node(0);
        // fold into a preceding convolution with constant weights
        if ((prod->type == "Convolution") && prod->input_node(1)->is_constant() && prod->outs[0].uses.size() == 1) {
            const Tensor& w = prod->input_node(1)->constant;
            auto wf = to_f32(w);
            const int64_t per = w.numel() / (int64_t)C;
            for (size_t c = 0; c < C; ++c) for (int64_t i = 0; i < per; ++i) wf[c * (size_t)per + (size_t)i] *= scale[c];
            auto nw = make_constant(from_f32(w.et, w.shape, wf));
            nw->name = prod->input_node(1)->name;
            auto conv = prod->clone_with_new_inputs({prod->input(0), nw->output(0)});
            conv->name = prod->name;
            auto add = op("Add", {conv->output(0), make_constant(from_f32(et, bs, shift))->output(0)});
            copy_runtime_info({prod, n}, {conv, add});
            replace_node(n, add);
        } else {
            auto mul = op("Multiply", {n->input(0), make_constant(from_f32(et, bs, scale))->output(0)});
            auto add = op("Add", {mul->output(0), make_constant(from_f32(et, bs, shift))->output(0)});
            copy_runtime_info({n}, {mul, add});
            replace_node(n, add);
        }
        changed = true;
    }
    return changed;
}

// ------------------------------------------------------------------------------------ fp16 compression of constants
bool compress_model_to_f16(const ModelPtr& m) {
    // Models that already carry compressed weights or FakeQuantize are left alone
    for (auto& n : m->ordered_ops()) {
        if (n->type == "FakeQuantize" || n->type == "FakeConvert") return false;
        if (n->type == "Convert" && n->input_node(0)->is_constant() && is_low_precision(n->input_node(0)->constant.et) && n->input_node(0)->constant.numel() >= 64) return false;
    }
    bool changed = false;
    for (auto& n : m->ordered_ops()) {
        if (!n->is_constant() || (n->constant.et != ET::f32 && n->constant.et != ET::f64)) continue;
        if (n->rt_info.count("disable_fp16_compression_0") || n->rt_info.count("keep_const_precision_0")) continue;
        // constants that feed shape-like ports stay as they are
        bool data_use = false;
        for (auto& u : n->outs[0].uses) {
            const std::string& t = u.node->type;
            const bool shape_port = (t == "Reshape" && u.input == 1) || (t == "Interpolate" && u.input > 0) || (t == "Range") || (t == "Broadcast" && u.input > 0) ||
                                    (t == "Tile" && u.input == 1) || (t == "Pad" && u.input > 0 && u.input < 3);
            if (!shape_port) data_use = true;
        }
        if (!data_use) continue;
        const int64_t cnt = n->constant.numel();
        if (cnt == 0) continue;
        // keep in full precision when too many values would be lost (out of f16 range or large relative error)
        auto v = to_f32(n->constant);
        int64_t bad = 0;
        std::vector<uint16_t> h((size_t)cnt);
        for (int64_t i = 0; i < cnt; ++i) {
            const float f = v[(size_t)i];
            h[(size_t)i] = f32_to_f16(f);
            const float back = f16_to_f32(h[(size_t)i]);
            if (std::isfinite(f) && (!std::isfinite(back) || (f != 0.f && back == 0.f) || std::fabs(back - f) > 1e-4f * std::max(1.f, std::fabs(f)) * 10.f)) ++bad;
        }
        if (double(bad) / double(cnt) >= 0.75) continue;
        Tensor t(ET::f16, n->constant.shape);
        std::memcpy(t.data(), h.data(), (size_t)cnt * 2);
        auto c16 = make_constant(t);
        c16->name = n->name + "_compressed";
        auto cvt = op("Convert", {c16->output(0)}, {{"destination_type", Attr::Type(n->constant.et)}});
        cvt->name = n->name;
        cvt->rt_info["decompression_0"] = Attr::Str("");
        cvt->outs[0].names = n->outs[0].names;
        replace_output(n->output(0), cvt->output(0));
        changed = true;
    }
    return changed;
}

// ------------------------------------------------------------------------------------ weight compression (int4 / int8)
// mode: "int4_asym", "int4_sym", "int8_asym", "int8_sym". Emits
//   Const(u4|i4|u8|i8)[N, G, gs] -> Convert(f16) -> [Subtract(Convert(Const zp [N, G, 1]))] -> Multiply(Const f16 [N, G, 1])
//   -> Reshape [N, K] -> [Convert(f32)] -> MatMul(transpose_b = true)
bool compress_weights(const ModelPtr& m, const std::string& mode, int64_t group_size, double ratio, bool all_layers) {
    (void)ratio;
    const bool int4 = mode.rfind("int4", 0) == 0;
    const bool sym = mode.find("sym") != std::string::npos && mode.find("asym") == std::string::npos;
    bool changed = false;
    auto order = m->ordered_ops();
    // the last MatMul (LM head) and embeddings stay int8 unless all_layers is set, like the default NNCF policy
    NodePtr last_matmul;
    for (auto& n : order) if (n->type == "MatMul") last_matmul = n;
    for (auto& n : order) {
        if (n->type != "MatMul") continue;
        NodePtr wnode = n->input_node(1);
        NodePtr cvt_after;
        if (wnode->type == "Convert" && wnode->input_node(0)->is_constant()) { cvt_after = wnode; wnode = wnode->input_node(0); }
        if (!wnode->is_constant() || !et_is_real(wnode->constant.et) || wnode->constant.shape.size() != 2) continue;
        if (wnode->constant.numel() < 4096) continue;
        const bool tb = n->attr_bool("transpose_b");
        Tensor w = wnode->constant;
        auto wf = to_f32(w);
        int64_t N = tb ? w.shape[0] : w.shape[1], K = tb ? w.shape[1] : w.shape[0];
        if (!tb) {   // store as [N, K]
            std::vector<float> t((size_t)(N * K));
            for (int64_t k = 0; k < K; ++k) for (int64_t j = 0; j < N; ++j) t[(size_t)(j * K + k)] = wf[(size_t)(k * N + j)];
            wf.swap(t);
        }
        const bool use4 = int4 && (all_layers || n != last_matmul);
        int64_t gs = (use4 && group_size > 0 && K % group_size == 0) ? group_size : K;
        const int64_t G = K / gs;
        const int levels = use4 ? 15 : 255;
        const ET qt = use4 ? (sym ? ET::i4 : ET::u4) : (sym ? ET::i8 : ET::u8);
        Tensor q(qt, Shape{N, G, gs}), scale(ET::f16, Shape{N, G, 1}), zp(qt, Shape{N, G, 1});
        for (int64_t r = 0; r < N; ++r) for (int64_t g = 0; g < G; ++g) {
            const float* p = wf.data() + r * K + g * gs;
            float mn = p[0], mx = p[0];
            for (int64_t i = 1; i < gs; ++i) { mn = std::min(mn, p[i]); mx = std::max(mx, p[i]); }
            float s, z;
            if (sym) {
                const float amax = std::max(std::fabs(mn), std::fabs(mx));
                s = amax / float(use4 ? 7 : 127);
                z = 0.f;
            } else {
                s = (mx - mn) / float(levels);
                z = 0.f;
            }
            if (s < 1e-8f) s = 1e-8f;
            s = f16_to_f32(f32_to_f16(s));
            if (s <= 0.f) s = 6e-8f;
            if (!sym) z = std::min(float(levels), std::max(0.f, std::nearbyint(-mn / s)));
            set_elem_f64(scale, r * G + g, s);
            set_elem_f64(zp, r * G + g, z);
            for (int64_t i = 0; i < gs; ++i) {
                float v = std::nearbyint(p[i] / s + z);
                if (sym) v = std::min(float(use4 ? 7 : 127), std::max(float(use4 ? -8 : -128), v));
                else v = std::min(float(levels), std::max(0.f, v));
                set_elem_f64(q, (r * G + g) * gs + i, v);
            }
        }
        auto qc = make_constant(q);
        qc->name = wnode->name;
        Output cur = op("Convert", {qc->output(0)}, {{"destination_type", Attr::Type(ET::f16)}})->output(0);
        cur.node->rt_info["decompression_0"] = Attr::Str("");
        if (!sym) {
            auto zc = op("Convert", {make_constant(zp)->output(0)}, {{"destination_type", Attr::Type(ET::f16)}});
            cur = op("Subtract", {cur, zc->output(0)})->output(0);
        }
        cur = op("Multiply", {cur, make_constant(scale)->output(0)})->output(0);
        if (G > 1 || true) cur = op("Reshape", {cur, c_i64({N, K})}, {{"special_zero", Attr::Bool(false)}})->output(0);
        const ET act = n->in_et(0);
        if (act != ET::f16) cur = op("Convert", {cur}, {{"destination_type", Attr::Type(act)}})->output(0);
        n->set_input(1, cur);
        n->set_attr("transpose_b", Attr::Bool(true));
        n->validate_and_infer();
        changed = true;
    }
    // embeddings (Gather over a float table) -> int8 per-row
    for (auto& n : order) {
        if (n->type != "Gather") continue;
        NodePtr wnode = n->input_node(0);
        if (!wnode->is_constant() || !et_is_real(wnode->constant.et) || wnode->constant.shape.size() != 2 || wnode->constant.numel() < 4096) continue;
        const Tensor& w = wnode->constant;
        const int64_t N = w.shape[0], K = w.shape[1];
        auto wf = to_f32(w);
        Tensor q(ET::u8, Shape{N, K}), scale(ET::f16, Shape{N, 1}), zp(ET::u8, Shape{N, 1});
        for (int64_t r = 0; r < N; ++r) {
            const float* p = wf.data() + r * K;
            float mn = p[0], mx = p[0];
            for (int64_t i = 1; i < K; ++i) { mn = std::min(mn, p[i]); mx = std::max(mx, p[i]); }
            float s = f16_to_f32(f32_to_f16(std::max((mx - mn) / 255.f, 1e-8f)));
            if (s <= 0.f) s = 6e-8f;
            const float z = std::min(255.f, std::max(0.f, std::nearbyint(-mn / s)));
            set_elem_f64(scale, r, s);
            set_elem_f64(zp, r, z);
            for (int64_t i = 0; i < K; ++i) q.data()[r * K + i] = uint8_t(std::min(255.f, std::max(0.f, std::nearbyint(p[i] / s + z))));
        }
        auto qc = make_constant(q);
        qc->name = wnode->name;
        Output cur = op("Convert", {qc->output(0)}, {{"destination_type", Attr::Type(ET::f16)}})->output(0);
        cur.node->rt_info["decompression_0"] = Attr::Str("");
        cur = op("Subtract", {cur, op("Convert", {make_constant(zp)->output(0)}, {{"destination_type", Attr::Type(ET::f16)}})->output(0)})->output(0);
        cur = op("Multiply", {cur, make_constant(scale)->output(0)})->output(0);
        if (n->in_et(0) != ET::f16) cur = op("Convert", {cur}, {{"destination_type", Attr::Type(n->in_et(0))}})->output(0);
        n->set_input(0, cur);
        n->validate_and_infer();
        changed = true;
    }
    if (changed) m->validate();
    return changed;
}

// ------------------------------------------------------------------------------------ stateful <-> stateless
bool make_stateful(const ModelPtr& m, const std::vector<std::pair<std::string, std::string>>& pairs) {
    bool changed = false;
    auto find_by_tensor_name = [&](const std::vector<NodePtr>& v, const std::string& nm) -> NodePtr {
        for (auto& n : v) if (n->name == nm || n->outs[0].names.count(nm)) return n;
        return nullptr;
    };
    for (auto& pr : pairs) {
        NodePtr p = find_by_tensor_name(m->params, pr.first), r = find_by_tensor_name(m->results, pr.second);
        OVC_CHECK(p && r, "MakeStateful: cannot find parameter '" << pr.first << "' / result '" << pr.second << "'");
        const std::string var_id = pr.first + pr.second;
        // the initial value is a zero tensor whose dynamic dims are taken as 0
        Shape z;
        const PShape& ps = p->outs[0].shape;
        OVC_CHECK(!ps.rank_dynamic, "MakeStateful: parameter '" << pr.first << "' has a dynamic rank");
        for (auto& d : ps.dims) z.push_back(d.is_static() ? d.lo : 0);
        Tensor init(p->outs[0].et, z);
        if (init.data()) std::memset(init.data(), 0, init.byte_size());
        auto rv = op("ReadValue", {make_constant(init)->output(0)},
                     {{"variable_id", Attr::Str(var_id)}, {"variable_type", Attr::Type(p->outs[0].et)}, {"variable_shape", Attr::Shape_(ps)}}, "opset6");
        rv->name = p->name;
        replace_output(p->output(0), rv->output(0));
        auto as = op("Assign", {r->input(0)}, {{"variable_id", Attr::Str(var_id)}}, "opset6");
        m->remove_parameter(p);
        m->remove_result(r);
        m->add_sinks({as});
        changed = true;
    }
    if (changed) m->validate();
    return changed;
}

bool stateful_to_stateless(const ModelPtr& m) {
    // ReadValue/Assign pairs become Parameter/Result pairs; names follow the
    // "past_key_values.N.keypresent.N.key" convention when the variable id uses it
    bool changed = false;
    std::map<std::string, NodePtr> reads, assigns;
    for (auto& n : m->ordered_ops()) {
        if (n->type == "ReadValue") reads[n->attr_str("variable_id")] = n;
        if (n->type == "Assign") assigns[n->attr_str("variable_id")] = n;
    }
    // "past_key_values.3.keypresent.3.key" -> ("past_key_values.3.key", "present.3.key"); plain string search on purpose:
    // std::regex must not be used in this module (its template code clashes with the copy exported by libtorch).
    auto split_kv_name = [](const std::string& id, std::string& in_name, std::string& out_name) {
        if (id.rfind("past_key_values.", 0) != 0) return false;
        const size_t pos = id.find("present.");
        if (pos == std::string::npos || pos == 0) return false;
        in_name = id.substr(0, pos);
        out_name = id.substr(pos);
        return true;
    };
    for (auto& kv : reads) {
        auto it = assigns.find(kv.first);
        if (it == assigns.end()) continue;
        std::string in_name = kv.first + "_in", out_name = kv.first + "_out";
        split_kv_name(kv.first, in_name, out_name);
        NodePtr rv = kv.second, as = it->second;
        auto p = make_parameter(rv->outs[0].et, rv->outs[0].shape, in_name);

        replace_output(rv->output(0), p->output(0));
        auto r = make_result(as->input(0));
        r->name = out_name;
        r->outs[0].names.insert(out_name);
        m->add_parameters({p});
        m->add_results({r});
        m->remove_sink(as);
        changed = true;
    }
    if (changed) m->validate();
    return changed;
}

// ------------------------------------------------------------------------------------ names
static bool init_node_info(const ModelPtr& m) {
    for (auto& n : m->ordered_ops()) if (!n->rt_info.count("fused_names_0")) n->rt_info["fused_names_0"] = Attr::Str(n->name);
    return false;
}
static bool fused_names_cleanup(const ModelPtr& m) {
    for (auto& n : m->ordered_ops()) n->rt_info.erase("fused_names_0");
    return false;
}

// ------------------------------------------------------------------------------------ ConvertPrecision (whole graph)
static bool convert_precision(const ModelPtr& m, ET from, ET to) {
    bool changed = false;
    for (auto& n : m->ordered_ops()) {
        // nodes of a precision-sensitive island (marked by MarkSugraphsToKeepInMixedPrecision or by hand) keep their type
        if (n->rt_info.count("disable_fp16_compression_0") && !n->is_parameter()) continue;
        if (n->is_parameter() && n->attr("element_type").et == from) { n->set_attr("element_type", Attr::Type(to)); changed = true; }
        else if (n->is_constant() && n->constant.et == from) { n->constant = convert_tensor(n->constant, to); changed = true; }
        else if (n->type == "Convert" && n->attr("destination_type").et == from) { n->set_attr("destination_type", Attr::Type(to)); changed = true; }
        else {
            for (const char* k : {"output_type", "index_element_type", "variable_type"})
                if (n->has_attr(k) && n->attr(k).kind == Attr::TYPE && n->attr(k).et == from) { n->set_attr(k, Attr::Type(to)); changed = true; }
        }
    }
    if (changed) m->validate();
    return changed;
}

// forward declarations of the LLM passes (transform_llm.cpp)
std::shared_ptr<MatcherPass> make_rms_fusion();
std::shared_ptr<MatcherPass> make_rope_fusion();
std::shared_ptr<MatcherPass> make_rope_fusion_interleaved();
std::shared_ptr<MatcherPass> make_rope_fusion_partial();
std::shared_ptr<MatcherPass> make_rope_fusion_qwen();
std::shared_ptr<MatcherPass> make_rope_fusion_chatglm();
std::shared_ptr<MatcherPass> make_lora_fusion();
std::shared_ptr<MatcherPass> make_matmul_to_fc();
std::shared_ptr<MatcherPass> make_fc_to_compressed();
std::shared_ptr<MatcherPass> make_swiglu_fusion();
std::shared_ptr<MatcherPass> make_sdpa_fusion();
bool fuse_moe_experts(const ModelPtr& m);

std::shared_ptr<ModelPass> make_pass(const std::string& name, const AttrMap& options) {
    auto lam = [&](std::function<bool(const ModelPtr&)> f) { return std::make_shared<LambdaPass>(name, std::move(f)); };
    auto wrap = [&](std::shared_ptr<MatcherPass> mp) { auto g = std::make_shared<GraphRewrite>(); g->name = name; g->add(std::move(mp)); return g; };
    auto opt_s = [&](const char* k, const std::string& d) { auto it = options.find(k); return it == options.end() ? d : (it->second.kind == Attr::STR ? it->second.s : it->second.to_string()); };
    auto opt_i = [&](const char* k, int64_t d) { auto it = options.find(k); return it == options.end() ? d : it->second.i; };
    if (name == "ConstantFolding") return lam(constant_folding);
    if (name == "NopElimination") return lam(nop_elimination);
    if (name == "BatchNormDecomposition") return lam(batch_norm_decomposition);
    if (name == "Validate") return lam([](const ModelPtr& m) { m->validate(); return false; });
    if (name == "InitNodeInfo") return lam(init_node_info);
    if (name == "FusedNamesCleanup") return lam(fused_names_cleanup);
    if (name == "CompressFloatConstants") return lam(compress_model_to_f16);
    if (name == "ConvertFP32ToFP16") return lam([](const ModelPtr& m) { return convert_precision(m, ET::f32, ET::f16); });
    if (name == "ConvertPrecision") { const ET f = et_from_name(opt_s("from", "f32")), t = et_from_name(opt_s("to", "f16")); return lam([f, t](const ModelPtr& m) { return convert_precision(m, f, t); }); }
    if (name == "StatefulToStateless") return lam(stateful_to_stateless);
    if (name == "CompressWeights") { const std::string mode = opt_s("mode", "int4_asym"); const int64_t gs = opt_i("group_size", 128); const bool all = opt_i("all_layers", 0) != 0;
        return lam([mode, gs, all](const ModelPtr& m) { return compress_weights(m, mode, gs, 1.0, all); }); }
    if (name == "RMSFusion") return wrap(make_rms_fusion());
    if (name == "RoPEFusion") {     // half-rotate, interleaved, the partial-rotary wrapper around either, then the fused-QKV forms of Qwen and ChatGLM
        auto g = std::make_shared<GraphRewrite>();
        g->name = name;
        g->add(make_rope_fusion());
        g->add(make_rope_fusion_interleaved());
        g->add(make_rope_fusion_partial());
        g->add(make_rope_fusion_qwen());
        g->add(make_rope_fusion_chatglm());
        return g;
    }
    if (name == "LoraSubgraphFusion") return wrap(make_lora_fusion());
    if (name == "ConvertMatMulToFullyConnected") return wrap(make_matmul_to_fc());
    if (name == "ConvertFullyConnectedToFullyConnectedCompressed") return wrap(make_fc_to_compressed());
    if (name == "GLUFusion") return wrap(make_swiglu_fusion());
    if (name == "SDPAFusion") return wrap(make_sdpa_fusion());
    if (name == "FuseMOEExperts") return lam(fuse_moe_experts);
    if (name == "SDPAToPagedAttention") { AttrMap o = options; return lam([o](const ModelPtr& m) { return sdpa_to_paged_attention(m, o); }); }
    if (name == "MOCTransformations") return lam([](const ModelPtr& m) { run_moc_transformations(m); return true; });
    throw Error("unknown pass '" + name + "'");
}

std::vector<std::string> available_passes() {
    return {"ConstantFolding", "NopElimination", "BatchNormDecomposition", "Validate", "InitNodeInfo", "FusedNamesCleanup", "CompressFloatConstants",
            "ConvertFP32ToFP16", "ConvertPrecision", "StatefulToStateless", "CompressWeights", "RMSFusion", "RoPEFusion",
            "ConvertMatMulToFullyConnected", "ConvertFullyConnectedToFullyConnectedCompressed", "GLUFusion", "SDPAFusion", "FuseMOEExperts",
            "SDPAToPagedAttention", "MOCTransformations", "LoraSubgraphFusion"};
}

void run_moc_transformations(const ModelPtr& m, bool cf) {
    PassManager pm;
    pm.add(make_pass("InitNodeInfo"));
    if (cf) pm.add(make_pass("ConstantFolding"));
    pm.add(make_pass("NopElimination"));
    pm.add(make_pass("BatchNormDecomposition"));
    if (cf) pm.add(make_pass("ConstantFolding"));
    pm.add(make_pass("SDPAFusion"));
    pm.add(make_pass("Validate"));
    pm.run(m);
}

void run_llm_fusions(const ModelPtr& m) {
    PassManager pm;
    pm.add(make_pass("RMSFusion"));
    pm.add(make_pass("RoPEFusion"));
    pm.add(make_pass("ConvertMatMulToFullyConnected"));
    pm.add(make_pass("ConvertFullyConnectedToFullyConnectedCompressed"));
    pm.add(make_pass("GLUFusion"));
    pm.add(make_pass("Validate"));
    pm.run(m);
}

}  // namespace ovc
