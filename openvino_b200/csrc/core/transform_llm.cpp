// LLM graph fusions and the SDPA -> PagedAttention rewrite.
//
// Reference counterparts (src/common/transformations/src/transformations/common_optimizations/):
// rms_fusion.cpp:21-173, fuse_rotary_positional_embeddings.cpp:180-262 (half-rotate form), glu_fusion.cpp,
// sdpa_fusion.cpp, fuse_moe_experts.cpp / moe_op_fusion.cpp, op_conversions/convert_fc_to_compressed.cpp:23-227,
// pattern_blocks/compressed_weights_block.cpp:17-75, and src/core/src/pass/sdpa_to_paged_attention.cpp:70-220
// with sdpa_to_paged_attention/state_management_pattern.cpp. The patterns here are written against the
// graphs this framework's own PyTorch frontend and model builders produce.
#include "pass.hpp"

namespace ovc {

using namespace pattern;

static NodePtr op(const std::string& type, const std::vector<Output>& in, const std::vector<std::pair<std::string, Attr>>& attrs = {},
                  const std::string& version = "") {
    return make_node(type, version, in, attrs);
}
static Output c_i64(const std::vector<int64_t>& v, bool scalar = false) { return make_constant_i64(v, ET::i64, scalar)->output(0); }
static Output c_i32(const std::vector<int64_t>& v, bool scalar = false) { return make_constant_i64(v, ET::i32, scalar)->output(0); }

static bool const_scalar_equals(const Output& o, double v, double tol = 1e-6) {
    Tensor t;
    if (!try_constant_value(o, t) || t.numel() != 1 || t.et == ET::string) return false;
    return std::fabs(get_elem_f64(t, 0) - v) <= tol * std::max(1.0, std::fabs(v));
}
static ValuePredicate scalar_eq(double v) { return [v](const Output& o) { return const_scalar_equals(o, v); }; }

// ------------------------------------------------------------------------------------ RMSFusion
// x * 1/sqrt(mean(x^2, -1) + eps) [* gamma]  ->  RMS(x, gamma)
std::shared_ptr<MatcherPass> make_rms_fusion() {
    auto x = any_input();
    auto xc = optional({"Convert"}, x);                       // fp32 island inside a half-precision model
    auto pow2 = any_of({wrap_type({"Power"}, {xc, wrap_const(scalar_eq(2.0))}), wrap_type({"Multiply"}, {xc, xc})});
    auto mean = wrap_type({"ReduceMean"}, {pow2, wrap_const()});
    auto eps = wrap_const();
    auto add = wrap_type({"Add"}, {mean, eps});
    auto sqrt = wrap_type({"Sqrt"}, {add});
    auto inv = any_of({wrap_type({"Divide"}, {wrap_const(scalar_eq(1.0)), sqrt}), wrap_type({"Power"}, {sqrt, wrap_const(scalar_eq(-1.0))}),
                       wrap_type({"Power"}, {add, wrap_const(scalar_eq(-0.5))})});
    auto mul1 = any_of({wrap_type({"Multiply"}, {xc, inv}), wrap_type({"Divide"}, {xc, sqrt})});
    auto mul1c = optional({"Convert"}, mul1);
    auto gamma = wrap_const();
    auto gamma_c = optional({"Convert"}, gamma);
    auto mul2 = wrap_type({"Multiply"}, {mul1c, gamma_c});
    auto root = any_of({mul2, mul1c});
    // a bare normalisation (no gamma) that is itself multiplied by gamma later must not match first: roots
    // are tried at every node, so the gamma form is preferred by checking the single consumer below.
    return std::make_shared<MatcherPass>("RMSFusion", root, [=](Matcher& m) {
        const bool with_gamma = m.has(mul2);
        const Output xin = m.at(x);
        if (xin.shape().rank_dynamic) return false;
        std::vector<int64_t> axes;
        if (!get_constant_ints(m.node(mean)->input(1), axes) || axes.size() != 1) return false;
        const int64_t rank = (int64_t)xin.shape().rank();
        if (axes[0] != -1 && axes[0] != rank - 1) return false;
        if (!m.node(mean)->attr_bool("keep_dims")) return false;
        Tensor et;
        if (!try_constant_value(m.at(eps), et) || et.numel() != 1) return false;
        NodePtr rootn = m.match_root();
        if (!with_gamma) {
            // leave it to the gamma form when the only consumer is a Multiply by a constant
            auto& uses = rootn->outs[0].uses;
            if (uses.size() == 1 && uses[0].node->type == "Multiply") {
                Node* c = uses[0].node;
                NodePtr other = c->input_node(uses[0].input == 0 ? 1 : 0);
                if (other->is_constant() || (other->type == "Convert" && other->input_node(0)->is_constant())) return false;
            }
        }
        Output g;
        if (with_gamma) {
            g = m.at(gamma);
            const PShape& gs = g.shape();
            if (!gs.is_static()) return false;
            // gamma must be a vector over the last axis
            int64_t n = 1;
            for (auto& d : gs.dims) n *= d.lo;
            if (!xin.shape().dims.back().is_static() || n != xin.shape().dims.back().lo) return false;
            if (gs.rank() != 1) g = op("Reshape", {g, c_i64({n})}, {{"special_zero", Attr::Bool(false)}})->output(0);
            if (g.et() != xin.et()) g = op("Convert", {g}, {{"destination_type", Attr::Type(xin.et())}})->output(0);
        } else {
            const int64_t n = xin.shape().dims.back().is_static() ? xin.shape().dims.back().lo : 1;
            g = make_constant(from_f32(xin.et(), Shape{n}, std::vector<float>((size_t)n, 1.0f)))->output(0);
        }
        auto rms = op("RMS", {xin, g}, {{"epsilon", Attr::Float(get_elem_f64(et, 0))}, {"output_type", Attr::Type(rootn->outs[0].et)},
                                        {"elementwise_affine", Attr::Bool(with_gamma)}});
        copy_runtime_info(m.matched_nodes(), {rms});
        replace_node(rootn, rms);
        return true;
    });
}

// ------------------------------------------------------------------------------------ RoPEFusion (half rotate)
// x * cos + concat(-x[..., h:], x[..., :h]) * sin  ->  RoPE(x, cos, sin)
std::shared_ptr<MatcherPass> make_rope_fusion() {
    auto x = any_input(rank_equals(4));
    auto cos = any_input();
    auto sin = any_input();
    auto slice_hi = wrap_type({"Slice", "StridedSlice"}, {x, any_input(), any_input(), any_input(), any_input()});
    auto slice_lo = wrap_type({"Slice", "StridedSlice"}, {x, any_input(), any_input(), any_input(), any_input()});
    auto neg = any_of({wrap_type({"Negative"}, {slice_hi}), wrap_type({"Multiply"}, {slice_hi, wrap_const(scalar_eq(-1.0))})});
    auto cat = wrap_type({"Concat"}, {neg, slice_lo});
    auto mul_cos = wrap_type({"Multiply"}, {x, cos});
    auto mul_sin = wrap_type({"Multiply"}, {cat, sin});
    auto add = wrap_type({"Add"}, {mul_cos, mul_sin});
    return std::make_shared<MatcherPass>("RoPEFusion", add, [=](Matcher& m) {
        const Output xin = m.at(x);
        const PShape& xs = xin.shape();
        if (!xs.dims[3].is_static()) return false;
        const int64_t S = xs.dims[3].lo, half = S / 2;
        auto check_slice = [&](const NodePtr& s, int64_t b, int64_t e_min) {
            std::vector<int64_t> vb, ve, vs, va;
            if (!get_constant_ints(s->input(1), vb) || !get_constant_ints(s->input(2), ve) || !get_constant_ints(s->input(3), vs)) return false;
            if (s->type == "Slice") {
                if (s->num_inputs() < 5 || !get_constant_ints(s->input(4), va) || va.size() != 1) return false;
                if (va[0] != -1 && va[0] != 3) return false;
                return vb.size() == 1 && vb[0] == b && ve[0] >= e_min && vs[0] == 1;
            }
            return false;
        };
        if (!check_slice(m.node(slice_hi), half, S) || !check_slice(m.node(slice_lo), 0, half)) return false;
        // a table laid out [1, positions, 1, S] belongs to x in [B, L, H, S] order: RoPE reads x as [B, H, L, S], so leave that form alone
        const PShape& cshape = m.at(cos).shape();
        if (!cshape.rank_dynamic && cshape.rank() == 4 && cshape.dims[2].is_static() && cshape.dims[2].lo == 1 && !(cshape.dims[1].is_static() && cshape.dims[1].lo == 1)) return false;
        if (m.node(slice_lo)->input(2).node->is_constant()) { std::vector<int64_t> ve; get_constant_ints(m.node(slice_lo)->input(2), ve); if (ve[0] != half) return false; }
        if (m.node(cat)->attr_int("axis") != -1 && m.node(cat)->attr_int("axis") != 3) return false;
        auto rope = op("RoPE", {xin, m.at(cos), m.at(sin)}, {{"rotary_ndims", Attr::Int(S)}, {"head_size", Attr::Int(S)},
                                                             {"head_cnt", Attr::Int(xs.dims[1].is_static() ? xs.dims[1].lo : 0)}});
        copy_runtime_info(m.matched_nodes(), {rope});
        replace_node(m.match_root(), rope);
        return true;
    });
}

// RoPE, interleaved (GPT-J "rotate every two") form:
//   x * cos + reshape(concat(unsqueeze(-x[..., 1::2]), unsqueeze(x[..., 0::2]), -1), shape(x)) * sin  ->  RoPE(x, cos, sin), is_interleaved
// (fuse_rotary_positional_embeddings.cpp, RoPEFusionGPTJ, in the reference).
std::shared_ptr<MatcherPass> make_rope_fusion_interleaved() {
    auto x = any_input(rank_equals(4));
    auto cos = any_input();
    auto sin = any_input();
    auto odd = wrap_type({"Slice"}, {x, any_input(), any_input(), any_input(), any_input()});
    auto even = wrap_type({"Slice"}, {x, any_input(), any_input(), any_input(), any_input()});
    auto neg = any_of({wrap_type({"Negative"}, {odd}), wrap_type({"Multiply"}, {odd, wrap_const(scalar_eq(-1.0))})});
    auto u_neg = wrap_type({"Unsqueeze"}, {neg, any_input()});
    auto u_even = wrap_type({"Unsqueeze"}, {even, any_input()});
    auto cat = wrap_type({"Concat"}, {u_neg, u_even});
    auto flat = wrap_type({"Reshape"}, {cat, any_input()});
    auto mul_cos = wrap_type({"Multiply"}, {x, cos});
    auto mul_sin = wrap_type({"Multiply"}, {flat, sin});
    auto add = wrap_type({"Add"}, {mul_cos, mul_sin});
    return std::make_shared<MatcherPass>("RoPEFusionInterleaved", add, [=](Matcher& m) {
        const Output xin = m.at(x);
        const PShape& xs = xin.shape();
        if (!xs.dims[3].is_static() || xs.dims[3].lo % 2) return false;
        const int64_t S = xs.dims[3].lo;
        auto strided = [&](const NodePtr& sl, int64_t start) {
            std::vector<int64_t> vb, ve, vs, va;
            if (!get_constant_ints(sl->input(1), vb) || !get_constant_ints(sl->input(2), ve) || !get_constant_ints(sl->input(3), vs) ||
                !get_constant_ints(sl->input(4), va)) return false;
            return vb.size() == 1 && vb[0] == start && vs[0] == 2 && ve[0] >= S - 1 + start && (va[0] == 3 || va[0] == -1);
        };
        if (!strided(m.node(odd), 1) || !strided(m.node(even), 0)) return false;
        const int64_t cat_axis = m.node(cat)->attr_int("axis");
        if (cat_axis != -1 && cat_axis != 4) return false;
        if (!(m.node(flat)->output(0).shape() == xs)) return false;
        auto rope = op("RoPE", {xin, m.at(cos), m.at(sin)}, {{"is_interleaved", Attr::Bool(true)}, {"rotary_ndims", Attr::Int(S)}, {"head_size", Attr::Int(S)},
                                                             {"head_cnt", Attr::Int(xs.dims[1].is_static() ? xs.dims[1].lo : 0)}});
        copy_runtime_info(m.matched_nodes(), {rope});
        replace_node(m.match_root(), rope);
        return true;
    });
}

// Partial rotary embedding (GPT-NeoX / Phi: only the first rotary_ndims of the head are rotated):
//   concat(RoPE(x[..., :r], cos, sin), x[..., r:], -1)  ->  RoPE(x, cos, sin) with rotary_ndims = r
std::shared_ptr<MatcherPass> make_rope_fusion_partial() {
    auto x = any_input(rank_equals(4));
    auto head = wrap_type({"Slice"}, {x, any_input(), any_input(), any_input(), any_input()});
    auto tail = wrap_type({"Slice"}, {x, any_input(), any_input(), any_input(), any_input()});
    auto rope_in = wrap_type({"RoPE"}, {head, any_input(), any_input()});
    auto cat = wrap_type({"Concat"}, {rope_in, tail});
    return std::make_shared<MatcherPass>("RoPEFusionPartial", cat, [=](Matcher& m) {
        const Output xin = m.at(x);
        const PShape& xs = xin.shape();
        if (!xs.dims[3].is_static()) return false;
        const int64_t S = xs.dims[3].lo;
        NodePtr r = m.node(rope_in);
        if (r->attr_bool("input_trans0213") || r->attr_bool("output_trans0213") || r->attr_int("slice_stop") > r->attr_int("slice_start")) return false;
        const int64_t rot = r->attr_int("rotary_ndims");
        auto range = [&](const NodePtr& sl, int64_t b, int64_t e) {
            std::vector<int64_t> vb, ve, vs, va;
            if (!get_constant_ints(sl->input(1), vb) || !get_constant_ints(sl->input(2), ve) || !get_constant_ints(sl->input(3), vs) ||
                !get_constant_ints(sl->input(4), va)) return false;
            return vb.size() == 1 && vb[0] == b && (ve[0] == e || (e == S && ve[0] >= S)) && vs[0] == 1 && (va[0] == 3 || va[0] == -1);
        };
        if (rot <= 0 || rot >= S || !range(m.node(head), 0, rot) || !range(m.node(tail), rot, S)) return false;
        const int64_t cat_axis = m.node(cat)->attr_int("axis");
        if (cat_axis != -1 && cat_axis != 3) return false;
        auto rope = op("RoPE", {xin, r->input(1), r->input(2)}, {{"is_interleaved", Attr::Bool(r->attr_bool("is_interleaved"))}, {"rotary_ndims", Attr::Int(rot)},
                                                                {"head_size", Attr::Int(S)}, {"head_cnt", Attr::Int(r->attr_int("head_cnt"))}});
        copy_runtime_info(m.matched_nodes(), {rope});
        replace_node(m.match_root(), rope);
        return true;
    });
}

// Where one output of a VariadicSplit over the last axis of a fused QKV projection starts and stops
static bool split_range(const NodePtr& split, size_t index, int64_t& start, int64_t& stop) {
    std::vector<int64_t> axis, lens;
    if (!get_constant_ints(split->input(1), axis) || !get_constant_ints(split->input(2), lens) || axis.size() != 1 || index >= lens.size()) return false;
    if (axis[0] != 2 && axis[0] != -1) return false;
    start = 0;
    for (size_t i = 0; i < index; ++i) { if (lens[i] < 0) return false; start += lens[i]; }
    if (lens[index] < 0) return false;
    stop = start + lens[index];
    return true;
}

// RoPE over a fused QKV projection, Qwen form (RoPEFusionQwen of fuse_rotary_positional_embeddings.cpp in the reference):
//   x = reshape(variadic_split(qkv [B, L, W], -1)[i], [B, L, H, S]);  h = split(reshape(x, [B, L, H, 2, S / 2]), -2)
//   x * cos + concat(squeeze(-h[1]), squeeze(h[0]), -1) * sin,  cos / sin [1, positions, 1, S]
//   ->  RoPE(qkv, cos, sin) {is_qwen, slice_start / stop, head_cnt, head_size}, output [B, L, H, S]
std::shared_ptr<MatcherPass> make_rope_fusion_qwen() {
    auto qkv = any_input(rank_equals(3));
    auto split = wrap_type({"VariadicSplit"}, {qkv, wrap_const(), wrap_const()});
    auto x = wrap_type({"Reshape"}, {split, any_input()}, rank_equals(4));
    auto cos = any_input(rank_equals(4));
    auto sin = any_input(rank_equals(4));
    auto halves = wrap_type({"Reshape"}, {x, any_input()}, rank_equals(5));
    auto hi = wrap_type({"Split"}, {halves, wrap_const()});
    auto lo = wrap_type({"Split"}, {halves, wrap_const()});
    auto neg = any_of({wrap_type({"Multiply"}, {hi, wrap_const(scalar_eq(-1.0))}), wrap_type({"Negative"}, {hi})});
    auto sq_neg = wrap_type({"Squeeze", "Reshape"}, {neg, any_input()});
    auto sq_lo = wrap_type({"Squeeze", "Reshape"}, {lo, any_input()});
    auto cat = wrap_type({"Concat"}, {sq_neg, sq_lo});
    auto add = wrap_type({"Add"}, {wrap_type({"Multiply"}, {x, cos}), wrap_type({"Multiply"}, {cat, sin})});
    return std::make_shared<MatcherPass>("RoPEFusionQwen", add, [=](Matcher& m) {
        const PShape& xs = m.at(x).shape();
        if (!xs.dims[2].is_static() || !xs.dims[3].is_static() || xs.dims[3].lo % 2) return false;
        const int64_t H = xs.dims[2].lo, S = xs.dims[3].lo;
        int64_t start = 0, stop = 0;
        if (!split_range(m.node(split), m.at(split).index, start, stop) || stop - start != H * S) return false;
        if (m.node(hi) != m.node(lo) || m.at(hi).index != 1 || m.at(lo).index != 0 || m.node(hi)->attr_int("num_splits") != 2) return false;
        std::vector<int64_t> ax;
        if (!get_constant_ints(m.node(hi)->input(1), ax) || ax.size() != 1 || (ax[0] != -2 && ax[0] != 3)) return false;
        const PShape& hs = m.at(halves).shape();
        if (!hs.dims[3].is_static() || hs.dims[3].lo != 2 || !hs.dims[4].is_static() || hs.dims[4].lo != S / 2) return false;
        const int64_t cat_axis = m.node(cat)->attr_int("axis");
        if (cat_axis != -1 && cat_axis != 3) return false;
        if (!(m.at(cat).shape().rank() == 4)) return false;
        for (const PatternPtr& t : {cos, sin}) {
            const PShape& ts = m.at(t).shape();
            if (!(ts.dims[2].is_static() && ts.dims[2].lo == 1 && ts.dims[3].is_static() && ts.dims[3].lo == S)) return false;
        }
        auto rope = op("RoPE", {m.at(qkv), m.at(cos), m.at(sin)},
                       {{"is_qwen", Attr::Bool(true)}, {"slice_start", Attr::Int(start)}, {"slice_stop", Attr::Int(stop)}, {"rotary_ndims", Attr::Int(S)},
                        {"head_cnt", Attr::Int(H)}, {"head_size", Attr::Int(S)}});
        copy_runtime_info(m.matched_nodes(), {rope});
        replace_node(m.match_root(), rope);
        return true;
    });
}

// RoPE over a fused QKV projection, ChatGLM form (RoPEFusionChatGLM in the reference): pairs of neighbouring elements of the
// first `rot` values of every head are rotated by a combined cache [L, B or 1, 1, rot / 2, 2] (cos, sin), the rest passes through:
//   x = reshape(variadic_split(qkv [L, B, W], -1)[i], [L, B, H, S]);  p = reshape(x[..., :rot], [L, B, H, rot / 2, 2])
//   concat(reshape(stack(p0 * c - p1 * s, p1 * c + p0 * s), [L, B, H, rot]), x[..., rot:], -1)
//   ->  RoPE(qkv, cache, cache) {is_chatglm, rotary_ndims, slice_start / stop, head_cnt, head_size}, output [L, B, H, S]
std::shared_ptr<MatcherPass> make_rope_fusion_chatglm() {
    auto qkv = any_input(rank_equals(3));
    auto split = wrap_type({"VariadicSplit"}, {qkv, wrap_const(), wrap_const()});
    auto x = wrap_type({"Reshape"}, {split, any_input()}, rank_equals(4));
    auto cache = any_input(rank_equals(5));
    auto head = wrap_type({"Slice"}, {x, any_input(), any_input(), any_input(), any_input()});
    auto tail = wrap_type({"Slice"}, {x, any_input(), any_input(), any_input(), any_input()});
    auto pairs = wrap_type({"Reshape"}, {head, any_input()}, rank_equals(5));
    auto p0 = wrap_type({"Gather"}, {pairs, wrap_const(scalar_eq(0.0)), wrap_const()});
    auto p1 = wrap_type({"Gather"}, {pairs, wrap_const(scalar_eq(1.0)), wrap_const()});
    auto c = wrap_type({"Gather"}, {cache, wrap_const(scalar_eq(0.0)), wrap_const()});
    auto s = wrap_type({"Gather"}, {cache, wrap_const(scalar_eq(1.0)), wrap_const()});
    auto o0 = wrap_type({"Subtract"}, {wrap_type({"Multiply"}, {p0, c}), wrap_type({"Multiply"}, {p1, s})});
    auto o1 = wrap_type({"Add"}, {wrap_type({"Multiply"}, {p1, c}), wrap_type({"Multiply"}, {p0, s})});
    auto stack = wrap_type({"Concat"}, {wrap_type({"Unsqueeze"}, {o0, any_input()}), wrap_type({"Unsqueeze"}, {o1, any_input()})});
    auto flat = wrap_type({"Reshape"}, {stack, any_input()}, rank_equals(4));
    auto root = wrap_type({"Concat"}, {flat, tail});
    return std::make_shared<MatcherPass>("RoPEFusionChatGLM", root, [=](Matcher& m) {
        const PShape& xs = m.at(x).shape();
        if (!xs.dims[2].is_static() || !xs.dims[3].is_static()) return false;
        const int64_t H = xs.dims[2].lo, S = xs.dims[3].lo;
        int64_t start = 0, stop = 0;
        if (!split_range(m.node(split), m.at(split).index, start, stop) || stop - start != H * S) return false;
        const PShape& ps = m.at(pairs).shape();
        if (!ps.dims[3].is_static() || !ps.dims[4].is_static() || ps.dims[4].lo != 2) return false;
        const int64_t rot = 2 * ps.dims[3].lo;
        auto range = [&](const NodePtr& sl, int64_t b, int64_t e) {
            std::vector<int64_t> vb, ve, vs, va;
            if (!get_constant_ints(sl->input(1), vb) || !get_constant_ints(sl->input(2), ve) || !get_constant_ints(sl->input(3), vs) ||
                !get_constant_ints(sl->input(4), va)) return false;
            return vb.size() == 1 && vb[0] == b && (ve[0] == e || (e == S && ve[0] >= S)) && vs[0] == 1 && (va[0] == 3 || va[0] == -1);
        };
        if (rot <= 0 || rot > S || !range(m.node(head), 0, rot) || (rot < S && !range(m.node(tail), rot, S))) return false;
        for (const PatternPtr& g : {p0, p1, c, s}) {
            std::vector<int64_t> ax;
            if (!get_constant_ints(m.node(g)->input(2), ax) || ax.size() != 1 || (ax[0] != -1 && ax[0] != 4)) return false;
        }
        const PShape& cs = m.at(cache).shape();
        if (!(cs.dims[3].is_static() && cs.dims[3].lo == rot / 2 && cs.dims[4].is_static() && cs.dims[4].lo == 2 && cs.dims[2].is_static() && cs.dims[2].lo == 1)) return false;
        const int64_t a0 = m.node(stack)->attr_int("axis"), a1 = m.node(root)->attr_int("axis");
        if ((a0 != -1 && a0 != 4) || (a1 != -1 && a1 != 3)) return false;
        auto rope = op("RoPE", {m.at(qkv), m.at(cache), m.at(cache)},
                       {{"is_chatglm", Attr::Bool(true)}, {"is_interleaved", Attr::Bool(true)}, {"slice_start", Attr::Int(start)}, {"slice_stop", Attr::Int(stop)},
                        {"rotary_ndims", Attr::Int(rot)}, {"head_cnt", Attr::Int(H)}, {"head_size", Attr::Int(S)}});
        copy_runtime_info(m.matched_nodes(), {rope});
        replace_node(m.match_root(), rope);
        return true;
    });
}

// ------------------------------------------------------------------------------------ LoRA
//   main(x) + ((x @ A^T) * alpha) @ B^T   with A, alpha, B read from variables (adapters switched by set_state at run time)
//   ->  LoraSubgraph(main(x), x, A, alpha, B)
// One operation per adapted projection lets a device run the low-rank path as two small GEMMs whose second epilogue adds
// into the main result (src/common/transformations/src/transformations/common_optimizations/lora_subgraph_fusion.cpp).
std::shared_ptr<MatcherPass> make_lora_fusion() {
    auto x = any_input();
    auto main = wrap_type({"MatMul", "FullyConnected", "FullyConnectedCompressed", "Convolution"});
    auto rv = [] { return optional({"Convert"}, wrap_type({"ReadValue"})); };
    auto a = rv(), alpha = rv(), b = rv();
    auto mm_a = wrap_type({"MatMul"}, {x, a});
    auto scaled = wrap_type({"Multiply"}, {mm_a, alpha});
    auto mm_b = wrap_type({"MatMul"}, {scaled, b});
    auto add = wrap_type({"Add"}, {main, mm_b});
    return std::make_shared<MatcherPass>("LoraSubgraphFusion", add, [=](Matcher& m) {
        NodePtr mn = m.node(main);
        // the adapter reads the projection's own input
        if (!(mn->input(0) == m.at(x))) return false;
        if (!m.node(mm_a)->attr_bool("transpose_b") || !m.node(mm_b)->attr_bool("transpose_b") || m.node(mm_a)->attr_bool("transpose_a") ||
            m.node(mm_b)->attr_bool("transpose_a")) return false;
        // (the optional Convert may be absent: take the operands from the matched nodes themselves)
        NodePtr sc = m.node(scaled);
        const Output a_in = m.node(mm_a)->input(1), b_in = m.node(mm_b)->input(1);
        const Output alpha_in = sc->input(0).node == m.node(mm_a) ? sc->input(1) : sc->input(0);
        auto lora = op("LoraSubgraph", {mn->output(0), m.at(x), a_in, alpha_in, b_in}, {}, "ie_internal_opset");
        copy_runtime_info({m.node(mm_a), m.node(scaled), m.node(mm_b), m.match_root()}, {lora});
        replace_node(m.match_root(), lora);
        return true;
    });
}

// ------------------------------------------------------------------------------------ compressed weights helpers
struct CompressedWeight {
    NodePtr weights;     // low-precision Constant
    NodePtr scales;      // Constant
    NodePtr zero_points; // Constant or null
    bool valid = false;
};
// Walks W <- [Convert] <- [Transpose] <- [Reshape] <- Multiply(scale) <- [Subtract(zp)] <- Convert <- Const(lp)
static CompressedWeight match_compressed(const Output& w) {
    CompressedWeight r;
    NodePtr n = w.node;
    if (n->type == "Convert" && !n->input_node(0)->is_constant()) n = n->input_node(0);
    if (n->type == "Reshape" && !n->input_node(0)->is_constant()) n = n->input_node(0);
    if (n->type != "Multiply") return r;
    NodePtr a = n->input_node(0), b = n->input_node(1);
    if (a->is_constant()) std::swap(a, b);
    if (!b->is_constant()) { if (b->type == "Convert" && b->input_node(0)->is_constant()) b = b->input_node(0); else return r; }
    r.scales = b;
    if (a->type == "Subtract") {
        NodePtr z = a->input_node(1);
        if (z->type == "Convert") z = z->input_node(0);
        if (!z->is_constant()) return r;
        r.zero_points = z;
        a = a->input_node(0);
    }
    if (a->type != "Convert" || !a->input_node(0)->is_constant()) return r;
    r.weights = a->input_node(0);
    const ET t = r.weights->constant.et;
    r.valid = t == ET::u4 || t == ET::i4 || t == ET::u8 || t == ET::i8 || t == ET::nf4 || t == ET::f4e2m1 || t == ET::f8e4m3 || t == ET::f8e5m2;
    return r;
}
static bool is_weight_like(const Output& w) {
    NodePtr n = w.node;
    if (n->is_constant()) return true;
    if (n->type == "Convert" && n->input_node(0)->is_constant()) return true;
    return match_compressed(w).valid;
}

// ------------------------------------------------------------------------------------ MatMul -> FullyConnected
std::shared_ptr<MatcherPass> make_matmul_to_fc() {
    auto a = any_input(has_static_rank());
    auto w = any_input([](const Output& o) { return o.shape().rank_is_static() && o.shape().rank() == 2 && is_weight_like(o); });
    auto mm = wrap_type({"MatMul"}, {a, w});
    return std::make_shared<MatcherPass>("ConvertMatMulToFullyConnected", mm, [=](Matcher& m) {
        NodePtr n = m.match_root();
        if (n->attr_bool("transpose_a")) return false;
        Output wv = m.at(w);
        if (!n->attr_bool("transpose_b")) {
            // FullyConnected wants [N, K]
            if (wv.node->is_constant()) {
                std::vector<Tensor> ins = {wv.node->constant, make_constant_i64({1, 0})->constant}, outs(1);
                auto tn = op("Transpose", {wv, c_i64({1, 0})});
                EvalContext ctx;
                tn->schema->eval(*tn, ins, outs, ctx);
                Tensor own(outs[0].et, outs[0].shape);
                std::memcpy(own.data(), outs[0].data(), own.byte_size());
                auto c = make_constant(own);
                c->name = wv.node->name;
                wv = c->output(0);
            } else return false;
        }
        Output bias = make_constant(Tensor(ET::dynamic, Shape{0}))->output(0);
        auto fc = op("FullyConnected", {m.at(a), wv, bias}, {{"output_type", Attr::Type(ET::dynamic)}});
        copy_runtime_info({n}, {fc});
        replace_node(n, fc);
        return true;
    });
}

// FullyConnected(x, decompress(Wq), bias) -> FullyConnectedCompressed(x, Wq[N,K], bias, scales[N,G], zp[N,G])
std::shared_ptr<MatcherPass> make_fc_to_compressed() {
    auto fc = wrap_type({"FullyConnected"});
    return std::make_shared<MatcherPass>("ConvertFullyConnectedToFullyConnectedCompressed", fc, [=](Matcher& m) {
        NodePtr n = m.match_root();
        CompressedWeight cw = match_compressed(n->input(1));
        if (!cw.valid) return false;
        const Tensor& w = cw.weights->constant;
        if (w.shape.size() < 2) return false;
        const int64_t N = w.shape[0], K = w.numel() / N;
        Tensor w2 = w;
        w2.shape = Shape{N, K};   // fold [N, G, gs] -> [N, K]; the bytes are unchanged
        auto wc = make_constant(w2);
        wc->name = cw.weights->name;
        auto fold = [&](const NodePtr& c) {
            Tensor t = c->constant;
            const int64_t G = std::max<int64_t>(1, t.numel() / N);
            t.shape = t.numel() == 1 ? Shape{} : Shape{N, G};
            auto k = make_constant(t);
            k->name = c->name;
            return k;
        };
        Output sc = fold(cw.scales)->output(0);
        Output zp = cw.zero_points ? fold(cw.zero_points)->output(0) : make_constant(Tensor(ET::dynamic, Shape{0}))->output(0);
        auto fcc = op("FullyConnectedCompressed", {n->input(0), wc->output(0), n->input(2), sc, zp}, {{"output_type", Attr::Type(n->outs[0].et)}});
        copy_runtime_info(m.matched_nodes(), {fcc});
        replace_node(n, fcc);
        return true;
    });
}

// ------------------------------------------------------------------------------------ SwiGLU
// Multiply(Swish(VariadicSplit(x)[0]), VariadicSplit(x)[1]) -> GLU(x)
std::shared_ptr<MatcherPass> make_swiglu_fusion() {
    auto x = any_input(has_static_rank());
    auto split = wrap_type({"VariadicSplit"}, {x, wrap_const(), wrap_const()});
    auto act = wrap_type({"Swish", "Gelu"}, {split});
    auto mul = wrap_type({"Multiply"}, {act, split});
    return std::make_shared<MatcherPass>("GLUFusion", mul, [=](Matcher& m) {
        NodePtr sp = m.node(split);
        if (sp->num_outputs() != 2) return false;
        std::vector<int64_t> axis, lens;
        if (!get_constant_ints(sp->input(1), axis) || !get_constant_ints(sp->input(2), lens) || lens.size() != 2 || lens[0] != lens[1]) return false;
        const int64_t rank = (int64_t)m.at(x).shape().rank();
        if (axis[0] != -1 && axis[0] != rank - 1) return false;
        NodePtr a = m.node(act);
        if (a->type == "Swish" && a->num_inputs() > 1) return false;
        NodePtr mu = m.match_root();
        const size_t gate_idx = a->input(0).index;
        // the other Multiply operand must be the other half
        Output other = mu->input(0).node == a ? mu->input(1) : mu->input(0);
        if (other.node != sp || other.index == gate_idx) return false;
        std::string gt = a->type == "Swish" ? "Swish" : (a->attr_str("approximation_mode") == "TANH" ? "Gelu_Tanh" : "Gelu");
        auto glu = op("GLU", {m.at(x)}, {{"axis", Attr::Int(-1)}, {"split_lengths", Attr::Int(lens[0])}, {"glu_type", Attr::Str(gt)},
                                        {"split_to_glu_idx", Attr::Int((int64_t)gate_idx)}, {"output_type", Attr::Type(mu->outs[0].et)}});
        copy_runtime_info(m.matched_nodes(), {glu});
        replace_node(mu, glu);
        return true;
    });
}

// ------------------------------------------------------------------------------------ SDPAFusion
// MatMul(Softmax(MatMul(q, k^T) * scale [+ mask]), v) -> ScaledDotProductAttention
std::shared_ptr<MatcherPass> make_sdpa_fusion() {
    auto q = any_input(), k = any_input(), v = any_input();
    auto qk = wrap_type({"MatMul"}, {q, k});
    auto scale = wrap_const();
    auto scaled = optional({"Multiply", "Divide"}, {qk, scale});
    auto mask = any_input();
    auto masked = optional({"Add"}, {scaled, mask});
    auto sm = wrap_type({"Softmax"}, {masked});
    auto out = wrap_type({"MatMul"}, {sm, v});
    return std::make_shared<MatcherPass>("SDPAFusion", out, [=](Matcher& m) {
        NodePtr mm1 = m.node(qk), mm2 = m.match_root();
        if (mm1->attr_bool("transpose_a") || !mm1->attr_bool("transpose_b") || mm2->attr_bool("transpose_a") || mm2->attr_bool("transpose_b")) return false;
        const PShape& qs = m.at(q).shape();
        if (qs.rank_dynamic || qs.rank() < 3) return false;
        NodePtr smn = m.node(sm);
        const int64_t ax = smn->attr_int("axis");
        if (ax != -1 && ax != (int64_t)qs.rank() - 1) return false;
        std::vector<Output> ins = {m.at(q), m.at(k), m.at(v)};
        const bool has_scale = m.has(scaled) && m.node(scaled) != mm1 && (m.node(scaled)->type == "Multiply" || m.node(scaled)->type == "Divide");
        const bool has_mask = m.has(masked) && m.node(masked)->type == "Add" && m.node(masked) != m.node(scaled);
        Output mk = has_mask ? m.at(mask) : make_constant(from_f32(m.at(q).et(), Shape{}, {0.f}))->output(0);
        ins.push_back(mk);
        if (has_scale) {
            Tensor st;
            if (!try_constant_value(m.at(scale), st) || st.numel() != 1) return false;
            double sv = get_elem_f64(st, 0);
            if (m.node(scaled)->type == "Divide") sv = 1.0 / sv;
            ins.push_back(make_constant(from_f32(m.at(q).et(), Shape{}, {float(sv)}))->output(0));
        } else {
            ins.push_back(make_constant(from_f32(m.at(q).et(), Shape{}, {1.0f}))->output(0));
        }
        auto sdpa = op("ScaledDotProductAttention", ins, {{"causal", Attr::Bool(false)}});
        copy_runtime_info(m.matched_nodes(), {sdpa});
        replace_node(mm2, sdpa);
        return true;
    });
}

// ------------------------------------------------------------------------------------ MoE expert fusion
// A chain  acc = acc + scatter/where(expert_e(x) * w_e)  built per expert by exporters is model specific; this
// framework's builders emit the MOE op directly, so the pass only normalises 2-D expert constants that were
// written per expert ("experts.{e}.gate/up/down") into the batched [E, ...] constants the MOE op expects.
bool fuse_moe_experts(const ModelPtr& m) {
    bool changed = false;
    for (auto& n : m->ordered_ops()) {
        if (n->type != "MOE") continue;
        for (size_t i = 3; i < std::min<size_t>(6, n->num_inputs()); ++i) {
            NodePtr w = n->input_node(i);
            if (w->type != "Concat") continue;
            bool all_const = true;
            for (auto& in : w->inputs()) all_const = all_const && in.node->is_constant();
            if (!all_const) continue;
            std::vector<Tensor> ins, outs(1);
            for (auto& in : w->inputs()) ins.push_back(in.node->constant);
            EvalContext ctx;
            if (!w->schema->eval(*w, ins, outs, ctx)) continue;
            auto c = make_constant(outs[0]);
            c->name = w->name + "/FusedMOEWeights";
            replace_output(w->output(0), c->output(0));
            changed = true;
        }
    }
    return changed;
}

// ------------------------------------------------------------------------------------ SDPA -> PagedAttention
namespace {
// Follows optional GQA head expansion / Convert / Transpose back to a Concat(ReadValue-like, current)
struct KvTrace {
    NodePtr concat;
    Output current;          // new K or V rows, [B, Hkv, L, S]
    NodePtr read_value;      // or past Parameter
    bool ok = false;
};
KvTrace trace_kv(Output v) {
    KvTrace t;
    NodePtr n = v.node;
    for (int guard = 0; guard < 12 && n; ++guard) {
        if (n->type == "Concat") break;
        if (n->type == "Reshape" || n->type == "Broadcast" || n->type == "Unsqueeze" || n->type == "Convert" || n->type == "Multiply" || n->type == "Gather") {
            // Gather(past, beam_idx) and broadcast helpers: data travels through input 0
            n = n->input_node(0);
            continue;
        }
        return t;
    }
    if (!n || n->type != "Concat" || n->num_inputs() != 2) return t;
    NodePtr past = n->input_node(0);
    for (int guard = 0; guard < 4 && past; ++guard) {
        if (past->type == "ReadValue" || past->is_parameter()) break;
        if (past->type == "Gather" || past->type == "Convert") { past = past->input_node(0); continue; }
        return t;
    }
    if (!past || (past->type != "ReadValue" && !past->is_parameter())) return t;
    t.concat = n;
    t.current = n->input(1);
    t.read_value = past;
    t.ok = true;
    return t;
}
}  // namespace


// What the attention mask of an SDPA encodes besides causality, read from the mask's own subgraph:
// * a sliding window: a comparison one side of which is a position shifted by a scalar integer constant W
//   (``k_pos > q_pos - W``, the form of the exported Mistral / Phi-3 / Gemma graphs): W keys stay visible
//   (W + 1 for the non-strict comparisons);
// * ALiBi: a per-head constant ([H, 1, 1] or [1, H, 1, 1]) multiplied into a position term that is added to the scores.
struct MaskFeatures {
    int64_t window = 0;
    Output alibi;            // the slopes constant when found
};

Output skip_shape_ops(Output o) {
    for (int i = 0; i < 4; ++i) {
        const std::string& t = o.node->type;
        if (t == "Convert" || t == "Unsqueeze" || t == "Squeeze" || t == "Reshape") o = o.node->input(0);
        else break;
    }
    return o;
}

MaskFeatures mask_features(const Output& mask, int64_t heads) {
    MaskFeatures f;
    std::vector<NodePtr> stack = {mask.node};
    std::set<Node*> seen;
    size_t budget = 400;
    while (!stack.empty() && budget--) {
        NodePtr n = stack.back();
        stack.pop_back();
        if (!seen.insert(n.get()).second) continue;
        if (n->is_parameter() || n->type == "ReadValue" || n->type == "Constant") continue;
        const bool strict = n->type == "Greater" || n->type == "Less";
        if (strict || n->type == "GreaterEqual" || n->type == "LessEqual") {
            for (size_t k = 0; k < 2 && f.window == 0; ++k) {
                Output side = skip_shape_ops(n->input(k));
                if (side.node->type != "Subtract" && side.node->type != "Add") continue;
                for (size_t j = 0; j < 2; ++j) {
                    std::vector<int64_t> c;
                    Output operand = skip_shape_ops(side.node->input(j));
                    if (operand.node->type == "Constant" && get_constant_ints(operand, c) && c.size() == 1 && std::llabs(c[0]) >= 2) {
                        f.window = std::llabs(c[0]) + (strict ? 0 : 1);
                        break;
                    }
                }
            }
        }
        if (n->type == "Multiply" && !f.alibi.node && heads > 1) {
            for (size_t k = 0; k < 2; ++k) {
                Output c = skip_shape_ops(n->input(k));
                if (c.node->type != "Constant" || !et_is_real(c.et())) continue;
                const PShape& cs = c.shape();
                if (!cs.is_static()) continue;
                int64_t total = 1, big = 0;
                for (auto& d : cs.dims) { total *= d.lo; if (d.lo > 1) big = d.lo; }
                if (total == heads && big == heads) { f.alibi = c; break; }
            }
        }
        for (size_t k = 0; k < n->num_inputs(); ++k) stack.push_back(n->input(k).node);
    }
    return f;
}

bool sdpa_to_paged_attention(const ModelPtr& m, const AttrMap& options) {
    auto opt_b = [&](const char* k) { auto it = options.find(k); return it != options.end() && it->second.i != 0; };
    (void)opt_b;
    std::vector<NodePtr> sdpas;
    for (auto& n : m->ordered_ops()) if (n->type == "ScaledDotProductAttention") sdpas.push_back(n);
    OVC_CHECK(!sdpas.empty(), "SDPAToPagedAttention: the model has no ScaledDotProductAttention");
    auto find_param = [&](const std::string& nm) -> NodePtr {
        for (auto& p : m->params) if (p->name == nm || p->outs[0].names.count(nm)) return p;
        return nullptr;
    };
    NodePtr input_ids = find_param("input_ids");
    if (!input_ids) input_ids = find_param("inputs_embeds");
    OVC_CHECK(input_ids, "SDPAToPagedAttention: the model has neither 'input_ids' nor 'inputs_embeds'");

    auto mk = [&](const char* nm, ET et, const PShape& s) { auto p = make_parameter(et, s, nm); return p; };
    NodePtr max_context_len = mk("max_context_len", ET::i32, PShape(Shape{}));
    NodePtr past_lens = mk("past_lens", ET::i32, PShape::dynamic(1));
    NodePtr subsequence_begins = mk("subsequence_begins", ET::i32, PShape::dynamic(1));
    NodePtr block_indices = mk("block_indices", ET::i32, PShape::dynamic(1));
    NodePtr block_indices_begins = mk("block_indices_begins", ET::i32, PShape::dynamic(1));
    std::vector<NodePtr> new_params = {max_context_len, past_lens, subsequence_begins, block_indices, block_indices_begins};

    // input_ids [B, L] -> [T] then Unsqueeze(1): the old batch axis now runs over tokens
    if (input_ids->name == "input_ids") {
        auto uses = input_ids->outs[0].uses;
        input_ids->set_attr("shape", Attr::Shape_(PShape::dynamic(1)));
        input_ids->validate_and_infer();
        auto uns = op("Unsqueeze", {input_ids->output(0), c_i64({1})});
        for (auto& u : uses) u.node->set_input(u.input, uns->output(0));
    }
    NodePtr position_ids = find_param("position_ids");
    if (!position_ids) {
        position_ids = mk("position_ids", ET::i64, PShape::dynamic(1));
        new_params.push_back(position_ids);
    } else {
        auto uses = position_ids->outs[0].uses;
        position_ids->set_attr("shape", Attr::Shape_(PShape::dynamic(1)));
        position_ids->validate_and_infer();
        auto uns = op("Unsqueeze", {position_ids->output(0), c_i64({1})});
        for (auto& u : uses) u.node->set_input(u.input, uns->output(0));
    }

    std::set<NodePtr> dead_assigns, dead_params;
    int layer = 0;
    for (auto& sdpa : sdpas) {
        KvTrace kt = trace_kv(sdpa->input(1)), vt = trace_kv(sdpa->input(2));
        OVC_CHECK(kt.ok && vt.ok, "SDPAToPagedAttention: cannot trace the KV cache of '" << sdpa->name << "'");
        const PShape& ks = kt.current.shape();
        const PShape& vs = vt.current.shape();
        OVC_CHECK(!ks.rank_dynamic && ks.rank() == 4 && ks.dims[1].is_static() && ks.dims[3].is_static(),
                  "SDPAToPagedAttention: key of '" << sdpa->name << "' must be [B, H, L, S] with static H and S, got " << ks.str());
        const int64_t Hk = ks.dims[1].lo, S = ks.dims[3].lo, Hv = vs.dims[1].lo, Sv = vs.dims[3].lo;
        const ET et = sdpa->outs[0].et;
        NodePtr kc = mk(("key_cache." + std::to_string(layer)).c_str(), ET::dynamic, PShape::dynamic(4));
        NodePtr vc = mk(("value_cache." + std::to_string(layer)).c_str(), ET::dynamic, PShape::dynamic(4));
        new_params.push_back(kc);
        new_params.push_back(vc);
        auto flat = [&](const Output& x) {   // [B, H, L, S] -> [T, H*S]
            auto t = op("Transpose", {x, c_i64({0, 2, 1, 3})});
            return op("Reshape", {t->output(0), c_i64({0, -1})}, {{"special_zero", Attr::Bool(true)}})->output(0);
        };
        Output q2 = flat(sdpa->input(0)), k2 = flat(kt.current), v2 = flat(vt.current);
        // fold [B, L, H*S] -> [B*L, H*S]: B*L = T
        auto flat2 = [&](const Output& x, int64_t width) { return op("Reshape", {x, c_i64({-1, width})}, {{"special_zero", Attr::Bool(false)}})->output(0); };
        const PShape& qs = sdpa->input(0).shape();
        OVC_CHECK(qs.dims[1].is_static(), "SDPAToPagedAttention: query head count must be static");
        const int64_t Hq = qs.dims[1].lo;
        q2 = flat2(q2, Hq * S); k2 = flat2(k2, Hk * S); v2 = flat2(v2, Hv * Sv);
        Output scale;
        if (sdpa->num_inputs() > 4) scale = sdpa->input(4);
        else scale = make_constant(from_f32(et == ET::dynamic ? ET::f32 : et, Shape{}, {1.0f / std::sqrt(float(S))}))->output(0);
        if (scale.shape().rank_is_static() && scale.shape().rank() > 0) scale = op("Squeeze", {scale})->output(0);
        auto empty_f = [&]() { return make_constant(Tensor(ET::f32, Shape{0}))->output(0); };
        auto empty_i = [&]() { return make_constant(Tensor(ET::i32, Shape{0}))->output(0); };
        // sliding window and ALiBi slopes: from the options when given, else from the structure of the mask
        MaskFeatures mf;
        if (sdpa->num_inputs() > 3) mf = mask_features(sdpa->input(3), Hq);
        if (auto it = options.find("sliding_window"); it != options.end() && it->second.i > 0) mf.window = it->second.i;
        Output alibi = empty_f();
        if (mf.alibi.node) {
            auto flat_slopes = op("Reshape", {mf.alibi, c_i64({-1})}, {{"special_zero", Attr::Bool(false)}});
            alibi = flat_slopes->output(0);
            if (alibi.et() != ET::f32) alibi = op("Convert", {alibi}, {{"destination_type", Attr::Type(ET::f32)}})->output(0);
        }
        std::vector<Output> ins = {q2, k2, v2, kc->output(0), vc->output(0), past_lens->output(0), subsequence_begins->output(0),
                                   block_indices->output(0), block_indices_begins->output(0), scale, c_i32({mf.window}, true), alibi,
                                   max_context_len->output(0)};
        // score_aggregation_window, rotated_block_indices, rotation_deltas, rotation_trig_lut, xattention_threshold,
        // xattention_block_size, xattention_stride, sinks, adaptive_rkv (4), token_type_ids, qq_bias, qq_bias_begins
        ins.push_back(empty_i()); ins.push_back(empty_i()); ins.push_back(empty_i()); ins.push_back(empty_f()); ins.push_back(empty_f());
        ins.push_back(c_i32({0}, true)); ins.push_back(c_i32({0}, true));
        ins.push_back(sdpa->num_inputs() > 5 ? sdpa->input(5) : empty_f());
        for (int i = 0; i < 4; ++i) ins.push_back(empty_i());
        ins.push_back(empty_i());
        ins.push_back(make_constant(Tensor(ET::u8, Shape{0}))->output(0));
        ins.push_back(empty_i());
        auto pa = make_node("PagedAttentionExtension", "extension", ins, {}, false);
        pa->rt_info["num_k_heads"] = Attr::Int(Hk);
        pa->rt_info["k_head_size"] = Attr::Int(S);
        pa->rt_info["num_v_heads"] = Attr::Int(Hv);
        pa->rt_info["v_head_size"] = Attr::Int(Sv);
        pa->validate_and_infer();
        pa->name = sdpa->name + "/PagedAttention";
        // [T, Hq*Sv] -> [T, 1, Hq, Sv] -> [T, Hq, 1, Sv]: the layout the consumers of the SDPA output expect
        auto r = op("Reshape", {pa->output(0), c_i64({0, 1, -1, Sv})}, {{"special_zero", Attr::Bool(true)}});
        auto t = op("Transpose", {r->output(0), c_i64({0, 2, 1, 3})});
        copy_runtime_info({sdpa}, {pa, r, t});
        replace_node(sdpa, t, false);
        // retire the state of this layer
        for (auto* tr : {&kt, &vt}) {
            for (auto& u : tr->concat->outs[0].uses) if (u.node->type == "Assign") dead_assigns.insert(u.node->shared_from_this());
            if (tr->read_value->is_parameter()) dead_params.insert(tr->read_value);
        }
        ++layer;
    }
    for (auto& a : dead_assigns) m->remove_sink(a);
    // Results that only exposed the present KV tensors go away with the cache
    for (auto& r : std::vector<NodePtr>(m->results)) {
        NodePtr src = r->input_node(0);
        if (src->type == "Concat" && src->num_inputs() == 2 && (src->input_node(0)->type == "ReadValue" || src->input_node(0)->is_parameter())) {
            bool is_kv = false;
            for (auto& nm : r->outs[0].names) if (nm.rfind("present", 0) == 0) is_kv = true;
            if (is_kv || r->name.rfind("present", 0) == 0) m->remove_result(r);
        }
    }
    for (auto& p : dead_params) m->remove_parameter(p);
    m->add_parameters(new_params);
    // beam_idx / attention_mask have no meaning for the paged form
    for (const char* nm : {"beam_idx", "attention_mask"}) {
        if (NodePtr p = find_param(nm)) {
            if (p->outs[0].uses.empty()) { m->remove_parameter(p); continue; }
            // the mask only fed the SDPA that is gone now; anything left keeps a neutral constant
            bool only_dead = true;
            for (auto& n : m->ordered_ops()) for (auto& i : n->inputs()) if (i.node == p) only_dead = false;
            if (only_dead) m->remove_parameter(p);
        }
    }
    m->validate();
    return true;
}

}  // namespace ovc
