// Recurrent-state operations of the internal operation set: the Mamba2 selective state-space recurrence and the gated
// delta rule (dense and paged forms), the paged causal 1-D convolution that feeds them, KV-cache token reordering for
// paged attention, and the attention-gated GRU cell / sequence: shape / type inference and reference evaluation.
//
// The paged forms keep one state snapshot per block of a state table: the first block slot of a sequence is read, the
// next slots are written each time the sequence crosses a multiple of its cache interval and once more at the end of
// the step. Tables are inputs that the operation updates in place, like the KV cache of paged attention.
//
// Reference counterparts: src/core/src/op/{selective_ssm,gated_delta_net,paged_selective_ssm,paged_gated_delta_net,
// paged_causal_conv1d,pa_kv_reorder}.cpp, src/common/transformations/src/ov_ops/{augru_cell,augru_sequence}.cpp and the
// specifications under docs/articles_en/documentation/openvino-ir-format/operation-sets/operation-specs/internal/.
#include <algorithm>
#include <cmath>
#include <cstring>

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
AttrSpec Af(const char* n, double d = 0) { AttrSpec s = A(n, K::FLOAT, Attr::Float(d)); s.f32 = true; return s; }
AttrSpec As(const char* n, const char* d = "") { return A(n, K::STR, Attr::Str(d)); }
AttrSpec Afs(const char* n) { return A(n, K::FLOATS, Attr::Floats({})); }
AttrSpec Ass(const char* n) { return A(n, K::STRS, Attr::Strs({})); }

void reg(const char* type, const char* version, std::vector<AttrSpec> attrs, InferFn infer, EvalFn eval, int min_in, int max_in, bool side_effects = false) {
    OpSchema s;
    s.type = type;
    s.version = version;
    s.attrs = std::move(attrs);
    s.infer = std::move(infer);
    s.eval = std::move(eval);
    s.min_inputs = min_in;
    s.max_inputs = max_in;
    s.has_side_effects = side_effects;
    OpRegistry::get().add(std::move(s));
}

Dim dim_of(const PShape& s, size_t i) { return (!s.rank_dynamic && i < s.dims.size()) ? s.dims[i] : Dim::dynamic(); }

// write fp32 values back into a tensor of any float type, in place
void store_f32(const Tensor& t, const std::vector<float>& v) {
    Tensor tmp = from_f32(t.et, t.shape, v);
    std::memcpy(t.data(), tmp.data(), t.byte_size());
}

// ------------------------------------------------------------------------------------------------ recurrences
// One token of the selective state-space recurrence for one head: state [P, S] (head_dim x state_size)
void ssm_step(float* state, int64_t P, int64_t S, float dA, float dt, const float* Bv, const float* x, const float* Cv, float* y) {
    for (int64_t p = 0; p < P; ++p) {
        float acc = 0;
        float* row = state + p * S;
        for (int64_t s = 0; s < S; ++s) {
            row[s] = row[s] * dA + dt * Bv[s] * x[p];
            acc += row[s] * Cv[s];
        }
        y[p] = acc;
    }
}

// One token of the gated delta rule for one value head. `state` is [Dk, Dv] (dense form) or [Dv, Dk] (paged form).
void gdn_step(float* state, int64_t Dk, int64_t Dv, bool v_major, const float* q, const float* k, const float* v, float g, float beta, float* out) {
    auto at = [&](int64_t ik, int64_t iv) -> float& { return v_major ? state[iv * Dk + ik] : state[ik * Dv + iv]; };
    const float decay = std::exp(g);
    for (int64_t iv = 0; iv < Dv; ++iv) {
        float mem = 0;
        for (int64_t ik = 0; ik < Dk; ++ik) {
            at(ik, iv) *= decay;
            mem += at(ik, iv) * k[ik];
        }
        const float delta = (v[iv] - mem) * beta;
        float o = 0;
        for (int64_t ik = 0; ik < Dk; ++ik) {
            at(ik, iv) += k[ik] * delta;
            o += at(ik, iv) * q[ik];
        }
        out[iv] = o;
    }
}

void l2_normalise(std::vector<float>& v, float eps, float extra_scale) {
    double s = 0;
    for (float a : v) s += (double)a * a;
    const float inv = (float)(1.0 / std::sqrt(s + eps)) * extra_scale;
    for (float& a : v) a *= inv;
}

// Walk of one sequence through the block slots of a paged state table: `load(block)`, then for every chunk of tokens
// up to the next multiple of the cache interval `run(token_begin, token_end)` and `save(block)`.
template <class Load, class Run, class Save>
void paged_walk(const Node& n, const std::vector<int64_t>& blocks, int64_t bb, int64_t be, int64_t tb, int64_t te, int64_t past, int64_t interval, int64_t table_rows,
                Load load, Run run, Save save) {
    OVC_CHECK(be > bb, n.description() << ": a sequence needs at least one state block");
    auto blk = [&](int64_t slot) {
        OVC_CHECK(bb + slot < be, n.description() << ": block slot " << slot << " is beyond the " << (be - bb) << " slots of the sequence");
        const int64_t b = blocks[(size_t)(bb + slot)];
        OVC_CHECK(b >= 0 && b < table_rows, n.description() << ": block index " << b << " outside the table of " << table_rows << " rows");
        return b;
    };
    load(blk(0));
    int64_t slot = 1, token = tb;
    int64_t to_boundary = interval > 0 ? ((past % interval) > 0 ? interval - past % interval : interval) : (te - tb);
    while (token < te) {
        const int64_t end = std::min(token + to_boundary, te);
        run(token, end);
        save(blk(slot++));
        token = end;
        if (interval > 0) to_boundary = interval;
    }
}

bool eval_selective_ssm(N n, Ins in, Outs out, C) {
    const auto Av = to_f32(in[0]), dt = to_f32(in[1]), Bm = to_f32(in[2]), x = to_f32(in[3]), Cm = to_f32(in[4]);
    auto state = to_f32(in[5]);
    const int64_t Bn = in[3].shape[0], L = in[3].shape[1], H = in[3].shape[2], P = in[3].shape[3], G = in[2].shape[2], S = in[2].shape[3];
    OVC_CHECK(G > 0 && H % G == 0 && (int64_t)Av.size() == H, n.description() << ": num_heads must be a multiple of num_groups and A needs one value per head");
    std::vector<float> y((size_t)(Bn * L * H * P));
    for (int64_t b = 0; b < Bn; ++b)
        for (int64_t t = 0; t < L; ++t)
            for (int64_t h = 0; h < H; ++h) {
                const float d = dt[(size_t)((b * L + t) * H + h)];
                const int64_t g = h / (H / G);
                ssm_step(state.data() + ((b * H + h) * P) * S, P, S, std::exp(Av[(size_t)h] * d), d, Bm.data() + ((b * L + t) * G + g) * S,
                         x.data() + ((b * L + t) * H + h) * P, Cm.data() + ((b * L + t) * G + g) * S, y.data() + ((b * L + t) * H + h) * P);
            }
    out[0] = from_f32(in[3].et, in[3].shape, y);
    out[1] = from_f32(in[5].et, in[5].shape, state);
    return true;
}

bool eval_gated_delta_net(N n, Ins in, Outs out, C) {
    const auto q = to_f32(in[0]), k = to_f32(in[1]), v = to_f32(in[2]), gate = to_f32(in[4]), beta = to_f32(in[5]);
    auto state = to_f32(in[3]);
    const int64_t Bn = in[0].shape[0], L = in[0].shape[1], Hq = in[0].shape[2], Dk = in[0].shape[3], Hv = in[2].shape[2], Dv = in[2].shape[3];
    OVC_CHECK(Hq > 0 && Hv % Hq == 0, n.description() << ": value heads must be a multiple of query / key heads");
    const bool norm = n.attr_bool("fuse_qk_l2norm");
    const float scale = 1.f / std::sqrt((float)Dk);
    std::vector<float> y((size_t)(Bn * L * Hv * Dv)), qv((size_t)Dk), kv((size_t)Dk);
    for (int64_t b = 0; b < Bn; ++b)
        for (int64_t t = 0; t < L; ++t)
            for (int64_t h = 0; h < Hv; ++h) {
                const int64_t hq = h / (Hv / Hq);
                std::copy_n(q.data() + ((b * L + t) * Hq + hq) * Dk, Dk, qv.begin());
                std::copy_n(k.data() + ((b * L + t) * Hq + hq) * Dk, Dk, kv.begin());
                if (norm) {
                    l2_normalise(qv, (float)n.attr_float("q_l2_norm_eps", 1e-6), scale);
                    l2_normalise(kv, (float)n.attr_float("k_l2_norm_eps", 1e-6), 1.f);
                } else {
                    for (float& a : qv) a *= scale;
                }
                gdn_step(state.data() + ((b * Hv + h) * Dk) * Dv, Dk, Dv, false, qv.data(), kv.data(), v.data() + ((b * L + t) * Hv + h) * Dv,
                         gate[(size_t)((b * L + t) * Hv + h)], beta[(size_t)((b * L + t) * Hv + h)], y.data() + ((b * L + t) * Hv + h) * Dv);
            }
    out[0] = from_f32(in[2].et, in[2].shape, y);
    out[1] = from_f32(in[3].et, in[3].shape, state);
    return true;
}

bool eval_paged_selective_ssm(N n, Ins in, Outs out, C) {
    const auto Av = to_f32(in[0]), dt = to_f32(in[1]), Bm = to_f32(in[2]), x = to_f32(in[3]), Cm = to_f32(in[4]);
    auto table = to_f32(in[5]);
    const auto begins = to_i64(in[6]), blocks = to_i64(in[7]), bbeg = to_i64(in[8]), past = to_i64(in[9]), interval = to_i64(in[10]);
    const int64_t H = in[3].shape[1], P = in[3].shape[2], G = in[2].shape[1], S = in[2].shape[2], rows = in[5].shape[0];
    OVC_CHECK(G > 0 && H % G == 0, n.description() << ": num_heads must be a multiple of num_groups");
    const int64_t per_block = H * P * S, seqs = (int64_t)begins.size() - 1;
    std::vector<float> y((size_t)(in[3].shape[0] * H * P)), state((size_t)per_block);
    for (int64_t s = 0; s < seqs; ++s)
        paged_walk(n, blocks, bbeg[(size_t)s], bbeg[(size_t)s + 1], begins[(size_t)s], begins[(size_t)s + 1], past[(size_t)s], interval[(size_t)s], rows,
                   [&](int64_t b) { std::copy_n(table.data() + b * per_block, per_block, state.begin()); },
                   [&](int64_t t0, int64_t t1) {
                       for (int64_t t = t0; t < t1; ++t)
                           for (int64_t h = 0; h < H; ++h) {
                               const float d = dt[(size_t)(t * H + h)];
                               const int64_t g = h / (H / G);
                               ssm_step(state.data() + h * P * S, P, S, std::exp(Av[(size_t)h] * d), d, Bm.data() + (t * G + g) * S, x.data() + (t * H + h) * P,
                                        Cm.data() + (t * G + g) * S, y.data() + (t * H + h) * P);
                           }
                   },
                   [&](int64_t b) { std::copy_n(state.begin(), per_block, table.data() + b * per_block); });
    store_f32(in[5], table);
    out[0] = from_f32(in[3].et, in[3].shape, y);
    return true;
}

bool eval_paged_gated_delta_net(N n, Ins in, Outs out, C) {
    const auto q = to_f32(in[0]), k = to_f32(in[1]), v = to_f32(in[2]), gate = to_f32(in[4]), beta = to_f32(in[5]);
    auto table = to_f32(in[3]);
    const auto begins = to_i64(in[6]), blocks = to_i64(in[7]), bbeg = to_i64(in[8]), past = to_i64(in[9]), interval = to_i64(in[10]);
    const int64_t Hq = in[0].shape[1], Dk = in[0].shape[2], Hv = in[2].shape[1], Dv = in[2].shape[2], rows = in[3].shape[0];
    OVC_CHECK(Hq > 0 && Hv % Hq == 0, n.description() << ": value heads must be a multiple of query / key heads");
    const bool norm = n.attr_bool("use_qk_l2norm");
    const float scale = 1.f / std::sqrt((float)Dk);
    const int64_t per_block = Hv * Dv * Dk, seqs = (int64_t)begins.size() - 1;
    std::vector<float> y((size_t)(in[2].shape[0] * Hv * Dv)), state((size_t)per_block), qv((size_t)Dk), kv((size_t)Dk);
    for (int64_t s = 0; s < seqs; ++s)
        paged_walk(n, blocks, bbeg[(size_t)s], bbeg[(size_t)s + 1], begins[(size_t)s], begins[(size_t)s + 1], past[(size_t)s], interval[(size_t)s], rows,
                   [&](int64_t b) { std::copy_n(table.data() + b * per_block, per_block, state.begin()); },
                   [&](int64_t t0, int64_t t1) {
                       for (int64_t t = t0; t < t1; ++t)
                           for (int64_t h = 0; h < Hv; ++h) {
                               const int64_t hq = h / (Hv / Hq);
                               std::copy_n(q.data() + (t * Hq + hq) * Dk, Dk, qv.begin());
                               std::copy_n(k.data() + (t * Hq + hq) * Dk, Dk, kv.begin());
                               if (norm) {
                                   l2_normalise(qv, (float)n.attr_float("q_l2_norm_eps", 1e-6), scale);
                                   l2_normalise(kv, (float)n.attr_float("k_l2_norm_eps", 1e-6), 1.f);
                               } else {
                                   for (float& a : qv) a *= scale;
                               }
                               gdn_step(state.data() + h * Dv * Dk, Dk, Dv, true, qv.data(), kv.data(), v.data() + (t * Hv + h) * Dv, gate[(size_t)(t * Hv + h)],
                                        beta[(size_t)(t * Hv + h)], y.data() + (t * Hv + h) * Dv);
                           }
                   },
                   [&](int64_t b) { std::copy_n(state.begin(), per_block, table.data() + b * per_block); });
    store_f32(in[3], table);
    out[0] = from_f32(in[2].et, in[2].shape, y);
    return true;
}

bool eval_paged_causal_conv1d(N n, Ins in, Outs out, C) {
    const auto x = to_f32(in[0]), w = to_f32(in[2]), bias = to_f32(in[3]);
    auto table = to_f32(in[1]);
    const auto begins = to_i64(in[4]), blocks = to_i64(in[5]), bbeg = to_i64(in[6]), past = to_i64(in[7]), interval = to_i64(in[8]);
    const int64_t Hd = in[0].shape[1], Kk = in[1].shape[2], OC = in[2].shape[0], ICg = in[2].shape[1], rows = in[1].shape[0];
    OVC_CHECK(OC == Hd && in[2].shape[2] == Kk && ICg > 0 && Hd % ICg == 0, n.description() << ": weights [hidden, hidden / groups, kernel] must match the state [hidden, kernel]");
    const int64_t groups = Hd / ICg, per_block = Hd * Kk, seqs = (int64_t)begins.size() - 1;
    std::vector<float> y((size_t)(in[0].shape[0] * Hd)), state((size_t)per_block);
    for (int64_t s = 0; s < seqs; ++s)
        paged_walk(n, blocks, bbeg[(size_t)s], bbeg[(size_t)s + 1], begins[(size_t)s], begins[(size_t)s + 1], past[(size_t)s], interval[(size_t)s], rows,
                   [&](int64_t b) { std::copy_n(table.data() + b * per_block, per_block, state.begin()); },
                   [&](int64_t t0, int64_t t1) {
                       for (int64_t t = t0; t < t1; ++t) {
                           for (int64_t c = 0; c < Hd; ++c) {          // the window moves one step: oldest value out, the new token in
                               float* row = state.data() + c * Kk;
                               std::copy(row + 1, row + Kk, row);
                               row[Kk - 1] = x[(size_t)(t * Hd + c)];
                           }
                           for (int64_t oc = 0; oc < OC; ++oc) {
                               const int64_t g = oc * groups / OC;
                               float acc = bias.empty() ? 0.f : bias[(size_t)oc];
                               for (int64_t ic = 0; ic < ICg; ++ic)
                                   for (int64_t kk = 0; kk < Kk; ++kk) acc += w[(size_t)((oc * ICg + ic) * Kk + kk)] * state[(size_t)((g * ICg + ic) * Kk + kk)];
                               y[(size_t)(t * Hd + oc)] = acc;
                           }
                       }
                   },
                   [&](int64_t b) { std::copy_n(state.begin(), per_block, table.data() + b * per_block); });
    store_f32(in[1], table);
    out[0] = from_f32(in[0].et, in[0].shape, y);
    return true;
}

// caches [blocks, kv_heads, block_size, head_size] of a whole-byte element type: rows move inside and between blocks
bool eval_pa_kv_reorder(N n, Ins in, Outs out, C) {
    const auto blocks = to_i64(in[2]), bbeg = to_i64(in[3]), upd = to_i64(in[4]), ubeg = to_i64(in[5]);
    for (int which = 0; which < 2; ++which) {
        const Tensor& cache = in[(size_t)which];
        OVC_CHECK(cache.shape.size() == 4 && cache.byte_size() % (size_t)cache.numel() == 0, n.description() << ": caches are [blocks, heads, block_size, head_size] of a whole-byte type");
        const int64_t Hn = cache.shape[1], BS = cache.shape[2], D = cache.shape[3];
        const size_t row = (size_t)D * (cache.byte_size() / (size_t)cache.numel());
        for (size_t s = 0; s + 1 < ubeg.size(); ++s) {
            const int64_t b0 = bbeg[s], b1 = bbeg[s + 1];
            for (int64_t op = ubeg[s]; op < ubeg[s + 1]; ++op) {
                const int64_t src = upd[(size_t)(2 * op)], dst = upd[(size_t)(2 * op + 1)];
                OVC_CHECK(src >= 0 && dst >= 0 && b0 + src / BS < b1 && b0 + dst / BS < b1, n.description() << ": token " << src << " -> " << dst << " is outside the blocks of sequence " << s);
                const int64_t sb = blocks[(size_t)(b0 + src / BS)], db = blocks[(size_t)(b0 + dst / BS)];
                OVC_CHECK(sb >= 0 && sb < cache.shape[0] && db >= 0 && db < cache.shape[0], n.description() << ": block index outside the cache");
                for (int64_t h = 0; h < Hn; ++h)
                    std::memmove(cache.data() + (size_t)(((db * Hn + h) * BS + dst % BS)) * row, cache.data() + (size_t)(((sb * Hn + h) * BS + src % BS)) * row, row);
            }
        }
    }
    out[0] = Tensor(ET::u8, {1});
    out[0].data()[0] = 0;
    return true;
}

// ------------------------------------------------------------------------------------------------ AUGRU
float act(const std::string& name, float v) {
    if (name == "tanh") return std::tanh(v);
    if (name == "relu") return std::max(v, 0.f);
    return 1.f / (1.f + std::exp(-v));
}

// one step for one batch row; gate order in W / R / B is update, reset, hidden
void augru_step(const float* x, float* h, const float* W, const float* R, const float* Bv, float a, int64_t I, int64_t Hs, float clip, const std::string& f, const std::string& g) {
    std::vector<float> z((size_t)Hs), r((size_t)Hs), hh((size_t)Hs);
    auto dot = [](const float* w, const float* v, int64_t len) { float s = 0; for (int64_t i = 0; i < len; ++i) s += w[i] * v[i]; return s; };
    auto clamp = [&](float v) { return clip > 0 ? std::min(std::max(v, -clip), clip) : v; };
    for (int64_t j = 0; j < Hs; ++j) {
        z[(size_t)j] = act(f, clamp(dot(W + j * I, x, I) + dot(R + j * Hs, h, Hs) + Bv[j]));
        r[(size_t)j] = act(f, clamp(dot(W + (Hs + j) * I, x, I) + dot(R + (Hs + j) * Hs, h, Hs) + Bv[Hs + j]));
    }
    std::vector<float> rh((size_t)Hs);
    for (int64_t j = 0; j < Hs; ++j) rh[(size_t)j] = r[(size_t)j] * h[j];
    for (int64_t j = 0; j < Hs; ++j)
        hh[(size_t)j] = act(g, clamp(dot(W + (2 * Hs + j) * I, x, I) + dot(R + (2 * Hs + j) * Hs, rh.data(), Hs) + Bv[2 * Hs + j]));
    for (int64_t j = 0; j < Hs; ++j) {
        const float zz = (1.f - a) * z[(size_t)j];
        h[j] = (1.f - zz) * hh[(size_t)j] + zz * h[j];
    }
}

void activations_of(const Node& n, std::string& f, std::string& g) {
    f = "sigmoid";
    g = "tanh";
    if (n.has_attr("activations")) {
        const auto& a = n.attr("activations").ss;
        if (a.size() > 0) f = a[0];
        if (a.size() > 1) g = a[1];
    }
}

}  // namespace

void register_recurrent_ops() {
    reg("SelectiveSSM", "ie_internal_opset", {},
        [](Node& n) {
            n.set_num_outputs(2);
            n.set_output(0, n.in_et(3), n.in_shape(3));
            n.set_output(1, n.in_et(5), n.in_shape(5));
        }, eval_selective_ssm, 6, 6);

    reg("GatedDeltaNet", "ie_internal_opset", {Ab("fuse_qk_l2norm"), Af("q_l2_norm_eps", 1e-6), Af("k_l2_norm_eps", 1e-6)},
        [](Node& n) {
            n.set_num_outputs(2);
            n.set_output(0, n.in_et(2), n.in_shape(2));
            n.set_output(1, n.in_et(3), n.in_shape(3));
        }, eval_gated_delta_net, 6, 6);

    reg("PagedSelectiveSSM", "ie_internal_opset", {}, [](Node& n) { n.set_output(0, n.in_et(3), n.in_shape(3)); }, eval_paged_selective_ssm, 11, 11, true);
    reg("PagedGatedDeltaNet", "ie_internal_opset", {Ab("use_qk_l2norm"), Af("q_l2_norm_eps", 1e-6), Af("k_l2_norm_eps", 1e-6)},
        [](Node& n) { n.set_output(0, n.in_et(2), n.in_shape(2)); }, eval_paged_gated_delta_net, 11, 11, true);
    reg("PagedCausalConv1D", "ie_internal_opset", {}, [](Node& n) { n.set_output(0, n.in_et(0), n.in_shape(0)); }, eval_paged_causal_conv1d, 9, 9, true);
    reg("PaKVReorder", "ie_internal_opset", {}, [](Node& n) { n.set_output(0, ET::u8, PShape({Dim(1)})); }, eval_pa_kv_reorder, 6, 6, true);

    const std::vector<AttrSpec> gru = {Ai("hidden_size", 0), Ass("activations"), Afs("activations_alpha"), Afs("activations_beta"), Af("clip", 0), Ab("linear_before_reset")};
    reg("AUGRUCell", "ie_internal_opset", gru,
        [](Node& n) { n.set_output(0, n.in_et(0), PShape({dim_of(n.in_shape(0), 0), Dim(n.attr_int("hidden_size"))})); },
        [](N n, Ins in, Outs out, C) {
            OVC_CHECK(!n.attr_bool("linear_before_reset"), n.description() << ": linear_before_reset is not part of the attention-gated cell");
            const auto x = to_f32(in[0]), W = to_f32(in[2]), R = to_f32(in[3]), Bv = to_f32(in[4]), a = to_f32(in[5]);
            auto h = to_f32(in[1]);
            const int64_t Bn = in[0].shape[0], I = in[0].shape[1], Hs = n.attr_int("hidden_size");
            std::string f, g;
            activations_of(n, f, g);
            for (int64_t b = 0; b < Bn; ++b) augru_step(x.data() + b * I, h.data() + b * Hs, W.data(), R.data(), Bv.data(), a[(size_t)b], I, Hs, (float)n.attr_float("clip"), f, g);
            out[0] = from_f32(in[0].et, {Bn, Hs}, h);
            return true;
        }, 6, 6);
    std::vector<AttrSpec> gru_seq = {As("direction", "forward")};
    gru_seq.insert(gru_seq.end(), gru.begin(), gru.end());
    reg("AUGRUSequence", "ie_internal_opset", gru_seq,
        [](Node& n) {
            n.set_num_outputs(2);
            const Dim Bn = dim_of(n.in_shape(0), 0), S = dim_of(n.in_shape(0), 1), Hs(n.attr_int("hidden_size"));
            n.set_output(0, n.in_et(0), PShape({Bn, Dim(1), S, Hs}));
            n.set_output(1, n.in_et(0), PShape({Bn, Dim(1), Hs}));
        },
        [](N n, Ins in, Outs out, C) {
            OVC_CHECK(n.attr_str("direction", "forward") == "forward" && !n.attr_bool("linear_before_reset"), n.description() << ": forward direction without linear_before_reset only");
            const auto x = to_f32(in[0]), W = to_f32(in[3]), R = to_f32(in[4]), Bv = to_f32(in[5]), a = to_f32(in[6]);
            const auto lens = to_i64(in[2]);
            auto h = to_f32(in[1]);
            const int64_t Bn = in[0].shape[0], S = in[0].shape[1], I = in[0].shape[2], Hs = n.attr_int("hidden_size");
            std::string f, g;
            activations_of(n, f, g);
            std::vector<float> y((size_t)(Bn * S * Hs), 0.f);
            for (int64_t b = 0; b < Bn; ++b)
                for (int64_t t = 0; t < std::min<int64_t>(S, lens[(size_t)b]); ++t) {
                    augru_step(x.data() + (b * S + t) * I, h.data() + b * Hs, W.data(), R.data(), Bv.data(), a[(size_t)(b * S + t)], I, Hs, (float)n.attr_float("clip"), f, g);
                    std::copy_n(h.data() + b * Hs, Hs, y.data() + (b * S + t) * Hs);
                }
            out[0] = from_f32(in[0].et, {Bn, 1, S, Hs}, y);
            out[1] = from_f32(in[0].et, {Bn, 1, Hs}, h);
            return true;
        }, 7, 7);
}

}  // namespace ovc
