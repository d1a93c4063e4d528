// Reference kernels of the LLM operations: PagedAttentionExtension, RoPE, MOE.
//
// PagedAttention follows the contract of
// docs/articles_en/documentation/openvino-ir-format/operation-sets/operation-specs/internal/paged-attention.rst
// and src/core/reference/include/openvino/reference/paged_attention.hpp: the new key/value rows of every
// sub-sequence are first written into the block cache, then every new token attends causally to the
// cached tokens of its own sequence. Cache layout of this executor: [num_blocks, kv_heads, block_size,
// head_size] for both K and V (the layout the "CPU" device asks for).
#include "graph.hpp"

namespace ovc {

using Ins = const std::vector<Tensor>&;
using Outs = std::vector<Tensor>&;

static int64_t rt_int(const Node& n, const char* key, int64_t def) {
    auto it = n.rt_info.find(key);
    if (it == n.rt_info.end()) return def;
    if (it->second.kind == Attr::INT) return it->second.i;
    if (it->second.kind == Attr::STR && !it->second.s.empty()) return std::stoll(it->second.s);
    return def;
}

bool eval_paged_attention(const Node& n, Ins in, Outs out, EvalContext&) {
    const Tensor &Q = in[0], &Kn = in[1], &Vn = in[2];
    Tensor kc = in[3], vc = in[4];   // shares the buffers: the caches are updated in place
    OVC_CHECK(kc.shape.size() == 4 && vc.shape.size() == 4, n.description() << ": caches must be [blocks, kv_heads, block_size, head_size]");
    const int64_t Hk = kc.shape[1], bs = kc.shape[2], S = kc.shape[3], Sv = vc.shape[3];
    const int64_t T = Q.shape[0];
    const int64_t Hq = Q.shape[1] / S;
    OVC_CHECK(Hq * S == Q.shape[1] && Kn.shape[1] == Hk * S && Vn.shape[1] == Hk * Sv, n.description() << ": query/key/value widths do not match the cache geometry");
    OVC_CHECK(rt_int(n, "num_k_heads", Hk) == Hk, n.description() << ": cache has " << Hk << " kv heads, the op was built for " << rt_int(n, "num_k_heads", Hk));
    const auto past = to_i64(in[5]), sb = to_i64(in[6]), bi = to_i64(in[7]), bib = to_i64(in[8]);
    const int64_t B = (int64_t)past.size();
    float scale = 1.0f / std::sqrt(float(S));
    if (in.size() > 9 && in[9].numel() > 0) scale = float(get_elem_f64(in[9], 0));
    const int64_t window = (in.size() > 10 && in[10].numel() > 0) ? get_elem_i64(in[10], 0) : 0;
    std::vector<float> alibi;
    if (in.size() > 11 && in[11].numel() > 0) alibi = to_f32(in[11]);
    std::vector<float> sinks;
    if (in.size() > 20 && in[20].numel() > 0) sinks = to_f32(in[20]);
    const int64_t G = Hq / Hk;
    // score aggregation (input 13): 0 = off, N > 0 = the last N new tokens of a sequence vote, N < 0 = all of them
    std::vector<int64_t> score_win;
    if (in.size() > 13 && in[13].numel() > 0) score_win = to_i64(in[13]);
    // re-rotation of cached keys (inputs 14..16): physical blocks whose keys still carry the position they had before an
    // eviction moved them; deltas name the row of the (cos | sin) table per block or per token of the block
    std::vector<int64_t> rot_blocks, rot_deltas;
    std::vector<float> rot_lut;
    int64_t rot_per_block = 1;
    if (in.size() > 16 && in[14].numel() > 0 && in[15].numel() > 0 && in[16].numel() > 0) {
        rot_blocks = to_i64(in[14]);
        rot_deltas = to_i64(in[15]);
        rot_lut = to_f32(in[16]);
        rot_per_block = std::max<int64_t>(1, (int64_t)rot_deltas.size() / (int64_t)rot_blocks.size());
        OVC_CHECK(rot_per_block == 1 || rot_per_block == bs, n.description() << ": rotation_deltas holds one row per block or one per token of a block");
        OVC_CHECK((int64_t)rot_lut.size() % S == 0, n.description() << ": rotation_trig_lut rows must be head_size wide");
    }
    auto q = to_f32(Q), kn = to_f32(Kn), vn = to_f32(Vn);
    const bool write = n.attr_bool("write_kv_cache", true);
    auto slot = [&](int64_t b, int64_t pos) -> int64_t {
        const int64_t blk_i = bib[(size_t)b] + pos / bs;
        OVC_CHECK(blk_i < bib[(size_t)b + 1] && blk_i < (int64_t)bi.size(), n.description() << ": sequence " << b << " has no block for position " << pos);
        return bi[(size_t)blk_i] * bs + pos % bs;
    };
    // 1. write the new rows
    if (write) {
        for (int64_t b = 0; b < B; ++b) {
            for (int64_t t = sb[(size_t)b]; t < sb[(size_t)b + 1]; ++t) {
                const int64_t pos = past[(size_t)b] + (t - sb[(size_t)b]);
                const int64_t sl = slot(b, pos), blk = sl / bs, off = sl % bs;
                for (int64_t h = 0; h < Hk; ++h) {
                    for (int64_t d = 0; d < S; ++d) set_elem_f64(kc, ((blk * Hk + h) * bs + off) * S + d, kn[(size_t)((t * Hk + h) * S + d)]);
                    for (int64_t d = 0; d < Sv; ++d) set_elem_f64(vc, ((blk * Hk + h) * bs + off) * Sv + d, vn[(size_t)((t * Hk + h) * Sv + d)]);
                }
            }
        }
    }
    // 2. attention
    std::vector<float> o((size_t)(T * Hq * Sv), 0.f);
    std::vector<float> s;
    int64_t total_ctx = 0;
    std::vector<int64_t> score_off((size_t)B, 0);
    for (int64_t b = 0; b < B; ++b) { score_off[(size_t)b] = total_ctx; total_ctx += past[(size_t)b] + (sb[(size_t)b + 1] - sb[(size_t)b]); }
    std::vector<float> scores((size_t)total_ctx, 0.f);
    std::vector<float> krow((size_t)S);
    for (int64_t b = 0; b < B; ++b) {
        const int64_t new_len = sb[(size_t)b + 1] - sb[(size_t)b];
        const int64_t win = score_win.empty() ? 0 : score_win[score_win.size() == 1 ? 0 : (size_t)b];
        for (int64_t t = sb[(size_t)b]; t < sb[(size_t)b + 1]; ++t) {
            const int64_t qpos = past[(size_t)b] + (t - sb[(size_t)b]);
            const bool votes = win != 0 && (win < 0 || (new_len - (t - sb[(size_t)b])) <= win);
            const int64_t lo = window > 0 ? std::max<int64_t>(0, qpos - window + 1) : 0;
            const int64_t cnt = qpos - lo + 1;
            s.resize((size_t)cnt);
            for (int64_t h = 0; h < Hq; ++h) {
                const int64_t hk = h / G;
                const float* qp = q.data() + (t * Hq + h) * S;
                float mx = -std::numeric_limits<float>::infinity();
                for (int64_t j = 0; j < cnt; ++j) {
                    const int64_t sl = slot(b, lo + j), blk = sl / bs, off = sl % bs;
                    const int64_t base = ((blk * Hk + hk) * bs + off) * S;
                    for (int64_t d = 0; d < S; ++d) krow[(size_t)d] = float(get_elem_f64(kc, base + d));
                    if (!rot_blocks.empty() && lo + j < past[(size_t)b]) {
                        const auto it = std::find(rot_blocks.begin(), rot_blocks.end(), blk);
                        if (it != rot_blocks.end()) {
                            const int64_t r = it - rot_blocks.begin();
                            const int64_t row = rot_deltas[(size_t)(r * rot_per_block + (rot_per_block == 1 ? 0 : off))];
                            OVC_CHECK(row >= 0 && (row + 1) * S <= (int64_t)rot_lut.size(), n.description() << ": rotation row " << row << " outside the table");
                            const float* lut = rot_lut.data() + row * S;
                            const int64_t half = S / 2;
                            for (int64_t d = 0; d < half; ++d) {
                                const float x0 = krow[(size_t)d], x1 = krow[(size_t)(d + half)];
                                krow[(size_t)d] = x0 * lut[d] - x1 * lut[d + half];
                                krow[(size_t)(d + half)] = x0 * lut[d + half] + x1 * lut[d];
                            }
                        }
                    }
                    float acc = 0;
                    for (int64_t d = 0; d < S; ++d) acc += qp[d] * krow[(size_t)d];
                    acc *= scale;
                    if (!alibi.empty()) acc += alibi[(size_t)h] * float((lo + j) - qpos);
                    s[(size_t)j] = acc;
                    mx = std::max(mx, acc);
                }
                if (!sinks.empty()) mx = std::max(mx, sinks[(size_t)(h % (int64_t)sinks.size())]);
                double sum = 0;
                for (int64_t j = 0; j < cnt; ++j) { s[(size_t)j] = std::exp(s[(size_t)j] - mx); sum += s[(size_t)j]; }
                if (!sinks.empty()) sum += std::exp(sinks[(size_t)(h % (int64_t)sinks.size())] - mx);
                const float inv = sum > 0 ? float(1.0 / sum) : 0.f;
                float* op = o.data() + (t * Hq + h) * Sv;
                for (int64_t j = 0; j < cnt; ++j) {
                    const int64_t sl = slot(b, lo + j), blk = sl / bs, off = sl % bs;
                    const int64_t base = ((blk * Hk + hk) * bs + off) * Sv;
                    const float p = s[(size_t)j] * inv;
                    for (int64_t d = 0; d < Sv; ++d) op[d] += p * float(get_elem_f64(vc, base + d));
                    if (votes) scores[(size_t)(score_off[(size_t)b] + lo + j)] += p;
                }
            }
        }
    }
    out[0] = from_f32(n.outs[0].et == ET::dynamic ? Q.et : n.outs[0].et, Shape{T, Hq * Sv}, o);
    // output 1: one region per sequence (past + new positions), the attention mass each cached position received from the
    // voting queries, summed over the heads; all zeros when aggregation is off
    out[1] = score_win.empty() ? Tensor(out[0].et, Shape{0}) : from_f32(out[0].et, Shape{total_ctx}, scores);
    out[2] = Tensor(out[0].et, Shape{0});
    return true;
}

// RoPE(x, cos, sin[, position ids]); half-rotate (LLaMA / GPT-NeoX) and interleaved (GPT-J) forms.
// x is [B, H, L, S] ([B, L, H, S] with input_trans0213); cos/sin broadcast to [B, 1, L, rotary_ndims]
// (tables of rotary_ndims or rotary_ndims/2 entries per position are both accepted).
// Fused-QKV forms. X is [a, b, W]; the head block [slice_start, slice_stop) of the last axis holds head_cnt heads of head_size.
// Qwen: a = batch, b = tokens; half rotation by tables [1, positions, 1, S] whose LAST b rows belong to these tokens (the
// tables are cut to the present length) unless position ids (input 3) name the rows.
// ChatGLM: a = tokens, b = batch; neighbouring pairs of the first rotary_ndims values rotate by a cache [a, b or 1, 1, rot / 2, 2].
static bool eval_rope_fused_qkv(const Node& n, Ins in, Outs out) {
    const Tensor& X = in[0];
    OVC_CHECK(X.shape.size() == 3, n.description() << ": the fused QKV input must be 3-D");
    const int64_t D0 = X.shape[0], D1 = X.shape[1], W = X.shape[2], H = n.attr_int("head_cnt"), S = n.attr_int("head_size"), s0 = n.attr_int("slice_start");
    OVC_CHECK(H > 0 && S > 0 && s0 >= 0 && s0 + H * S <= W, n.description() << ": heads [" << s0 << ", " << s0 + H * S << ") do not fit the projection of width " << W);
    int64_t rot = n.attr_int("rotary_ndims");
    if (rot <= 0) rot = S;
    const int64_t half = rot / 2;
    const auto x = to_f32(X), c = to_f32(in[1]), s = to_f32(in[2]);
    std::vector<float> o((size_t)(D0 * D1 * H * S));
    if (n.attr_bool("is_qwen")) {
        const int64_t cw = in[1].shape.back(), rows = in[1].numel() / std::max<int64_t>(cw, 1);
        OVC_CHECK(cw == rot, n.description() << ": tables must hold " << rot << " values per position");
        std::vector<int64_t> pos;
        if (in.size() > 3 && in[3].numel() > 0) pos = to_i64(in[3]);
        for (int64_t b = 0; b < D0; ++b) for (int64_t l = 0; l < D1; ++l) {
            int64_t row = rows >= D1 ? rows - D1 + l : std::min(l, rows - 1);
            if (!pos.empty()) row = pos[(size_t)((b * D1 + l) % (int64_t)pos.size())];
            OVC_CHECK(row >= 0 && row < rows, n.description() << ": position " << row << " outside the tables of " << rows << " rows");
            for (int64_t h = 0; h < H; ++h) {
                const float* xp = x.data() + (b * D1 + l) * W + s0 + h * S;
                float* op = o.data() + ((b * D1 + l) * H + h) * S;
                for (int64_t i = 0; i < half; ++i) {
                    op[i] = xp[i] * c[(size_t)(row * cw + i)] - xp[i + half] * s[(size_t)(row * cw + i)];
                    op[i + half] = xp[i + half] * c[(size_t)(row * cw + i + half)] + xp[i] * s[(size_t)(row * cw + i + half)];
                }
                for (int64_t i = rot; i < S; ++i) op[i] = xp[i];
            }
        }
    } else {
        const Shape& cs = in[1].shape;
        OVC_CHECK(cs.size() == 5 && cs[0] >= D0 && cs[3] == half && cs[4] == 2, n.description() << ": the cache must be [tokens, batch or 1, 1, " << half << ", 2]");
        const int64_t Bc = cs[1];
        for (int64_t l = 0; l < D0; ++l) for (int64_t b = 0; b < D1; ++b) for (int64_t h = 0; h < H; ++h) {
            const float* xp = x.data() + (l * D1 + b) * W + s0 + h * S;
            float* op = o.data() + ((l * D1 + b) * H + h) * S;
            const float* cp = c.data() + ((l * Bc + (Bc == 1 ? 0 : b)) * half) * 2;
            for (int64_t i = 0; i < half; ++i) {
                const float x0 = xp[2 * i], x1 = xp[2 * i + 1], cc = cp[2 * i], ss = cp[2 * i + 1];
                op[2 * i] = x0 * cc - x1 * ss;
                op[2 * i + 1] = x1 * cc + x0 * ss;
            }
            for (int64_t i = rot; i < S; ++i) op[i] = xp[i];
        }
    }
    out[0] = from_f32(X.et, Shape{D0, D1, H, S}, o);
    return true;
}

bool eval_rope(const Node& n, Ins in, Outs out, EvalContext&) {
    if (n.attr_bool("is_qwen") || n.attr_bool("is_chatglm")) return eval_rope_fused_qkv(n, in, out);
    const Tensor& X = in[0];
    OVC_CHECK(X.shape.size() == 4, n.description() << ": input must be 4-D");
    const bool it = n.attr_bool("input_trans0213"), ot = n.attr_bool("output_trans0213");
    const int64_t B = X.shape[0], H = it ? X.shape[2] : X.shape[1], L = it ? X.shape[1] : X.shape[2];
    int64_t S = X.shape[3];
    const int64_t s0 = n.attr_int("slice_start"), s1 = n.attr_int("slice_stop");
    const int64_t Sfull = S;
    if (s1 > s0) S = s1 - s0;
    int64_t rot = n.attr_int("rotary_ndims");
    if (rot <= 0) rot = S;
    const int64_t half = rot / 2;
    const bool inter = n.attr_bool("is_interleaved");
    auto x = to_f32(X), c = to_f32(in[1]), s = to_f32(in[2]);
    std::vector<int64_t> pos;
    if (in.size() > 3 && in[3].numel() > 0) pos = to_i64(in[3]);
    // table geometry: last dim = rot or half; the dim before it (if any) runs over positions
    const Shape& cs = in[1].shape;
    const int64_t cw = cs.empty() ? 1 : cs.back();
    const int64_t crow = cs.size() >= 2 ? cs[cs.size() - 2] : 1;
    const int64_t cbatch = in[1].numel() / std::max<int64_t>(1, cw * crow);
    std::vector<float> o((size_t)(B * H * L * S));
    for (int64_t b = 0; b < B; ++b) for (int64_t h = 0; h < H; ++h) for (int64_t l = 0; l < L; ++l) {
        const float* xp = x.data() + (it ? ((b * L + l) * H + h) : ((b * H + h) * L + l)) * Sfull + (s1 > s0 ? s0 : 0);
        float* op = o.data() + (ot ? ((b * L + l) * H + h) : ((b * H + h) * L + l)) * S;
        int64_t row = l;
        if (!pos.empty()) row = pos[(size_t)((pos.size() == (size_t)L) ? l : (b * L + l) % (int64_t)pos.size())];
        if (crow == 1) row = 0; else row = std::min(row, crow - 1);
        const int64_t cb = cbatch > 1 ? std::min(b, cbatch - 1) : 0;
        const float* cp = c.data() + (cb * crow + row) * cw;
        const float* sp = s.data() + (cb * crow + row) * cw;
        for (int64_t i = 0; i < half; ++i) {
            if (inter) {
                const float x0 = xp[2 * i], x1 = xp[2 * i + 1];
                const float cc = cp[cw == rot ? 2 * i : i], ss = sp[cw == rot ? 2 * i : i];
                op[2 * i] = x0 * cc - x1 * ss;
                op[2 * i + 1] = x1 * cc + x0 * ss;
            } else {
                const float x0 = xp[i], x1 = xp[i + half];
                const float c0 = cp[i], sn0 = sp[i];
                const float c1 = cp[cw == rot ? i + half : i], sn1 = sp[cw == rot ? i + half : i];
                op[i] = x0 * c0 - x1 * sn0;
                op[i + half] = x1 * c1 + x0 * sn1;
            }
        }
        for (int64_t i = rot; i < S; ++i) op[i] = xp[i];
    }
    Shape os = ot ? Shape{B, L, H, S} : Shape{B, H, L, S};
    out[0] = from_f32(X.et, os, o);
    return true;
}

// MOE (GEMM3_SWIGLU): hidden [.., H], routing weights [T, k], expert indices [T, k],
// w_gate [E, F, H], w_up [E, F, H], w_down [E, H, F]
bool eval_moe(const Node& n, Ins in, Outs out, EvalContext&) {
    const Tensor& X = in[0];
    const int64_t H = X.shape.back(), T = X.numel() / H;
    auto x = to_f32(X), rw = to_f32(in[1]);
    auto idx = to_i64(in[2]);
    const int64_t k = (int64_t)idx.size() / std::max<int64_t>(T, 1);
    OVC_CHECK(n.attr_str("expert_type") == "GEMM3_SWIGLU", n.description() << ": only GEMM3_SWIGLU experts are implemented by the reference executor");
    const Tensor &W0 = in[3], &W1 = in[4], &W2 = in[5];
    const int64_t E = W0.shape[0], F = W0.shape[1];
    auto w0 = to_f32(W0), w1 = to_f32(W1), w2 = to_f32(W2);
    std::vector<float> o((size_t)(T * H), 0.f), hbuf((size_t)F);
    for (int64_t t = 0; t < T; ++t) for (int64_t j = 0; j < k; ++j) {
        const int64_t e = idx[(size_t)(t * k + j)];
        OVC_CHECK(e >= 0 && e < E, n.description() << ": expert index " << e << " out of range");
        const float wgt = rw[(size_t)(t * k + j)];
        const float* xp = x.data() + t * H;
        for (int64_t f = 0; f < F; ++f) {
            const float* g = w0.data() + (e * F + f) * H;
            const float* u = w1.data() + (e * F + f) * H;
            float ag = 0, au = 0;
            for (int64_t d = 0; d < H; ++d) { ag += xp[d] * g[d]; au += xp[d] * u[d]; }
            hbuf[(size_t)f] = ag / (1.0f + std::exp(-ag)) * au;
        }
        for (int64_t d = 0; d < H; ++d) {
            const float* dw = w2.data() + (e * H + d) * F;
            float acc = 0;
            for (int64_t f = 0; f < F; ++f) acc += hbuf[(size_t)f] * dw[f];
            o[(size_t)(t * H + d)] += wgt * acc;
        }
    }
    out[0] = from_f32(X.et, X.shape, o);
    return true;
}

}  // namespace ovc
