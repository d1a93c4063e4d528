// More of the operation set: attribute schemas (reference visit_attributes order), shape / type inference and the
// reference evaluation of data-movement, detection, signal, recurrent and embedding operations.
//
// Reference counterparts: src/core/src/op/{batch_to_space,space_to_batch,space_to_depth,shuffle_channels,reverse_sequence,
// bucketize,eye,lrn,grn,search_sorted,segment_max,slice_scatter,gather_tree,unique,col2im,inverse,reorg_yolo,roi_align,
// roi_pooling,non_max_suppression,grid_sample,dft,idft,rdft,irdft,lstm_cell,lstm_sequence,gru_cell,gru_sequence,rnn_cell,
// rnn_sequence,ctc_greedy_decoder,ctc_greedy_decoder_seq_len,embeddingbag_offsets_sum,embeddingbag_packedsum,
// embedding_segments_sum,adaptive_max_pool,convolution,group_conv,grouped_matmul,convert_promote_types,random_uniform,
// multinomial,identity,erfinv,bitwise_left_shift,bitwise_right_shift}.cpp and the kernels of the same names under
// src/core/reference/include/openvino/reference/. Real types are computed in fp32 / fp64, integers in int64.
#include <algorithm>
#include <cmath>
#include <complex>
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
AttrSpec Ass(const char* n, std::vector<std::string> d = {}) { return A(n, K::STRS, Attr::Strs(std::move(d))); }
AttrSpec At(const char* n, ET d = ET::dynamic) { return A(n, K::TYPE, Attr::Type(d)); }

void reg(const char* type, const char* version, std::vector<AttrSpec> attrs, InferFn infer, EvalFn eval, int min_in, int max_in,
         bool side_effects = false) {
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

void infer_same(Node& n) { n.set_output(0, n.in_et(0), n.in_shape(0)); }

int64_t norm_axis(int64_t a, int64_t rank, const Node& n) {
    OVC_CHECK(a >= -rank && a < std::max<int64_t>(rank, 1), n.description() << ": axis " << a << " out of range for rank " << rank);
    return a < 0 ? a + rank : a;
}

std::vector<int64_t> strides_of(const Shape& s) {
    std::vector<int64_t> st(s.size(), 1);
    for (int64_t i = (int64_t)s.size() - 2; i >= 0; --i) st[(size_t)i] = st[(size_t)i + 1] * s[(size_t)i + 1];
    return st;
}

// Copy elements of any type by index (bytes per element known; packed sub-byte types are not handled by these ops).
struct Mover {
    size_t es;
    const uint8_t* src;
    uint8_t* dst;
    Mover(const Tensor& in, Tensor& out) : es(et_byte_size(in.et, 1)), src(in.data()), dst(out.data()) {
        OVC_CHECK(et_byte_size(in.et, 8) == 8 * es && es > 0, "sub-byte element types are not supported by this operation");
    }
    void operator()(int64_t to, int64_t from) const { std::memcpy(dst + (size_t)to * es, src + (size_t)from * es, es); }
};

Dim dim_mul(const Dim& d, int64_t k) { return d.is_static() ? Dim(d.lo * k) : Dim::dynamic(); }
Dim dim_div(const Dim& d, int64_t k) { return d.is_static() ? Dim(d.lo / k) : Dim::dynamic(); }

// ------------------------------------------------------------------------------------ activations of the recurrent cells
float activate(const std::string& name, float v, float alpha, float beta) {
    if (name == "sigmoid") return 1.0f / (1.0f + std::exp(-v));
    if (name == "tanh") return std::tanh(v);
    if (name == "relu") return v > 0 ? v : 0.f;
    if (name == "hardsigmoid") return std::min(1.0f, std::max(0.0f, alpha * v + beta));
    OVC_CHECK(false, "unsupported recurrent activation '" << name << "'");
    return 0.f;
}

struct CellAttrs {
    int64_t hidden;
    std::vector<std::string> acts;
    std::vector<double> alpha, beta;
    float clip;
    float act(size_t i, float v) const {
        const float a = i < alpha.size() ? (float)alpha[i] : 0.2f, b = i < beta.size() ? (float)beta[i] : 0.5f;
        return activate(acts.at(i), v, a, b);
    }
    float clipv(float v) const { return clip > 0.f ? std::min(std::max(v, -clip), clip) : v; }
};
CellAttrs cell_attrs(N n, std::vector<std::string> default_acts) {
    CellAttrs c;
    c.hidden = n.attr_int("hidden_size");
    c.acts = n.has_attr("activations") && !n.attr("activations").ss.empty() ? n.attr("activations").ss : default_acts;
    if (n.has_attr("activations_alpha")) c.alpha = n.attr("activations_alpha").fs;
    if (n.has_attr("activations_beta")) c.beta = n.attr("activations_beta").fs;
    c.clip = (float)n.attr_float("clip");
    return c;
}
std::vector<AttrSpec> cell_specs(std::vector<std::string> acts) {
    return {Ai("hidden_size", 0), Ass("activations", std::move(acts)), Afs("activations_alpha"), Afs("activations_beta"), Af("clip", 0.0)};
}

// y[b, :] = x[b, :] W^T + h[b, :] R^T + bias for `gates` stacked blocks of `hidden` rows
void gemv_gates(const float* x, int64_t I, const float* h, int64_t H, const float* W, const float* R, const float* B, int64_t rows, float* y) {
    for (int64_t r = 0; r < rows; ++r) {
        float acc = B ? B[r] : 0.f;
        for (int64_t i = 0; i < I; ++i) acc += x[i] * W[r * I + i];
        for (int64_t i = 0; i < H; ++i) acc += h[i] * R[r * H + i];
        y[r] = acc;
    }
}

// One LSTM step for a batch row. Gate order of the weights: f, i, c, o (the order of the operation set).
void lstm_step(const CellAttrs& a, const float* x, int64_t I, float* h, float* c, const float* W, const float* R, const float* B, std::vector<float>& g) {
    const int64_t H = a.hidden;
    g.resize((size_t)(4 * H));
    gemv_gates(x, I, h, H, W, R, B, 4 * H, g.data());
    for (int64_t k = 0; k < H; ++k) {
        const float f = a.act(0, a.clipv(g[(size_t)k])), i = a.act(0, a.clipv(g[(size_t)(H + k)]));
        const float cc = a.act(1, a.clipv(g[(size_t)(2 * H + k)])), o = a.act(0, a.clipv(g[(size_t)(3 * H + k)]));
        c[k] = f * c[k] + i * cc;
        h[k] = o * a.act(2, c[k]);
    }
}

// One GRU step. Gate order: z, r, h. With linear_before_reset the bias has 4 * H entries (the last block is the recurrent
// bias of the candidate gate, applied before the reset gate multiplies).
void gru_step(const CellAttrs& a, bool lbr, const float* x, int64_t I, float* h, const float* W, const float* R, const float* B, std::vector<float>& tmp) {
    const int64_t H = a.hidden;
    tmp.assign((size_t)(4 * H), 0.f);
    float* zr = tmp.data();            // 2H: z and r pre-activations
    float* hh = tmp.data() + 2 * H;    // H: candidate
    float* rh = tmp.data() + 3 * H;    // H: scratch
    gemv_gates(x, I, h, H, W, R, B, 2 * H, zr);
    for (int64_t k = 0; k < 2 * H; ++k) zr[k] = a.act(0, a.clipv(zr[k]));
    const float* Wh = W + 2 * H * I;
    const float* Rh = R + 2 * H * H;
    if (lbr) {
        for (int64_t k = 0; k < H; ++k) {
            float xw = B ? B[2 * H + k] : 0.f, hr = B ? B[3 * H + k] : 0.f;
            for (int64_t i = 0; i < I; ++i) xw += x[i] * Wh[k * I + i];
            for (int64_t i = 0; i < H; ++i) hr += h[i] * Rh[k * H + i];
            hh[k] = a.act(1, a.clipv(xw + zr[H + k] * hr));
        }
    } else {
        for (int64_t k = 0; k < H; ++k) rh[k] = zr[H + k] * h[k];
        for (int64_t k = 0; k < H; ++k) {
            float acc = B ? B[2 * H + k] : 0.f;
            for (int64_t i = 0; i < I; ++i) acc += x[i] * Wh[k * I + i];
            for (int64_t i = 0; i < H; ++i) acc += rh[i] * Rh[k * H + i];
            hh[k] = a.act(1, a.clipv(acc));
        }
    }
    for (int64_t k = 0; k < H; ++k) h[k] = (1.f - zr[k]) * hh[k] + zr[k] * h[k];
}

void rnn_step(const CellAttrs& a, const float* x, int64_t I, float* h, const float* W, const float* R, const float* B, std::vector<float>& tmp) {
    const int64_t H = a.hidden;
    tmp.resize((size_t)H);
    gemv_gates(x, I, h, H, W, R, B, H, tmp.data());
    for (int64_t k = 0; k < H; ++k) h[k] = a.act(0, a.clipv(tmp[(size_t)k]));
}

// Sequence ops: X [B, T, I], H0 [B, D, H] (, C0), seq_lens [B], W [D, G*H, I], R [D, G*H, H], Bias [D, G'*H];
// outputs Y [B, D, T, H], Ho [B, D, H] (, Co). kind: 0 LSTM, 1 GRU, 2 RNN.
bool eval_sequence(N n, Ins in, Outs out, int kind) {
    const bool lstm = kind == 0;
    const CellAttrs a = cell_attrs(n, kind == 0 ? std::vector<std::string>{"sigmoid", "tanh", "tanh"}
                                                : kind == 1 ? std::vector<std::string>{"sigmoid", "tanh"} : std::vector<std::string>{"tanh"});
    const std::string dir = n.attr_str("direction", "forward");
    const bool lbr = kind == 1 && n.attr_bool("linear_before_reset");
    const Tensor& X = in[0];
    const int64_t Bn = X.shape[0], T = X.shape[1], I = X.shape[2], H = a.hidden;
    const size_t off = lstm ? 1 : 0;
    const auto x = to_f32(X), h0 = to_f32(in[1]), W = to_f32(in[3 + off]), R = to_f32(in[4 + off]), Bi = to_f32(in[5 + off]);
    std::vector<float> c0;
    if (lstm) c0 = to_f32(in[2]);
    const auto lens = to_i64(in[2 + off]);
    const int64_t D = in[1].shape[1], G = kind == 0 ? 4 : kind == 1 ? 3 : 1, GB = (kind == 1 && lbr) ? 4 : G;
    std::vector<float> Y((size_t)(Bn * D * T * H), 0.f), Ho((size_t)(Bn * D * H)), Co(lstm ? (size_t)(Bn * D * H) : 0);
    std::vector<float> tmp;
    for (int64_t d = 0; d < D; ++d) {
        const bool reverse = dir == "reverse" || (dir == "bidirectional" && d == 1);
        const float* Wd = W.data() + d * G * H * I;
        const float* Rd = R.data() + d * G * H * H;
        const float* Bd = Bi.data() + d * GB * H;
        for (int64_t b = 0; b < Bn; ++b) {
            std::vector<float> h(h0.begin() + (b * D + d) * H, h0.begin() + (b * D + d + 1) * H), c;
            if (lstm) c.assign(c0.begin() + (b * D + d) * H, c0.begin() + (b * D + d + 1) * H);
            const int64_t L = std::min<int64_t>(std::max<int64_t>(lens[(size_t)b], 0), T);
            for (int64_t s = 0; s < L; ++s) {
                const int64_t t = reverse ? L - 1 - s : s;
                const float* xt = x.data() + (b * T + t) * I;
                if (kind == 0) lstm_step(a, xt, I, h.data(), c.data(), Wd, Rd, Bd, tmp);
                else if (kind == 1) gru_step(a, lbr, xt, I, h.data(), Wd, Rd, Bd, tmp);
                else rnn_step(a, xt, I, h.data(), Wd, Rd, Bd, tmp);
                std::copy(h.begin(), h.end(), Y.begin() + ((b * D + d) * T + t) * H);
            }
            std::copy(h.begin(), h.end(), Ho.begin() + (b * D + d) * H);
            if (lstm) std::copy(c.begin(), c.end(), Co.begin() + (b * D + d) * H);
        }
    }
    out[0] = from_f32(X.et, Shape{Bn, D, T, H}, Y);
    out[1] = from_f32(X.et, Shape{Bn, D, H}, Ho);
    if (lstm) out[2] = from_f32(X.et, Shape{Bn, D, H}, Co);
    return true;
}

void infer_sequence(Node& n, bool lstm) {
    const PShape& x = n.in_shape(0);
    const PShape& h0 = n.in_shape(1);
    const Dim B = x.rank_dynamic ? Dim::dynamic() : x.dims[0], T = x.rank_dynamic ? Dim::dynamic() : x.dims[1];
    const Dim D = h0.rank_dynamic ? Dim::dynamic() : h0.dims[1];
    const Dim H(n.attr_int("hidden_size"));
    n.set_num_outputs(lstm ? 3 : 2);
    PShape y;
    y.dims = {B, D, T, H};
    PShape hs;
    hs.dims = {B, D, H};
    n.set_output(0, n.in_et(0), y);
    n.set_output(1, n.in_et(0), hs);
    if (lstm) n.set_output(2, n.in_et(0), hs);
}

void infer_cell(Node& n, bool lstm) {
    const PShape& x = n.in_shape(0);
    PShape hs;
    hs.dims = {x.rank_dynamic ? Dim::dynamic() : x.dims[0], Dim(n.attr_int("hidden_size"))};
    n.set_num_outputs(lstm ? 2 : 1);
    n.set_output(0, n.in_et(0), hs);
    if (lstm) n.set_output(1, n.in_et(0), hs);
}

// ------------------------------------------------------------------------------------ bilinear sampling helper
float bilinear(const float* img, int64_t Hh, int64_t Ww, float y, float x) {
    if (y < -1.0f || y > (float)Hh || x < -1.0f || x > (float)Ww) return 0.f;
    y = std::max(y, 0.f);
    x = std::max(x, 0.f);
    int64_t y0 = (int64_t)y, x0 = (int64_t)x, y1, x1;
    if (y0 >= Hh - 1) { y0 = y1 = Hh - 1; y = (float)y0; } else y1 = y0 + 1;
    if (x0 >= Ww - 1) { x0 = x1 = Ww - 1; x = (float)x0; } else x1 = x0 + 1;
    const float ly = y - (float)y0, lx = x - (float)x0, hy = 1.f - ly, hx = 1.f - lx;
    return hy * hx * img[y0 * Ww + x0] + hy * lx * img[y0 * Ww + x1] + ly * hx * img[y1 * Ww + x0] + ly * lx * img[y1 * Ww + x1];
}

// ------------------------------------------------------------------------------------ DFT family
// Complex tensors carry a trailing dimension of 2. Plain O(n^2) transform along one axis at a time.
void dft_axis(std::vector<std::complex<double>>& data, const Shape& shape, size_t axis, int64_t out_len, bool inverse, Shape& new_shape) {
    const int64_t n_in = shape[axis];
    new_shape = shape;
    new_shape[axis] = out_len;
    const auto st_in = strides_of(shape), st_out = strides_of(new_shape);
    std::vector<std::complex<double>> out((size_t)shape_size(new_shape));
    const int64_t outer = shape_size(shape) / n_in;
    const double sign = inverse ? 2.0 * M_PI : -2.0 * M_PI;
    std::vector<int64_t> idx(shape.size());
    for (int64_t o = 0; o < outer; ++o) {
        // decompose o over all dims except `axis`
        int64_t rem = o, base_in = 0, base_out = 0;
        for (int64_t d = (int64_t)shape.size() - 1; d >= 0; --d) {
            if ((size_t)d == axis) continue;
            const int64_t i = rem % shape[(size_t)d];
            rem /= shape[(size_t)d];
            base_in += i * st_in[(size_t)d];
            base_out += i * st_out[(size_t)d];
        }
        for (int64_t k = 0; k < out_len; ++k) {
            std::complex<double> acc(0, 0);
            const int64_t lim = std::min(n_in, out_len);     // the signal is cropped or zero padded to out_len
            for (int64_t t = 0; t < lim; ++t) {
                const double ang = sign * (double)((k * t) % out_len) / (double)out_len;
                acc += data[(size_t)(base_in + t * st_in[axis])] * std::complex<double>(std::cos(ang), std::sin(ang));
            }
            if (inverse) acc /= (double)out_len;
            out[(size_t)(base_out + k * st_out[axis])] = acc;
        }
    }
    data.swap(out);
}

std::vector<int64_t> fft_axes(Ins in, int64_t rank_no_complex) {
    auto axes = to_i64(in[1]);
    for (auto& a : axes) if (a < 0) a += rank_no_complex;
    return axes;
}

// kind: 0 DFT, 1 IDFT, 2 RDFT, 3 IRDFT
bool eval_fft(N, Ins in, Outs out, int kind) {
    const Tensor& x = in[0];
    const bool real_in = kind == 2, real_out = kind == 3;
    Shape cs = x.shape;                       // shape without the trailing 2
    if (!real_in) cs.pop_back();
    const auto axes = fft_axes(in, (int64_t)cs.size());
    std::vector<int64_t> sizes;
    if (in.size() > 2) sizes = to_i64(in[2]);
    const auto v = to_f64(x);
    std::vector<std::complex<double>> data((size_t)shape_size(cs));
    for (size_t i = 0; i < data.size(); ++i) data[i] = real_in ? std::complex<double>(v[i], 0.0) : std::complex<double>(v[2 * i], v[2 * i + 1]);
    Shape cur = cs;
    for (size_t ai = 0; ai < axes.size(); ++ai) {
        const size_t ax = (size_t)axes[ai];
        int64_t len = cur[ax];
        const bool last = ai + 1 == axes.size();
        if (!sizes.empty() && sizes[ai] > 0) len = sizes[ai];
        else if (real_out && last) len = 2 * (cur[ax] - 1);
        if (real_out && last) {
            // rebuild the Hermitian-symmetric spectrum of length `len` along the last transformed axis
            Shape full = cur;
            full[ax] = len;
            const auto si = strides_of(cur), so = strides_of(full);
            std::vector<std::complex<double>> ext((size_t)shape_size(full));
            const int64_t total = shape_size(full);
            for (int64_t o = 0; o < total; ++o) {
                int64_t rem = o, k = 0, src = 0;
                std::vector<int64_t> id(full.size());
                for (int64_t d = (int64_t)full.size() - 1; d >= 0; --d) { id[(size_t)d] = rem % full[(size_t)d]; rem /= full[(size_t)d]; }
                k = id[ax];
                if (k < cur[ax]) {
                    for (size_t d = 0; d < full.size(); ++d) src += id[d] * si[d];
                    ext[(size_t)o] = data[(size_t)src];
                } else {
                    // X[k] = conj(X[len - k]); the other transformed axes are back in the signal domain already (this axis is
                    // the last one to be inverted), so their indices stay as they are
                    for (size_t d = 0; d < full.size(); ++d) src += (d == ax ? len - k : id[d]) * si[d];
                    ext[(size_t)o] = (len - k) < cur[ax] ? std::conj(data[(size_t)src]) : std::complex<double>(0, 0);
                }
            }
            data.swap(ext);
            cur = full;
        }
        Shape ns;
        dft_axis(data, cur, ax, len, kind == 1 || kind == 3, ns);
        cur = ns;
    }
    if (kind == 2) {
        // keep the non-redundant half along the last transformed axis
        const size_t ax = (size_t)axes.back();
        Shape half = cur;
        half[ax] = cur[ax] / 2 + 1;
        const auto si = strides_of(cur), so = strides_of(half);
        std::vector<std::complex<double>> h((size_t)shape_size(half));
        for (int64_t o = 0; o < shape_size(half); ++o) {
            int64_t rem = o, src = 0;
            for (int64_t d = (int64_t)half.size() - 1; d >= 0; --d) { src += (rem % half[(size_t)d]) * si[(size_t)d]; rem /= half[(size_t)d]; }
            h[(size_t)o] = data[(size_t)src];
        }
        data.swap(h);
        cur = half;
    }
    std::vector<double> res;
    Shape os = cur;
    if (real_out) {
        res.resize(data.size());
        for (size_t i = 0; i < data.size(); ++i) res[i] = data[i].real();
    } else {
        res.resize(2 * data.size());
        for (size_t i = 0; i < data.size(); ++i) { res[2 * i] = data[i].real(); res[2 * i + 1] = data[i].imag(); }
        os.push_back(2);
    }
    out[0] = from_f64(x.et, os, res);
    return true;
}

void infer_fft(Node& n, int kind) {
    const PShape& x = n.in_shape(0);
    std::vector<int64_t> axes, sizes;
    if (x.rank_dynamic || !get_constant_ints(n.input(1), axes)) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
    const bool has_sizes = n.num_inputs() > 2 && get_constant_ints(n.input(2), sizes);
    if (n.num_inputs() > 2 && !has_sizes) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
    PShape out = x;
    if (kind != 2) out.dims.pop_back();
    const int64_t r = (int64_t)out.rank();
    for (size_t i = 0; i < axes.size(); ++i) {
        const size_t ax = (size_t)(axes[i] < 0 ? axes[i] + r : axes[i]);
        OVC_CHECK(ax < out.rank(), n.description() << ": axis out of range");
        const bool last = i + 1 == axes.size();
        if (has_sizes && sizes[i] > 0) out.dims[ax] = Dim(sizes[i]);
        else if (kind == 3 && last) out.dims[ax] = out.dims[ax].is_static() ? Dim(2 * (out.dims[ax].lo - 1)) : Dim::dynamic();
        if (kind == 2 && last) out.dims[ax] = out.dims[ax].is_static() ? Dim(out.dims[ax].lo / 2 + 1) : Dim::dynamic();
    }
    if (kind != 3) out.dims.push_back(Dim(2));
    n.set_output(0, n.in_et(0), out);
}

// ------------------------------------------------------------------------------------ boxes
float iou_corner(const float* a, const float* b) {
    const float ay0 = std::min(a[0], a[2]), ax0 = std::min(a[1], a[3]), ay1 = std::max(a[0], a[2]), ax1 = std::max(a[1], a[3]);
    const float by0 = std::min(b[0], b[2]), bx0 = std::min(b[1], b[3]), by1 = std::max(b[0], b[2]), bx1 = std::max(b[1], b[3]);
    const float ih = std::min(ay1, by1) - std::max(ay0, by0), iw = std::min(ax1, bx1) - std::max(ax0, bx0);
    if (ih <= 0 || iw <= 0) return 0.f;
    const float inter = ih * iw, uni = (ay1 - ay0) * (ax1 - ax0) + (by1 - by0) * (bx1 - bx0) - inter;
    return uni > 0 ? inter / uni : 0.f;
}

// Philox 4x32-10 counter-based generator (one block of four 32-bit words per counter value).
struct Philox {
    uint32_t key[2];
    uint64_t counter;
    uint64_t n_extra;
    Philox(uint64_t global_seed, uint64_t op_seed) : counter(0), n_extra(op_seed) {
        key[0] = (uint32_t)global_seed;
        key[1] = (uint32_t)(global_seed >> 32);
    }
    void block(uint32_t out[4]) {
        uint32_t c[4] = {(uint32_t)counter, (uint32_t)(counter >> 32), (uint32_t)n_extra, (uint32_t)(n_extra >> 32)};
        uint32_t k0 = key[0], k1 = key[1];
        for (int r = 0; r < 10; ++r) {
            const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
            const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n1 = (uint32_t)p1, n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1, n3 = (uint32_t)p0;
            c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
            k0 += 0x9E3779B9u;
            k1 += 0xBB67AE85u;
        }
        for (int i = 0; i < 4; ++i) out[i] = c[i];
        ++counter;
    }
    // uniform doubles in [0, 1)
    void fill(std::vector<double>& v) {
        uint32_t w[4];
        for (size_t i = 0; i < v.size(); i += 2) {
            block(w);
            v[i] = (double)((((uint64_t)w[1] & 0x1FFFFFu) << 32) | w[0]) / 9007199254740992.0;
            if (i + 1 < v.size()) v[i + 1] = (double)((((uint64_t)w[3] & 0x1FFFFFu) << 32) | w[2]) / 9007199254740992.0;
        }
    }
};

}  // namespace

void register_ext_ops() {
    // ---- plumbing / element-wise
    reg("Identity", "opset16", {}, infer_same, [](N, Ins in, Outs out, C) { out[0] = in[0]; return true; }, 1, 1);
    reg("ErfInv", "opset17", {}, infer_same,
        [](N, Ins in, Outs out, C) {
            auto v = to_f64(in[0]);
            for (auto& x : v) {
                if (x <= -1.0) { x = x == -1.0 ? -INFINITY : NAN; continue; }
                if (x >= 1.0) { x = x == 1.0 ? INFINITY : NAN; continue; }
                // Winitzki's start value, then Newton steps on erf(y) - x (converges to double precision in three)
                const double a = 0.147, ln = std::log(1.0 - x * x), t = 2.0 / (M_PI * a) + ln / 2.0;
                double y = std::copysign(std::sqrt(std::sqrt(t * t - ln / a) - t), x);
                for (int it = 0; it < 4; ++it) y -= (std::erf(y) - x) / (2.0 / std::sqrt(M_PI) * std::exp(-y * y));
                x = y;
            }
            out[0] = from_f64(in[0].et, in[0].shape, v);
            return true;
        }, 1, 1);
    for (const char* t : {"BitwiseLeftShift", "BitwiseRightShift"}) {
        const bool left = std::string(t) == "BitwiseLeftShift";
        reg(t, "opset15", {As("auto_broadcast", "numpy")},
            [](Node& n) {
                const PShape &a = n.in_shape(0), &b = n.in_shape(1);
                PShape o = PShape::dynamic();
                if (!a.rank_dynamic && !b.rank_dynamic) {
                    const size_t r = std::max(a.rank(), b.rank());
                    o = PShape::dynamic(r);
                    for (size_t i = 0; i < r; ++i) {
                        const Dim da = i < r - a.rank() ? Dim(1) : a.dims[i - (r - a.rank())], db = i < r - b.rank() ? Dim(1) : b.dims[i - (r - b.rank())];
                        o.dims[i] = (da.is_static() && da.lo == 1) ? db : da;
                    }
                }
                n.set_output(0, n.in_et(0), o);
            },
            [left](N, Ins in, Outs out, C) {
                const Shape &sa = in[0].shape, &sb = in[1].shape;
                const size_t r = std::max(sa.size(), sb.size());
                Shape os(r);
                for (size_t i = 0; i < r; ++i) {
                    const int64_t da = i < r - sa.size() ? 1 : sa[i - (r - sa.size())], db = i < r - sb.size() ? 1 : sb[i - (r - sb.size())];
                    os[i] = da == 1 ? db : da;
                }
                const auto a = to_i64(in[0]), b = to_i64(in[1]);
                const auto sta = strides_of(sa), stb = strides_of(sb), sto = strides_of(os);
                std::vector<int64_t> o((size_t)shape_size(os));
                for (int64_t i = 0; i < (int64_t)o.size(); ++i) {
                    int64_t ia = 0, ib = 0, rem = i;
                    for (size_t d = 0; d < r; ++d) {
                        const int64_t id = rem / sto[d];
                        rem %= sto[d];
                        if (d >= r - sa.size() && sa[d - (r - sa.size())] != 1) ia += id * sta[d - (r - sa.size())];
                        if (d >= r - sb.size() && sb[d - (r - sb.size())] != 1) ib += id * stb[d - (r - sb.size())];
                    }
                    const int64_t sh = b[(size_t)ib];
                    o[(size_t)i] = sh < 0 || sh >= 64 ? 0 : (left ? (int64_t)((uint64_t)a[(size_t)ia] << sh) : (a[(size_t)ia] >> sh));
                }
                out[0] = from_i64(in[0].et, os, o);
                return true;
            }, 2, 2);
    }
    reg("ConvertPromoteTypes", "opset14", {Ab("promote_unsafe", false), Ab("pytorch_scalar_promotion", false), At("u64_integer_promotion_target", ET::f32)},
        [](Node& n) {
            const ET a = n.in_et(0), b = n.in_et(1);
            ET t = a;
            if (a != b && a != ET::dynamic && b != ET::dynamic) {
                const bool ra = et_is_real(a), rb = et_is_real(b);
                auto bits = [](ET e) { return (int)et_byte_size(e, 8); };      // bits per element
                if (ra != rb) t = ra ? a : b;                                   // a real type wins over an integer one
                else if (ra) t = bits(a) >= bits(b) ? a : b;
                else {
                    const bool sa = a == ET::i8 || a == ET::i16 || a == ET::i32 || a == ET::i64 || a == ET::i4;
                    const bool sb = b == ET::i8 || b == ET::i16 || b == ET::i32 || b == ET::i64 || b == ET::i4;
                    if (a == ET::boolean) t = b;
                    else if (b == ET::boolean) t = a;
                    else if (sa == sb) t = bits(a) >= bits(b) ? a : b;
                    else {
                        // signed with unsigned: the signed type when it is wider, else the next wider signed type
                        const ET s = sa ? a : b, u = sa ? b : a;
                        if (bits(s) > bits(u)) t = s;
                        else t = bits(u) < 16 ? ET::i16 : bits(u) < 32 ? ET::i32 : bits(u) < 64 ? ET::i64 : n.attr("u64_integer_promotion_target").et;
                    }
                }
            }
            n.set_num_outputs(2);
            n.set_output(0, t, n.in_shape(0));
            n.set_output(1, t, n.in_shape(1));
        },
        [](N n, Ins in, Outs out, C) {
            out[0] = convert_tensor(in[0], n.outs[0].et);
            out[1] = convert_tensor(in[1], n.outs[1].et);
            return true;
        }, 2, 2);

    // ---- layout
    reg("SpaceToDepth", "opset1", {Ai("block_size", 1), As("mode", "blocks_first")},
        [](Node& n) {
            const PShape& in = n.in_shape(0);
            if (in.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
            const int64_t b = n.attr_int("block_size");
            PShape o = in;
            int64_t mul = 1;
            for (size_t i = 2; i < in.rank(); ++i) { o.dims[i] = dim_div(in.dims[i], b); mul *= b; }
            o.dims[1] = dim_mul(in.dims[1], mul);
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const int64_t b = n.attr_int("block_size");
            const bool first = n.attr_str("mode") == "blocks_first";
            const size_t sp = x.shape.size() - 2;
            Shape os = x.shape;
            int64_t blocks = 1;
            for (size_t i = 0; i < sp; ++i) { os[2 + i] /= b; blocks *= b; }
            os[1] *= blocks;
            Tensor o(x.et, os);
            Mover mv(x, o);
            const auto si = strides_of(x.shape), so = strides_of(os);
            const int64_t Cin = x.shape[1];
            for (int64_t i = 0; i < x.numel(); ++i) {
                int64_t rem = i, nb = rem / si[0];
                rem %= si[0];
                const int64_t c = rem / si[1];
                rem %= si[1];
                int64_t blk = 0, dst = nb * so[0];
                for (size_t d = 0; d < sp; ++d) {
                    const int64_t p = rem / si[2 + d];
                    rem %= si[2 + d];
                    blk = blk * b + p % b;
                    dst += (p / b) * so[2 + d];
                }
                const int64_t oc = first ? blk * Cin + c : c * blocks + blk;
                mv(dst + oc * so[1], i);
            }
            out[0] = o;
            return true;
        }, 1, 1);
    auto infer_b2s = [](Node& n, bool to_batch) {
        const PShape& in = n.in_shape(0);
        std::vector<int64_t> bs, pb, pe;
        if (in.rank_dynamic || !get_constant_ints(n.input(1), bs) || !get_constant_ints(n.input(2), pb) || !get_constant_ints(n.input(3), pe)) {
            n.set_output(0, n.in_et(0), in.rank_dynamic ? PShape::dynamic() : PShape::dynamic(in.rank()));
            return;
        }
        PShape o = in;
        int64_t prod = 1;
        for (auto b : bs) prod *= b;
        for (size_t i = 1; i < in.rank(); ++i) {
            if (!in.dims[i].is_static()) { o.dims[i] = Dim::dynamic(); continue; }
            o.dims[i] = to_batch ? Dim((in.dims[i].lo + pb[i] + pe[i]) / bs[i]) : Dim(in.dims[i].lo * bs[i] - pb[i] - pe[i]);
        }
        o.dims[0] = to_batch ? dim_mul(in.dims[0], prod) : dim_div(in.dims[0], prod);
        n.set_output(0, n.in_et(0), o);
    };
    // SpaceToBatch: pad, then move block offsets of every spatial axis into the batch (batch index = offset-major)
    reg("SpaceToBatch", "opset2", {}, [infer_b2s](Node& n) { infer_b2s(n, true); },
        [](N, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const auto bs = to_i64(in[1]), pb = to_i64(in[2]), pe = to_i64(in[3]);
            const size_t r = x.shape.size();
            Shape padded = x.shape, os = x.shape;
            int64_t prod = 1;
            for (size_t i = 1; i < r; ++i) { padded[i] += pb[i] + pe[i]; os[i] = padded[i] / bs[i]; prod *= bs[i]; }
            os[0] = x.shape[0] * prod;
            Tensor o(x.et, os);
            std::memset(o.data(), 0, o.byte_size());
            Mover mv(x, o);
            const auto si = strides_of(x.shape), so = strides_of(os);
            for (int64_t i = 0; i < x.numel(); ++i) {
                int64_t rem = i, dst = 0, off = 0;
                const int64_t nb = rem / si[0];
                rem %= si[0];
                for (size_t d = 1; d < r; ++d) {
                    const int64_t p = rem / si[d] + pb[d];
                    rem %= si[d];
                    off = off * bs[d] + p % bs[d];
                    dst += (p / bs[d]) * so[d];
                }
                mv(dst + (off * x.shape[0] + nb) * so[0], i);
            }
            out[0] = o;
            return true;
        }, 4, 4);
    reg("BatchToSpace", "opset2", {}, [infer_b2s](Node& n) { infer_b2s(n, false); },
        [](N, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const auto bs = to_i64(in[1]), cb = to_i64(in[2]), ce = to_i64(in[3]);
            const size_t r = x.shape.size();
            int64_t prod = 1;
            for (size_t i = 1; i < r; ++i) prod *= bs[i];
            Shape os = x.shape;
            os[0] = x.shape[0] / prod;
            for (size_t i = 1; i < r; ++i) os[i] = x.shape[i] * bs[i] - cb[i] - ce[i];
            Tensor o(x.et, os);
            Mover mv(x, o);
            const auto si = strides_of(x.shape), so = strides_of(os);
            for (int64_t i = 0; i < x.numel(); ++i) {
                int64_t rem = i;
                const int64_t b_in = rem / si[0];
                rem %= si[0];
                int64_t off = b_in / os[0];
                const int64_t nb = b_in % os[0];
                // offsets were packed first-axis-major
                std::vector<int64_t> offs(r, 0);
                for (size_t d = r - 1; d >= 1; --d) { offs[d] = off % bs[d]; off /= bs[d]; }
                int64_t dst = nb * so[0];
                bool inside = true;
                for (size_t d = 1; d < r; ++d) {
                    const int64_t p = (rem / si[d]) * bs[d] + offs[d] - cb[d];
                    rem %= si[d];
                    if (p < 0 || p >= os[d]) { inside = false; break; }
                    dst += p * so[d];
                }
                if (inside) mv(dst, i);
            }
            out[0] = o;
            return true;
        }, 4, 4);
    reg("ShuffleChannels", "opset1", {Ai("axis", 1), Ai("group", 1)}, infer_same,
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const int64_t ax = norm_axis(n.attr_int("axis"), (int64_t)x.shape.size(), n), g = n.attr_int("group");
            const int64_t Cn = x.shape[(size_t)ax], per = Cn / g;
            int64_t outer = 1, inner = 1;
            for (int64_t i = 0; i < ax; ++i) outer *= x.shape[(size_t)i];
            for (size_t i = (size_t)ax + 1; i < x.shape.size(); ++i) inner *= x.shape[i];
            Tensor o(x.et, x.shape);
            const size_t es = et_byte_size(x.et, 1);
            for (int64_t a = 0; a < outer; ++a)
                for (int64_t c = 0; c < Cn; ++c) {
                    const int64_t dc = (c % per) * g + c / per;
                    std::memcpy(o.data() + (size_t)((a * Cn + dc) * inner) * es, x.data() + (size_t)((a * Cn + c) * inner) * es, (size_t)inner * es);
                }
            out[0] = o;
            return true;
        }, 1, 1);
    reg("ReverseSequence", "opset1", {Ai("batch_axis", 0), Ai("seq_axis", 1)}, infer_same,
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const int64_t r = (int64_t)x.shape.size(), ba = norm_axis(n.attr_int("batch_axis"), r, n), sa = norm_axis(n.attr_int("seq_axis"), r, n);
            const auto lens = to_i64(in[1]);
            Tensor o(x.et, x.shape);
            Mover mv(x, o);
            const auto st = strides_of(x.shape);
            for (int64_t i = 0; i < x.numel(); ++i) {
                const int64_t b = (i / st[(size_t)ba]) % x.shape[(size_t)ba], s = (i / st[(size_t)sa]) % x.shape[(size_t)sa];
                const int64_t L = lens[(size_t)b];
                const int64_t ns = s < L ? L - 1 - s : s;
                mv(i + (ns - s) * st[(size_t)sa], i);
            }
            out[0] = o;
            return true;
        }, 2, 2);
    reg("ReorgYolo", "opset2", {Ais("stride", {1})},
        [](Node& n) {
            const PShape& in = n.in_shape(0);
            if (in.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
            const int64_t s = n.attr_ints("stride").at(0);
            PShape o = in;
            o.dims[1] = dim_mul(in.dims[1], s * s);
            for (size_t i = 2; i < in.rank(); ++i) o.dims[i] = dim_div(in.dims[i], s);
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const int64_t s = n.attr_ints("stride").at(0), B = x.shape[0], Cc = x.shape[1], H = x.shape[2], W = x.shape[3];
            Shape os{B, Cc * s * s, H / s, W / s};
            Tensor o(x.et, os);
            Mover mv(x, o);
            // the darknet reorg: the output is indexed like the input and reads from the "expanded" view
            const int64_t oc = Cc / (s * s);
            for (int64_t b = 0; b < B; ++b)
                for (int64_t k = 0; k < Cc; ++k)
                    for (int64_t j = 0; j < H; ++j)
                        for (int64_t i = 0; i < W; ++i) {
                            const int64_t c2 = k % oc, offset = k / oc;
                            const int64_t w2 = i * s + offset % s, h2 = j * s + offset / s;
                            mv(i + W * (j + H * (k + Cc * b)), w2 + W * s * (h2 + H * s * (c2 + oc * b)));
                        }
            out[0] = o;
            return true;
        }, 1, 1);

    // ---- search / bucket / generate
    reg("Bucketize", "opset3", {At("output_type", ET::i64), Ab("with_right_bound", true)},
        [](Node& n) { n.set_output(0, n.attr("output_type").et, n.in_shape(0)); },
        [](N n, Ins in, Outs out, C) {
            const auto v = to_f64(in[0]), b = to_f64(in[1]);
            const bool right = n.attr_bool("with_right_bound");
            std::vector<int64_t> o(v.size());
            for (size_t i = 0; i < v.size(); ++i)
                o[i] = right ? std::lower_bound(b.begin(), b.end(), v[i]) - b.begin() : std::upper_bound(b.begin(), b.end(), v[i]) - b.begin();
            out[0] = from_i64(n.attr("output_type").et, in[0].shape, o);
            return true;
        }, 2, 2);
    reg("SearchSorted", "opset15", {Ab("right_mode", false), At("output_type", ET::i64)},
        [](Node& n) { n.set_output(0, n.attr("output_type").et, n.in_shape(1)); },
        [](N n, Ins in, Outs out, C) {
            const auto s = to_f64(in[0]), v = to_f64(in[1]);
            const int64_t L = in[0].shape.back(), M = in[1].shape.back();
            const bool right = n.attr_bool("right_mode");
            std::vector<int64_t> o(v.size());
            for (size_t i = 0; i < v.size(); ++i) {
                const int64_t row = (int64_t)i / M;
                auto b = s.begin() + row * L, e = b + L;
                o[i] = (right ? std::upper_bound(b, e, v[i]) : std::lower_bound(b, e, v[i])) - b;
            }
            out[0] = from_i64(n.attr("output_type").et, in[1].shape, o);
            return true;
        }, 2, 2);
    reg("Eye", "opset9", {At("output_type", ET::f32)},
        [](Node& n) {
            std::vector<int64_t> r, c, bsh;
            PShape o = PShape::dynamic();
            if (get_constant_ints(n.input(0), r) && get_constant_ints(n.input(1), c)) {
                o = PShape();
                if (n.num_inputs() > 3) {
                    if (!get_constant_ints(n.input(3), bsh)) { n.set_output(0, n.attr("output_type").et, PShape::dynamic()); return; }
                    for (auto b : bsh) o.dims.push_back(Dim(b));
                }
                o.dims.push_back(Dim(r.at(0)));
                o.dims.push_back(Dim(c.at(0)));
            }
            n.set_output(0, n.attr("output_type").et, o);
        },
        [](N n, Ins in, Outs out, C) {
            const int64_t R = to_i64(in[0]).at(0), Cc = to_i64(in[1]).at(0), k = to_i64(in[2]).at(0);
            Shape os;
            if (in.size() > 3) for (auto b : to_i64(in[3])) os.push_back(b);
            int64_t batch = 1;
            for (auto b : os) batch *= b;
            os.push_back(R);
            os.push_back(Cc);
            std::vector<double> v((size_t)(batch * R * Cc), 0.0);
            for (int64_t b = 0; b < batch; ++b)
                for (int64_t i = 0; i < R; ++i) if (i + k >= 0 && i + k < Cc) v[(size_t)((b * R + i) * Cc + i + k)] = 1.0;
            out[0] = from_f64(n.attr("output_type").et, os, v);
            return true;
        }, 3, 4);
    reg("RandomUniform", "opset8", {At("output_type", ET::f32), Ai("op_seed", 0), Ai("global_seed", 0), As("alignment", "TENSORFLOW")},
        [](Node& n) {
            std::vector<int64_t> sh;
            PShape o = PShape::dynamic();
            if (get_constant_ints(n.input(0), sh)) { o = PShape(); for (auto d : sh) o.dims.push_back(Dim(d)); }
            n.set_output(0, n.attr("output_type").et, o);
        },
        [](N n, Ins in, Outs out, C) {
            Shape os;
            for (auto d : to_i64(in[0])) os.push_back(d);
            const double lo = get_elem_f64(in[1], 0), hi = get_elem_f64(in[2], 0);
            std::vector<double> u((size_t)shape_size(os));
            Philox(n.attr_int("global_seed"), n.attr_int("op_seed")).fill(u);
            const ET et = n.attr("output_type").et;
            if (et_is_real(et)) {
                for (auto& x : u) x = lo + x * (hi - lo);
                out[0] = from_f64(et, os, u);
            } else {
                std::vector<int64_t> v(u.size());
                for (size_t i = 0; i < u.size(); ++i) v[i] = (int64_t)std::floor(lo + u[i] * (hi - lo));
                out[0] = from_i64(et, os, v);
            }
            return true;
        }, 3, 3, /*side_effects=*/true);
    reg("Multinomial", "opset13", {At("convert_type", ET::i64), Ab("with_replacement", false), Ab("log_probs", false), Ai("global_seed", 0), Ai("op_seed", 0)},
        [](Node& n) {
            const PShape& p = n.in_shape(0);
            std::vector<int64_t> ns;
            PShape o = PShape::dynamic(2);
            if (!p.rank_dynamic) o.dims[0] = p.dims[0];
            if (get_constant_ints(n.input(1), ns)) o.dims[1] = Dim(ns.at(0));
            n.set_output(0, n.attr("convert_type").et, o);
        },
        [](N n, Ins in, Outs out, C) {
            auto p = to_f64(in[0]);
            const int64_t B = in[0].shape[0], V = in[0].shape[1], S = to_i64(in[1]).at(0);
            const bool repl = n.attr_bool("with_replacement");
            if (n.attr_bool("log_probs")) for (auto& x : p) x = std::exp(x);
            std::vector<double> u((size_t)(B * S));
            Philox(n.attr_int("global_seed"), n.attr_int("op_seed")).fill(u);
            std::vector<int64_t> o((size_t)(B * S));
            for (int64_t b = 0; b < B; ++b) {
                std::vector<double> w(p.begin() + b * V, p.begin() + (b + 1) * V);
                for (int64_t s = 0; s < S; ++s) {
                    const double total = std::accumulate(w.begin(), w.end(), 0.0);
                    double target = u[(size_t)(b * S + s)] * total, acc = 0;
                    int64_t pick = V - 1;
                    for (int64_t v = 0; v < V; ++v) { acc += w[(size_t)v]; if (acc > target) { pick = v; break; } }
                    o[(size_t)(b * S + s)] = pick;
                    if (!repl) w[(size_t)pick] = 0.0;
                }
            }
            out[0] = from_i64(n.attr("convert_type").et, Shape{B, S}, o);
            return true;
        }, 2, 2, /*side_effects=*/true);

    // ---- normalisation across channels
    reg("LRN", "opset1", {Af("alpha", 1.0, false), Af("beta", 1.0, false), Af("bias", 1.0, false), Ai("size", 1)}, infer_same,
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const auto v = to_f32(x);
            auto axes = to_i64(in[1]);
            const int64_t r = (int64_t)x.shape.size(), size = n.attr_int("size");
            for (auto& a : axes) if (a < 0) a += r;
            const double alpha = n.attr_float("alpha"), beta = n.attr_float("beta"), bias = n.attr_float("bias");
            const auto st = strides_of(x.shape);
            std::vector<float> o(v.size());
            const int64_t lo = -(size - 1) / 2, hi = size / 2;     // window [i + lo, i + hi]
            const double norm = alpha / std::pow((double)size, (double)axes.size());
            for (int64_t i = 0; i < (int64_t)v.size(); ++i) {
                // enumerate the window over all normalised axes
                double sq = 0;
                std::vector<int64_t> off(axes.size(), lo);
                for (;;) {
                    int64_t j = i;
                    bool ok = true;
                    for (size_t a = 0; a < axes.size(); ++a) {
                        const int64_t ax = axes[a], pos = (i / st[(size_t)ax]) % x.shape[(size_t)ax] + off[a];
                        if (pos < 0 || pos >= x.shape[(size_t)ax]) { ok = false; break; }
                        j += off[a] * st[(size_t)ax];
                    }
                    if (ok) sq += (double)v[(size_t)j] * v[(size_t)j];
                    size_t a = 0;
                    while (a < off.size() && ++off[a] > hi) { off[a] = lo; ++a; }
                    if (a == off.size()) break;
                }
                o[(size_t)i] = (float)(v[(size_t)i] / std::pow(bias + norm * sq, beta));
            }
            out[0] = from_f32(x.et, x.shape, o);
            return true;
        }, 2, 2);
    reg("GRN", "opset1", {Af("bias", 1.0)}, infer_same,
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const auto v = to_f32(x);
            const int64_t B = x.shape[0], Cc = x.shape[1], inner = x.numel() / (B * Cc);
            const float bias = (float)n.attr_float("bias");
            std::vector<float> o(v.size());
            for (int64_t b = 0; b < B; ++b)
                for (int64_t i = 0; i < inner; ++i) {
                    float sq = bias;
                    for (int64_t c = 0; c < Cc; ++c) { const float e = v[(size_t)((b * Cc + c) * inner + i)]; sq += e * e; }
                    const float inv = 1.0f / std::sqrt(sq);
                    for (int64_t c = 0; c < Cc; ++c) o[(size_t)((b * Cc + c) * inner + i)] = v[(size_t)((b * Cc + c) * inner + i)] * inv;
                }
            out[0] = from_f32(x.et, x.shape, o);
            return true;
        }, 1, 1);

    // ---- segments / scatter / trees
    reg("SegmentMax", "opset16", {As("fill_mode", "ZERO")},
        [](Node& n) {
            const PShape& d = n.in_shape(0);
            if (d.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
            PShape o = d;
            std::vector<int64_t> ns, ids;
            if (n.num_inputs() > 2 && get_constant_ints(n.input(2), ns)) o.dims[0] = Dim(ns.at(0));
            else if (get_constant_ints(n.input(1), ids) && !ids.empty()) o.dims[0] = Dim(ids.back() + 1);
            else o.dims[0] = Dim::dynamic();
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const auto v = to_f64(x);
            const auto ids = to_i64(in[1]);
            const int64_t rows = x.shape[0], inner = rows ? x.numel() / rows : 0;
            int64_t segs = ids.empty() ? 0 : ids.back() + 1;
            if (in.size() > 2) segs = to_i64(in[2]).at(0);
            const bool lowest = n.attr_str("fill_mode") == "LOWEST";
            const double fill = lowest ? (et_is_real(x.et) ? -std::numeric_limits<double>::max() : (double)std::numeric_limits<int32_t>::min()) : 0.0;
            std::vector<double> o((size_t)(segs * inner), fill);
            std::vector<char> seen((size_t)segs, 0);
            for (int64_t r = 0; r < rows; ++r) {
                const int64_t s = ids[(size_t)r];
                if (s < 0 || s >= segs) continue;
                for (int64_t i = 0; i < inner; ++i) {
                    double& d = o[(size_t)(s * inner + i)];
                    d = seen[(size_t)s] ? std::max(d, v[(size_t)(r * inner + i)]) : v[(size_t)(r * inner + i)];
                }
                seen[(size_t)s] = 1;
            }
            Shape os = x.shape;
            os[0] = segs;
            out[0] = from_f64(x.et, os, o);
            return true;
        }, 2, 3);
    reg("SliceScatter", "opset15", {}, infer_same,
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const Tensor& u = in[1];
            const auto start = to_i64(in[2]), stop = to_i64(in[3]), step = to_i64(in[4]);
            const int64_t r = (int64_t)x.shape.size();
            std::vector<int64_t> axes(start.size());
            std::iota(axes.begin(), axes.end(), 0);
            if (in.size() > 5) axes = to_i64(in[5]);
            std::vector<int64_t> b(r, 0), s(r, 1);
            for (size_t i = 0; i < axes.size(); ++i) {
                const int64_t ax = norm_axis(axes[i], r, n), dim = x.shape[(size_t)ax];
                int64_t st = start[i];
                if (st < 0) st += dim;
                st = step[i] > 0 ? std::min(std::max<int64_t>(st, 0), dim) : std::min(std::max<int64_t>(st, -1), dim - 1);
                b[(size_t)ax] = st;
                s[(size_t)ax] = step[i];
                (void)stop;
            }
            Tensor o(x.et, x.shape);
            std::memcpy(o.data(), x.data(), x.byte_size());
            Mover mv(u, o);
            const auto su = strides_of(u.shape), sx = strides_of(x.shape);
            for (int64_t i = 0; i < u.numel(); ++i) {
                int64_t rem = i, dst = 0;
                for (int64_t d = 0; d < r; ++d) {
                    const int64_t id = rem / su[(size_t)d];
                    rem %= su[(size_t)d];
                    dst += (b[(size_t)d] + id * s[(size_t)d]) * sx[(size_t)d];
                }
                mv(dst, i);
            }
            out[0] = o;
            return true;
        }, 5, 6);
    reg("GatherTree", "opset1", {}, infer_same,
        [](N, Ins in, Outs out, C) {
            // step_ids / parent_idx [T, B, beam]; max_seq_len [B]; end_token scalar
            const auto ids = to_i64(in[0]), par = to_i64(in[1]), len = to_i64(in[2]);
            const int64_t end = to_i64(in[3]).at(0), T = in[0].shape[0], B = in[0].shape[1], W = in[0].shape[2];
            std::vector<int64_t> o(ids.size(), end);
            for (int64_t b = 0; b < B; ++b)
                for (int64_t w = 0; w < W; ++w) {
                    const int64_t L = std::min<int64_t>(len[(size_t)b], T);
                    if (L <= 0) continue;
                    int64_t parent = w;
                    for (int64_t t = L - 1; t >= 0; --t) {
                        o[(size_t)((t * B + b) * W + w)] = ids[(size_t)((t * B + b) * W + parent)];
                        parent = par[(size_t)((t * B + b) * W + parent)];
                    }
                    bool finished = false;
                    for (int64_t t = 0; t < L; ++t) {
                        int64_t& e = o[(size_t)((t * B + b) * W + w)];
                        if (finished) e = end;
                        else if (e == end) finished = true;
                    }
                }
            out[0] = from_i64(in[0].et, in[0].shape, o);
            return true;
        }, 4, 4);
    reg("Unique", "opset10", {Ab("sorted", true), At("index_element_type", ET::i64), At("count_element_type", ET::i64)},
        [](Node& n) {
            const PShape& in = n.in_shape(0);
            n.set_num_outputs(4);
            PShape flat = PShape::dynamic(1);
            if (in.is_static()) flat.dims[0] = Dim(1, std::max<int64_t>(1, shape_size(in.to_shape())));
            PShape uq = flat;
            if (n.num_inputs() > 1 && !in.rank_dynamic) {
                std::vector<int64_t> ax;
                uq = PShape::dynamic(in.rank());
                if (get_constant_ints(n.input(1), ax)) {
                    const size_t a = (size_t)(ax.at(0) < 0 ? ax.at(0) + (int64_t)in.rank() : ax.at(0));
                    uq = in;
                    uq.dims[a] = in.dims[a].is_static() ? Dim(1, std::max<int64_t>(in.dims[a].lo, 1)) : Dim::dynamic();
                    flat = PShape::dynamic(1);
                    flat.dims[0] = uq.dims[a];
                }
            }
            n.set_output(0, n.in_et(0), uq);
            n.set_output(1, n.attr("index_element_type").et, flat);
            PShape rev = PShape::dynamic(1);
            if (in.is_static()) rev.dims[0] = Dim(n.num_inputs() > 1 ? -1 : shape_size(in.to_shape()));
            n.set_output(2, n.attr("index_element_type").et, n.num_inputs() > 1 ? PShape::dynamic(1) : rev);
            n.set_output(3, n.attr("count_element_type").et, flat);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const bool sorted = n.attr_bool("sorted");
            int64_t axis = -1;
            if (in.size() > 1) axis = norm_axis(to_i64(in[1]).at(0), (int64_t)x.shape.size(), n);
            const auto v = to_f64(x);
            // a "slice" is one element (flattened) or one hyper-plane along `axis`
            int64_t count = x.numel(), outer = 1, inner = 1;
            if (axis >= 0) {
                count = x.shape[(size_t)axis];
                for (int64_t i = 0; i < axis; ++i) outer *= x.shape[(size_t)i];
                for (size_t i = (size_t)axis + 1; i < x.shape.size(); ++i) inner *= x.shape[i];
            }
            auto slice = [&](int64_t s) {
                std::vector<double> r;
                if (axis < 0) { r.push_back(v[(size_t)s]); return r; }
                for (int64_t o = 0; o < outer; ++o) for (int64_t i = 0; i < inner; ++i) r.push_back(v[(size_t)((o * count + s) * inner + i)]);
                return r;
            };
            std::vector<std::vector<double>> uniq;
            std::vector<int64_t> first, rev((size_t)count), cnt;
            for (int64_t s = 0; s < count; ++s) {
                const auto sl = slice(s);
                size_t u = 0;
                for (; u < uniq.size(); ++u) if (uniq[u] == sl) break;
                if (u == uniq.size()) { uniq.push_back(sl); first.push_back(s); cnt.push_back(0); }
                rev[(size_t)s] = (int64_t)u;
                ++cnt[u];
            }
            std::vector<size_t> order(uniq.size());
            std::iota(order.begin(), order.end(), 0);
            if (sorted) std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return uniq[a] < uniq[b]; });
            std::vector<int64_t> pos(uniq.size());
            for (size_t i = 0; i < order.size(); ++i) pos[order[i]] = (int64_t)i;
            const int64_t U = (int64_t)uniq.size();
            Shape us = axis < 0 ? Shape{U} : x.shape;
            if (axis >= 0) us[(size_t)axis] = U;
            std::vector<double> uv((size_t)shape_size(us));
            std::vector<int64_t> f((size_t)U), c((size_t)U);
            for (int64_t i = 0; i < U; ++i) {
                const size_t u = order[(size_t)i];
                f[(size_t)i] = first[u];
                c[(size_t)i] = cnt[u];
                if (axis < 0) uv[(size_t)i] = uniq[u][0];
                else for (int64_t o = 0; o < outer; ++o) for (int64_t k = 0; k < inner; ++k) uv[(size_t)((o * U + i) * inner + k)] = uniq[u][(size_t)(o * inner + k)];
            }
            for (auto& r : rev) r = pos[(size_t)r];
            out[0] = from_f64(x.et, us, uv);
            out[1] = from_i64(n.attr("index_element_type").et, Shape{U}, f);
            out[2] = from_i64(n.attr("index_element_type").et, Shape{count}, rev);
            out[3] = from_i64(n.attr("count_element_type").et, Shape{U}, c);
            return true;
        }, 1, 2);

    // ---- linear algebra
    reg("Inverse", "opset14", {Ab("adjoint", false)}, infer_same,
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const int64_t M = x.shape.back(), batch = x.numel() / (M * M);
            auto v = to_f64(x);
            std::vector<double> o(v.size());
            for (int64_t b = 0; b < batch; ++b) {
                // Gauss-Jordan with partial pivoting on [A | I]
                std::vector<double> a(v.begin() + b * M * M, v.begin() + (b + 1) * M * M), inv((size_t)(M * M), 0.0);
                for (int64_t i = 0; i < M; ++i) inv[(size_t)(i * M + i)] = 1.0;
                for (int64_t col = 0; col < M; ++col) {
                    int64_t piv = col;
                    for (int64_t r = col + 1; r < M; ++r) if (std::fabs(a[(size_t)(r * M + col)]) > std::fabs(a[(size_t)(piv * M + col)])) piv = r;
                    if (piv != col) for (int64_t k = 0; k < M; ++k) { std::swap(a[(size_t)(col * M + k)], a[(size_t)(piv * M + k)]); std::swap(inv[(size_t)(col * M + k)], inv[(size_t)(piv * M + k)]); }
                    const double d = a[(size_t)(col * M + col)];
                    for (int64_t k = 0; k < M; ++k) { a[(size_t)(col * M + k)] /= d; inv[(size_t)(col * M + k)] /= d; }
                    for (int64_t r = 0; r < M; ++r) {
                        if (r == col) continue;
                        const double f = a[(size_t)(r * M + col)];
                        if (f == 0.0) continue;
                        for (int64_t k = 0; k < M; ++k) { a[(size_t)(r * M + k)] -= f * a[(size_t)(col * M + k)]; inv[(size_t)(r * M + k)] -= f * inv[(size_t)(col * M + k)]; }
                    }
                }
                const bool adj = n.attr_bool("adjoint");
                for (int64_t i = 0; i < M; ++i) for (int64_t j = 0; j < M; ++j) o[(size_t)(b * M * M + i * M + j)] = adj ? inv[(size_t)(j * M + i)] : inv[(size_t)(i * M + j)];
            }
            out[0] = from_f64(x.et, x.shape, o);
            return true;
        }, 1, 1);
    // mat_a [G, M, K] x mat_b [G, N, K]^T -> [G, M, N]; with offsets: mat_a [sum M, K], rows up to offsets[g] use expert g -> [sum M, N]
    reg("GroupedMatMul", "opset17", {},
        [](Node& n) {
            const PShape &a = n.in_shape(0), &b = n.in_shape(1);
            if (a.rank_dynamic || b.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
            PShape o;
            if (n.num_inputs() > 2) o.dims = {a.dims[0], b.dims[1]};
            else o.dims = {a.dims[0], a.dims[1], b.dims[1]};
            n.set_output(0, n.in_et(0), o);
        },
        [](N, Ins in, Outs out, C) {
            const auto a = to_f32(in[0]), b = to_f32(in[1]);
            const int64_t G = in[1].shape[0], Nn = in[1].shape[1], Kk = in[1].shape[2];
            if (in.size() > 2) {
                const auto offs = to_i64(in[2]);
                const int64_t rows = in[0].shape[0];
                std::vector<float> o((size_t)(rows * Nn), 0.f);
                int64_t begin = 0;
                for (int64_t g = 0; g < G; ++g) {
                    const int64_t end = std::min<int64_t>(offs[(size_t)g], rows);
                    for (int64_t r = begin; r < end; ++r)
                        for (int64_t j = 0; j < Nn; ++j) {
                            float acc = 0;
                            for (int64_t k = 0; k < Kk; ++k) acc += a[(size_t)(r * Kk + k)] * b[(size_t)((g * Nn + j) * Kk + k)];
                            o[(size_t)(r * Nn + j)] = acc;
                        }
                    begin = std::max(begin, end);
                }
                out[0] = from_f32(in[0].et, Shape{rows, Nn}, o);
            } else {
                const int64_t M = in[0].shape[1];
                std::vector<float> o((size_t)(G * M * Nn));
                for (int64_t g = 0; g < G; ++g)
                    for (int64_t r = 0; r < M; ++r)
                        for (int64_t j = 0; j < Nn; ++j) {
                            float acc = 0;
                            for (int64_t k = 0; k < Kk; ++k) acc += a[(size_t)((g * M + r) * Kk + k)] * b[(size_t)((g * Nn + j) * Kk + k)];
                            o[(size_t)((g * M + r) * Nn + j)] = acc;
                        }
                out[0] = from_f32(in[0].et, Shape{G, M, Nn}, o);
            }
            return true;
        }, 2, 3);

    // ---- transposed convolution: data [N, C, spatial], filters [C, O, k...] (grouped: [G, C/G, O/G, k...])
    auto infer_deconv = [](Node& n, bool grouped) {
        const PShape &x = n.in_shape(0), &w = n.in_shape(1);
        if (x.rank_dynamic || w.rank_dynamic) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
        const size_t sp = x.rank() - 2, wo = grouped ? 1 : 0;
        PShape o = PShape::dynamic(x.rank());
        o.dims[0] = x.dims[0];
        o.dims[1] = grouped ? (w.dims[0].is_static() && w.dims[2].is_static() ? Dim(w.dims[0].lo * w.dims[2].lo) : Dim::dynamic()) : w.dims[1];
        std::vector<int64_t> forced;
        if (n.num_inputs() > 2 && get_constant_ints(n.input(2), forced)) {
            for (size_t i = 0; i < sp; ++i) o.dims[2 + i] = Dim(forced.at(i));
            n.set_output(0, n.in_et(0), o);
            return;
        }
        const auto strides = n.attr_ints("strides"), dil = n.attr_ints("dilations"), pb = n.attr_ints("pads_begin"), pe = n.attr_ints("pads_end"),
                   op = n.attr_ints("output_padding");
        const std::string ap = n.attr_str("auto_pad", "explicit");
        for (size_t i = 0; i < sp; ++i) {
            const Dim &xi = x.dims[2 + i], &ki = w.dims[2 + wo + i];
            if (!xi.is_static() || !ki.is_static()) continue;
            const int64_t s = i < strides.size() ? strides[i] : 1, d = i < dil.size() ? dil[i] : 1, opad = i < op.size() ? op[i] : 0;
            int64_t pads = (i < pb.size() ? pb[i] : 0) + (i < pe.size() ? pe[i] : 0);
            if (ap == "same_upper" || ap == "same_lower") { o.dims[2 + i] = Dim(xi.lo * s); continue; }
            if (ap == "valid") pads = 0;
            o.dims[2 + i] = Dim(s * (xi.lo - 1) + d * (ki.lo - 1) + 1 - pads + opad);
        }
        n.set_output(0, n.in_et(0), o);
    };
    auto eval_deconv = [](N n, Ins in, Outs out, bool grouped) {
        const Tensor &x = in[0], &w = in[1];
        const auto xv = to_f32(x), wv = to_f32(w);
        const size_t sp = x.shape.size() - 2, wo = grouped ? 1 : 0;
        OVC_CHECK(sp >= 1 && sp <= 3, n.description() << ": 1 to 3 spatial dimensions are supported");
        const int64_t G = grouped ? w.shape[0] : 1, Cg = w.shape[wo], Og = w.shape[wo + 1], Nb = x.shape[0];
        Shape os = n.outs[0].shape.is_static() ? n.outs[0].shape.to_shape() : Shape{};
        auto strides = n.attr_ints("strides"), dil = n.attr_ints("dilations"), pb = n.attr_ints("pads_begin"), pe = n.attr_ints("pads_end");
        strides.resize(sp, 1);
        dil.resize(sp, 1);
        pb.resize(sp, 0);
        pe.resize(sp, 0);
        const std::string ap = n.attr_str("auto_pad", "explicit");
        if (os.empty() || in.size() > 2 || ap != "explicit") {
            // sizes given by the third input or by auto_pad: derive the padding from the requested output size
            os = Shape{Nb, G * Og};
            std::vector<int64_t> forced;
            if (in.size() > 2) forced = to_i64(in[2]);
            for (size_t i = 0; i < sp; ++i) {
                const int64_t full = strides[i] * (x.shape[2 + i] - 1) + dil[i] * (w.shape[2 + wo + i] - 1) + 1;
                int64_t want = !forced.empty() ? forced[i] : (ap == "valid" ? full : ap == "explicit" ? full - pb[i] - pe[i] : x.shape[2 + i] * strides[i]);
                if (ap == "valid") { pb[i] = pe[i] = 0; }
                else if (ap != "explicit" || !forced.empty()) {
                    const int64_t total = std::max<int64_t>(full - want, 0);
                    if (ap == "same_lower") { pb[i] = total - total / 2; pe[i] = total / 2; } else if (ap != "explicit") { pb[i] = total / 2; pe[i] = total - total / 2; }
                }
                os.push_back(want);
            }
        }
        std::vector<float> o((size_t)shape_size(os), 0.f);
        Shape xs3{1, 1, 1}, ks3{1, 1, 1}, os3{1, 1, 1};
        int64_t s3[3] = {1, 1, 1}, d3[3] = {1, 1, 1}, p3[3] = {0, 0, 0};
        for (size_t i = 0; i < sp; ++i) {
            const size_t j = 3 - sp + i;
            xs3[j] = x.shape[2 + i]; ks3[j] = w.shape[2 + wo + i]; os3[j] = os[2 + i];
            s3[j] = strides[i]; d3[j] = dil[i]; p3[j] = pb[i];
        }
        const int64_t xsp = xs3[0] * xs3[1] * xs3[2], ksp = ks3[0] * ks3[1] * ks3[2], osp = os3[0] * os3[1] * os3[2];
        for (int64_t b = 0; b < Nb; ++b)
            for (int64_t g = 0; g < G; ++g)
                for (int64_t c = 0; c < Cg; ++c)
                    for (int64_t oc = 0; oc < Og; ++oc) {
                        const float* wk = wv.data() + (((g * Cg + c) * Og + oc) * ksp);
                        const float* xi = xv.data() + ((b * G * Cg + g * Cg + c) * xsp);
                        float* oo = o.data() + ((b * G * Og + g * Og + oc) * osp);
                        for (int64_t z = 0; z < xs3[0]; ++z) for (int64_t y = 0; y < xs3[1]; ++y) for (int64_t xx = 0; xx < xs3[2]; ++xx) {
                            const float v = xi[(z * xs3[1] + y) * xs3[2] + xx];
                            if (v == 0.f) continue;
                            for (int64_t kz = 0; kz < ks3[0]; ++kz) for (int64_t ky = 0; ky < ks3[1]; ++ky) for (int64_t kx = 0; kx < ks3[2]; ++kx) {
                                const int64_t oz = z * s3[0] + kz * d3[0] - p3[0], oy = y * s3[1] + ky * d3[1] - p3[1], ox = xx * s3[2] + kx * d3[2] - p3[2];
                                if (oz < 0 || oz >= os3[0] || oy < 0 || oy >= os3[1] || ox < 0 || ox >= os3[2]) continue;
                                oo[(oz * os3[1] + oy) * os3[2] + ox] += v * wk[(kz * ks3[1] + ky) * ks3[2] + kx];
                            }
                        }
                    }
        out[0] = from_f32(x.et, os, o);
        return true;
    };
    const std::vector<AttrSpec> deconv_attrs = {Ais("strides"), Ais("dilations"), Ais("pads_begin"), Ais("pads_end"), As("auto_pad", "explicit"), Ais("output_padding")};
    reg("ConvolutionBackpropData", "opset1", deconv_attrs, [infer_deconv](Node& n) { infer_deconv(n, false); },
        [eval_deconv](N n, Ins in, Outs out, C) { return eval_deconv(n, in, out, false); }, 2, 3);
    reg("GroupConvolutionBackpropData", "opset1", deconv_attrs, [infer_deconv](Node& n) { infer_deconv(n, true); },
        [eval_deconv](N n, Ins in, Outs out, C) { return eval_deconv(n, in, out, true); }, 2, 3);
    reg("Col2Im", "opset15", {Ais("strides", {1, 1}), Ais("dilations", {1, 1}), Ais("pads_begin", {0, 0}), Ais("pads_end", {0, 0})},
        [](Node& n) {
            const PShape& x = n.in_shape(0);
            std::vector<int64_t> osz, ks;
            if (x.rank_dynamic || !get_constant_ints(n.input(1), osz) || !get_constant_ints(n.input(2), ks)) { n.set_output(0, n.in_et(0), PShape::dynamic()); return; }
            PShape o;
            const bool batched = x.rank() == 3;
            if (batched) o.dims.push_back(x.dims[0]);
            const Dim& ck = x.dims[batched ? 1 : 0];
            o.dims.push_back(ck.is_static() ? Dim(ck.lo / (ks[0] * ks[1])) : Dim::dynamic());
            o.dims.push_back(Dim(osz[0]));
            o.dims.push_back(Dim(osz[1]));
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const auto v = to_f32(x);
            const auto osz = to_i64(in[1]), ks = to_i64(in[2]);
            const auto st = n.attr_ints("strides"), dl = n.attr_ints("dilations"), pb = n.attr_ints("pads_begin"), pe = n.attr_ints("pads_end");
            const bool batched = x.shape.size() == 3;
            const int64_t B = batched ? x.shape[0] : 1, CK = x.shape[batched ? 1 : 0], L = x.shape[batched ? 2 : 1], Cc = CK / (ks[0] * ks[1]);
            const int64_t H = osz[0], W = osz[1];
            const int64_t nh = (H + pb[0] + pe[0] - dl[0] * (ks[0] - 1) - 1) / st[0] + 1, nw = (W + pb[1] + pe[1] - dl[1] * (ks[1] - 1) - 1) / st[1] + 1;
            OVC_CHECK(nh * nw == L, n.description() << ": the number of blocks does not match the output size");
            std::vector<float> o((size_t)(B * Cc * H * W), 0.f);
            for (int64_t b = 0; b < B; ++b)
                for (int64_t c = 0; c < Cc; ++c)
                    for (int64_t ky = 0; ky < ks[0]; ++ky) for (int64_t kx = 0; kx < ks[1]; ++kx)
                        for (int64_t by = 0; by < nh; ++by) for (int64_t bx = 0; bx < nw; ++bx) {
                            const int64_t y = by * st[0] - pb[0] + ky * dl[0], xx = bx * st[1] - pb[1] + kx * dl[1];
                            if (y < 0 || y >= H || xx < 0 || xx >= W) continue;
                            o[(size_t)(((b * Cc + c) * H + y) * W + xx)] += v[(size_t)((b * CK + (c * ks[0] + ky) * ks[1] + kx) * L + by * nw + bx)];
                        }
            Shape os = batched ? Shape{B, Cc, H, W} : Shape{Cc, H, W};
            out[0] = from_f32(x.et, os, o);
            return true;
        }, 3, 3);

    // ---- pooling / regions
    reg("AdaptiveMaxPool", "opset8", {At("index_element_type", ET::i64)},
        [](Node& n) {
            const PShape& x = n.in_shape(0);
            n.set_num_outputs(2);
            PShape o = x.rank_dynamic ? PShape::dynamic() : x;
            std::vector<int64_t> sz;
            if (!x.rank_dynamic) {
                const bool known = get_constant_ints(n.input(1), sz);
                for (size_t i = 2; i < x.rank(); ++i) o.dims[i] = known ? Dim(sz.at(i - 2)) : Dim::dynamic();
            }
            n.set_output(0, n.in_et(0), o);
            n.set_output(1, n.attr("index_element_type").et, o);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const auto v = to_f32(x);
            const auto sz = to_i64(in[1]);
            const size_t sp = x.shape.size() - 2;
            Shape is3{1, 1, 1}, os3{1, 1, 1};
            for (size_t i = 0; i < sp; ++i) { is3[3 - sp + i] = x.shape[2 + i]; os3[3 - sp + i] = sz[i]; }
            const int64_t NC = x.shape[0] * x.shape[1], isp = is3[0] * is3[1] * is3[2], osp = os3[0] * os3[1] * os3[2];
            std::vector<float> o((size_t)(NC * osp));
            std::vector<int64_t> idx((size_t)(NC * osp));
            auto lo = [](int64_t i, int64_t in_n, int64_t out_n) { return (i * in_n) / out_n; };
            auto hi = [](int64_t i, int64_t in_n, int64_t out_n) { return ((i + 1) * in_n + out_n - 1) / out_n; };
            for (int64_t c = 0; c < NC; ++c)
                for (int64_t z = 0; z < os3[0]; ++z) for (int64_t y = 0; y < os3[1]; ++y) for (int64_t xx = 0; xx < os3[2]; ++xx) {
                    float best = -INFINITY;
                    int64_t bi = 0;
                    for (int64_t a = lo(z, is3[0], os3[0]); a < hi(z, is3[0], os3[0]); ++a)
                        for (int64_t b = lo(y, is3[1], os3[1]); b < hi(y, is3[1], os3[1]); ++b)
                            for (int64_t d = lo(xx, is3[2], os3[2]); d < hi(xx, is3[2], os3[2]); ++d) {
                                const int64_t p = (a * is3[1] + b) * is3[2] + d;
                                if (v[(size_t)(c * isp + p)] > best) { best = v[(size_t)(c * isp + p)]; bi = p; }
                            }
                    o[(size_t)(c * osp + (z * os3[1] + y) * os3[2] + xx)] = best;
                    idx[(size_t)(c * osp + (z * os3[1] + y) * os3[2] + xx)] = bi;
                }
            Shape os{x.shape[0], x.shape[1]};
            for (size_t i = 0; i < sp; ++i) os.push_back(sz[i]);
            out[0] = from_f32(x.et, os, o);
            out[1] = from_i64(n.attr("index_element_type").et, os, idx);
            return true;
        }, 2, 2);
    auto infer_roi = [](Node& n, const char* ph, const char* pw) {
        const PShape &x = n.in_shape(0), &rois = n.in_shape(1);
        PShape o;
        o.dims = {rois.rank_dynamic ? Dim::dynamic() : rois.dims[0], x.rank_dynamic ? Dim::dynamic() : x.dims[1], Dim(n.attr_int(ph)), Dim(n.attr_int(pw))};
        n.set_output(0, n.in_et(0), o);
    };
    auto eval_roi_align = [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        const auto v = to_f32(x), rois = to_f32(in[1]);
        const auto bidx = to_i64(in[2]);
        const int64_t Cc = x.shape[1], H = x.shape[2], W = x.shape[3], R = in[1].shape[0];
        const int64_t ph = n.attr_int("pooled_h"), pw = n.attr_int("pooled_w"), sr = n.attr_int("sampling_ratio");
        const float scale = (float)n.attr_float("spatial_scale");
        const bool avg = n.attr_str("mode", "avg") == "avg";
        const std::string am = n.attr_str("aligned_mode", "asymmetric");
        const float off_in = am == "half_pixel_for_nn" ? -0.5f : (am == "half_pixel" ? 0.5f : 0.f), off_out = am == "half_pixel" ? -0.5f : 0.f;
        std::vector<float> o((size_t)(R * Cc * ph * pw));
        for (int64_t r = 0; r < R; ++r) {
            const float x1 = (rois[(size_t)(r * 4)] + off_in) * scale + off_out, y1 = (rois[(size_t)(r * 4 + 1)] + off_in) * scale + off_out;
            const float x2 = (rois[(size_t)(r * 4 + 2)] + off_in) * scale + off_out, y2 = (rois[(size_t)(r * 4 + 3)] + off_in) * scale + off_out;
            float rw = x2 - x1, rh = y2 - y1;
            if (am == "asymmetric") { rw = std::max(rw, 1.f); rh = std::max(rh, 1.f); }
            const float bw = rw / (float)pw, bh = rh / (float)ph;
            const int64_t sx = sr > 0 ? sr : (int64_t)std::ceil(bw), sy = sr > 0 ? sr : (int64_t)std::ceil(bh);
            for (int64_t c = 0; c < Cc; ++c) {
                const float* img = v.data() + ((bidx[(size_t)r] * Cc + c) * H * W);
                for (int64_t py = 0; py < ph; ++py)
                    for (int64_t px = 0; px < pw; ++px) {
                        float acc = avg ? 0.f : -INFINITY;
                        for (int64_t iy = 0; iy < sy; ++iy)
                            for (int64_t ix = 0; ix < sx; ++ix) {
                                const float yy = y1 + (float)py * bh + ((float)iy + 0.5f) * bh / (float)sy;
                                const float xx = x1 + (float)px * bw + ((float)ix + 0.5f) * bw / (float)sx;
                                const float s = bilinear(img, H, W, yy, xx);
                                acc = avg ? acc + s : std::max(acc, s);
                            }
                        o[(size_t)(((r * Cc + c) * ph + py) * pw + px)] = avg ? acc / (float)std::max<int64_t>(sx * sy, 1) : acc;
                    }
            }
        }
        out[0] = from_f32(x.et, Shape{R, Cc, ph, pw}, o);
        return true;
    };
    reg("ROIAlign", "opset3", {Ai("pooled_h", 1), Ai("pooled_w", 1), Ai("sampling_ratio", 1), Af("spatial_scale", 1.0), As("mode", "avg")},
        [infer_roi](Node& n) { infer_roi(n, "pooled_h", "pooled_w"); }, eval_roi_align, 3, 3);
    reg("ROIAlign", "opset9", {Ai("pooled_h", 1), Ai("pooled_w", 1), Ai("sampling_ratio", 1), Af("spatial_scale", 1.0), As("mode", "avg"), As("aligned_mode", "asymmetric")},
        [infer_roi](Node& n) { infer_roi(n, "pooled_h", "pooled_w"); }, eval_roi_align, 3, 3);
    reg("ROIPooling", "opset2", {Ais("output_size", {1, 1}), Af("spatial_scale", 1.0), As("method", "max")},
        [](Node& n) {
            const PShape &x = n.in_shape(0), &rois = n.in_shape(1);
            const auto os = n.attr_ints("output_size");
            PShape o;
            o.dims = {rois.rank_dynamic ? Dim::dynamic() : rois.dims[0], x.rank_dynamic ? Dim::dynamic() : x.dims[1], Dim(os.at(0)), Dim(os.at(1))};
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const auto v = to_f32(x), rois = to_f32(in[1]);
            const int64_t Cc = x.shape[1], H = x.shape[2], W = x.shape[3], R = in[1].shape[0];
            const auto os = n.attr_ints("output_size");
            const int64_t ph = os[0], pw = os[1];
            const float scale = (float)n.attr_float("spatial_scale");
            const bool is_max = n.attr_str("method", "max") == "max";
            std::vector<float> o((size_t)(R * Cc * ph * pw), 0.f);
            for (int64_t r = 0; r < R; ++r) {
                const int64_t b = (int64_t)rois[(size_t)(r * 5)];
                if (is_max) {
                    const int64_t x1 = (int64_t)std::round(rois[(size_t)(r * 5 + 1)] * scale), y1 = (int64_t)std::round(rois[(size_t)(r * 5 + 2)] * scale);
                    const int64_t x2 = (int64_t)std::round(rois[(size_t)(r * 5 + 3)] * scale), y2 = (int64_t)std::round(rois[(size_t)(r * 5 + 4)] * scale);
                    const int64_t rh = std::max<int64_t>(y2 - y1 + 1, 1), rw = std::max<int64_t>(x2 - x1 + 1, 1);
                    for (int64_t c = 0; c < Cc; ++c) {
                        const float* img = v.data() + ((b * Cc + c) * H * W);
                        for (int64_t py = 0; py < ph; ++py)
                            for (int64_t px = 0; px < pw; ++px) {
                                int64_t hs = (int64_t)std::floor((double)py * rh / ph) + y1, he = (int64_t)std::ceil((double)(py + 1) * rh / ph) + y1;
                                int64_t ws = (int64_t)std::floor((double)px * rw / pw) + x1, we = (int64_t)std::ceil((double)(px + 1) * rw / pw) + x1;
                                hs = std::min(std::max<int64_t>(hs, 0), H); he = std::min(std::max<int64_t>(he, 0), H);
                                ws = std::min(std::max<int64_t>(ws, 0), W); we = std::min(std::max<int64_t>(we, 0), W);
                                float best = (he <= hs || we <= ws) ? 0.f : -INFINITY;
                                for (int64_t yy = hs; yy < he; ++yy) for (int64_t xx = ws; xx < we; ++xx) best = std::max(best, img[yy * W + xx]);
                                o[(size_t)(((r * Cc + c) * ph + py) * pw + px)] = best;
                            }
                    }
                } else {
                    // bilinear: ROI corners are fractions of the feature map
                    const float x1 = rois[(size_t)(r * 5 + 1)], y1 = rois[(size_t)(r * 5 + 2)], x2 = rois[(size_t)(r * 5 + 3)], y2 = rois[(size_t)(r * 5 + 4)];
                    const float rh = (y2 - y1) * (float)(H - 1), rw = (x2 - x1) * (float)(W - 1);
                    for (int64_t c = 0; c < Cc; ++c) {
                        const float* img = v.data() + ((b * Cc + c) * H * W);
                        for (int64_t py = 0; py < ph; ++py)
                            for (int64_t px = 0; px < pw; ++px) {
                                const float yy = (ph > 1 ? (float)py * rh / (float)(ph - 1) : 0.5f * rh) + y1 * (float)(H - 1);
                                const float xx = (pw > 1 ? (float)px * rw / (float)(pw - 1) : 0.5f * rw) + x1 * (float)(W - 1);
                                o[(size_t)(((r * Cc + c) * ph + py) * pw + px)] = bilinear(img, H, W, yy, xx);
                            }
                    }
                }
            }
            out[0] = from_f32(x.et, Shape{R, Cc, ph, pw}, o);
            return true;
        }, 2, 2);
    reg("GridSample", "opset9", {Ab("align_corners", false), As("mode", "bilinear"), As("padding_mode", "zeros")},
        [](Node& n) {
            const PShape &x = n.in_shape(0), &g = n.in_shape(1);
            PShape o = PShape::dynamic(4);
            if (!x.rank_dynamic) { o.dims[0] = x.dims[0]; o.dims[1] = x.dims[1]; }
            if (!g.rank_dynamic) { o.dims[2] = g.dims[1]; o.dims[3] = g.dims[2]; }
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            const Tensor& x = in[0];
            const auto v = to_f32(x), g = to_f32(in[1]);
            const int64_t B = x.shape[0], Cc = x.shape[1], H = x.shape[2], W = x.shape[3], Ho = in[1].shape[1], Wo = in[1].shape[2];
            const bool ac = n.attr_bool("align_corners");
            const std::string mode = n.attr_str("mode"), pad = n.attr_str("padding_mode");
            auto unnorm = [&](float c, int64_t size) { return ac ? (c + 1.f) / 2.f * (float)(size - 1) : ((c + 1.f) * (float)size - 1.f) / 2.f; };
            auto reflect = [&](float c, int64_t size) {
                // reflect about the borders of the sampling domain, then clamp
                const float lo = ac ? 0.f : -0.5f, span = ac ? (float)(size - 1) : (float)size;
                if (span <= 0) return 0.f;
                float t = std::fabs(c - lo);
                const float extra = std::fmod(t, span);
                const int64_t flips = (int64_t)std::floor(t / span);
                const float r = (flips % 2 == 0) ? extra + lo : span - extra + lo;
                return std::min(std::max(r, 0.f), (float)(size - 1));
            };
            auto at = [&](const float* img, int64_t y, int64_t xx) -> float {
                if (pad == "border") { y = std::min(std::max<int64_t>(y, 0), H - 1); xx = std::min(std::max<int64_t>(xx, 0), W - 1); }
                else if (pad == "reflection") { y = (int64_t)std::lround(reflect((float)y, H)); xx = (int64_t)std::lround(reflect((float)xx, W)); }
                if (y < 0 || y >= H || xx < 0 || xx >= W) return 0.f;
                return img[y * W + xx];
            };
            auto cubic = [](float t, float w[4]) {
                const float A = -0.75f;
                w[0] = ((A * (t + 1) - 5 * A) * (t + 1) + 8 * A) * (t + 1) - 4 * A;
                w[1] = ((A + 2) * t - (A + 3)) * t * t + 1;
                w[2] = ((A + 2) * (1 - t) - (A + 3)) * (1 - t) * (1 - t) + 1;
                w[3] = ((A * (2 - t) - 5 * A) * (2 - t) + 8 * A) * (2 - t) - 4 * A;
            };
            std::vector<float> o((size_t)(B * Cc * Ho * Wo));
            for (int64_t b = 0; b < B; ++b)
                for (int64_t y = 0; y < Ho; ++y)
                    for (int64_t xx = 0; xx < Wo; ++xx) {
                        float gx = unnorm(g[(size_t)(((b * Ho + y) * Wo + xx) * 2)], W), gy = unnorm(g[(size_t)(((b * Ho + y) * Wo + xx) * 2 + 1)], H);
                        // bilinear / nearest pad the sampling position itself; bicubic pads every neighbour it reads instead
                        if (mode != "bicubic") {
                            if (pad == "border") { gx = std::min(std::max(gx, 0.f), (float)(W - 1)); gy = std::min(std::max(gy, 0.f), (float)(H - 1)); }
                            else if (pad == "reflection") { gx = reflect(gx, W); gy = reflect(gy, H); }
                        }
                        for (int64_t c = 0; c < Cc; ++c) {
                            const float* img = v.data() + ((b * Cc + c) * H * W);
                            float r;
                            if (mode == "nearest") r = at(img, (int64_t)std::nearbyint(gy), (int64_t)std::nearbyint(gx));
                            else if (mode == "bicubic") {
                                const int64_t x0 = (int64_t)std::floor(gx), y0 = (int64_t)std::floor(gy);
                                float wx[4], wy[4];
                                cubic(gx - (float)x0, wx);
                                cubic(gy - (float)y0, wy);
                                r = 0;
                                for (int i = 0; i < 4; ++i) for (int j = 0; j < 4; ++j) r += wy[i] * wx[j] * at(img, y0 - 1 + i, x0 - 1 + j);
                            } else {
                                const int64_t x0 = (int64_t)std::floor(gx), y0 = (int64_t)std::floor(gy);
                                const float lx = gx - (float)x0, ly = gy - (float)y0;
                                r = (1 - ly) * (1 - lx) * at(img, y0, x0) + (1 - ly) * lx * at(img, y0, x0 + 1) + ly * (1 - lx) * at(img, y0 + 1, x0) + ly * lx * at(img, y0 + 1, x0 + 1);
                            }
                            o[(size_t)(((b * Cc + c) * Ho + y) * Wo + xx)] = r;
                        }
                    }
            out[0] = from_f32(x.et, Shape{B, Cc, Ho, Wo}, o);
            return true;
        }, 2, 2);
    // boxes [B, N, 4], scores [B, C, N]; outputs selected_indices [K, 3], selected_scores [K, 3], valid_outputs [1]
    auto infer_nms = [](Node& n) {
        const PShape &boxes = n.in_shape(0), &scores = n.in_shape(1);
        n.set_num_outputs(3);
        PShape sel = PShape::dynamic(2);
        sel.dims[1] = Dim(3);
        std::vector<int64_t> mo;
        if (boxes.is_static() && scores.is_static() && n.num_inputs() > 2 && get_constant_ints(n.input(2), mo))
            sel.dims[0] = Dim(0, scores.dims[0].lo * scores.dims[1].lo * std::min<int64_t>(boxes.dims[1].lo, mo.at(0)));
        const ET it = n.has_attr("output_type") ? n.attr("output_type").et : ET::i64;
        n.set_output(0, it, sel);
        n.set_output(1, ET::f32, sel);
        PShape one;
        one.dims = {Dim(1)};
        n.set_output(2, it, one);
    };
    auto eval_nms = [](N n, Ins in, Outs out, C) {
        const auto boxes = to_f32(in[0]), scores = to_f32(in[1]);
        const int64_t B = in[0].shape[0], Nb = in[0].shape[1], Cc = in[1].shape[1];
        const int64_t max_out = in.size() > 2 ? to_i64(in[2]).at(0) : 0;
        const float iou_t = in.size() > 3 ? (float)get_elem_f64(in[3], 0) : 0.f, score_t = in.size() > 4 ? (float)get_elem_f64(in[4], 0) : 0.f;
        const float sigma = in.size() > 5 ? (float)get_elem_f64(in[5], 0) : 0.f;
        const bool center = n.attr_str("box_encoding", "corner") == "center";
        struct Sel { float score; int64_t b, c, i; };
        std::vector<Sel> all;
        for (int64_t b = 0; b < B; ++b)
            for (int64_t c = 0; c < Cc; ++c) {
                std::vector<std::pair<float, int64_t>> cand;
                for (int64_t i = 0; i < Nb; ++i) { const float s = scores[(size_t)((b * Cc + c) * Nb + i)]; if (s > score_t) cand.push_back({s, i}); }
                std::vector<Sel> kept;
                auto box = [&](int64_t i, float o[4]) {
                    const float* p = boxes.data() + (b * Nb + i) * 4;
                    if (center) { o[0] = p[1] - p[3] / 2; o[1] = p[0] - p[2] / 2; o[2] = p[1] + p[3] / 2; o[3] = p[0] + p[2] / 2; }
                    else { o[0] = p[0]; o[1] = p[1]; o[2] = p[2]; o[3] = p[3]; }
                };
                // greedy selection; with soft-NMS (sigma > 0) scores decay instead of boxes being dropped
                while (!cand.empty() && (int64_t)kept.size() < max_out) {
                    auto best = std::max_element(cand.begin(), cand.end(), [](const std::pair<float, int64_t>& x, const std::pair<float, int64_t>& y) {
                        return x.first < y.first || (x.first == y.first && x.second > y.second);
                    });
                    const auto cur = *best;
                    cand.erase(best);
                    if (cur.first <= score_t) break;
                    float cb[4];
                    box(cur.second, cb);
                    bool keep = true;
                    if (sigma <= 0.f) {
                        for (auto& k : kept) { float kb[4]; box(k.i, kb); if (iou_corner(cb, kb) > iou_t) { keep = false; break; } }
                    }
                    if (!keep) continue;
                    kept.push_back({cur.first, b, c, cur.second});
                    if (sigma > 0.f)
                        for (auto& o : cand) {
                            float ob[4];
                            box(o.second, ob);
                            const float iou = iou_corner(cb, ob);
                            o.first *= iou <= iou_t ? std::exp(-0.5f * iou * iou / sigma) : 0.f;
                        }
                }
                all.insert(all.end(), kept.begin(), kept.end());
            }
        if (n.attr_bool("sort_result_descending", true))
            std::stable_sort(all.begin(), all.end(), [](const Sel& x, const Sel& y) { return x.score > y.score; });
        const int64_t Kk = (int64_t)all.size();
        std::vector<int64_t> idx((size_t)(Kk * 3));
        std::vector<float> sc((size_t)(Kk * 3));
        for (int64_t k = 0; k < Kk; ++k) {
            idx[(size_t)(k * 3)] = all[(size_t)k].b; idx[(size_t)(k * 3 + 1)] = all[(size_t)k].c; idx[(size_t)(k * 3 + 2)] = all[(size_t)k].i;
            sc[(size_t)(k * 3)] = (float)all[(size_t)k].b; sc[(size_t)(k * 3 + 1)] = (float)all[(size_t)k].c; sc[(size_t)(k * 3 + 2)] = all[(size_t)k].score;
        }
        const ET it = n.has_attr("output_type") ? n.attr("output_type").et : ET::i64;
        out[0] = from_i64(it, Shape{Kk, 3}, idx);
        out[1] = from_f32(ET::f32, Shape{Kk, 3}, sc);
        out[2] = from_i64(it, Shape{1}, {Kk});
        return true;
    };
    reg("NonMaxSuppression", "opset5", {As("box_encoding", "corner"), Ab("sort_result_descending", true), At("output_type", ET::i64)}, infer_nms, eval_nms, 2, 6);
    reg("NonMaxSuppression", "opset9", {As("box_encoding", "corner"), Ab("sort_result_descending", true), At("output_type", ET::i64)}, infer_nms, eval_nms, 2, 6);

    // ---- signal processing
    for (int kind = 0; kind < 4; ++kind) {
        static const char* names[4] = {"DFT", "IDFT", "RDFT", "IRDFT"};
        reg(names[kind], kind < 2 ? "opset7" : "opset9", {}, [kind](Node& n) { infer_fft(n, kind); },
            [kind](N n, Ins in, Outs out, C) { return eval_fft(n, in, out, kind); }, 2, 3);
    }

    // ---- recurrent cells and sequences
    reg("LSTMCell", "opset4", cell_specs({"sigmoid", "tanh", "tanh"}), [](Node& n) { infer_cell(n, true); },
        [](N n, Ins in, Outs out, C) {
            const CellAttrs a = cell_attrs(n, {"sigmoid", "tanh", "tanh"});
            const int64_t B = in[0].shape[0], I = in[0].shape[1], H = a.hidden;
            const auto x = to_f32(in[0]), W = to_f32(in[3]), R = to_f32(in[4]);
            auto h = to_f32(in[1]), c = to_f32(in[2]);
            std::vector<float> bias = in.size() > 5 ? to_f32(in[5]) : std::vector<float>((size_t)(4 * H), 0.f), tmp;
            for (int64_t b = 0; b < B; ++b) lstm_step(a, x.data() + b * I, I, h.data() + b * H, c.data() + b * H, W.data(), R.data(), bias.data(), tmp);
            out[0] = from_f32(in[0].et, Shape{B, H}, h);
            out[1] = from_f32(in[0].et, Shape{B, H}, c);
            return true;
        }, 5, 6);
    {
        auto specs = cell_specs({"sigmoid", "tanh"});
        specs.insert(specs.begin(), Ab("linear_before_reset", false));
        reg("GRUCell", "opset3", specs, [](Node& n) { infer_cell(n, false); },
            [](N n, Ins in, Outs out, C) {
                const CellAttrs a = cell_attrs(n, {"sigmoid", "tanh"});
                const bool lbr = n.attr_bool("linear_before_reset");
                const int64_t B = in[0].shape[0], I = in[0].shape[1], H = a.hidden;
                const auto x = to_f32(in[0]), W = to_f32(in[2]), R = to_f32(in[3]);
                auto h = to_f32(in[1]);
                std::vector<float> bias = in.size() > 4 ? to_f32(in[4]) : std::vector<float>((size_t)((lbr ? 4 : 3) * H), 0.f), tmp;
                for (int64_t b = 0; b < B; ++b) gru_step(a, lbr, x.data() + b * I, I, h.data() + b * H, W.data(), R.data(), bias.data(), tmp);
                out[0] = from_f32(in[0].et, Shape{B, H}, h);
                return true;
            }, 4, 5);
    }
    reg("RNNCell", "opset1", cell_specs({"tanh"}), [](Node& n) { infer_cell(n, false); },
        [](N n, Ins in, Outs out, C) {
            const CellAttrs a = cell_attrs(n, {"tanh"});
            const int64_t B = in[0].shape[0], I = in[0].shape[1], H = a.hidden;
            const auto x = to_f32(in[0]), W = to_f32(in[2]), R = to_f32(in[3]);
            auto h = to_f32(in[1]);
            std::vector<float> bias = in.size() > 4 ? to_f32(in[4]) : std::vector<float>((size_t)H, 0.f), tmp;
            for (int64_t b = 0; b < B; ++b) rnn_step(a, x.data() + b * I, I, h.data() + b * H, W.data(), R.data(), bias.data(), tmp);
            out[0] = from_f32(in[0].et, Shape{B, H}, h);
            return true;
        }, 4, 5);
    {
        auto specs = cell_specs({"sigmoid", "tanh", "tanh"});
        specs.insert(specs.begin(), As("direction", "forward"));
        reg("LSTMSequence", "opset5", specs, [](Node& n) { infer_sequence(n, true); }, [](N n, Ins in, Outs out, C) { return eval_sequence(n, in, out, 0); }, 7, 7);
    }
    {
        auto specs = cell_specs({"sigmoid", "tanh"});
        specs.insert(specs.begin(), Ab("linear_before_reset", false));
        specs.insert(specs.begin(), As("direction", "forward"));
        reg("GRUSequence", "opset5", specs, [](Node& n) { infer_sequence(n, false); }, [](N n, Ins in, Outs out, C) { return eval_sequence(n, in, out, 1); }, 6, 6);
    }
    {
        auto specs = cell_specs({"tanh"});
        specs.insert(specs.begin(), As("direction", "forward"));
        reg("RNNSequence", "opset5", specs, [](Node& n) { infer_sequence(n, false); }, [](N n, Ins in, Outs out, C) { return eval_sequence(n, in, out, 2); }, 6, 6);
    }

    // ---- CTC
    reg("CTCGreedyDecoder", "opset1", {Ab("ctc_merge_repeated", true)},
        [](Node& n) {
            const PShape& x = n.in_shape(0);
            PShape o = PShape::dynamic(4);
            if (!x.rank_dynamic) { o.dims[0] = x.dims[1]; o.dims[1] = x.dims[0]; }
            o.dims[2] = Dim(1);
            o.dims[3] = Dim(1);
            n.set_output(0, n.in_et(0), o);
        },
        [](N n, Ins in, Outs out, C) {
            // data [T, B, classes], sequence mask [T, B]; output [B, T, 1, 1] padded with -1; the last class is the blank
            const auto v = to_f32(in[0]), mask = to_f32(in[1]);
            const int64_t T = in[0].shape[0], B = in[0].shape[1], Cc = in[0].shape[2];
            const bool merge = n.attr_bool("ctc_merge_repeated");
            std::vector<float> o((size_t)(B * T), -1.f);
            for (int64_t b = 0; b < B; ++b) {
                int64_t prev = -1, k = 0;
                for (int64_t t = 0; t < T && mask[(size_t)(t * B + b)] != 0.f; ++t) {
                    const float* p = v.data() + (t * B + b) * Cc;
                    const int64_t best = std::max_element(p, p + Cc) - p;
                    if (best != Cc - 1 && !(merge && best == prev)) o[(size_t)(b * T + k++)] = (float)best;
                    prev = best;
                }
            }
            out[0] = from_f32(in[0].et, Shape{B, T, 1, 1}, o);
            return true;
        }, 2, 2);
    reg("CTCGreedyDecoderSeqLen", "opset6", {Ab("merge_repeated", true), At("classes_index_type", ET::i32), At("sequence_length_type", ET::i32)},
        [](Node& n) {
            const PShape& x = n.in_shape(0);
            n.set_num_outputs(2);
            PShape o = PShape::dynamic(2), l = PShape::dynamic(1);
            if (!x.rank_dynamic) { o.dims[0] = x.dims[0]; o.dims[1] = x.dims[1]; l.dims[0] = x.dims[0]; }
            n.set_output(0, n.attr("classes_index_type").et, o);
            n.set_output(1, n.attr("sequence_length_type").et, l);
        },
        [](N n, Ins in, Outs out, C) {
            // data [B, T, classes], sequence lengths [B], optional blank index (default: the last class)
            const auto v = to_f32(in[0]);
            const auto lens = to_i64(in[1]);
            const int64_t B = in[0].shape[0], T = in[0].shape[1], Cc = in[0].shape[2];
            const int64_t blank = in.size() > 2 ? to_i64(in[2]).at(0) : Cc - 1;
            const bool merge = n.attr_bool("merge_repeated");
            std::vector<int64_t> o((size_t)(B * T), -1), ol((size_t)B, 0);
            for (int64_t b = 0; b < B; ++b) {
                int64_t prev = -1, k = 0;
                for (int64_t t = 0; t < std::min<int64_t>(lens[(size_t)b], T); ++t) {
                    const float* p = v.data() + (b * T + t) * Cc;
                    const int64_t best = std::max_element(p, p + Cc) - p;
                    if (best != blank && !(merge && best == prev)) o[(size_t)(b * T + k++)] = best;
                    prev = best;
                }
                ol[(size_t)b] = k;
            }
            out[0] = from_i64(n.attr("classes_index_type").et, Shape{B, T}, o);
            out[1] = from_i64(n.attr("sequence_length_type").et, Shape{B}, ol);
            return true;
        }, 2, 3);

    // ---- embedding bags: rows of a table summed per bag (optionally weighted)
    auto infer_bag = [](Node& n, int bags_input, bool packed) {
        const PShape& tab = n.in_shape(0);
        PShape o = tab.rank_dynamic ? PShape::dynamic() : tab;
        if (!tab.rank_dynamic) {
            if (packed) o.dims[0] = n.in_shape(1).rank_dynamic ? Dim::dynamic() : n.in_shape(1).dims[0];
            else if (bags_input >= 0) o.dims[0] = n.in_shape((size_t)bags_input).rank_dynamic ? Dim::dynamic() : n.in_shape((size_t)bags_input).dims[0];
        }
        n.set_output(0, n.in_et(0), o);
    };
    auto bag_sum = [](const std::vector<float>& tab, int64_t width, const std::vector<int64_t>& idx, int64_t b, int64_t e, const std::vector<float>* w, float* dst, bool mean) {
        for (int64_t k = 0; k < width; ++k) dst[k] = 0.f;
        for (int64_t i = b; i < e; ++i)
            for (int64_t k = 0; k < width; ++k) dst[k] += tab[(size_t)(idx[(size_t)i] * width + k)] * (w ? (*w)[(size_t)i] : 1.f);
        if (mean && e > b) for (int64_t k = 0; k < width; ++k) dst[k] /= (float)(e - b);
    };
    auto eval_offsets = [bag_sum](N n, Ins in, Outs out, C) {
        const auto tab = to_f32(in[0]);
        auto idx = to_i64(in[1]);
        const auto offs = to_i64(in[2]);
        const int64_t rows = in[0].shape[0], width = rows ? in[0].numel() / rows : 0, bags = (int64_t)offs.size();
        const int64_t def = in.size() > 3 && in[3].numel() > 0 ? to_i64(in[3]).at(0) : -1;
        std::vector<float> w;
        if (in.size() > 4) w = to_f32(in[4]);
        const bool mean = n.has_attr("reduction") && (n.attr_str("reduction") == "mean" || n.attr_str("reduction") == "MEAN");
        std::vector<float> o((size_t)(bags * width), 0.f);
        for (int64_t b = 0; b < bags; ++b) {
            const int64_t s = offs[(size_t)b], e = b + 1 < bags ? offs[(size_t)b + 1] : (int64_t)idx.size();
            if (e > s) bag_sum(tab, width, idx, s, e, in.size() > 4 ? &w : nullptr, o.data() + b * width, mean);
            else if (def >= 0) for (int64_t k = 0; k < width; ++k) o[(size_t)(b * width + k)] = tab[(size_t)(def * width + k)];
        }
        Shape os = in[0].shape;
        os[0] = bags;
        out[0] = from_f32(in[0].et, os, o);
        return true;
    };
    auto eval_packed = [bag_sum](N n, Ins in, Outs out, C) {
        const auto tab = to_f32(in[0]);
        const auto idx = to_i64(in[1]);
        const int64_t rows = in[0].shape[0], width = rows ? in[0].numel() / rows : 0, bags = in[1].shape[0], per = in[1].shape[1];
        std::vector<float> w;
        if (in.size() > 2) w = to_f32(in[2]);
        const bool mean = n.has_attr("reduction") && (n.attr_str("reduction") == "mean" || n.attr_str("reduction") == "MEAN");
        std::vector<float> o((size_t)(bags * width));
        for (int64_t b = 0; b < bags; ++b) bag_sum(tab, width, idx, b * per, (b + 1) * per, in.size() > 2 ? &w : nullptr, o.data() + b * width, mean);
        Shape os = in[0].shape;
        os[0] = bags;
        out[0] = from_f32(in[0].et, os, o);
        return true;
    };
    reg("EmbeddingBagOffsetsSum", "opset3", {}, [infer_bag](Node& n) { infer_bag(n, 2, false); }, eval_offsets, 3, 5);
    reg("EmbeddingBagPackedSum", "opset3", {}, [infer_bag](Node& n) { infer_bag(n, -1, true); }, eval_packed, 2, 3);
    reg("EmbeddingBagOffsets", "opset15", {As("reduction", "sum")}, [infer_bag](Node& n) { infer_bag(n, 2, false); }, eval_offsets, 3, 5);
    reg("EmbeddingBagPacked", "opset15", {As("reduction", "sum")}, [infer_bag](Node& n) { infer_bag(n, -1, true); }, eval_packed, 2, 3);
    reg("EmbeddingSegmentsSum", "opset3", {},
        [](Node& n) {
            const PShape& tab = n.in_shape(0);
            PShape o = tab.rank_dynamic ? PShape::dynamic() : tab;
            std::vector<int64_t> ns;
            if (!tab.rank_dynamic) o.dims[0] = get_constant_ints(n.input(3), ns) ? Dim(ns.at(0)) : Dim::dynamic();
            n.set_output(0, n.in_et(0), o);
        },
        [](N, Ins in, Outs out, C) {
            const auto tab = to_f32(in[0]);
            const auto idx = to_i64(in[1]), seg = to_i64(in[2]);
            const int64_t rows = in[0].shape[0], width = rows ? in[0].numel() / rows : 0, segs = to_i64(in[3]).at(0);
            const int64_t def = in.size() > 4 && in[4].numel() > 0 ? to_i64(in[4]).at(0) : -1;
            std::vector<float> w;
            if (in.size() > 5) w = to_f32(in[5]);
            std::vector<float> o((size_t)(segs * width), 0.f);
            std::vector<char> used((size_t)segs, 0);
            for (size_t i = 0; i < idx.size(); ++i) {
                const int64_t s = seg[i];
                if (s < 0 || s >= segs) continue;
                used[(size_t)s] = 1;
                for (int64_t k = 0; k < width; ++k) o[(size_t)(s * width + k)] += tab[(size_t)(idx[i] * width + k)] * (in.size() > 5 ? w[i] : 1.f);
            }
            if (def >= 0)
                for (int64_t s = 0; s < segs; ++s)
                    if (!used[(size_t)s]) for (int64_t k = 0; k < width; ++k) o[(size_t)(s * width + k)] = tab[(size_t)(def * width + k)];
            Shape os = in[0].shape;
            os[0] = segs;
            out[0] = from_f32(in[0].et, os, o);
            return true;
        }, 4, 6);
}

}  // namespace ovc
