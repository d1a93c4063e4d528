// Reference kernels: a plain C++ implementation of every registered operation, used by constant
// folding, by Model::evaluate, by the "CPU" device and as the numerical oracle of the CUDA plugin.
//
// Same role as src/core/reference/include/openvino/reference/*.hpp (matmul.hpp, convolution.hpp,
// softmax.hpp, scaled_dot_product_attention.hpp, rms_norm.hpp, paged_attention.hpp, ...). Real types
// are computed in fp32 (f64 in double), integer types in int64; results are rounded to the output type.
#include <numeric>
#include <thread>

#include "graph.hpp"

namespace ovc {

namespace {

// ------------------------------------------------------------------------------------ utilities
void parallel_for(int64_t n, int threads, const std::function<void(int64_t, int64_t)>& fn) {
    if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
    threads = (int)std::min<int64_t>(threads, std::max<int64_t>(1, n));
    if (threads <= 1 || n < 2) { fn(0, n); return; }
    std::vector<std::thread> pool;
    const int64_t chunk = (n + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const int64_t b = t * chunk, e = std::min(n, b + chunk);
        if (b >= e) break;
        pool.emplace_back([=, &fn] { fn(b, e); });
    }
    for (auto& th : pool) th.join();
}

std::vector<int64_t> strides_of(const Shape& s) {
    std::vector<int64_t> st(s.size(), 1);
    for (int64_t i = (int64_t)s.size() - 2; i >= 0; --i) st[(size_t)i] = st[(size_t)i + 1] * s[(size_t)i + 1];
    return st;
}

Shape broadcast_shape(const Shape& a, const Shape& b) {
    const size_t r = std::max(a.size(), b.size());
    Shape out(r);
    for (size_t i = 0; i < r; ++i) {
        const int64_t da = i < r - a.size() ? 1 : a[i - (r - a.size())];
        const int64_t db = i < r - b.size() ? 1 : b[i - (r - b.size())];
        OVC_CHECK(da == db || da == 1 || db == 1, "shapes " << PShape(a).str() << " and " << PShape(b).str() << " do not broadcast");
        out[i] = da == 1 ? db : da;
    }
    return out;
}
// strides of `s` viewed in the broadcast `out` shape (0 where broadcast)
std::vector<int64_t> bstrides(const Shape& s, const Shape& out) {
    std::vector<int64_t> st(out.size(), 0);
    const auto own = strides_of(s);
    const size_t off = out.size() - s.size();
    for (size_t i = 0; i < s.size(); ++i) st[off + i] = s[i] == 1 ? 0 : own[i];
    return st;
}

template <class T, class F>
void broadcast_apply(const Shape& out, const std::vector<int64_t>& sa, const std::vector<int64_t>& sb, const T* a, const T* b, T* o, F f) {
    const int64_t n = shape_size(out);
    const size_t r = out.size();
    if (r == 0) { o[0] = f(a[0], b[0]); return; }
    std::vector<int64_t> idx(r, 0);
    int64_t ia = 0, ib = 0;
    for (int64_t i = 0; i < n; ++i) {
        o[i] = f(a[ia], b[ib]);
        for (int64_t d = (int64_t)r - 1; d >= 0; --d) {
            ++idx[(size_t)d];
            ia += sa[(size_t)d];
            ib += sb[(size_t)d];
            if (idx[(size_t)d] < out[(size_t)d]) break;
            ia -= sa[(size_t)d] * out[(size_t)d];
            ib -= sb[(size_t)d] * out[(size_t)d];
            idx[(size_t)d] = 0;
        }
    }
}

bool is_f64(ET t) { return t == ET::f64; }

using Ins = const std::vector<Tensor>&;
using Outs = std::vector<Tensor>&;

// unary over real / integer types
template <class FR, class FI>
bool unary(Ins in, Outs out, FR fr, FI fi) {
    const Tensor& x = in[0];
    const int64_t n = x.numel();
    if (et_is_real(x.et)) {
        if (x.et == ET::f64) {
            Tensor r(ET::f64, x.shape);
            for (int64_t i = 0; i < n; ++i) r.ptr<double>()[i] = fr(x.ptr<double>()[i]);
            out[0] = r;
        } else if (x.et == ET::f32) {
            // fp32 in, fp32 out: no staging copies, large tensors are split over threads
            Tensor r(ET::f32, x.shape);
            const float* p = x.ptr<float>();
            float* q = r.ptr<float>();
            parallel_for(n, n >= (1 << 16) ? 0 : 1, [&](int64_t i0, int64_t i1) {
                for (int64_t i = i0; i < i1; ++i) q[i] = float(fr(double(p[i])));
            });
            out[0] = r;
        } else {
            auto v = to_f32(x);
            for (auto& e : v) e = float(fr(double(e)));
            out[0] = from_f32(x.et, x.shape, v);
        }
    } else {
        auto v = to_i64(x);
        for (auto& e : v) e = fi(e);
        out[0] = from_i64(x.et, x.shape, v);
    }
    return true;
}
template <class FR>
bool unary_real(Ins in, Outs out, FR fr) {
    return unary(in, out, fr, [&](int64_t v) { return (int64_t)fr((double)v); });
}

template <class FR, class FI>
bool binary(const Node& n, Ins in, Outs out, FR fr, FI fi) {
    const Tensor &a = in[0], &b = in[1];
    const Shape os = broadcast_shape(a.shape, b.shape);
    const auto sa = bstrides(a.shape, os), sb = bstrides(b.shape, os);
    const ET et = n.outs[0].et == ET::dynamic ? a.et : (n.outs[0].et == ET::boolean && a.et != ET::boolean ? a.et : n.outs[0].et);
    const ET cet = a.et;
    (void)et;
    if (et_is_real(cet)) {
        if (is_f64(cet)) {
            auto va = to_f64(a), vb = to_f64(b);
            std::vector<double> vo((size_t)shape_size(os));
            broadcast_apply(os, sa, sb, va.data(), vb.data(), vo.data(), fr);
            out[0] = from_f64(cet, os, vo);
        } else if (a.et == ET::f32 && b.et == ET::f32 && (n.outs[0].et == ET::f32 || n.outs[0].et == ET::dynamic)) {
            // fp32 operands: straight from the tensors' memory into the result
            Tensor r(ET::f32, os);
            const float* pa = a.ptr<float>();
            const float* pb = b.ptr<float>();
            float* po = r.ptr<float>();
            const int64_t total = shape_size(os);
            if (a.shape == b.shape) {
                parallel_for(total, total >= (1 << 16) ? 0 : 1, [&](int64_t i0, int64_t i1) {
                    for (int64_t i = i0; i < i1; ++i) po[i] = float(fr(pa[i], pb[i]));
                });
            } else {
                broadcast_apply(os, sa, sb, pa, pb, po, [&](float x, float y) { return float(fr(x, y)); });
            }
            out[0] = r;
        } else {
            auto va = to_f32(a), vb = to_f32(b);
            std::vector<float> vo((size_t)shape_size(os));
            broadcast_apply(os, sa, sb, va.data(), vb.data(), vo.data(), [&](float x, float y) { return float(fr(x, y)); });
            out[0] = from_f32(cet, os, vo);
        }
    } else {
        auto va = to_i64(a), vb = to_i64(b);
        std::vector<int64_t> vo((size_t)shape_size(os));
        broadcast_apply(os, sa, sb, va.data(), vb.data(), vo.data(), fi);
        out[0] = from_i64(cet, os, vo);
    }
    return true;
}

template <class FR, class FI>
bool compare(Ins in, Outs out, FR fr, FI fi) {
    const Tensor &a = in[0], &b = in[1];
    const Shape os = broadcast_shape(a.shape, b.shape);
    const auto sa = bstrides(a.shape, os), sb = bstrides(b.shape, os);
    Tensor r(ET::boolean, os);
    const int64_t n = shape_size(os);
    if (et_is_real(a.et)) {
        auto va = to_f64(a), vb = to_f64(b);
        std::vector<double> vo((size_t)n);
        broadcast_apply(os, sa, sb, va.data(), vb.data(), vo.data(), [&](double x, double y) { return fr(x, y) ? 1.0 : 0.0; });
        for (int64_t i = 0; i < n; ++i) r.data()[i] = vo[(size_t)i] != 0;
    } else {
        auto va = to_i64(a), vb = to_i64(b);
        std::vector<int64_t> vo((size_t)n);
        broadcast_apply(os, sa, sb, va.data(), vb.data(), vo.data(), [&](int64_t x, int64_t y) { return (int64_t)fi(x, y); });
        for (int64_t i = 0; i < n; ++i) r.data()[i] = vo[(size_t)i] != 0;
    }
    out[0] = r;
    return true;
}

std::vector<int64_t> norm_axes(const Tensor& axes, int64_t rank) {
    std::vector<int64_t> a = to_i64(axes);
    for (auto& v : a) { if (v < 0) v += rank; OVC_CHECK(v >= 0 && v < std::max<int64_t>(rank, 1), "axis out of range"); }
    return a;
}

// generic reduction over a set of axes; `init`, `acc`, `fin(value, count)`
template <class Acc, class Fin>
bool reduce(const Node& n, Ins in, Outs out, double init, Acc acc, Fin fin) {
    const Tensor& x = in[0];
    const int64_t rank = (int64_t)x.shape.size();
    auto axes = norm_axes(in[1], rank);
    const bool keep = n.attr_bool("keep_dims");
    std::vector<bool> red((size_t)rank, false);
    for (auto a : axes) red[(size_t)a] = true;
    Shape os, os_keep;
    for (int64_t i = 0; i < rank; ++i) {
        if (red[(size_t)i]) { os_keep.push_back(1); if (keep) os.push_back(1); }
        else { os_keep.push_back(x.shape[(size_t)i]); os.push_back(x.shape[(size_t)i]); }
    }
    const auto ost = strides_of(os_keep);
    const int64_t on = shape_size(os_keep), total = x.numel();
    std::vector<double> accv((size_t)on, init);
    std::vector<int64_t> cnt((size_t)on, 0);
    auto v = to_f64(x);
    std::vector<int64_t> idx((size_t)rank, 0);
    for (int64_t i = 0; i < total; ++i) {
        int64_t o = 0;
        for (int64_t d = 0; d < rank; ++d) if (!red[(size_t)d]) o += idx[(size_t)d] * ost[(size_t)d];
        accv[(size_t)o] = acc(accv[(size_t)o], v[(size_t)i]);
        ++cnt[(size_t)o];
        for (int64_t d = rank - 1; d >= 0; --d) { if (++idx[(size_t)d] < x.shape[(size_t)d]) break; idx[(size_t)d] = 0; }
    }
    const int64_t per = on ? std::max<int64_t>(1, total / std::max<int64_t>(on, 1)) : 1;
    for (int64_t o = 0; o < on; ++o) accv[(size_t)o] = fin(accv[(size_t)o], cnt[(size_t)o] ? cnt[(size_t)o] : per);
    const ET oet = n.type.rfind("ReduceLogical", 0) == 0 ? ET::boolean : x.et;
    out[0] = et_is_real(oet) ? from_f64(oet, os, accv) : [&] { std::vector<int64_t> iv(accv.size()); for (size_t i = 0; i < accv.size(); ++i) iv[i] = (int64_t)std::llround(accv[i]); return from_i64(oet, os, iv); }();
    return true;
}

// Inner block of the fp32 GEMM: rows [m0, m1) x columns [n0, n1) += A[:, k0:k1] * B[k0:k1, :]. Four rows share every load
// of a B row, the column loop is unit stride so that the compiler vectorises it; the function is cloned for AVX-512, AVX2
// and baseline x86-64 and the loader picks the clone that the machine supports.
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
#define OVC_SIMD_CLONES __attribute__((target_clones("arch=x86-64-v4", "arch=x86-64-v3", "default"), optimize("O3")))
#else
#define OVC_SIMD_CLONES
#endif
OVC_SIMD_CLONES
void sgemm_block(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int64_t N, int64_t K, int64_t m0, int64_t m1,
                 int64_t k0, int64_t k1, int64_t n0, int64_t n1) {
    int64_t m = m0;
    for (; m + 4 <= m1; m += 4) {
        float* __restrict__ c0 = C + m * N;
        float* __restrict__ c1 = c0 + N;
        float* __restrict__ c2 = c1 + N;
        float* __restrict__ c3 = c2 + N;
        for (int64_t k = k0; k < k1; ++k) {
            const float a0 = A[m * K + k], a1 = A[(m + 1) * K + k], a2 = A[(m + 2) * K + k], a3 = A[(m + 3) * K + k];
            const float* __restrict__ b = B + k * N;
            for (int64_t nn = n0; nn < n1; ++nn) {
                const float bv = b[nn];
                c0[nn] += a0 * bv;
                c1[nn] += a1 * bv;
                c2[nn] += a2 * bv;
                c3[nn] += a3 * bv;
            }
        }
    }
    for (; m < m1; ++m) {
        float* __restrict__ c = C + m * N;
        for (int64_t k = k0; k < k1; ++k) {
            const float a = A[m * K + k];
            const float* __restrict__ b = B + k * N;
            for (int64_t nn = n0; nn < n1; ++nn) c[nn] += a * b[nn];
        }
    }
}

// C[M,N] (+)= A[M,K] * B[K,N] (row-major, fp32): cache blocking over K and N (the B block stays in L2), the work is split
// over threads along M, or along N when there are fewer rows than threads
void sgemm(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int threads, bool accumulate = false) {
    if (threads <= 0) threads = (int)std::max(1u, std::thread::hardware_concurrency());
    const int64_t KB = 128, NB = 256;
    if (M >= 4 * threads || N < 64 * threads) {
        parallel_for((M + 3) / 4, threads, [&](int64_t q0, int64_t q1) {
            const int64_t m0 = q0 * 4, m1 = std::min(M, q1 * 4);
            for (int64_t m = m0; m < m1; ++m) if (!accumulate) std::fill(C + m * N, C + (m + 1) * N, 0.f);
            for (int64_t k0 = 0; k0 < K; k0 += KB)
                for (int64_t n0 = 0; n0 < N; n0 += NB)
                    sgemm_block(A, B, C, N, K, m0, m1, k0, std::min(K, k0 + KB), n0, std::min(N, n0 + NB));
        });
    } else {
        const int64_t nblocks = (N + NB - 1) / NB;
        parallel_for(nblocks, threads, [&](int64_t b0, int64_t b1) {
            for (int64_t nb = b0; nb < b1; ++nb) {
                const int64_t n0 = nb * NB, n1 = std::min(N, n0 + NB);
                if (!accumulate) for (int64_t m = 0; m < M; ++m) std::fill(C + m * N + n0, C + m * N + n1, 0.f);
                for (int64_t k0 = 0; k0 < K; k0 += KB) sgemm_block(A, B, C, N, K, 0, M, k0, std::min(K, k0 + KB), n0, n1);
            }
        });
    }
}
// C[M,N] = A[M,K] * B[N,K]^T
void sgemm_nt(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K, int threads) {
    parallel_for(M * ((N + 63) / 64), threads, [&](int64_t j0, int64_t j1) {
        const int64_t nb = (N + 63) / 64;
        for (int64_t j = j0; j < j1; ++j) {
            const int64_t m = j / nb, n0 = (j % nb) * 64, n1 = std::min(N, n0 + 64);
            const float* a = A + m * K;
            for (int64_t nn = n0; nn < n1; ++nn) {
                const float* b = B + nn * K;
                float acc0 = 0, acc1 = 0, acc2 = 0, acc3 = 0;
                int64_t k = 0;
                for (; k + 4 <= K; k += 4) { acc0 += a[k] * b[k]; acc1 += a[k + 1] * b[k + 1]; acc2 += a[k + 2] * b[k + 2]; acc3 += a[k + 3] * b[k + 3]; }
                for (; k < K; ++k) acc0 += a[k] * b[k];
                C[m * N + nn] = (acc0 + acc1) + (acc2 + acc3);
            }
        }
    });
}

std::vector<float> transpose2d(const float* a, int64_t r, int64_t c) {
    std::vector<float> t((size_t)(r * c));
    for (int64_t i = 0; i < r; ++i) for (int64_t j = 0; j < c; ++j) t[(size_t)(j * r + i)] = a[i * c + j];
    return t;
}

bool eval_matmul(const Node& n, Ins in, Outs out, EvalContext& ctx, bool ta, bool tb, ET oet) {
    const Tensor &A = in[0], &B = in[1];
    Shape as = A.shape, bs = B.shape;
    const bool a1 = as.size() == 1, b1 = bs.size() == 1;
    if (a1) { as.insert(as.begin(), 1); ta = false; }
    if (b1) { bs.push_back(1); tb = false; }
    const int64_t ar = as[as.size() - 2], ac = as.back(), br = bs[bs.size() - 2], bc = bs.back();
    const int64_t M = ta ? ac : ar, K = ta ? ar : ac, K2 = tb ? bc : br, N = tb ? br : bc;
    OVC_CHECK(K == K2, n.description() << ": inner dimensions differ (" << K << " vs " << K2 << ")");
    Shape ba(as.begin(), as.end() - 2), bb(bs.begin(), bs.end() - 2);
    const Shape bo = broadcast_shape(ba, bb);
    const auto sa = bstrides(ba, bo), sb = bstrides(bb, bo);
    const int64_t nb = shape_size(bo);
    auto va = to_f32(A), vb = to_f32(B);
    std::vector<float> vo((size_t)(nb * M * N));
    std::vector<int64_t> idx(bo.size(), 0);
    for (int64_t bi = 0; bi < nb; ++bi) {
        int64_t oa = 0, ob = 0;
        for (size_t d = 0; d < bo.size(); ++d) { oa += idx[d] * sa[d]; ob += idx[d] * sb[d]; }
        const float* pa = va.data() + oa * ar * ac;
        const float* pb = vb.data() + ob * br * bc;
        std::vector<float> ta_buf, tb_buf;
        if (ta) { ta_buf = transpose2d(pa, ar, ac); pa = ta_buf.data(); }
        if (tb) sgemm_nt(pa, pb, vo.data() + bi * M * N, M, N, K, ctx.num_threads);
        else sgemm(pa, pb, vo.data() + bi * M * N, M, N, K, ctx.num_threads);
        for (int64_t d = (int64_t)bo.size() - 1; d >= 0; --d) { if (++idx[(size_t)d] < bo[(size_t)d]) break; idx[(size_t)d] = 0; }
    }
    Shape os = bo;
    if (!a1) os.push_back(M);
    if (!b1) os.push_back(N);
    out[0] = from_f32(oet == ET::dynamic ? A.et : oet, os, vo);
    return true;
}

void resolve_pads(const Node& n, const Shape& in_sp, const std::vector<int64_t>& k, const std::vector<int64_t>& st,
                  const std::vector<int64_t>& dil, std::vector<int64_t>& pb, std::vector<int64_t>& pe) {
    const std::string ap = n.attr_str("auto_pad", "explicit");
    const size_t sp = k.size();
    if (ap == "same_upper" || ap == "same_lower") {
        pb.assign(sp, 0); pe.assign(sp, 0);
        for (size_t i = 0; i < sp; ++i) {
            const int64_t o = (in_sp[i] + st[i] - 1) / st[i];
            const int64_t total = std::max<int64_t>(0, (o - 1) * st[i] + dil[i] * (k[i] - 1) + 1 - in_sp[i]);
            const int64_t half = total / 2;
            if (ap == "same_upper") { pb[i] = half; pe[i] = total - half; } else { pe[i] = half; pb[i] = total - half; }
        }
    } else if (ap == "valid") { pb.assign(sp, 0); pe.assign(sp, 0); }
}

// 1-D/2-D/3-D convolution through im2col + GEMM, groups supported
bool eval_conv(const Node& n, Ins in, Outs out, EvalContext& ctx, bool group) {
    const Tensor &X = in[0], &W = in[1];
    const size_t sp = X.shape.size() - 2;
    OVC_CHECK(sp >= 1 && sp <= 3, n.description() << ": only 1-3 spatial dimensions are supported");
    auto st = n.attr_ints("strides"), dil = n.attr_ints("dilations"), pb = n.attr_ints("pads_begin"), pe = n.attr_ints("pads_end");
    if (st.empty()) st.assign(sp, 1);
    if (dil.empty()) dil.assign(sp, 1);
    if (pb.empty()) pb.assign(sp, 0);
    if (pe.empty()) pe.assign(sp, 0);
    const int64_t G = group ? W.shape[0] : 1;
    const size_t wo = group ? 1 : 0;
    const int64_t Cout_g = W.shape[wo], Cin_g = W.shape[wo + 1];
    const int64_t N = X.shape[0], Cin = X.shape[1];
    OVC_CHECK(Cin == Cin_g * G, n.description() << ": channel mismatch");
    Shape isp(X.shape.begin() + 2, X.shape.end()), ksp(W.shape.begin() + (long)wo + 2, W.shape.end());
    resolve_pads(n, isp, ksp, st, dil, pb, pe);
    Shape osp(sp);
    for (size_t i = 0; i < sp; ++i) osp[i] = (isp[i] + pb[i] + pe[i] - (dil[i] * (ksp[i] - 1) + 1)) / st[i] + 1;
    // pad to 3 spatial dims
    auto pad3 = [&](Shape s, int64_t v) { while (s.size() < 3) s.insert(s.begin(), v); return s; };
    const Shape I = pad3(isp, 1), Kk = pad3(ksp, 1), O = pad3(osp, 1);
    auto pad3v = [&](std::vector<int64_t> s, int64_t v) { while (s.size() < 3) s.insert(s.begin(), v); return s; };
    const auto S = pad3v(st, 1), D = pad3v(dil, 1), PB = pad3v(pb, 0);
    const int64_t ksz = Kk[0] * Kk[1] * Kk[2], osz = O[0] * O[1] * O[2], isz = I[0] * I[1] * I[2];
    // fp32 tensors are read and written in place; other types go through fp32 copies
    std::vector<float> vx_c, vw_c, vo_c;
    if (X.et != ET::f32) vx_c = to_f32(X);
    if (W.et != ET::f32) vw_c = to_f32(W);
    const float* vx_p = X.et == ET::f32 ? X.ptr<float>() : vx_c.data();
    const float* vw_p = W.et == ET::f32 ? W.ptr<float>() : vw_c.data();
    Shape os = {N, G * Cout_g};
    os.insert(os.end(), osp.begin(), osp.end());
    Tensor result;
    float* vo_p;
    if (X.et == ET::f32) {
        result = Tensor(ET::f32, os);
        vo_p = result.ptr<float>();
    } else {
        vo_c.resize((size_t)(N * G * Cout_g * osz));
        vo_p = vo_c.data();
    }
    const int64_t Kdim = Cin_g * ksz;
    std::vector<float> col((size_t)(Kdim * osz));
    for (int64_t b = 0; b < N; ++b) {
        for (int64_t g = 0; g < G; ++g) {
            const float* xg = vx_p + (b * Cin + g * Cin_g) * isz;
            parallel_for(Kdim, ctx.num_threads, [&](int64_t r0, int64_t r1) {
                for (int64_t r = r0; r < r1; ++r) {
                    const int64_t c = r / ksz, kk = r % ksz;
                    const int64_t kz = kk / (Kk[1] * Kk[2]), ky = (kk / Kk[2]) % Kk[1], kx = kk % Kk[2];
                    float* dst = col.data() + r * osz;
                    const float* src = xg + c * isz;
                    for (int64_t oz = 0; oz < O[0]; ++oz) {
                        const int64_t iz = oz * S[0] - PB[0] + kz * D[0];
                        for (int64_t oy = 0; oy < O[1]; ++oy) {
                            const int64_t iy = oy * S[1] - PB[1] + ky * D[1];
                            for (int64_t ox = 0; ox < O[2]; ++ox) {
                                const int64_t ix = ox * S[2] - PB[2] + kx * D[2];
                                const bool ok = iz >= 0 && iz < I[0] && iy >= 0 && iy < I[1] && ix >= 0 && ix < I[2];
                                dst[(oz * O[1] + oy) * O[2] + ox] = ok ? src[(iz * I[1] + iy) * I[2] + ix] : 0.f;
                            }
                        }
                    }
                }
            });
            sgemm(vw_p + g * Cout_g * Kdim, col.data(), vo_p + (b * G + g) * Cout_g * osz, Cout_g, osz, Kdim, ctx.num_threads);
        }
    }
    out[0] = X.et == ET::f32 ? result : from_f32(X.et, os, vo_c);
    return true;
}

bool eval_pool(const Node& n, Ins in, Outs out, EvalContext& ctx, bool maxpool) {
    const Tensor& X = in[0];
    const size_t sp = X.shape.size() - 2;
    OVC_CHECK(sp >= 1 && sp <= 3, n.description() << ": only 1-3 spatial dimensions are supported");
    auto k = n.attr_ints("kernel"), st = n.attr_ints("strides"), pb = n.attr_ints("pads_begin"), pe = n.attr_ints("pads_end");
    auto dil = n.has_attr("dilations") ? n.attr_ints("dilations") : std::vector<int64_t>();
    if (dil.empty()) dil.assign(sp, 1);
    if (st.empty()) st.assign(sp, 1);
    if (pb.empty()) pb.assign(sp, 0);
    if (pe.empty()) pe.assign(sp, 0);
    Shape isp(X.shape.begin() + 2, X.shape.end());
    resolve_pads(n, isp, k, st, dil, pb, pe);
    const Shape osp_full = n.outs[0].shape.is_static() ? n.outs[0].shape.to_shape() : Shape();
    Shape osp(sp);
    const std::string rt = n.attr_str("rounding_type", "floor");
    const bool ceil_mode = rt != "floor";
    for (size_t i = 0; i < sp; ++i) {
        const int64_t eff = dil[i] * (k[i] - 1) + 1, num = isp[i] + pb[i] + pe[i] - eff;
        int64_t o = (ceil_mode ? (num + st[i] - 1) / st[i] : num / st[i]) + 1;
        if (ceil_mode && (o - 1) * st[i] >= isp[i] + pb[i]) --o;
        osp[i] = o;
    }
    auto pad3 = [&](std::vector<int64_t> s, int64_t v) { while (s.size() < 3) s.insert(s.begin(), v); return s; };
    const auto I = pad3(isp, 1), Kk = pad3(k, 1), O = pad3(osp, 1), S = pad3(st, 1), D = pad3(dil, 1), PB = pad3(pb, 0), PE = pad3(pe, 0);
    const int64_t NC = X.shape[0] * X.shape[1], isz = I[0] * I[1] * I[2], osz = O[0] * O[1] * O[2];
    auto vx = to_f32(X);
    std::vector<float> vo((size_t)(NC * osz));
    std::vector<int64_t> vi(maxpool && n.num_outputs() > 1 ? (size_t)(NC * osz) : 0);
    const bool exclude_pad = n.attr_bool("exclude-pad");
    parallel_for(NC, ctx.num_threads, [&](int64_t c0, int64_t c1) {
        for (int64_t c = c0; c < c1; ++c) {
            const float* src = vx.data() + c * isz;
            for (int64_t oz = 0; oz < O[0]; ++oz) for (int64_t oy = 0; oy < O[1]; ++oy) for (int64_t ox = 0; ox < O[2]; ++ox) {
                float best = -std::numeric_limits<float>::infinity(), sum = 0.f;
                int64_t besti = 0, cnt = 0, cnt_pad = 0;
                for (int64_t kz = 0; kz < Kk[0]; ++kz) for (int64_t ky = 0; ky < Kk[1]; ++ky) for (int64_t kx = 0; kx < Kk[2]; ++kx) {
                    const int64_t iz = oz * S[0] - PB[0] + kz * D[0], iy = oy * S[1] - PB[1] + ky * D[1], ix = ox * S[2] - PB[2] + kx * D[2];
                    const bool inside = iz >= 0 && iz < I[0] && iy >= 0 && iy < I[1] && ix >= 0 && ix < I[2];
                    // positions inside the declared padding count for include-pad averages; ceil-mode overhang does not
                    const bool in_padded = iz < I[0] + PE[0] && iy < I[1] + PE[1] && ix < I[2] + PE[2];
                    if (in_padded) ++cnt_pad;
                    if (!inside) continue;
                    const int64_t ii = (iz * I[1] + iy) * I[2] + ix;
                    const float v = src[ii];
                    if (v > best) { best = v; besti = ii; }
                    sum += v;
                    ++cnt;
                }
                const int64_t oi = c * osz + (oz * O[1] + oy) * O[2] + ox;
                if (maxpool) { vo[(size_t)oi] = best; if (!vi.empty()) vi[(size_t)oi] = besti; }
                else vo[(size_t)oi] = sum / float(std::max<int64_t>(1, exclude_pad ? cnt : cnt_pad));
            }
        }
    });
    Shape os = {X.shape[0], X.shape[1]};
    os.insert(os.end(), osp.begin(), osp.end());
    (void)osp_full;
    out[0] = from_f32(X.et, os, vo);
    if (!vi.empty()) out[1] = from_i64(n.outs[1].et, os, vi);
    return true;
}

bool eval_softmax(const Node& n, Ins in, Outs out, bool log) {
    const Tensor& x = in[0];
    const int64_t rank = (int64_t)x.shape.size();
    int64_t axis = n.attr_int("axis");
    if (axis < 0) axis += rank;
    int64_t outer = 1, inner = 1;
    for (int64_t i = 0; i < axis; ++i) outer *= x.shape[(size_t)i];
    for (int64_t i = axis + 1; i < rank; ++i) inner *= x.shape[(size_t)i];
    const int64_t A = rank ? x.shape[(size_t)axis] : 1;
    auto v = to_f32(x);
    for (int64_t o = 0; o < outer; ++o) for (int64_t i = 0; i < inner; ++i) {
        float* p = v.data() + o * A * inner + i;
        float mx = -std::numeric_limits<float>::infinity();
        for (int64_t a = 0; a < A; ++a) mx = std::max(mx, p[a * inner]);
        double s = 0;
        for (int64_t a = 0; a < A; ++a) { const float e = (mx == -std::numeric_limits<float>::infinity()) ? 0.f : std::exp(p[a * inner] - mx); if (!log) p[a * inner] = e; s += e; }
        if (log) { const float ls = float(std::log(s)); for (int64_t a = 0; a < A; ++a) p[a * inner] = p[a * inner] - mx - ls; }
        else { const float inv = s > 0 ? float(1.0 / s) : 0.f; for (int64_t a = 0; a < A; ++a) p[a * inner] *= inv; }
    }
    out[0] = from_f32(x.et, x.shape, v);
    return true;
}

// copy with generic permutation/strides: out[idx] = in[sum idx[d]*src_stride[d] + offset]
Tensor gather_strided(const Tensor& x, const Shape& os, const std::vector<int64_t>& src_strides, int64_t offset) {
    const int64_t n = shape_size(os);
    const size_t r = os.size();
    const int bits = et_bits(x.et);
    Tensor o(x.et, os);
    if (x.et == ET::string) {
        std::vector<int64_t> idx(r, 0);
        int64_t src = offset;
        for (int64_t i = 0; i < n; ++i) {
            o.strings[(size_t)i] = x.strings[(size_t)src];
            for (int64_t d = (int64_t)r - 1; d >= 0; --d) { ++idx[(size_t)d]; src += src_strides[(size_t)d]; if (idx[(size_t)d] < os[(size_t)d]) break; src -= src_strides[(size_t)d] * os[(size_t)d]; idx[(size_t)d] = 0; }
        }
        return o;
    }
    if (bits % 8 != 0) {
        std::vector<int64_t> idx(r, 0);
        int64_t src = offset;
        for (int64_t i = 0; i < n; ++i) {
            set_elem_f64(o, i, get_elem_f64(x, src));
            for (int64_t d = (int64_t)r - 1; d >= 0; --d) { ++idx[(size_t)d]; src += src_strides[(size_t)d]; if (idx[(size_t)d] < os[(size_t)d]) break; src -= src_strides[(size_t)d] * os[(size_t)d]; idx[(size_t)d] = 0; }
        }
        return o;
    }
    const size_t es = (size_t)bits / 8;
    const uint8_t* sp = x.data();
    uint8_t* dp = o.data();
    // innermost contiguous run
    if (r == 0) { std::memcpy(dp, sp + (size_t)offset * es, es); return o; }
    std::vector<int64_t> idx(r, 0);
    int64_t src = offset;
    const bool inner_contig = src_strides[r - 1] == 1;
    const int64_t inner = os[r - 1];
    if (inner_contig && inner > 0) {
        const int64_t rows = n / inner;
        for (int64_t row = 0; row < rows; ++row) {
            std::memcpy(dp + (size_t)(row * inner) * es, sp + (size_t)src * es, (size_t)inner * es);
            for (int64_t d = (int64_t)r - 2; d >= 0; --d) { ++idx[(size_t)d]; src += src_strides[(size_t)d]; if (idx[(size_t)d] < os[(size_t)d]) break; src -= src_strides[(size_t)d] * os[(size_t)d]; idx[(size_t)d] = 0; }
        }
        return o;
    }
    for (int64_t i = 0; i < n; ++i) {
        std::memcpy(dp + (size_t)i * es, sp + (size_t)src * es, es);
        for (int64_t d = (int64_t)r - 1; d >= 0; --d) { ++idx[(size_t)d]; src += src_strides[(size_t)d]; if (idx[(size_t)d] < os[(size_t)d]) break; src -= src_strides[(size_t)d] * os[(size_t)d]; idx[(size_t)d] = 0; }
    }
    return o;
}

Tensor reshape_view(const Tensor& x, const Shape& s) {
    Tensor o = x;
    o.shape = s;
    return o;
}

bool eval_reshape(const Node& n, Ins in, Outs out) {
    const Tensor& x = in[0];
    auto pat = to_i64(in[1]);
    const bool sz = n.attr_bool("special_zero");
    Shape os(pat.size());
    int64_t known = 1;
    int neg = -1;
    for (size_t i = 0; i < pat.size(); ++i) {
        if (pat[i] == -1) { neg = (int)i; continue; }
        os[i] = (pat[i] == 0 && sz) ? x.shape.at(i) : pat[i];
        known *= os[i];
    }
    if (neg >= 0) os[(size_t)neg] = known ? x.numel() / known : 0;
    OVC_CHECK(shape_size(os) == x.numel(), n.description() << ": cannot reshape " << PShape(x.shape).str() << " to " << PShape(os).str());
    out[0] = reshape_view(x, os);
    return true;
}

bool eval_concat(const Node& n, Ins in, Outs out) {
    const int64_t rank = (int64_t)in[0].shape.size();
    int64_t axis = n.attr_int("axis");
    if (axis < 0) axis += rank;
    Shape os = in[0].shape;
    os[(size_t)axis] = 0;
    for (auto& t : in) os[(size_t)axis] += t.shape[(size_t)axis];
    Tensor o(in[0].et, os);
    int64_t outer = 1, inner = 1;
    for (int64_t i = 0; i < axis; ++i) outer *= os[(size_t)i];
    for (int64_t i = axis + 1; i < rank; ++i) inner *= os[(size_t)i];
    const int bits = et_bits(o.et);
    if (o.et == ET::string || bits % 8 != 0) {
        int64_t pos = 0;
        for (int64_t ou = 0; ou < outer; ++ou) for (auto& t : in) {
            const int64_t len = t.shape[(size_t)axis] * inner;
            for (int64_t i = 0; i < len; ++i) {
                if (o.et == ET::string) o.strings[(size_t)pos] = t.strings[(size_t)(ou * len + i)];
                else set_elem_f64(o, pos, get_elem_f64(t, ou * len + i));
                ++pos;
            }
        }
    } else {
        const size_t es = (size_t)bits / 8;
        uint8_t* dp = o.data();
        for (int64_t ou = 0; ou < outer; ++ou) for (auto& t : in) {
            const size_t len = (size_t)(t.shape[(size_t)axis] * inner) * es;
            if (len) std::memcpy(dp, t.data() + (size_t)ou * len, len);
            dp += len;
        }
    }
    out[0] = o;
    return true;
}

Tensor slice_axis(const Tensor& x, int64_t axis, int64_t begin, int64_t count, int64_t step = 1) {
    Shape os = x.shape;
    os[(size_t)axis] = count;
    auto st = strides_of(x.shape);
    const int64_t off = begin * st[(size_t)axis];
    st[(size_t)axis] *= step;
    return gather_strided(x, os, st, off);
}

bool eval_gather(const Node& n, Ins in, Outs out) {
    const Tensor &d = in[0], &idx = in[1];
    const int64_t rank = (int64_t)d.shape.size();
    int64_t axis = to_i64(in[2]).at(0);
    if (axis < 0) axis += rank;
    int64_t bd = n.attr_int("batch_dims");
    if (bd < 0) bd += (int64_t)idx.shape.size();
    auto iv = to_i64(idx);
    const int64_t A = d.shape[(size_t)axis];
    int64_t batch = 1, outer = 1, inner = 1, ipb = 1;
    for (int64_t i = 0; i < bd; ++i) batch *= d.shape[(size_t)i];
    for (int64_t i = bd; i < axis; ++i) outer *= d.shape[(size_t)i];
    for (int64_t i = axis + 1; i < rank; ++i) inner *= d.shape[(size_t)i];
    for (size_t i = (size_t)bd; i < idx.shape.size(); ++i) ipb *= idx.shape[i];
    Shape os;
    for (int64_t i = 0; i < axis; ++i) os.push_back(d.shape[(size_t)i]);
    for (size_t i = (size_t)bd; i < idx.shape.size(); ++i) os.push_back(idx.shape[i]);
    for (int64_t i = axis + 1; i < rank; ++i) os.push_back(d.shape[(size_t)i]);
    Tensor o(d.et, os);
    const int bits = et_bits(d.et);
    const bool bytes = d.et != ET::string && bits % 8 == 0;
    const size_t es = bytes ? (size_t)bits / 8 : 0;
    int64_t pos = 0;
    for (int64_t b = 0; b < batch; ++b) for (int64_t ou = 0; ou < outer; ++ou) for (int64_t k = 0; k < ipb; ++k) {
        int64_t i = iv[(size_t)(b * ipb + k)];
        if (i < 0) i += A;
        const bool ok = i >= 0 && i < A;
        const int64_t src = ((b * outer + ou) * A + (ok ? i : 0)) * inner;
        if (bytes) {
            if (ok) std::memcpy(o.data() + (size_t)pos * es, d.data() + (size_t)src * es, (size_t)inner * es);
            else std::memset(o.data() + (size_t)pos * es, 0, (size_t)inner * es);
        } else {
            for (int64_t j = 0; j < inner; ++j) {
                if (d.et == ET::string) o.strings[(size_t)(pos + j)] = ok ? d.strings[(size_t)(src + j)] : std::string();
                else set_elem_f64(o, pos + j, ok ? get_elem_f64(d, src + j) : 0.0);
            }
        }
        pos += inner;
    }
    out[0] = o;
    return true;
}

float gelu_erf(float v) { return 0.5f * v * (1.0f + std::erf(v * 0.70710678118654752f)); }
float gelu_tanh(float v) { return 0.5f * v * (1.0f + std::tanh(0.7978845608028654f * (v + 0.044715f * v * v * v))); }

// scaled dot product attention over [..., L, E] x [..., S, E] x [..., S, Ev]
bool eval_sdpa(const Node& n, Ins in, Outs out, EvalContext& ctx) {
    const Tensor &Q = in[0], &Kt = in[1], &V = in[2];
    const size_t r = Q.shape.size();
    OVC_CHECK(r >= 2, n.description() << ": rank must be at least 2");
    const int64_t L = Q.shape[r - 2], E = Q.shape[r - 1], S = Kt.shape[Kt.shape.size() - 2], Ev = V.shape.back();
    Shape bq(Q.shape.begin(), Q.shape.end() - 2), bk(Kt.shape.begin(), Kt.shape.end() - 2), bv(V.shape.begin(), V.shape.end() - 2);
    const Shape bo = broadcast_shape(bq, broadcast_shape(bk, bv));
    const auto sq = bstrides(bq, bo), sk = bstrides(bk, bo), sv = bstrides(bv, bo);
    const int64_t nb = shape_size(bo);
    const bool causal = n.attr_bool("causal");
    float scale = 1.0f / std::sqrt(float(E));
    if (in.size() > 4 && in[4].numel() > 0) scale = float(get_elem_f64(in[4], 0));
    std::vector<float> mask;
    Shape mshape;
    bool bool_mask = false;
    if (in.size() > 3 && in[3].numel() > 0 && !causal) {
        mshape = in[3].shape;
        bool_mask = in[3].et == ET::boolean;
        mask = to_f32(in[3]);
    }
    std::vector<float> sinks;
    if (in.size() > 5 && in[5].numel() > 0) sinks = to_f32(in[5]);
    Shape full = bo; full.push_back(L); full.push_back(S);
    std::vector<int64_t> ms;
    if (!mask.empty()) ms = bstrides(mshape, full);
    auto vq = to_f32(Q), vk = to_f32(Kt), vv = to_f32(V);
    std::vector<float> vo((size_t)(nb * L * Ev));
    parallel_for(nb, ctx.num_threads, [&](int64_t b0, int64_t b1) {
        std::vector<float> s((size_t)S);
        for (int64_t b = b0; b < b1; ++b) {
            std::vector<int64_t> idx(bo.size());
            int64_t rem = b;
            for (int64_t d = (int64_t)bo.size() - 1; d >= 0; --d) { idx[(size_t)d] = rem % bo[(size_t)d]; rem /= bo[(size_t)d]; }
            int64_t oq = 0, ok = 0, ov = 0, om = 0;
            for (size_t d = 0; d < bo.size(); ++d) { oq += idx[d] * sq[d]; ok += idx[d] * sk[d]; ov += idx[d] * sv[d]; if (!ms.empty()) om += idx[d] * ms[d]; }
            const float* q = vq.data() + oq * L * E;
            const float* k = vk.data() + ok * S * E;
            const float* v = vv.data() + ov * S * Ev;
            for (int64_t l = 0; l < L; ++l) {
                float mx = -std::numeric_limits<float>::infinity();
                for (int64_t j = 0; j < S; ++j) {
                    float acc = 0;
                    for (int64_t e = 0; e < E; ++e) acc += q[l * E + e] * k[j * E + e];
                    acc *= scale;
                    if (causal) { if (j > l + (S - L)) acc = -std::numeric_limits<float>::infinity(); }
                    else if (!mask.empty()) {
                        const float m = mask[(size_t)(om + l * ms[bo.size()] + j * ms[bo.size() + 1])];
                        if (bool_mask) { if (m == 0.f) acc = -std::numeric_limits<float>::infinity(); } else acc += m;
                    }
                    s[(size_t)j] = acc;
                    mx = std::max(mx, acc);
                }
                float sink = 0.f;
                bool has_sink = false;
                if (!sinks.empty()) { has_sink = true; sink = sinks[(size_t)(idx.size() >= 2 ? idx[idx.size() - 1] % (int64_t)sinks.size() : 0)]; mx = std::max(mx, sink); }
                double sum = 0;
                for (int64_t j = 0; j < S; ++j) { s[(size_t)j] = (mx == -std::numeric_limits<float>::infinity()) ? 0.f : std::exp(s[(size_t)j] - mx); sum += s[(size_t)j]; }
                if (has_sink) sum += std::exp(sink - mx);
                const float inv = sum > 0 ? float(1.0 / sum) : 0.f;
                float* o = vo.data() + (b * L + l) * Ev;
                std::fill(o, o + Ev, 0.f);
                for (int64_t j = 0; j < S; ++j) { const float p = s[(size_t)j] * inv; if (p == 0.f) continue; for (int64_t e = 0; e < Ev; ++e) o[e] += p * v[j * Ev + e]; }
            }
        }
    });
    Shape os = bo; os.push_back(L); os.push_back(Ev);
    out[0] = from_f32(Q.et, os, vo);
    return true;
}

// Dequantise a compressed weight [N, K] given scales [N, G(,1)] and optional zero points
std::vector<float> dequant_weight(const Tensor& w, const Tensor& scales, const Tensor* zp) {
    OVC_CHECK(w.shape.size() >= 2, "compressed weight must have rank >= 2");
    const int64_t N = w.shape[0];
    const int64_t K = w.numel() / N;
    const int64_t G = std::max<int64_t>(1, scales.numel() / N);
    const int64_t gs = K / G;
    std::vector<float> out((size_t)(N * K));
    auto vs = to_f32(scales);
    std::vector<float> vz;
    if (zp && zp->numel() > 0) vz = to_f32(*zp);
    for (int64_t nrow = 0; nrow < N; ++nrow) for (int64_t k = 0; k < K; ++k) {
        const int64_t g = k / gs;
        const float s = vs[(size_t)(vs.size() == 1 ? 0 : nrow * G + g)];
        const float z = vz.empty() ? 0.f : vz[(size_t)(vz.size() == 1 ? 0 : nrow * G + g)];
        out[(size_t)(nrow * K + k)] = (float(get_elem_f64(w, nrow * K + k)) - z) * s;
    }
    return out;
}

bool eval_if_loop(const Node& n, Ins in, Outs out, EvalContext& ctx) {
    auto triples = [](const std::vector<int64_t>& v, size_t w) { std::vector<std::vector<int64_t>> r; for (size_t i = 0; i + w <= v.size(); i += w) r.emplace_back(v.begin() + (long)i, v.begin() + (long)(i + w)); return r; };
    if (n.type == "If") {
        const bool cond = get_elem_f64(in[0], 0) != 0;
        const Model& body = *n.bodies[cond ? 0 : 1];
        const auto im = triples(n.attr_ints(cond ? "input_map" : "else_input_map"), 3);
        const auto om = triples(n.attr_ints(cond ? "output_map" : "else_output_map"), 2);
        std::vector<Tensor> bin(body.params.size());
        for (auto& t : im) bin.at((size_t)t[1]) = in.at((size_t)t[0]);
        auto res = evaluate_model(body, bin, ctx);
        for (size_t i = 0; i < om.size(); ++i) out.at(i) = res.at((size_t)om[i][0]);
        return true;
    }
    // Loop / TensorIterator
    const Model& body = *n.bodies[0];
    const auto im = triples(n.attr_ints("input_map"), 3);
    const auto om = triples(n.attr_ints("output_map"), 2);
    const auto be = triples(n.attr_ints("back_edges"), 2);   // (body result, body parameter)
    const bool is_loop = n.type == "Loop";
    int64_t trip = -1;
    bool cond = true;
    if (is_loop) {
        trip = get_elem_i64(in[0], 0);
        cond = get_elem_f64(in[1], 0) != 0;
    }
    // sliced inputs define the trip count of a TensorIterator
    for (auto& t : im) if (t[2] >= 0) { const int64_t len = in.at((size_t)t[0]).shape.at((size_t)t[2]); if (trip < 0 || len < trip) trip = len; }
    if (trip < 0) trip = std::numeric_limits<int64_t>::max();
    std::vector<Tensor> bin(body.params.size());
    for (auto& t : im) if (t[2] < 0) bin.at((size_t)t[1]) = in.at((size_t)t[0]);
    const int64_t cur_iter = n.attr_int("current_iteration_input", -1), cond_out = n.attr_int("body_condition_output", -1);
    std::vector<std::vector<Tensor>> collected(om.size());
    std::vector<Tensor> last;
    for (int64_t it = 0; it < trip && cond; ++it) {
        for (auto& t : im) if (t[2] >= 0) {
            Tensor sl = slice_axis(in.at((size_t)t[0]), t[2], it, 1);
            bin.at((size_t)t[1]) = sl;
        }
        if (cur_iter >= 0) bin.at((size_t)cur_iter) = from_i64(body.params.at((size_t)cur_iter)->outs[0].et, body.params.at((size_t)cur_iter)->outs[0].shape.is_static() ? body.params.at((size_t)cur_iter)->outs[0].shape.to_shape() : Shape{1}, {it});
        last = evaluate_model(body, bin, ctx);
        for (auto& e : be) bin.at((size_t)e[1]) = last.at((size_t)e[0]);
        for (size_t i = 0; i < om.size(); ++i) if (om[i][1] >= 0) collected[i].push_back(last.at((size_t)om[i][0]));
        if (cond_out >= 0) cond = get_elem_f64(last.at((size_t)cond_out), 0) != 0;
    }
    for (size_t i = 0; i < om.size(); ++i) {
        if (om[i][1] >= 0) {
            OVC_CHECK(!collected[i].empty(), n.description() << ": zero iterations with concatenated outputs");
            auto cn = make_node("Concat", "opset1", {make_constant(collected[i][0])->output(0)}, {{"axis", Attr::Int(om[i][1])}}, false);
            std::vector<Tensor> o1(1);
            eval_concat(*cn, collected[i], o1);
            out.at(i) = o1[0];
        } else {
            OVC_CHECK(!last.empty(), n.description() << ": zero iterations");
            out.at(i) = last.at((size_t)om[i][0]);
        }
    }
    return true;
}

void set_eval(const char* type, EvalFn fn) {
    auto& r = OpRegistry::get();
    bool any = false;
    for (auto* s : r.all()) if (s->type == type) { const_cast<OpSchema*>(s)->eval = fn; any = true; }
    OVC_CHECK(any, "set_eval: unknown op " << type);
}

}  // namespace

// Paged attention over host tensors; defined in eval_llm.cpp
bool eval_paged_attention(const Node& n, Ins in, Outs out, EvalContext& ctx);
bool eval_rope(const Node& n, Ins in, Outs out, EvalContext& ctx);
bool eval_moe(const Node& n, Ins in, Outs out, EvalContext& ctx);

void register_eval_functions() {
    using N = const Node&;
    using C = EvalContext&;
    set_eval("Parameter", [](N, Ins, Outs, C) { return false; });
    set_eval("Result", [](N, Ins in, Outs out, C) { out[0] = in[0]; return true; });
    set_eval("Constant", [](N n, Ins, Outs out, C) { out[0] = n.constant; return true; });
    set_eval("Convert", [](N n, Ins in, Outs out, C) { out[0] = convert_tensor(in[0], n.attr("destination_type").et); return true; });
    set_eval("ConvertLike", [](N, Ins in, Outs out, C) { out[0] = convert_tensor(in[0], in[1].et); return true; });

#define UNARY_REAL(NAME, EXPR) set_eval(NAME, [](N, Ins in, Outs out, C) { return unary_real(in, out, [](double v) -> double { return EXPR; }); })
    UNARY_REAL("Acos", std::acos(v)); UNARY_REAL("Asin", std::asin(v)); UNARY_REAL("Atan", std::atan(v));
    UNARY_REAL("Cos", std::cos(v)); UNARY_REAL("Cosh", std::cosh(v)); UNARY_REAL("Erf", std::erf(v));
    UNARY_REAL("Exp", std::exp(v)); UNARY_REAL("Log", std::log(v)); UNARY_REAL("Sin", std::sin(v)); UNARY_REAL("Sinh", std::sinh(v));
    UNARY_REAL("Sqrt", std::sqrt(v)); UNARY_REAL("Tan", std::tan(v)); UNARY_REAL("Tanh", std::tanh(v));
    UNARY_REAL("Asinh", std::asinh(v)); UNARY_REAL("Acosh", std::acosh(v)); UNARY_REAL("Atanh", std::atanh(v));
    UNARY_REAL("Sigmoid", 1.0 / (1.0 + std::exp(-v)));
    UNARY_REAL("Mish", v * std::tanh(std::log1p(std::exp(v))));
    UNARY_REAL("HSwish", v * std::min(std::max(v + 3.0, 0.0), 6.0) / 6.0);
    UNARY_REAL("HSigmoid", std::min(std::max(v + 3.0, 0.0), 6.0) / 6.0);
    UNARY_REAL("SoftPlus", v > 20.0 ? v : std::log1p(std::exp(v)));
    UNARY_REAL("SoftSign", v / (1.0 + std::fabs(v)));
#undef UNARY_REAL
    set_eval("Abs", [](N, Ins in, Outs out, C) { return unary(in, out, [](double v) { return std::fabs(v); }, [](int64_t v) { return v < 0 ? -v : v; }); });
    set_eval("Negative", [](N, Ins in, Outs out, C) { return unary(in, out, [](double v) { return -v; }, [](int64_t v) { return -v; }); });
    set_eval("Ceiling", [](N, Ins in, Outs out, C) { return unary(in, out, [](double v) { return std::ceil(v); }, [](int64_t v) { return v; }); });
    set_eval("Floor", [](N, Ins in, Outs out, C) { return unary(in, out, [](double v) { return std::floor(v); }, [](int64_t v) { return v; }); });
    set_eval("Sign", [](N, Ins in, Outs out, C) { return unary(in, out, [](double v) { return double((v > 0) - (v < 0)); }, [](int64_t v) { return int64_t((v > 0) - (v < 0)); }); });
    set_eval("Relu", [](N, Ins in, Outs out, C) { return unary(in, out, [](double v) { return v > 0 ? v : 0.0; }, [](int64_t v) { return v > 0 ? v : 0; }); });
    set_eval("Round", [](N n, Ins in, Outs out, C) {
        const bool even = n.attr_str("mode") == "half_to_even";
        return unary(in, out, [even](double v) { return even ? std::nearbyint(v) : std::round(v); }, [](int64_t v) { return v; });
    });
    set_eval("Gelu", [](N n, Ins in, Outs out, C) {
        const bool th = n.has_attr("approximation_mode") && (n.attr_str("approximation_mode") == "TANH" || n.attr_str("approximation_mode") == "tanh");
        auto v = to_f32(in[0]);
        for (auto& e : v) e = th ? gelu_tanh(e) : gelu_erf(e);
        out[0] = from_f32(in[0].et, in[0].shape, v);
        return true;
    });
    set_eval("Swish", [](N, Ins in, Outs out, C) {
        const float beta = in.size() > 1 ? float(get_elem_f64(in[1], 0)) : 1.0f;
        auto v = to_f32(in[0]);
        for (auto& e : v) e = e / (1.0f + std::exp(-beta * e));
        out[0] = from_f32(in[0].et, in[0].shape, v);
        return true;
    });
    set_eval("Elu", [](N n, Ins in, Outs out, C) { const double a = n.attr_float("alpha"); return unary_real(in, out, [a](double v) { return v >= 0 ? v : a * (std::exp(v) - 1.0); }); });
    set_eval("Clamp", [](N n, Ins in, Outs out, C) {
        const double lo = n.attr_float("min"), hi = n.attr_float("max");
        return unary(in, out, [=](double v) { return std::min(std::max(v, lo), hi); },
                     [=](int64_t v) { return (int64_t)std::min<double>(std::max<double>((double)v, std::ceil(lo)), std::floor(hi)); });
    });
    set_eval("LogicalNot", [](N, Ins in, Outs out, C) { Tensor r(ET::boolean, in[0].shape); for (int64_t i = 0; i < r.numel(); ++i) r.data()[i] = get_elem_f64(in[0], i) == 0; out[0] = r; return true; });
    set_eval("IsNaN", [](N, Ins in, Outs out, C) { Tensor r(ET::boolean, in[0].shape); for (int64_t i = 0; i < r.numel(); ++i) r.data()[i] = std::isnan(get_elem_f64(in[0], i)); out[0] = r; return true; });
    set_eval("IsFinite", [](N, Ins in, Outs out, C) { Tensor r(ET::boolean, in[0].shape); for (int64_t i = 0; i < r.numel(); ++i) r.data()[i] = std::isfinite(get_elem_f64(in[0], i)); out[0] = r; return true; });
    set_eval("IsInf", [](N n, Ins in, Outs out, C) {
        Tensor r(ET::boolean, in[0].shape);
        const bool neg = n.attr_bool("detect_negative", true), pos = n.attr_bool("detect_positive", true);
        for (int64_t i = 0; i < r.numel(); ++i) { const double v = get_elem_f64(in[0], i); r.data()[i] = std::isinf(v) && ((v > 0 && pos) || (v < 0 && neg)); }
        out[0] = r;
        return true;
    });
    set_eval("BitwiseNot", [](N, Ins in, Outs out, C) { return unary(in, out, [](double v) { return v; }, [](int64_t v) { return ~v; }); });
    set_eval("PRelu", [](N n, Ins in, Outs out, C) {
        // slope broadcasts along the channel axis (1) when it is 1-D
        Tensor slope = in[1];
        if (slope.shape.size() == 1 && in[0].shape.size() > 1 && slope.shape[0] == in[0].shape[1]) {
            Shape s(in[0].shape.size(), 1);
            s[1] = slope.shape[0];
            slope = reshape_view(slope, s);
        }
        std::vector<Tensor> i2 = {in[0], slope};
        return binary(n, i2, out, [](double x, double s) { return x >= 0 ? x : x * s; }, [](int64_t x, int64_t s) { return x >= 0 ? x : x * s; });
    });
    set_eval("HardSigmoid", [](N, Ins in, Outs out, C) { const double a = get_elem_f64(in[1], 0), b = get_elem_f64(in[2], 0); std::vector<Tensor> i1 = {in[0]}; return unary_real(i1, out, [=](double v) { return std::min(1.0, std::max(0.0, a * v + b)); }); });
    set_eval("Selu", [](N, Ins in, Outs out, C) { const double a = get_elem_f64(in[1], 0), l = get_elem_f64(in[2], 0); std::vector<Tensor> i1 = {in[0]}; return unary_real(i1, out, [=](double v) { return l * (v > 0 ? v : a * (std::exp(v) - 1.0)); }); });

#define BINARY(NAME, FR, FI) set_eval(NAME, [](N n, Ins in, Outs out, C) { return binary(n, in, out, [](double x, double y) -> double { return FR; }, [](int64_t x, int64_t y) -> int64_t { return FI; }); })
    BINARY("Add", x + y, x + y);
    BINARY("Subtract", x - y, x - y);
    BINARY("Multiply", x * y, x * y);
    BINARY("Maximum", std::max(x, y), std::max(x, y));
    BINARY("Minimum", std::min(x, y), std::min(x, y));
    BINARY("Power", std::pow(x, y), (int64_t)std::llround(std::pow((double)x, (double)y)));
    BINARY("SquaredDifference", (x - y) * (x - y), (x - y) * (x - y));
    BINARY("Mod", std::fmod(x, y), (y == 0 ? 0 : x % y));
    BINARY("FloorMod", (y == 0 ? std::nan("") : x - std::floor(x / y) * y), (y == 0 ? 0 : ((x % y) + y) % y));
    BINARY("BitwiseAnd", x, x & y);
    BINARY("BitwiseOr", x, x | y);
    BINARY("BitwiseXor", x, x ^ y);
#undef BINARY
    set_eval("Divide", [](N n, Ins in, Outs out, C) {
        const bool py = n.attr_bool("m_pythondiv", true);
        return binary(n, in, out, [](double x, double y) { return x / y; },
                      [py](int64_t x, int64_t y) -> int64_t { if (y == 0) return 0; int64_t q = x / y; if (py && (x % y != 0) && ((x < 0) != (y < 0))) --q; return q; });
    });
#define COMPARE(NAME, OP) set_eval(NAME, [](N, Ins in, Outs out, C) { return compare(in, out, [](double x, double y) { return x OP y; }, [](int64_t x, int64_t y) { return x OP y; }); })
    COMPARE("Equal", ==); COMPARE("NotEqual", !=); COMPARE("Less", <); COMPARE("LessEqual", <=); COMPARE("Greater", >); COMPARE("GreaterEqual", >=);
#undef COMPARE
    set_eval("LogicalAnd", [](N, Ins in, Outs out, C) { return compare(in, out, [](double x, double y) { return x != 0 && y != 0; }, [](int64_t x, int64_t y) { return x != 0 && y != 0; }); });
    set_eval("LogicalOr", [](N, Ins in, Outs out, C) { return compare(in, out, [](double x, double y) { return x != 0 || y != 0; }, [](int64_t x, int64_t y) { return x != 0 || y != 0; }); });
    for (const char* t : {"LogicalXor", "Xor"})
        set_eval(t, [](N, Ins in, Outs out, C) { return compare(in, out, [](double x, double y) { return (x != 0) != (y != 0); }, [](int64_t x, int64_t y) { return (x != 0) != (y != 0); }); });
    set_eval("Select", [](N, Ins in, Outs out, C) {
        const Shape os = broadcast_shape(in[0].shape, broadcast_shape(in[1].shape, in[2].shape));
        const auto sc = bstrides(in[0].shape, os), sa = bstrides(in[1].shape, os), sb = bstrides(in[2].shape, os);
        Tensor r(in[1].et, os);
        const int64_t n = shape_size(os);
        std::vector<int64_t> idx(os.size(), 0);
        for (int64_t i = 0; i < n; ++i) {
            int64_t ic = 0, ia = 0, ib = 0;
            for (size_t d = 0; d < os.size(); ++d) { ic += idx[d] * sc[d]; ia += idx[d] * sa[d]; ib += idx[d] * sb[d]; }
            const bool c = get_elem_f64(in[0], ic) != 0;
            if (et_is_real(r.et)) set_elem_f64(r, i, c ? get_elem_f64(in[1], ia) : get_elem_f64(in[2], ib));
            else set_elem_i64(r, i, c ? get_elem_i64(in[1], ia) : get_elem_i64(in[2], ib));
            for (int64_t d = (int64_t)os.size() - 1; d >= 0; --d) { if (++idx[(size_t)d] < os[(size_t)d]) break; idx[(size_t)d] = 0; }
        }
        out[0] = r;
        return true;
    });

    const double inf = std::numeric_limits<double>::infinity();
    set_eval("ReduceSum", [](N n, Ins in, Outs out, C) { return reduce(n, in, out, 0.0, [](double a, double v) { return a + v; }, [](double a, int64_t) { return a; }); });
    set_eval("ReduceMean", [](N n, Ins in, Outs out, C) { return reduce(n, in, out, 0.0, [](double a, double v) { return a + v; }, [](double a, int64_t c) { return a / double(c); }); });
    set_eval("ReduceProd", [](N n, Ins in, Outs out, C) { return reduce(n, in, out, 1.0, [](double a, double v) { return a * v; }, [](double a, int64_t) { return a; }); });
    set_eval("ReduceMax", [inf](N n, Ins in, Outs out, C) { return reduce(n, in, out, -inf, [](double a, double v) { return std::max(a, v); }, [](double a, int64_t) { return a; }); });
    set_eval("ReduceMin", [inf](N n, Ins in, Outs out, C) { return reduce(n, in, out, inf, [](double a, double v) { return std::min(a, v); }, [](double a, int64_t) { return a; }); });
    set_eval("ReduceL1", [](N n, Ins in, Outs out, C) { return reduce(n, in, out, 0.0, [](double a, double v) { return a + std::fabs(v); }, [](double a, int64_t) { return a; }); });
    set_eval("ReduceL2", [](N n, Ins in, Outs out, C) { return reduce(n, in, out, 0.0, [](double a, double v) { return a + v * v; }, [](double a, int64_t) { return std::sqrt(a); }); });
    set_eval("ReduceLogicalAnd", [](N n, Ins in, Outs out, C) { return reduce(n, in, out, 1.0, [](double a, double v) { return (a != 0 && v != 0) ? 1.0 : 0.0; }, [](double a, int64_t) { return a; }); });
    set_eval("ReduceLogicalOr", [](N n, Ins in, Outs out, C) { return reduce(n, in, out, 0.0, [](double a, double v) { return (a != 0 || v != 0) ? 1.0 : 0.0; }, [](double a, int64_t) { return a; }); });

    set_eval("MatMul", [](N n, Ins in, Outs out, C c) { return eval_matmul(n, in, out, c, n.attr_bool("transpose_a"), n.attr_bool("transpose_b"), ET::dynamic); });
    set_eval("Convolution", [](N n, Ins in, Outs out, C c) { return eval_conv(n, in, out, c, false); });
    set_eval("GroupConvolution", [](N n, Ins in, Outs out, C c) { return eval_conv(n, in, out, c, true); });
    set_eval("MaxPool", [](N n, Ins in, Outs out, C c) { return eval_pool(n, in, out, c, true); });
    set_eval("AvgPool", [](N n, Ins in, Outs out, C c) { return eval_pool(n, in, out, c, false); });
    set_eval("AdaptiveAvgPool", [](N, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        auto osz = to_i64(in[1]);
        const size_t sp = osz.size();
        OVC_CHECK(sp >= 1 && sp <= 2 && x.shape.size() == sp + 2, "AdaptiveAvgPool: only 1-D/2-D are supported");
        const int64_t NC = x.shape[0] * x.shape[1];
        const int64_t IH = sp == 2 ? x.shape[2] : 1, IW = x.shape.back(), OH = sp == 2 ? osz[0] : 1, OW = osz.back();
        auto v = to_f32(x);
        std::vector<float> o((size_t)(NC * OH * OW));
        for (int64_t c = 0; c < NC; ++c) for (int64_t oh = 0; oh < OH; ++oh) for (int64_t ow = 0; ow < OW; ++ow) {
            const int64_t h0 = (oh * IH) / OH, h1 = ((oh + 1) * IH + OH - 1) / OH, w0 = (ow * IW) / OW, w1 = ((ow + 1) * IW + OW - 1) / OW;
            double s = 0;
            for (int64_t h = h0; h < h1; ++h) for (int64_t w = w0; w < w1; ++w) s += v[(size_t)((c * IH + h) * IW + w)];
            o[(size_t)((c * OH + oh) * OW + ow)] = float(s / double((h1 - h0) * (w1 - w0)));
        }
        Shape os = {x.shape[0], x.shape[1]};
        for (auto d : osz) os.push_back(d);
        out[0] = from_f32(x.et, os, o);
        return true;
    });
    set_eval("BatchNormInference", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        auto v = to_f32(x), g = to_f32(in[1]), b = to_f32(in[2]), m = to_f32(in[3]), var = to_f32(in[4]);
        const float eps = float(n.attr_float("epsilon"));
        const int64_t Cc = x.shape.size() > 1 ? x.shape[1] : 1;
        int64_t inner = 1;
        for (size_t i = 2; i < x.shape.size(); ++i) inner *= x.shape[i];
        for (int64_t i = 0; i < x.numel(); ++i) { const int64_t c = (i / inner) % Cc; v[(size_t)i] = (v[(size_t)i] - m[(size_t)c]) / std::sqrt(var[(size_t)c] + eps) * g[(size_t)c] + b[(size_t)c]; }
        out[0] = from_f32(x.et, x.shape, v);
        return true;
    });
    set_eval("MVN", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        const int64_t rank = (int64_t)x.shape.size();
        auto axes = norm_axes(in[1], rank);
        std::vector<bool> red((size_t)rank, false);
        for (auto a : axes) red[(size_t)a] = true;
        // group elements by their non-reduced coordinates
        Shape keep;
        for (int64_t i = 0; i < rank; ++i) keep.push_back(red[(size_t)i] ? 1 : x.shape[(size_t)i]);
        const auto kst = strides_of(keep);
        const int64_t groups = shape_size(keep);
        std::vector<double> sum((size_t)groups, 0), sq((size_t)groups, 0);
        std::vector<int64_t> cnt((size_t)groups, 0), gid((size_t)x.numel());
        auto v = to_f32(x);
        std::vector<int64_t> idx((size_t)rank, 0);
        for (int64_t i = 0; i < x.numel(); ++i) {
            int64_t g = 0;
            for (int64_t d = 0; d < rank; ++d) if (!red[(size_t)d]) g += idx[(size_t)d] * kst[(size_t)d];
            gid[(size_t)i] = g; sum[(size_t)g] += v[(size_t)i]; ++cnt[(size_t)g];
            for (int64_t d = rank - 1; d >= 0; --d) { if (++idx[(size_t)d] < x.shape[(size_t)d]) break; idx[(size_t)d] = 0; }
        }
        for (int64_t i = 0; i < x.numel(); ++i) { const int64_t g = gid[(size_t)i]; const double d = v[(size_t)i] - sum[(size_t)g] / cnt[(size_t)g]; sq[(size_t)g] += d * d; }
        const bool nv = n.attr_bool("normalize_variance", true);
        const double eps = n.attr_float("eps");
        const bool inside = n.attr_str("eps_mode") == "inside_sqrt" || n.attr_str("eps_mode") == "INSIDE_SQRT";
        for (int64_t i = 0; i < x.numel(); ++i) {
            const int64_t g = gid[(size_t)i];
            double d = v[(size_t)i] - sum[(size_t)g] / cnt[(size_t)g];
            if (nv) { const double var = sq[(size_t)g] / cnt[(size_t)g]; d /= inside ? std::sqrt(var + eps) : (std::sqrt(var) + eps); }
            v[(size_t)i] = float(d);
        }
        out[0] = from_f32(x.et, x.shape, v);
        return true;
    });
    set_eval("NormalizeL2", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        Node& nn = const_cast<Node&>(n);
        (void)nn;
        const int64_t rank = (int64_t)x.shape.size();
        auto axes = norm_axes(in[1], rank);
        std::vector<bool> red((size_t)rank, false);
        for (auto a : axes) red[(size_t)a] = true;
        Shape keep;
        for (int64_t i = 0; i < rank; ++i) keep.push_back(red[(size_t)i] ? 1 : x.shape[(size_t)i]);
        const auto kst = strides_of(keep);
        std::vector<double> sq((size_t)shape_size(keep), 0);
        std::vector<int64_t> gid((size_t)x.numel());
        auto v = to_f32(x);
        std::vector<int64_t> idx((size_t)rank, 0);
        for (int64_t i = 0; i < x.numel(); ++i) {
            int64_t g = 0;
            for (int64_t d = 0; d < rank; ++d) if (!red[(size_t)d]) g += idx[(size_t)d] * kst[(size_t)d];
            gid[(size_t)i] = g; sq[(size_t)g] += double(v[(size_t)i]) * v[(size_t)i];
            for (int64_t d = rank - 1; d >= 0; --d) { if (++idx[(size_t)d] < x.shape[(size_t)d]) break; idx[(size_t)d] = 0; }
        }
        const double eps = n.attr_float("eps");
        const bool add = n.attr_str("eps_mode") == "add" || n.attr_str("eps_mode") == "ADD";
        for (int64_t i = 0; i < x.numel(); ++i) { const double s = sq[(size_t)gid[(size_t)i]]; v[(size_t)i] = float(v[(size_t)i] / std::sqrt(add ? s + eps : std::max(s, eps))); }
        out[0] = from_f32(x.et, x.shape, v);
        return true;
    });
    set_eval("GroupNormalization", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        auto v = to_f32(x), g = to_f32(in[1]), b = to_f32(in[2]);
        const int64_t Nn = x.shape[0], Cc = x.shape[1], G = n.attr_int("num_groups");
        int64_t inner = 1;
        for (size_t i = 2; i < x.shape.size(); ++i) inner *= x.shape[i];
        const int64_t cpg = Cc / G, gsz = cpg * inner;
        const double eps = n.attr_float("epsilon");
        for (int64_t bn = 0; bn < Nn * G; ++bn) {
            float* p = v.data() + bn * gsz;
            double s = 0, sq = 0;
            for (int64_t i = 0; i < gsz; ++i) s += p[i];
            const double mean = s / gsz;
            for (int64_t i = 0; i < gsz; ++i) sq += (p[i] - mean) * (p[i] - mean);
            const double inv = 1.0 / std::sqrt(sq / gsz + eps);
            const int64_t c0 = (bn % G) * cpg;
            for (int64_t i = 0; i < gsz; ++i) { const int64_t c = c0 + i / inner; p[i] = float((p[i] - mean) * inv * g[(size_t)c] + b[(size_t)c]); }
        }
        out[0] = from_f32(x.et, x.shape, v);
        return true;
    });
    set_eval("Softmax", [](N n, Ins in, Outs out, C) { return eval_softmax(n, in, out, false); });
    set_eval("LogSoftmax", [](N n, Ins in, Outs out, C) { return eval_softmax(n, in, out, true); });
    set_eval("ScaledDotProductAttention", [](N n, Ins in, Outs out, C c) { return eval_sdpa(n, in, out, c); });
    set_eval("FakeQuantize", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        const Shape os = x.shape;
        const double levels = double(n.attr_int("levels"));
        auto v = to_f32(x);
        std::vector<std::vector<float>> p;
        std::vector<std::vector<int64_t>> st;
        for (int k = 1; k < 5; ++k) { p.push_back(to_f32(in[(size_t)k])); st.push_back(bstrides(in[(size_t)k].shape, os)); }
        std::vector<int64_t> idx(os.size(), 0);
        for (int64_t i = 0; i < x.numel(); ++i) {
            int64_t o[4] = {0, 0, 0, 0};
            for (size_t d = 0; d < os.size(); ++d) for (int k = 0; k < 4; ++k) o[k] += idx[d] * st[(size_t)k][d];
            const float il = p[0][(size_t)o[0]], ih = p[1][(size_t)o[1]], ol = p[2][(size_t)o[2]], oh = p[3][(size_t)o[3]];
            float r;
            if (v[(size_t)i] <= std::min(il, ih)) r = ol;
            else if (v[(size_t)i] > std::max(il, ih)) r = oh;
            else r = float(std::nearbyint((v[(size_t)i] - il) / (ih - il) * (levels - 1)) / (levels - 1) * (oh - ol) + ol);
            v[(size_t)i] = r;
            for (int64_t d = (int64_t)os.size() - 1; d >= 0; --d) { if (++idx[(size_t)d] < os[(size_t)d]) break; idx[(size_t)d] = 0; }
        }
        out[0] = from_f32(x.et, os, v);
        return true;
    });
    set_eval("Interpolate", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        const int64_t rank = (int64_t)x.shape.size();
        const bool v11 = n.version == "opset11";
        const size_t axes_port = v11 ? 2 : 3;
        std::vector<int64_t> axes;
        if (in.size() > axes_port) axes = norm_axes(in[axes_port], rank); else { axes.resize((size_t)rank); std::iota(axes.begin(), axes.end(), 0); }
        const std::string scm = n.attr_str("shape_calculation_mode", "sizes");
        Shape os = x.shape;
        std::vector<double> scales((size_t)rank, 1.0);
        if (scm == "sizes") {
            auto sz = to_i64(in[1]);
            for (size_t i = 0; i < axes.size(); ++i) { os[(size_t)axes[i]] = sz[i]; scales[(size_t)axes[i]] = double(sz[i]) / double(x.shape[(size_t)axes[i]]); }
        } else {
            auto sc = to_f32(in[v11 ? 1 : 2]);
            for (size_t i = 0; i < axes.size(); ++i) { scales[(size_t)axes[i]] = sc[i]; os[(size_t)axes[i]] = int64_t(std::floor(x.shape[(size_t)axes[i]] * double(sc[i]) + 1e-5)); }
        }
        const std::string mode = n.attr_str("mode"), ctm = n.attr_str("coordinate_transformation_mode"), nm = n.attr_str("nearest_mode");
        OVC_CHECK(mode == "nearest" || mode == "linear" || mode == "linear_onnx" || mode == "bilinear_pillow", "Interpolate: mode " << mode << " is not supported by the reference executor");
        auto src_coord = [&](int64_t o, int64_t d) -> double {
            const double sc = scales[(size_t)d], in_len = double(x.shape[(size_t)d]), out_len = double(os[(size_t)d]);
            if (ctm == "half_pixel") return (o + 0.5) / sc - 0.5;
            if (ctm == "pytorch_half_pixel") return out_len > 1 ? (o + 0.5) / sc - 0.5 : 0.0;
            if (ctm == "asymmetric") return o / sc;
            if (ctm == "tf_half_pixel_for_nn") return (o + 0.5) / sc;
            if (ctm == "align_corners") return out_len == 1 ? 0.0 : o * (in_len - 1) / (out_len - 1);
            return o / sc;
        };
        auto v = to_f32(x);
        const auto ist = strides_of(x.shape);
        std::vector<float> o((size_t)shape_size(os));
        std::vector<int64_t> idx((size_t)rank, 0);
        const int64_t total = shape_size(os);
        for (int64_t i = 0; i < total; ++i) {
            if (mode == "nearest") {
                int64_t src = 0;
                for (int64_t d = 0; d < rank; ++d) {
                    int64_t c = idx[(size_t)d];
                    if (os[(size_t)d] != x.shape[(size_t)d]) {
                        const double f = src_coord(idx[(size_t)d], d);
                        if (nm == "floor") c = (int64_t)std::floor(f);
                        else if (nm == "ceil") c = (int64_t)std::ceil(f);
                        else if (nm == "round_prefer_ceil") c = (int64_t)std::round(f);
                        else if (nm == "simple") c = scales[(size_t)d] < 1 ? (int64_t)std::ceil(f) : (int64_t)f;
                        else c = (f == std::floor(f) + 0.5) ? (int64_t)std::floor(f) : (int64_t)std::round(f);
                        c = std::min(std::max<int64_t>(c, 0), x.shape[(size_t)d] - 1);
                    }
                    src += c * ist[(size_t)d];
                }
                o[(size_t)i] = v[(size_t)src];
            } else {
                // separable linear interpolation over the resized axes
                std::vector<std::pair<int64_t, double>> terms = {{0, 1.0}};
                for (int64_t d = 0; d < rank; ++d) {
                    std::vector<std::pair<int64_t, double>> next;
                    if (os[(size_t)d] == x.shape[(size_t)d]) { for (auto& t : terms) next.emplace_back(t.first + idx[(size_t)d] * ist[(size_t)d], t.second); }
                    else {
                        double f = src_coord(idx[(size_t)d], d);
                        f = std::min(std::max(f, 0.0), double(x.shape[(size_t)d] - 1));
                        const int64_t c0 = (int64_t)std::floor(f), c1 = std::min(c0 + 1, x.shape[(size_t)d] - 1);
                        const double w1 = f - c0, w0 = 1.0 - w1;
                        for (auto& t : terms) { next.emplace_back(t.first + c0 * ist[(size_t)d], t.second * w0); if (w1 > 0) next.emplace_back(t.first + c1 * ist[(size_t)d], t.second * w1); }
                    }
                    terms.swap(next);
                }
                double acc = 0;
                for (auto& t : terms) acc += t.second * v[(size_t)t.first];
                o[(size_t)i] = float(acc);
            }
            for (int64_t d = rank - 1; d >= 0; --d) { if (++idx[(size_t)d] < os[(size_t)d]) break; idx[(size_t)d] = 0; }
        }
        out[0] = from_f32(x.et, os, o);
        return true;
    });

    set_eval("Reshape", [](N n, Ins in, Outs out, C) { return eval_reshape(n, in, out); });
    set_eval("Squeeze", [](N, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        Shape os;
        if (in.size() > 1) {
            auto ax = norm_axes(in[1], (int64_t)x.shape.size());
            std::set<int64_t> s(ax.begin(), ax.end());
            for (size_t i = 0; i < x.shape.size(); ++i) if (!(s.count((int64_t)i) && x.shape[i] == 1)) os.push_back(x.shape[i]);
        } else for (auto d : x.shape) if (d != 1) os.push_back(d);
        out[0] = reshape_view(x, os);
        return true;
    });
    set_eval("Unsqueeze", [](N, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        auto ax = to_i64(in[1]);
        const int64_t r = (int64_t)x.shape.size() + (int64_t)ax.size();
        std::set<int64_t> s;
        for (auto a : ax) s.insert(a < 0 ? a + r : a);
        Shape os;
        size_t k = 0;
        for (int64_t i = 0; i < (int64_t)x.shape.size() + (int64_t)s.size(); ++i) os.push_back(s.count(i) ? 1 : x.shape[k++]);
        out[0] = reshape_view(x, os);
        return true;
    });
    set_eval("Transpose", [](N, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        auto order = to_i64(in[1]);
        const int64_t r = (int64_t)x.shape.size();
        if (order.empty()) for (int64_t i = r - 1; i >= 0; --i) order.push_back(i);
        const auto st = strides_of(x.shape);
        Shape os((size_t)r);
        std::vector<int64_t> ss((size_t)r);
        for (int64_t i = 0; i < r; ++i) { const int64_t a = order[(size_t)i] < 0 ? order[(size_t)i] + r : order[(size_t)i]; os[(size_t)i] = x.shape[(size_t)a]; ss[(size_t)i] = st[(size_t)a]; }
        out[0] = gather_strided(x, os, ss, 0);
        return true;
    });
    set_eval("Concat", [](N n, Ins in, Outs out, C) { return eval_concat(n, in, out); });
    set_eval("Split", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        int64_t axis = to_i64(in[1]).at(0);
        if (axis < 0) axis += (int64_t)x.shape.size();
        const int64_t parts = n.attr_int("num_splits"), len = x.shape[(size_t)axis] / parts;
        for (int64_t i = 0; i < parts; ++i) out[(size_t)i] = slice_axis(x, axis, i * len, len);
        return true;
    });
    set_eval("VariadicSplit", [](N, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        int64_t axis = to_i64(in[1]).at(0);
        if (axis < 0) axis += (int64_t)x.shape.size();
        auto lens = to_i64(in[2]);
        int64_t known = 0;
        for (auto l : lens) if (l >= 0) known += l;
        int64_t pos = 0;
        for (size_t i = 0; i < lens.size(); ++i) { const int64_t l = lens[i] < 0 ? x.shape[(size_t)axis] - known : lens[i]; out[i] = slice_axis(x, axis, pos, l); pos += l; }
        return true;
    });
    set_eval("Slice", [](N, Ins in, Outs out, C) {
        Tensor x = in[0];
        auto b = to_i64(in[1]), e = to_i64(in[2]), s = to_i64(in[3]);
        std::vector<int64_t> axes;
        if (in.size() > 4) axes = norm_axes(in[4], (int64_t)x.shape.size()); else { axes.resize(b.size()); std::iota(axes.begin(), axes.end(), 0); }
        for (size_t k = 0; k < axes.size(); ++k) {
            const int64_t a = axes[k], dim = x.shape[(size_t)a], st = s[k];
            int64_t bb = b[k] < 0 ? b[k] + dim : b[k], ee = e[k] < 0 ? e[k] + dim : e[k], cnt;
            if (st > 0) { bb = std::max<int64_t>(0, std::min(bb, dim)); ee = std::max<int64_t>(0, std::min(ee, dim)); cnt = ee > bb ? (ee - bb + st - 1) / st : 0; }
            else { bb = std::max<int64_t>(-1, std::min(bb, dim - 1)); ee = std::max<int64_t>(-1, std::min(ee, dim - 1)); cnt = bb > ee ? (bb - ee + (-st) - 1) / (-st) : 0; }
            x = slice_axis(x, a, cnt ? bb : 0, cnt, st);
        }
        out[0] = x;
        return true;
    });
    set_eval("StridedSlice", [](N n, Ins in, Outs out, C) {
        Tensor x = in[0];
        auto b = to_i64(in[1]), e = to_i64(in[2]);
        std::vector<int64_t> st = in.size() > 3 ? to_i64(in[3]) : std::vector<int64_t>(b.size(), 1);
        auto mask = [&](const char* k, size_t i) { auto v = n.attr_ints(k); return i < v.size() && v[i] != 0; };
        const size_t nspec = b.size();
        Shape final_shape;
        size_t in_d = 0;
        const size_t rank = x.shape.size();
        for (size_t i = 0; i < nspec; ++i) {
            if (mask("ellipsis_mask", i)) {
                size_t rem_new = 0;
                for (size_t j = i + 1; j < nspec; ++j) if (mask("new_axis_mask", j)) ++rem_new;
                const size_t take = rank - in_d - (nspec - i - 1 - rem_new);
                for (size_t k = 0; k < take; ++k) final_shape.push_back(x.shape[in_d++]);
                continue;
            }
            if (mask("new_axis_mask", i)) { final_shape.push_back(1); continue; }
            const int64_t dim = x.shape[in_d], s = st[i];
            int64_t bb = b[i] < 0 ? b[i] + dim : b[i], ee = e[i] < 0 ? e[i] + dim : e[i], cnt;
            if (mask("shrink_axis_mask", i)) { x = slice_axis(x, (int64_t)in_d, std::min(std::max<int64_t>(bb, 0), dim - 1), 1, 1); ++in_d; continue; }
            if (s > 0) {
                if (mask("begin_mask", i)) bb = 0;
                if (mask("end_mask", i)) ee = dim;
                bb = std::max<int64_t>(0, std::min(bb, dim)); ee = std::max<int64_t>(0, std::min(ee, dim));
                cnt = ee > bb ? (ee - bb + s - 1) / s : 0;
            } else {
                if (mask("begin_mask", i)) bb = dim - 1;
                if (mask("end_mask", i)) ee = -1; else ee = std::max<int64_t>(-1, std::min(ee, dim - 1));
                bb = std::max<int64_t>(-1, std::min(bb, dim - 1));
                cnt = bb > ee ? (bb - ee + (-s) - 1) / (-s) : 0;
            }
            x = slice_axis(x, (int64_t)in_d, cnt ? bb : 0, cnt, s);
            final_shape.push_back(cnt);
            ++in_d;
        }
        while (in_d < rank) final_shape.push_back(x.shape[in_d++]);
        out[0] = reshape_view(x, final_shape);
        return true;
    });
    set_eval("Gather", [](N n, Ins in, Outs out, C) { return eval_gather(n, in, out); });
    set_eval("GatherElements", [](N n, Ins in, Outs out, C) {
        const Tensor &d = in[0], &idx = in[1];
        int64_t axis = n.attr_int("axis");
        const int64_t rank = (int64_t)d.shape.size();
        if (axis < 0) axis += rank;
        const auto dst = strides_of(d.shape);
        Tensor o(d.et, idx.shape);
        auto iv = to_i64(idx);
        std::vector<int64_t> id((size_t)rank, 0);
        for (int64_t i = 0; i < idx.numel(); ++i) {
            int64_t src = 0;
            for (int64_t k = 0; k < rank; ++k) { int64_t c = id[(size_t)k]; if (k == axis) { c = iv[(size_t)i]; if (c < 0) c += d.shape[(size_t)axis]; } src += c * dst[(size_t)k]; }
            set_elem_f64(o, i, get_elem_f64(d, src));
            for (int64_t k = rank - 1; k >= 0; --k) { if (++id[(size_t)k] < idx.shape[(size_t)k]) break; id[(size_t)k] = 0; }
        }
        out[0] = o;
        return true;
    });
    set_eval("GatherND", [](N n, Ins in, Outs out, C) {
        const Tensor &d = in[0], &idx = in[1];
        const int64_t bd = n.attr_int("batch_dims"), k = idx.shape.back();
        const auto dst = strides_of(d.shape);
        Shape os(idx.shape.begin(), idx.shape.end() - 1);
        for (size_t a = (size_t)(bd + k); a < d.shape.size(); ++a) os.push_back(d.shape[a]);
        int64_t inner = 1;
        for (size_t a = (size_t)(bd + k); a < d.shape.size(); ++a) inner *= d.shape[a];
        int64_t batch = 1;
        for (int64_t a = 0; a < bd; ++a) batch *= d.shape[(size_t)a];
        const int64_t tuples = idx.numel() / k, per_batch = tuples / std::max<int64_t>(batch, 1);
        const int64_t batch_stride = d.numel() / std::max<int64_t>(batch, 1);
        auto iv = to_i64(idx);
        Tensor o(d.et, os);
        for (int64_t t = 0; t < tuples; ++t) {
            const int64_t b = t / std::max<int64_t>(per_batch, 1);
            int64_t src = b * batch_stride;
            for (int64_t j = 0; j < k; ++j) { int64_t c = iv[(size_t)(t * k + j)]; if (c < 0) c += d.shape[(size_t)(bd + j)]; src += c * dst[(size_t)(bd + j)]; }
            for (int64_t j = 0; j < inner; ++j) set_elem_f64(o, t * inner + j, get_elem_f64(d, src + j));
        }
        out[0] = o;
        return true;
    });
    set_eval("ScatterUpdate", [](N, Ins in, Outs out, C) {
        const Tensor &d = in[0], &idx = in[1], &upd = in[2];
        int64_t axis = to_i64(in[3]).at(0);
        const int64_t rank = (int64_t)d.shape.size();
        if (axis < 0) axis += rank;
        Tensor o(d.et, d.shape);
        std::memcpy(o.data(), d.data(), d.byte_size());
        int64_t outer = 1, inner = 1;
        for (int64_t i = 0; i < axis; ++i) outer *= d.shape[(size_t)i];
        for (int64_t i = axis + 1; i < rank; ++i) inner *= d.shape[(size_t)i];
        auto iv = to_i64(idx);
        const int64_t ni = (int64_t)iv.size(), A = d.shape[(size_t)axis];
        for (int64_t ou = 0; ou < outer; ++ou) for (int64_t k = 0; k < ni; ++k) {
            int64_t t = iv[(size_t)k]; if (t < 0) t += A;
            for (int64_t j = 0; j < inner; ++j) set_elem_f64(o, (ou * A + t) * inner + j, get_elem_f64(upd, (ou * ni + k) * inner + j));
        }
        out[0] = o;
        return true;
    });
    set_eval("ScatterNDUpdate", [](N n, Ins in, Outs out, C) {
        const Tensor &d = in[0], &idx = in[1], &upd = in[2];
        Tensor o(d.et, d.shape);
        std::memcpy(o.data(), d.data(), d.byte_size());
        const int64_t k = idx.shape.back(), tuples = idx.numel() / k;
        const auto dst = strides_of(d.shape);
        int64_t inner = 1;
        for (size_t a = (size_t)k; a < d.shape.size(); ++a) inner *= d.shape[a];
        auto iv = to_i64(idx);
        const std::string red = n.has_attr("reduction") ? n.attr_str("reduction") : "none";
        for (int64_t t = 0; t < tuples; ++t) {
            int64_t dsto = 0;
            for (int64_t j = 0; j < k; ++j) { int64_t c = iv[(size_t)(t * k + j)]; if (c < 0) c += d.shape[(size_t)j]; dsto += c * dst[(size_t)j]; }
            for (int64_t j = 0; j < inner; ++j) {
                const double u = get_elem_f64(upd, t * inner + j), cur = get_elem_f64(o, dsto + j);
                double r = u;
                if (red == "sum") r = cur + u; else if (red == "sub") r = cur - u; else if (red == "prod") r = cur * u;
                else if (red == "min") r = std::min(cur, u); else if (red == "max") r = std::max(cur, u);
                set_elem_f64(o, dsto + j, r);
            }
        }
        out[0] = o;
        return true;
    });
    set_eval("ScatterElementsUpdate", [](N n, Ins in, Outs out, C) {
        const Tensor &d = in[0], &idx = in[1], &upd = in[2];
        int64_t axis = to_i64(in[3]).at(0);
        const int64_t rank = (int64_t)d.shape.size();
        if (axis < 0) axis += rank;
        Tensor o(d.et, d.shape);
        std::memcpy(o.data(), d.data(), d.byte_size());
        const auto dst = strides_of(d.shape);
        auto iv = to_i64(idx);
        const std::string red = n.has_attr("reduction") ? n.attr_str("reduction") : "none";
        std::vector<int64_t> id((size_t)rank, 0);
        for (int64_t i = 0; i < idx.numel(); ++i) {
            int64_t pos = 0;
            for (int64_t k = 0; k < rank; ++k) { int64_t c = id[(size_t)k]; if (k == axis) { c = iv[(size_t)i]; if (c < 0) c += d.shape[(size_t)axis]; } pos += c * dst[(size_t)k]; }
            const double u = get_elem_f64(upd, i), cur = get_elem_f64(o, pos);
            double r = u;
            if (red == "sum") r = cur + u; else if (red == "prod") r = cur * u; else if (red == "min") r = std::min(cur, u); else if (red == "max") r = std::max(cur, u);
            set_elem_f64(o, pos, r);
            for (int64_t k = rank - 1; k >= 0; --k) { if (++id[(size_t)k] < idx.shape[(size_t)k]) break; id[(size_t)k] = 0; }
        }
        out[0] = o;
        return true;
    });
    set_eval("ShapeOf", [](N n, Ins in, Outs out, C) { out[0] = from_i64(n.outs[0].et == ET::dynamic ? ET::i64 : n.outs[0].et, Shape{(int64_t)in[0].shape.size()}, in[0].shape); return true; });
    set_eval("Broadcast", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        Shape target = to_i64(in[1]);
        const std::string mode = n.attr_str("mode", "numpy");
        Shape xs = x.shape;
        if (mode == "explicit") {
            auto axes = to_i64(in[2]);
            Shape e(target.size(), 1);
            for (size_t i = 0; i < axes.size(); ++i) e[(size_t)axes[i]] = xs[i];
            xs = e;
        }
        const Shape os = mode == "bidirectional" ? broadcast_shape(xs, target) : target;
        out[0] = gather_strided(reshape_view(x, xs), os, bstrides(xs, os), 0);
        return true;
    });
    set_eval("Tile", [](N, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        auto rep = to_i64(in[1]);
        const size_t r = std::max(x.shape.size(), rep.size());
        Shape xs = x.shape;
        while (xs.size() < r) xs.insert(xs.begin(), 1);
        while (rep.size() < r) rep.insert(rep.begin(), 1);
        // view as [r0, d0, r1, d1, ...] with stride 0 on repeat axes
        Shape os2;
        std::vector<int64_t> st2;
        const auto st = strides_of(xs);
        Shape os(r);
        for (size_t i = 0; i < r; ++i) { os2.push_back(rep[i]); st2.push_back(0); os2.push_back(xs[i]); st2.push_back(st[i]); os[i] = rep[i] * xs[i]; }
        out[0] = reshape_view(gather_strided(reshape_view(x, xs), os2, st2, 0), os);
        return true;
    });
    set_eval("Pad", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        auto pb = to_i64(in[1]), pe = to_i64(in[2]);
        const std::string mode = n.attr_str("pad_mode", "constant");
        const int64_t rank = (int64_t)x.shape.size();
        Shape os((size_t)rank);
        for (int64_t i = 0; i < rank; ++i) os[(size_t)i] = x.shape[(size_t)i] + pb[(size_t)i] + pe[(size_t)i];
        const double pv = (in.size() > 3 && in[3].numel() > 0) ? get_elem_f64(in[3], 0) : 0.0;
        Tensor o(x.et, os);
        const auto ist = strides_of(x.shape);
        std::vector<int64_t> idx((size_t)rank, 0);
        for (int64_t i = 0; i < o.numel(); ++i) {
            int64_t src = 0;
            bool inside = true;
            for (int64_t d = 0; d < rank; ++d) {
                int64_t c = idx[(size_t)d] - pb[(size_t)d];
                const int64_t len = x.shape[(size_t)d];
                if (c < 0 || c >= len) {
                    if (mode == "constant") { inside = false; break; }
                    if (mode == "edge") c = std::min(std::max<int64_t>(c, 0), len - 1);
                    else if (mode == "reflect") { while (c < 0 || c >= len) c = c < 0 ? -c : 2 * (len - 1) - c; }
                    else if (mode == "symmetric") { while (c < 0 || c >= len) c = c < 0 ? -c - 1 : 2 * len - 1 - c; }
                }
                src += c * ist[(size_t)d];
            }
            set_elem_f64(o, i, inside ? get_elem_f64(x, src) : pv);
            for (int64_t d = rank - 1; d >= 0; --d) { if (++idx[(size_t)d] < os[(size_t)d]) break; idx[(size_t)d] = 0; }
        }
        out[0] = o;
        return true;
    });
    set_eval("Range", [](N n, Ins in, Outs out, C) {
        const ET et = n.attr("output_type").et;
        const double s = get_elem_f64(in[0], 0), e = get_elem_f64(in[1], 0), st = get_elem_f64(in[2], 0);
        const int64_t cnt = std::max<int64_t>(0, (int64_t)std::ceil((e - s) / st));
        std::vector<double> v((size_t)cnt);
        for (int64_t i = 0; i < cnt; ++i) v[(size_t)i] = s + i * st;
        out[0] = from_f64(et, Shape{cnt}, v);
        return true;
    });
    set_eval("OneHot", [](N n, Ins in, Outs out, C) {
        const Tensor& idx = in[0];
        const int64_t depth = get_elem_i64(in[1], 0);
        int64_t axis = n.attr_int("axis");
        const int64_t r = (int64_t)idx.shape.size();
        if (axis < 0) axis += r + 1;
        Shape os = idx.shape;
        os.insert(os.begin() + axis, depth);
        Tensor o(in[2].et, os);
        int64_t outer = 1, inner = 1;
        for (int64_t i = 0; i < axis; ++i) outer *= idx.shape[(size_t)i];
        for (int64_t i = axis; i < r; ++i) inner *= idx.shape[(size_t)i];
        const double on = get_elem_f64(in[2], 0), off = get_elem_f64(in[3], 0);
        auto iv = to_i64(idx);
        for (int64_t ou = 0; ou < outer; ++ou) for (int64_t d = 0; d < depth; ++d) for (int64_t j = 0; j < inner; ++j)
            set_elem_f64(o, (ou * depth + d) * inner + j, iv[(size_t)(ou * inner + j)] == d ? on : off);
        out[0] = o;
        return true;
    });
    set_eval("CumSum", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        int64_t axis = in.size() > 1 ? get_elem_i64(in[1], 0) : 0;
        const int64_t rank = (int64_t)x.shape.size();
        if (axis < 0) axis += rank;
        const bool excl = n.attr_bool("exclusive"), rev = n.attr_bool("reverse");
        int64_t outer = 1, inner = 1;
        for (int64_t i = 0; i < axis; ++i) outer *= x.shape[(size_t)i];
        for (int64_t i = axis + 1; i < rank; ++i) inner *= x.shape[(size_t)i];
        const int64_t A = x.shape[(size_t)axis];
        auto v = to_f64(x);
        std::vector<double> o(v.size());
        for (int64_t ou = 0; ou < outer; ++ou) for (int64_t j = 0; j < inner; ++j) {
            double acc = 0;
            for (int64_t k = 0; k < A; ++k) {
                const int64_t a = rev ? A - 1 - k : k;
                const size_t p = (size_t)((ou * A + a) * inner + j);
                if (excl) { o[p] = acc; acc += v[p]; } else { acc += v[p]; o[p] = acc; }
            }
        }
        out[0] = from_f64(x.et, x.shape, o);
        return true;
    });
    set_eval("TopK", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        const int64_t k = get_elem_i64(in[1], 0);
        const int64_t rank = (int64_t)x.shape.size();
        int64_t axis = n.attr_int("axis");
        if (axis < 0) axis += rank;
        const bool mx = n.attr_str("mode") == "max";
        const std::string sort = n.attr_str("sort");
        int64_t outer = 1, inner = 1;
        for (int64_t i = 0; i < axis; ++i) outer *= x.shape[(size_t)i];
        for (int64_t i = axis + 1; i < rank; ++i) inner *= x.shape[(size_t)i];
        const int64_t A = x.shape[(size_t)axis];
        Shape os = x.shape;
        os[(size_t)axis] = k;
        auto v = to_f64(x);
        std::vector<double> ov((size_t)(outer * k * inner));
        std::vector<int64_t> oi(ov.size());
        std::vector<int64_t> order((size_t)A);
        for (int64_t ou = 0; ou < outer; ++ou) for (int64_t j = 0; j < inner; ++j) {
            std::iota(order.begin(), order.end(), 0);
            auto val = [&](int64_t a) { return v[(size_t)((ou * A + a) * inner + j)]; };
            std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return mx ? val(a) > val(b) : val(a) < val(b); });
            std::vector<int64_t> top(order.begin(), order.begin() + std::min(k, A));
            if (sort == "index") std::sort(top.begin(), top.end());
            for (int64_t t = 0; t < (int64_t)top.size(); ++t) { const size_t p = (size_t)((ou * k + t) * inner + j); ov[p] = val(top[(size_t)t]); oi[p] = top[(size_t)t]; }
        }
        out[0] = from_f64(x.et, os, ov);
        out[1] = from_i64(n.attr("index_element_type").et, os, oi);
        return true;
    });
    set_eval("NonZero", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        const int64_t rank = std::max<int64_t>(1, (int64_t)x.shape.size());
        std::vector<std::vector<int64_t>> coords;
        std::vector<int64_t> idx((size_t)rank, 0);
        for (int64_t i = 0; i < x.numel(); ++i) {
            if (get_elem_f64(x, i) != 0) coords.push_back(idx);
            for (int64_t d = rank - 1; d >= 0 && !x.shape.empty(); --d) { if (++idx[(size_t)d] < x.shape[(size_t)d]) break; idx[(size_t)d] = 0; }
        }
        const int64_t cnt = (int64_t)coords.size();
        std::vector<int64_t> o((size_t)(rank * cnt));
        for (int64_t c = 0; c < cnt; ++c) for (int64_t d = 0; d < rank; ++d) o[(size_t)(d * cnt + c)] = coords[(size_t)c][(size_t)d];
        out[0] = from_i64(n.attr("output_type").et, Shape{rank, cnt}, o);
        return true;
    });
    set_eval("Roll", [](N, Ins in, Outs out, C) {
        Tensor x = in[0];
        auto shift = to_i64(in[1]);
        auto axes = norm_axes(in[2], (int64_t)x.shape.size());
        for (size_t k = 0; k < axes.size(); ++k) {
            const int64_t a = axes[k], len = x.shape[(size_t)a];
            if (len == 0) continue;
            int64_t s = ((shift[shift.size() == 1 ? 0 : k] % len) + len) % len;
            if (s == 0) continue;
            auto cn = make_node("Concat", "opset1", {make_constant(x)->output(0)}, {{"axis", Attr::Int(a)}}, false);
            std::vector<Tensor> parts = {slice_axis(x, a, len - s, s), slice_axis(x, a, 0, len - s)}, o1(1);
            eval_concat(*cn, parts, o1);
            x = o1[0];
        }
        out[0] = x;
        return true;
    });
    set_eval("DepthToSpace", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        OVC_CHECK(x.shape.size() == 4, "DepthToSpace: only 4-D is supported");
        const int64_t b = n.attr_int("block_size"), Nn = x.shape[0], Cc = x.shape[1], H = x.shape[2], W = x.shape[3], Co = Cc / (b * b);
        const bool blocks_first = n.attr_str("mode") == "blocks_first";
        // blocks_first: [N, b, b, Co, H, W] -> [N, Co, H, b, W, b]; depth_first: [N, Co, b, b, H, W] -> same target
        Shape os6 = {Nn, Co, H, b, W, b};
        std::vector<int64_t> st;
        if (blocks_first) { const auto s = strides_of({Nn, b, b, Co, H, W}); st = {s[0], s[3], s[4], s[1], s[5], s[2]}; }
        else { const auto s = strides_of({Nn, Co, b, b, H, W}); st = {s[0], s[1], s[4], s[2], s[5], s[3]}; }
        out[0] = reshape_view(gather_strided(x, os6, st, 0), {Nn, Co, H * b, W * b});
        return true;
    });
    set_eval("ArgMaxMin_internal", [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        const int64_t rank = (int64_t)x.shape.size();
        int64_t axis = n.attr_int("axis");
        if (axis < 0) axis += rank;
        const bool mx = n.attr_str("mode") == "max";
        int64_t outer = 1, inner = 1;
        for (int64_t i = 0; i < axis; ++i) outer *= x.shape[(size_t)i];
        for (int64_t i = axis + 1; i < rank; ++i) inner *= x.shape[(size_t)i];
        const int64_t A = x.shape[(size_t)axis];
        auto v = to_f64(x);
        std::vector<int64_t> o((size_t)(outer * inner));
        for (int64_t ou = 0; ou < outer; ++ou) for (int64_t j = 0; j < inner; ++j) {
            int64_t best = 0;
            for (int64_t a = 1; a < A; ++a) { const double c = v[(size_t)((ou * A + a) * inner + j)], bv = v[(size_t)((ou * A + best) * inner + j)]; if (mx ? c > bv : c < bv) best = a; }
            o[(size_t)(ou * inner + j)] = best;
        }
        Shape os;
        for (int64_t i = 0; i < rank; ++i) { if (i == axis) { if (n.attr_bool("keep_dims")) os.push_back(1); } else os.push_back(x.shape[(size_t)i]); }
        out[0] = from_i64(n.attr("index_element_type").et, os, o);
        return true;
    });

    // ---- stateful
    set_eval("ReadValue", [](N n, Ins in, Outs out, C c) {
        const std::string id = n.attr_str("variable_id");
        if (c.variables) {
            auto it = c.variables->values.find(id);
            if (it != c.variables->values.end()) { out[0] = it->second; return true; }
        }
        if (!in.empty()) { out[0] = in[0]; return true; }
        const PShape& s = n.outs[0].shape;
        Shape z;
        if (!s.rank_dynamic) for (auto& d : s.dims) z.push_back(d.is_static() ? d.lo : 0);
        out[0] = Tensor(n.outs[0].et, z);
        if (out[0].data()) std::memset(out[0].data(), 0, out[0].byte_size());
        return true;
    });
    set_eval("Assign", [](N n, Ins in, Outs out, C c) { if (c.variables) c.variables->values[n.attr_str("variable_id")] = in[0]; out[0] = in[0]; return true; });
    set_eval("If", [](N n, Ins in, Outs out, C c) { return eval_if_loop(n, in, out, c); });
    set_eval("Loop", [](N n, Ins in, Outs out, C c) { return eval_if_loop(n, in, out, c); });
    set_eval("TensorIterator", [](N n, Ins in, Outs out, C c) { return eval_if_loop(n, in, out, c); });

    // ---- LLM / internal
    auto rms = [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        const int64_t H = x.shape.back(), rows = x.numel() / std::max<int64_t>(H, 1);
        const float eps = float(n.attr_float("epsilon"));
        auto v = to_f32(x);
        std::vector<float> g;
        const Tensor* gt = nullptr;
        if (n.type == "RMS") { if (in.size() > 1 && in[1].numel() > 0) gt = &in[1]; }
        else if (in.size() > 2 && in[2].numel() > 0) gt = &in[2]; else if (n.type == "RMSNorm" && in.size() == 2) gt = nullptr;
        if (gt) g = to_f32(*gt);
        for (int64_t r = 0; r < rows; ++r) {
            float* p = v.data() + r * H;
            double s = 0;
            for (int64_t i = 0; i < H; ++i) s += double(p[i]) * p[i];
            const float inv = 1.0f / std::sqrt(float(s / H) + eps);
            for (int64_t i = 0; i < H; ++i) p[i] = p[i] * inv * (g.empty() ? 1.0f : g[(size_t)(g.size() == 1 ? 0 : i)]);
        }
        out[0] = from_f32(n.outs[0].et == ET::dynamic ? x.et : n.outs[0].et, x.shape, v);
        return true;
    };
    set_eval("RMS", rms);
    set_eval("RMSNorm", rms);
    set_eval("RoPE", eval_rope);
    set_eval("FullyConnected", [](N n, Ins in, Outs out, C c) {
        std::vector<Tensor> o1(1);
        eval_matmul(n, in, o1, c, false, true, n.outs[0].et);
        if (in.size() > 2 && in[2].numel() > 0) {
            auto v = to_f32(o1[0]), b = to_f32(in[2]);
            const int64_t Nn = o1[0].shape.back();
            for (size_t i = 0; i < v.size(); ++i) v[i] += b[(size_t)(b.size() == 1 ? 0 : (int64_t)i % Nn)];
            o1[0] = from_f32(o1[0].et, o1[0].shape, v);
        }
        out[0] = o1[0];
        return true;
    });
    set_eval("FullyConnectedCompressed", [](N n, Ins in, Outs out, C c) {
        // inputs: X, W (compressed [N, K] or [N, G, gs]), bias, scales, [zero points]
        const Tensor& W = in[1];
        const int64_t Nn = W.shape[0], K = W.numel() / Nn;
        auto wf = dequant_weight(W, in[3], in.size() > 4 ? &in[4] : nullptr);
        std::vector<Tensor> i2 = {in[0], from_f32(ET::f32, Shape{Nn, K}, wf)}, o1(1);
        i2[0] = convert_tensor(in[0], ET::f32);
        eval_matmul(n, i2, o1, c, false, true, ET::f32);
        auto v = to_f32(o1[0]);
        if (in[2].numel() > 0) { auto b = to_f32(in[2]); for (size_t i = 0; i < v.size(); ++i) v[i] += b[(size_t)(b.size() == 1 ? 0 : (int64_t)i % Nn)]; }
        out[0] = from_f32(n.outs[0].et == ET::dynamic ? in[0].et : n.outs[0].et, o1[0].shape, v);
        return true;
    });
    auto glu = [](N n, Ins in, Outs out, C) {
        const Tensor& x = in[0];
        const int64_t rank = (int64_t)x.shape.size();
        int64_t axis = n.type == "GLU" ? n.attr_int("axis") : -1;
        if (axis < 0) axis += rank;
        const int64_t A = x.shape[(size_t)axis];
        const int64_t len = n.type == "GLU" ? n.attr_int("split_lengths") : A / 2;
        const int64_t gate_idx = n.type == "GLU" ? n.attr_int("split_to_glu_idx") : 0;
        const std::string gt = n.type == "GLU" ? n.attr_str("glu_type") : "Swish";
        int64_t outer = 1, inner = 1;
        for (int64_t i = 0; i < axis; ++i) outer *= x.shape[(size_t)i];
        for (int64_t i = axis + 1; i < rank; ++i) inner *= x.shape[(size_t)i];
        auto v = to_f32(x);
        std::vector<float> o((size_t)(outer * len * inner));
        for (int64_t ou = 0; ou < outer; ++ou) for (int64_t a = 0; a < len; ++a) for (int64_t j = 0; j < inner; ++j) {
            const float first = v[(size_t)((ou * A + a) * inner + j)], second = v[(size_t)((ou * A + len + a) * inner + j)];
            const float g = gate_idx == 0 ? first : second, u = gate_idx == 0 ? second : first;
            float act;
            if (gt == "Gelu") act = gelu_erf(g); else if (gt == "Gelu_Tanh") act = gelu_tanh(g); else act = g / (1.0f + std::exp(-g));
            o[(size_t)((ou * len + a) * inner + j)] = act * u;
        }
        Shape os = x.shape;
        os[(size_t)axis] = len;
        out[0] = from_f32(n.outs[0].et == ET::dynamic ? x.et : n.outs[0].et, os, o);
        return true;
    };
    set_eval("GLU", glu);
    set_eval("SwiGLU_internal", glu);
    set_eval("PagedAttentionExtension", eval_paged_attention);
    set_eval("MOE", eval_moe);
}

}  // namespace ovc
