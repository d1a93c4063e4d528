// Linear-recurrence layers of hybrid LLMs: the selective state-space scan (Mamba-2 form) and the gated delta rule
// (Gated DeltaNet / Qwen3-Next linear attention). Both walk the tokens of a sequence in order with the recurrent state
// of one head resident in registers: one warp owns one row (state-space) or one column (delta rule) of the state matrix,
// its 32 lanes hold the row's elements, and the two dot products of a token are warp shuffles. The state is read from
// and written to HBM once per launch; per token only the token's own vectors are read and one output element per warp is
// written.
//
// Reference counterparts: the SelectiveSSM and GatedDeltaNet internal operations
// (src/common/transformations/include/ov_ops/, executed by the CPU plugin's recurrent kernels).
#include <type_traits>

#include "common.cuh"

namespace ovb {

namespace {

constexpr int REC_WARPS = 8;     // warps (state rows / columns) per CTA
constexpr int REC_MAXV = 8;      // state elements per lane: state widths up to 256

__device__ __forceinline__ float rec_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// state[b, h, p, :] <- state * exp(A[h] * dt) + dt * B[b, t, g, :] * x[b, t, h, p];  y[b, t, h, p] = <state, C[b, t, g, :]>
template <int NV>
__global__ void __launch_bounds__(REC_WARPS * 32)
selective_ssm_kernel(const float* __restrict__ A, const float* __restrict__ dt, const float* __restrict__ Bm, const float* __restrict__ x,
                     const float* __restrict__ Cm, float* __restrict__ state, float* __restrict__ y, int rows, int L, int H, int P, int G, int S) {
    const int row = blockIdx.x * REC_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const int p = row % P, h = (row / P) % H, b = row / (P * H), g = h / (H / G);
    float st[NV];
    float* srow = state + (size_t)row * S;
#pragma unroll
    for (int i = 0; i < NV; ++i) st[i] = (lane + 32 * i < S) ? srow[lane + 32 * i] : 0.f;
    const float a = A[h];
    for (int t = 0; t < L; ++t) {
        const size_t tok = (size_t)b * L + t;
        const float d = dt[tok * H + h], xv = x[(tok * H + h) * P + p];
        const float dA = expf(a * d), dx = d * xv;
        const float* bv = Bm + (tok * G + g) * S;
        const float* cv = Cm + (tok * G + g) * S;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int s = lane + 32 * i;
            if (s < S) {
                st[i] = st[i] * dA + bv[s] * dx;
                acc += st[i] * cv[s];
            }
        }
        acc = rec_warp_sum(acc);
        if (lane == 0) y[(tok * H + h) * P + p] = acc;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (lane + 32 * i < S) srow[lane + 32 * i] = st[i];
}

// One value column iv of the state [Dk, Dv] of (b, hv):  S *= exp(g);  delta = (v - <S, k>) * beta;  S += k * delta;  y = <S, q>.
// q arrives scaled (and normalised where the layer asks for it), k normalised likewise.
template <int NV>
__global__ void __launch_bounds__(REC_WARPS * 32)
gated_delta_rule_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ gate,
                        const float* __restrict__ beta, float* __restrict__ state, float* __restrict__ y, int cols, int L, int Hq, int Hv, int Dk, int Dv) {
    const int col = blockIdx.x * REC_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (col >= cols) return;
    const int iv = col % Dv, h = (col / Dv) % Hv, b = col / (Dv * Hv), hq = h / (Hv / Hq);
    float st[NV];
    float* sbase = state + ((size_t)(b * Hv + h) * Dk) * Dv + iv;
#pragma unroll
    for (int i = 0; i < NV; ++i) st[i] = (lane + 32 * i < Dk) ? sbase[(size_t)(lane + 32 * i) * Dv] : 0.f;
    for (int t = 0; t < L; ++t) {
        const size_t tok = (size_t)b * L + t;
        const float* qv = q + (tok * Hq + hq) * Dk;
        const float* kv = k + (tok * Hq + hq) * Dk;
        const float decay = expf(gate[tok * Hv + h]), bt = beta[tok * Hv + h], vv = v[(tok * Hv + h) * Dv + iv];
        float kr[NV], qr[NV], mem = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = lane + 32 * i;
            kr[i] = d < Dk ? kv[d] : 0.f;
            qr[i] = d < Dk ? qv[d] : 0.f;
            st[i] *= decay;
            mem += st[i] * kr[i];
        }
        mem = rec_warp_sum(mem);
        const float delta = (vv - mem) * bt;
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            st[i] += kr[i] * delta;
            o += st[i] * qr[i];
        }
        o = rec_warp_sum(o);
        if (lane == 0) y[(tok * Hv + h) * Dv + iv] = o;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (lane + 32 * i < Dk) sbase[(size_t)(lane + 32 * i) * Dv] = st[i];
}

template <class Launch>
int dispatch_width(int width, Launch launch) {
    if (width <= 32) return launch(std::integral_constant<int, 1>());
    if (width <= 64) return launch(std::integral_constant<int, 2>());
    if (width <= 128) return launch(std::integral_constant<int, 4>());
    return launch(std::integral_constant<int, REC_MAXV>());
}

}  // namespace

}  // namespace ovb

extern "C" {

int ovb_selective_ssm(const float* A, const float* dt, const float* Bm, const float* x, const float* Cm, float* state, float* y, int B, int L, int H, int P,
                      int G, int S, ovb_stream_t stream_) {
    using namespace ovb;
    OVB_REQUIRE(A && dt && Bm && x && Cm && state && y, "ovb_selective_ssm: null argument");
    OVB_REQUIRE(B > 0 && L >= 0 && H > 0 && P > 0 && G > 0 && S > 0 && H % G == 0, "ovb_selective_ssm: bad sizes (heads %d, groups %d)", H, G);
    if (S > 32 * REC_MAXV) {
        set_error("ovb_selective_ssm: state size %d above %d", S, 32 * REC_MAXV);
        return ERR_UNSUPPORTED;
    }
    OVB_REQUIRE((long long)B * H * P < (1ll << 31), "ovb_selective_ssm: too many state rows");
    const int rows = B * H * P;
    cudaStream_t stream = (cudaStream_t)stream_;
    return dispatch_width(S, [&](auto nv) -> int {
        selective_ssm_kernel<decltype(nv)::value><<<ceil_div(rows, REC_WARPS), REC_WARPS * 32, 0, stream>>>(A, dt, Bm, x, Cm, state, y, rows, L, H, P, G, S);
        OVB_CHECK_CUDA(cudaGetLastError());
        return 0;
    });
}

int ovb_gated_delta_rule(const float* q, const float* k, const float* v, const float* gate, const float* beta, float* state, float* y, int B, int L, int Hq,
                         int Hv, int Dk, int Dv, ovb_stream_t stream_) {
    using namespace ovb;
    OVB_REQUIRE(q && k && v && gate && beta && state && y, "ovb_gated_delta_rule: null argument");
    OVB_REQUIRE(B > 0 && L >= 0 && Hq > 0 && Hv > 0 && Dk > 0 && Dv > 0 && Hv % Hq == 0, "ovb_gated_delta_rule: bad sizes (value heads %d, key heads %d)", Hv, Hq);
    if (Dk > 32 * REC_MAXV) {
        set_error("ovb_gated_delta_rule: key width %d above %d", Dk, 32 * REC_MAXV);
        return ERR_UNSUPPORTED;
    }
    OVB_REQUIRE((long long)B * Hv * Dv < (1ll << 31), "ovb_gated_delta_rule: too many state columns");
    const int cols = B * Hv * Dv;
    cudaStream_t stream = (cudaStream_t)stream_;
    return dispatch_width(Dk, [&](auto nv) -> int {
        gated_delta_rule_kernel<decltype(nv)::value><<<ceil_div(cols, REC_WARPS), REC_WARPS * 32, 0, stream>>>(q, k, v, gate, beta, state, y, cols, L, Hq, Hv, Dk, Dv);
        OVB_CHECK_CUDA(cudaGetLastError());
        return 0;
    });
}

}  // extern "C"
