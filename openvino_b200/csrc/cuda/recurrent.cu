// Linear-recurrence layers of hybrid LLMs: the selective state-space scan (Mamba-2 form) and the gated delta rule
// (Gated DeltaNet / Qwen3-Next linear attention). Both walk the tokens of a sequence in order with the recurrent state
// of one head resident in registers: one warp owns four rows (state-space) or four columns (delta rule) of the state
// matrix, its 32 lanes hold the rows' elements, and the dot products of a token are warp shuffles (four sums share six
// shuffles). The state is read from and written to HBM once per launch; the token vectors every row of a head shares are
// staged in shared memory sixteen tokens at a time.
//
// Reference counterparts: the SelectiveSSM and GatedDeltaNet internal operations
// (src/common/transformations/include/ov_ops/, executed by the CPU plugin's recurrent kernels).
#include <stdlib.h>

#include <type_traits>

#include "common.cuh"

namespace ovb {

namespace {

constexpr int REC_WARPS = 8;     // warps per CTA
constexpr int REC_PER_WARP = 4;  // state rows (state-space) / columns (delta rule) per warp
constexpr int REC_TILE = REC_WARPS * REC_PER_WARP;   // rows / columns of one head per CTA
constexpr int REC_CHUNK = 16;    // tokens staged in shared memory at a time
constexpr int REC_MAXV = 8;      // state elements per lane: state widths up to 256

// Sums four per-lane values over the warp with 6 shuffles instead of 20: after each exchange a lane keeps only the values
// its half is responsible for. The total of v0 ends in lanes 0-7, v1 in 16-23, v2 in 8-15, v3 in 24-31.
__device__ __forceinline__ float rec_reduce4(float v0, float v1, float v2, float v3, int lane) {
    const bool up16 = lane & 16, up8 = lane & 8;
    float a = (up16 ? v1 : v0) + __shfl_xor_sync(0xffffffffu, up16 ? v0 : v1, 16);
    float b = (up16 ? v3 : v2) + __shfl_xor_sync(0xffffffffu, up16 ? v2 : v3, 16);
    float c = (up8 ? b : a) + __shfl_xor_sync(0xffffffffu, up8 ? a : b, 8);
    c += __shfl_xor_sync(0xffffffffu, c, 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    return c;
}
// Lane that holds the total of value r after rec_reduce4, and the value index a lane holds
__device__ __forceinline__ int rec_owner_lane(int r) { return ((r & 1) << 4) | ((r >> 1) << 3); }
__device__ __forceinline__ int rec_owned_value(int lane) { return ((lane >> 4) & 1) | (((lane >> 3) & 1) << 1); }

// Sums eight per-lane values over the warp with 9 shuffles. The total of value r ends in the four lanes whose bits 4, 3, 2
// spell r & 1, (r >> 1) & 1, (r >> 2) & 1.
__device__ __forceinline__ float rec_reduce8(const float (&v)[8], int lane) {
    const bool up16 = lane & 16, up8 = lane & 8, up4 = lane & 4;
    float a[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = (up16 ? v[2 * i + 1] : v[2 * i]) + __shfl_xor_sync(0xffffffffu, up16 ? v[2 * i] : v[2 * i + 1], 16);
    float b0 = (up8 ? a[1] : a[0]) + __shfl_xor_sync(0xffffffffu, up8 ? a[0] : a[1], 8);
    float b1 = (up8 ? a[3] : a[2]) + __shfl_xor_sync(0xffffffffu, up8 ? a[2] : a[3], 8);
    float c = (up4 ? b1 : b0) + __shfl_xor_sync(0xffffffffu, up4 ? b0 : b1, 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    return c;
}
__device__ __forceinline__ int rec_owned_value8(int lane) { return ((lane >> 4) & 1) | (((lane >> 3) & 1) << 1) | (((lane >> 2) & 1) << 2); }

// state[b, h, p, :] <- state * exp(A[h] * dt) + dt * B[b, t, g, :] * x[b, t, h, p];  y[b, t, h, p] = <state, C[b, t, g, :]>
// One CTA owns RW * 8 rows p of one (b, h), each warp RW of them; the token vectors B, C (shared by all rows and by the
// heads of a group) are staged in shared memory REC_CHUNK tokens at a time, so that they cross L2 once per CTA and not
// once per row, and the outputs of a chunk leave through shared memory as whole rows of y.
template <int NV, int RW>
__global__ void __launch_bounds__(REC_WARPS * 32)
selective_ssm_kernel(const float* __restrict__ A, const float* __restrict__ dt, const float* __restrict__ Bm, const float* __restrict__ x,
                     const float* __restrict__ Cm, float* __restrict__ state, float* __restrict__ y, int L, int H, int P, int G, int S) {
    constexpr int TILE = REC_WARPS * RW;
    __shared__ float sB[REC_CHUNK][NV * 32], sC[REC_CHUNK][NV * 32], sX[REC_CHUNK][TILE], sY[REC_CHUNK][TILE], sD[REC_CHUNK], sDA[REC_CHUNK];
    const int bh = blockIdx.y, b = bh / H, h = bh % H, g = h / (H / G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, p0 = blockIdx.x * TILE, pw = p0 + warp * RW;
    float st[RW][NV];
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int i = 0; i < NV; ++i) st[r][i] = (pw + r < P && lane + 32 * i < S) ? state[((size_t)bh * P + pw + r) * S + lane + 32 * i] : 0.f;
    const float a = A[h];
    const int mine = RW == 8 ? rec_owned_value8(lane) : rec_owned_value(lane);
    const bool writer = RW == 8 ? (lane & 3) == 0 : (lane & 7) == 0;
    for (int t0 = 0; t0 < L; t0 += REC_CHUNK) {
        const int nt = min(REC_CHUNK, L - t0);
        const size_t tok0 = (size_t)b * L + t0;
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * NV * 32; idx += REC_WARPS * 32) {
            const int tt = idx / (NV * 32), s = idx % (NV * 32);
            sB[tt][s] = s < S ? Bm[((tok0 + tt) * G + g) * S + s] : 0.f;
            sC[tt][s] = s < S ? Cm[((tok0 + tt) * G + g) * S + s] : 0.f;
        }
        for (int idx = threadIdx.x; idx < nt * TILE; idx += REC_WARPS * 32) {
            const int tt = idx / TILE, r = idx % TILE;
            sX[tt][r] = p0 + r < P ? x[((tok0 + tt) * H + h) * P + p0 + r] : 0.f;
        }
        if (threadIdx.x < nt) {
            const float d = dt[(tok0 + threadIdx.x) * H + h];
            sD[threadIdx.x] = d;
            sDA[threadIdx.x] = expf(a * d);
        }
        __syncthreads();
#pragma unroll 2
        for (int tt = 0; tt < nt; ++tt) {
            const float d = sD[tt], dA = sDA[tt];
            float bv[NV], cv[NV], acc[RW];
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                bv[i] = sB[tt][lane + 32 * i] * d;
                cv[i] = sC[tt][lane + 32 * i];
            }
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                const float xv = sX[tt][warp * RW + r];
                acc[r] = 0.f;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    st[r][i] = st[r][i] * dA + bv[i] * xv;
                    acc[r] += st[r][i] * cv[i];
                }
            }
            float total;
            if constexpr (RW == 8) total = rec_reduce8(acc, lane);
            else total = rec_reduce4(acc[0], acc[1], acc[2], acc[3], lane);
            if (writer) sY[tt][warp * RW + mine] = total;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * TILE; idx += REC_WARPS * 32) {
            const int tt = idx / TILE, r = idx % TILE;
            if (p0 + r < P) y[((tok0 + tt) * H + h) * P + p0 + r] = sY[tt][r];
        }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (pw + r < P && lane + 32 * i < S) state[((size_t)bh * P + pw + r) * S + lane + 32 * i] = st[r][i];
}

// Value columns iv of the state [Dk, Dv] of (b, hv):  S *= exp(g);  delta = (v - <S, k>) * beta;  S += k * delta;  y = <S, q>.
// q arrives scaled (and normalised where the layer asks for it), k normalised likewise. One CTA owns CW * 8 columns of one
// (b, hv), each warp CW of them; q and k of the head (shared by all its columns) are staged in shared memory REC_CHUNK
// tokens at a time, and the outputs of a chunk leave through shared memory as whole rows of y.
template <int NV, int CW>
__global__ void __launch_bounds__(REC_WARPS * 32)
gated_delta_rule_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ gate,
                        const float* __restrict__ beta, float* __restrict__ state, float* __restrict__ y, int L, int Hq, int Hv, int Dk, int Dv) {
    constexpr int TILE = REC_WARPS * CW;
    __shared__ float sQ[REC_CHUNK][NV * 32], sK[REC_CHUNK][NV * 32], sV[REC_CHUNK][TILE], sY[REC_CHUNK][TILE], sG[REC_CHUNK], sBt[REC_CHUNK];
    const int bh = blockIdx.y, b = bh / Hv, h = bh % Hv, hq = h / (Hv / Hq);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, c0 = blockIdx.x * TILE, cw = c0 + warp * CW;
    float st[CW][NV];
    float* sbase = state + (size_t)bh * Dk * Dv;
#pragma unroll
    for (int c = 0; c < CW; ++c)
#pragma unroll
        for (int i = 0; i < NV; ++i) st[c][i] = (cw + c < Dv && lane + 32 * i < Dk) ? sbase[(size_t)(lane + 32 * i) * Dv + cw + c] : 0.f;
    const int mine = CW == 8 ? rec_owned_value8(lane) : rec_owned_value(lane);
    const bool writer = CW == 8 ? (lane & 3) == 0 : (lane & 7) == 0;
    for (int t0 = 0; t0 < L; t0 += REC_CHUNK) {
        const int nt = min(REC_CHUNK, L - t0);
        const size_t tok0 = (size_t)b * L + t0;
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * NV * 32; idx += REC_WARPS * 32) {
            const int tt = idx / (NV * 32), d = idx % (NV * 32);
            sQ[tt][d] = d < Dk ? q[((tok0 + tt) * Hq + hq) * Dk + d] : 0.f;
            sK[tt][d] = d < Dk ? k[((tok0 + tt) * Hq + hq) * Dk + d] : 0.f;
        }
        for (int idx = threadIdx.x; idx < nt * TILE; idx += REC_WARPS * 32) {
            const int tt = idx / TILE, c = idx % TILE;
            sV[tt][c] = c0 + c < Dv ? v[((tok0 + tt) * Hv + h) * Dv + c0 + c] : 0.f;
        }
        if (threadIdx.x < nt) {
            sG[threadIdx.x] = expf(gate[(tok0 + threadIdx.x) * Hv + h]);
            sBt[threadIdx.x] = beta[(tok0 + threadIdx.x) * Hv + h];
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float decay = sG[tt], bt = sBt[tt];
            float kr[NV], qr[NV], mem[CW], o[CW];
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                kr[i] = sK[tt][lane + 32 * i];
                qr[i] = sQ[tt][lane + 32 * i];
            }
#pragma unroll
            for (int c = 0; c < CW; ++c) {
                mem[c] = 0.f;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    st[c][i] *= decay;
                    mem[c] += st[c][i] * kr[i];
                }
            }
            float m;
            if constexpr (CW == 8) m = rec_reduce8(mem, lane);
            else m = rec_reduce4(mem[0], mem[1], mem[2], mem[3], lane);
#pragma unroll
            for (int c = 0; c < CW; ++c) {
                const int owner = CW == 8 ? (((c & 1) << 4) | (((c >> 1) & 1) << 3) | (((c >> 2) & 1) << 2)) : rec_owner_lane(c);
                const float delta = (sV[tt][warp * CW + c] - __shfl_sync(0xffffffffu, m, owner)) * bt;
                o[c] = 0.f;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    st[c][i] += kr[i] * delta;
                    o[c] += st[c][i] * qr[i];
                }
            }
            float total;
            if constexpr (CW == 8) total = rec_reduce8(o, lane);
            else total = rec_reduce4(o[0], o[1], o[2], o[3], lane);
            if (writer) sY[tt][warp * CW + mine] = total;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * TILE; idx += REC_WARPS * 32) {
            const int tt = idx / TILE, c = idx % TILE;
            if (c0 + c < Dv) y[((tok0 + tt) * Hv + h) * Dv + c0 + c] = sY[tt][c];
        }
    }
#pragma unroll
    for (int c = 0; c < CW; ++c)
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (cw + c < Dv && lane + 32 * i < Dk) sbase[(size_t)(lane + 32 * i) * Dv + cw + c] = st[c][i];
}

// OVB_SSM_ROWS_PER_WARP = 4 keeps the four-row (four-column) form of both kernels for every shape (8 by default where it applies)
int env_rows_per_warp() {
    const char* e = getenv("OVB_SSM_ROWS_PER_WARP");
    return e && atoi(e) == 4 ? 4 : 8;
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
    OVB_REQUIRE((long long)B * H <= 65535, "ovb_selective_ssm: batch x heads above 65535");
    cudaStream_t stream = (cudaStream_t)stream_;
    static const int rows_per_warp = env_rows_per_warp();
    return dispatch_width(S, [&](auto nv) -> int {
        constexpr int NV = decltype(nv)::value;
        // eight rows per warp halve the shared-memory reads and shuffles per row; they need 8 * NV state registers per lane
        if (NV <= 4 && P >= 64 && rows_per_warp == 8)
            selective_ssm_kernel<NV, 8><<<dim3(ceil_div(P, REC_WARPS * 8), B * H), REC_WARPS * 32, 0, stream>>>(A, dt, Bm, x, Cm, state, y, L, H, P, G, S);
        else
            selective_ssm_kernel<NV, 4><<<dim3(ceil_div(P, REC_WARPS * 4), B * H), REC_WARPS * 32, 0, stream>>>(A, dt, Bm, x, Cm, state, y, L, H, P, G, S);
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
    OVB_REQUIRE((long long)B * Hv <= 65535, "ovb_gated_delta_rule: batch x value heads above 65535");
    cudaStream_t stream = (cudaStream_t)stream_;
    static const int cols_per_warp = env_rows_per_warp();
    return dispatch_width(Dk, [&](auto nv) -> int {
        constexpr int NV = decltype(nv)::value;
        if (NV <= 4 && Dv >= 64 && cols_per_warp == 8)
            gated_delta_rule_kernel<NV, 8><<<dim3(ceil_div(Dv, REC_WARPS * 8), B * Hv), REC_WARPS * 32, 0, stream>>>(q, k, v, gate, beta, state, y, L, Hq, Hv, Dk, Dv);
        else
            gated_delta_rule_kernel<NV, 4><<<dim3(ceil_div(Dv, REC_WARPS * 4), B * Hv), REC_WARPS * 32, 0, stream>>>(q, k, v, gate, beta, state, y, L, Hq, Hv, Dk, Dv);
        OVB_CHECK_CUDA(cudaGetLastError());
        return 0;
    });
}

}  // extern "C"
