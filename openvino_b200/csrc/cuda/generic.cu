// Generic primitives of the CUDA device's graph executor: unary and binary element-wise operations with broadcasting,
// softmax / log-softmax along any axis, reductions, strided copies (transpose, concat, slice, broadcast, tile) and 2-D pooling.
// All of them are bandwidth bound: one pass over the data, 16-byte accesses on the contiguous fast paths, fp32 arithmetic
// whatever the storage type (fp32, fp16, bf16). Role in the reference: the element-wise, softmax, reduce, reorder and
// pooling kernel families of src/plugins/intel_gpu/src/kernel_selector/cl_kernels (eltwise_simple_vload8.cl,
// softmax_gpu_ref.cl, reduce_ref.cl, reorder_data.cl, pooling_gpu_ref.cl).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ovb {

template <class T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ------------------------------------------------------------------------------------ unary
__device__ __forceinline__ float unary_apply(int op, float v, float a, float b) {
    switch (op) {
        case OVB_UN_RELU: return v > 0.f ? v : 0.f;
        case OVB_UN_SIGMOID: return 1.f / (1.f + __expf(-v));
        case OVB_UN_TANH: return tanhf(v);
        case OVB_UN_GELU_ERF: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
        case OVB_UN_GELU_TANH: return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        case OVB_UN_SWISH: return v / (1.f + __expf(-a * v));
        case OVB_UN_EXP: return expf(v);
        case OVB_UN_LOG: return logf(v);
        case OVB_UN_SQRT: return sqrtf(v);
        case OVB_UN_ABS: return fabsf(v);
        case OVB_UN_NEG: return -v;
        case OVB_UN_HSWISH: return v * fminf(fmaxf(v + 3.f, 0.f), 6.f) * (1.f / 6.f);
        case OVB_UN_HSIGMOID: return fminf(fmaxf(v + 3.f, 0.f), 6.f) * (1.f / 6.f);
        case OVB_UN_MISH: return v * tanhf(v > 20.f ? v : log1pf(expf(v)));
        case OVB_UN_SOFTPLUS: return v > 20.f ? v : log1pf(expf(v));
        case OVB_UN_ERF: return erff(v);
        case OVB_UN_FLOOR: return floorf(v);
        case OVB_UN_CEIL: return ceilf(v);
        case OVB_UN_SIGN: return v > 0.f ? 1.f : (v < 0.f ? -1.f : 0.f);
        case OVB_UN_CLAMP: return fminf(fmaxf(v, a), b);
        case OVB_UN_ELU: return v > 0.f ? v : a * (expf(v) - 1.f);
        case OVB_UN_SIN: return sinf(v);
        case OVB_UN_COS: return cosf(v);
        case OVB_UN_RSQRT: return rsqrtf(v);
        case OVB_UN_SOFTSIGN: return v / (1.f + fabsf(v));
        case OVB_UN_ROUND_EVEN: return rintf(v);
        case OVB_UN_ROUND_AWAY: return roundf(v);
        case OVB_UN_SCALE_SHIFT: return v * a + b;
        default: return v;
    }
}

template <class T>
__global__ void unary_kernel(int op, const T* __restrict__ x, T* __restrict__ y, size_t n, float a, float b) {
    pdl_enter();
    constexpr int V = 16 / sizeof(T);
    const size_t nv = n / V;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nv; i += stride) {
        union { uint4 u; T e[V]; } in, out;
        in.u = reinterpret_cast<const uint4*>(x)[i];
#pragma unroll
        for (int j = 0; j < V; ++j) out.e[j] = from_f<T>(unary_apply(op, to_f(in.e[j]), a, b));
        reinterpret_cast<uint4*>(y)[i] = out.u;
    }
    for (size_t i = nv * V + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += stride)
        y[i] = from_f<T>(unary_apply(op, to_f(x[i]), a, b));
}

// ------------------------------------------------------------------------------------ binary with broadcasting
__device__ __forceinline__ float binary_apply(int op, float a, float b) {
    switch (op) {
        case OVB_BIN_ADD: return a + b;
        case OVB_BIN_SUB: return a - b;
        case OVB_BIN_MUL: return a * b;
        case OVB_BIN_DIV: return a / b;
        case OVB_BIN_MAX: return fmaxf(a, b);
        case OVB_BIN_MIN: return fminf(a, b);
        case OVB_BIN_POW: return powf(a, b);
        case OVB_BIN_SQDIFF: return (a - b) * (a - b);
        case OVB_BIN_PRELU: return a >= 0.f ? a : a * b;
        default: return a;
    }
}

struct Dims {
    int nd;
    int shape[OVB_MAX_DIMS];
    int64_t sa[OVB_MAX_DIMS];   // element strides (0 on a broadcast axis)
    int64_t sb[OVB_MAX_DIMS];
};

// Offsets of flat index i in both operands. 32-bit index arithmetic when the element count allows it (64-bit division is
// an order of magnitude slower and would bound the copy).
__device__ __forceinline__ void offsets_of(size_t i, bool small, const Dims& d, int64_t& oa, int64_t& ob) {
    oa = 0;
    ob = 0;
    if (small) {
        uint32_t r = (uint32_t)i;
#pragma unroll
        for (int k = OVB_MAX_DIMS - 1; k >= 0; --k) {
            if (k < d.nd) {
                const uint32_t q = r / (uint32_t)d.shape[k];
                const uint32_t c = r - q * (uint32_t)d.shape[k];
                r = q;
                oa += (int64_t)c * d.sa[k];
                ob += (int64_t)c * d.sb[k];
            }
        }
    } else {
        size_t r = i;
#pragma unroll
        for (int k = OVB_MAX_DIMS - 1; k >= 0; --k) {
            if (k < d.nd) {
                const int c = int(r % d.shape[k]);
                r /= d.shape[k];
                oa += c * d.sa[k];
                ob += c * d.sb[k];
            }
        }
    }
}

template <class T>
__global__ void binary_same_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, size_t n) {
    pdl_enter();
    constexpr int V = 16 / sizeof(T);
    const size_t nv = n / V;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nv; i += stride) {
        union { uint4 u; T e[V]; } ia, ib, out;
        ia.u = reinterpret_cast<const uint4*>(a)[i];
        ib.u = reinterpret_cast<const uint4*>(b)[i];
#pragma unroll
        for (int j = 0; j < V; ++j) out.e[j] = from_f<T>(binary_apply(op, to_f(ia.e[j]), to_f(ib.e[j])));
        reinterpret_cast<uint4*>(y)[i] = out.u;
    }
    for (size_t i = nv * V + blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += stride)
        y[i] = from_f<T>(binary_apply(op, to_f(a[i]), to_f(b[i])));
}

template <class T>
__global__ void binary_bcast_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, size_t n, Dims d) {
    pdl_enter();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const bool small = n <= 0xFFFFFFFFull;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t oa, ob;
        offsets_of(i, small, d, oa, ob);
        y[i] = from_f<T>(binary_apply(op, to_f(a[oa]), to_f(b[ob])));
    }
}

// ------------------------------------------------------------------------------------ strided copy
// y (contiguous, `shape`) = x read through element strides `sa` (any layout: transposed, sliced, broadcast with stride 0).
// The output may itself be a slice of a larger tensor along one axis (concat): row pitch handled by the caller through
// `sb` = output element strides.
template <class T>
__global__ void strided_copy_kernel(const T* __restrict__ x, T* __restrict__ y, size_t n, Dims d) {
    pdl_enter();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const bool small = n <= 0xFFFFFFFFull;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t oa, ob;
        offsets_of(i, small, d, oa, ob);
        y[ob] = x[oa];
    }
}

// Transpose of the two innermost axes of [batch, R, C] through a padded shared-memory tile: both sides coalesced.
template <class T>
__global__ void transpose2d_kernel(const T* __restrict__ x, T* __restrict__ y, int R, int C) {
    pdl_enter();
    __shared__ T tile[32][33];
    const size_t base = (size_t)blockIdx.z * R * C;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int r = r0 + j, c = c0 + threadIdx.x;
        if (r < R && c < C) tile[j][threadIdx.x] = x[base + (size_t)r * C + c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int c = c0 + j, r = r0 + threadIdx.x;
        if (r < R && c < C) y[base + (size_t)c * R + r] = tile[threadIdx.x][j];
    }
}

// ------------------------------------------------------------------------------------ softmax / reductions over [outer, dim, inner]
__device__ __forceinline__ float warp_max(float v) {
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
template <bool MAX>
__device__ __forceinline__ float block_reduce(float v, float* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = MAX ? warp_max(v) : warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float r = MAX ? -INFINITY : 0.f;
    for (int w = 0; w < nw; ++w) r = MAX ? fmaxf(r, sh[w]) : r + sh[w];
    return r;
}

// inner == 1: one block per row, the row is read once into registers when it fits (dim <= 8 * blockDim), else three passes.
template <class T, int PER>
__global__ void softmax_rows_kernel(const T* __restrict__ x, T* __restrict__ y, int dim, int log_out) {
    pdl_enter();
    __shared__ float sh[32];
    const T* xr = x + (size_t)blockIdx.x * dim;
    T* yr = y + (size_t)blockIdx.x * dim;
    float v[PER];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        v[j] = c < dim ? to_f(xr[c]) : -INFINITY;
        m = fmaxf(m, v[j]);
    }
    m = block_reduce<true>(m, sh);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < dim) { v[j] = log_out ? v[j] - m : __expf(v[j] - m); s += log_out ? __expf(v[j]) : v[j]; }
    }
    s = block_reduce<false>(s, sh);
    const float inv = log_out ? logf(s) : 1.f / s;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int c = threadIdx.x + j * blockDim.x;
        if (c < dim) yr[c] = from_f<T>(log_out ? v[j] - inv : v[j] * inv);
    }
}

// general form: one thread per (outer, inner) column, strided walk over dim (coalesced across inner)
template <class T>
__global__ void softmax_strided_kernel(const T* __restrict__ x, T* __restrict__ y, size_t outer, int dim, size_t inner, int log_out) {
    pdl_enter();
    const size_t total = outer * inner;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t o = i / inner, in = i - o * inner;
        const T* xp = x + o * dim * inner + in;
        T* yp = y + o * dim * inner + in;
        float m = -INFINITY;
        for (int k = 0; k < dim; ++k) m = fmaxf(m, to_f(xp[(size_t)k * inner]));
        float s = 0.f;
        for (int k = 0; k < dim; ++k) s += __expf(to_f(xp[(size_t)k * inner]) - m);
        const float inv = log_out ? logf(s) : 1.f / s;
        for (int k = 0; k < dim; ++k) {
            const float t = to_f(xp[(size_t)k * inner]) - m;
            yp[(size_t)k * inner] = from_f<T>(log_out ? t - inv : __expf(t) * inv);
        }
    }
}

__device__ __forceinline__ float red_init(int op) {
    return op == OVB_RED_MAX ? -INFINITY : (op == OVB_RED_MIN ? INFINITY : (op == OVB_RED_PROD ? 1.f : 0.f));
}
__device__ __forceinline__ float red_step(int op, float acc, float v) {
    switch (op) {
        case OVB_RED_MAX: return fmaxf(acc, v);
        case OVB_RED_MIN: return fminf(acc, v);
        case OVB_RED_PROD: return acc * v;
        case OVB_RED_L2: return acc + v * v;
        case OVB_RED_L1: return acc + fabsf(v);
        default: return acc + v;   // SUM, MEAN
    }
}
__device__ __forceinline__ float red_merge(int op, float a, float b) {
    switch (op) {
        case OVB_RED_MAX: return fmaxf(a, b);
        case OVB_RED_MIN: return fminf(a, b);
        case OVB_RED_PROD: return a * b;
        default: return a + b;
    }
}
__device__ __forceinline__ float red_final(int op, float acc, int dim) {
    return op == OVB_RED_MEAN ? acc / (float)dim : (op == OVB_RED_L2 ? sqrtf(acc) : acc);
}

// inner == 1: one warp per output (rows of `dim` contiguous elements)
template <class T>
__global__ void reduce_rows_kernel(int op, const T* __restrict__ x, T* __restrict__ y, size_t outer, int dim) {
    pdl_enter();
    const size_t row = blockIdx.x * (size_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= outer) return;
    const int lane = threadIdx.x & 31;
    const T* xr = x + row * dim;
    float acc = red_init(op);
    for (int c = lane; c < dim; c += 32) acc = red_step(op, acc, to_f(xr[c]));
    for (int o = 16; o; o >>= 1) acc = red_merge(op, acc, __shfl_xor_sync(0xffffffffu, acc, o));
    if (lane == 0) y[row] = from_f<T>(red_final(op, acc, dim));
}

template <class T>
__global__ void reduce_strided_kernel(int op, const T* __restrict__ x, T* __restrict__ y, size_t outer, int dim, size_t inner) {
    pdl_enter();
    const size_t total = outer * inner;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t o = i / inner, in = i - o * inner;
        const T* xp = x + o * dim * inner + in;
        float acc = red_init(op);
        for (int k = 0; k < dim; ++k) acc = red_step(op, acc, to_f(xp[(size_t)k * inner]));
        y[i] = from_f<T>(red_final(op, acc, dim));
    }
}

// ------------------------------------------------------------------------------------ 2-D pooling, NCHW
template <class T>
__global__ void pool2d_kernel(const T* __restrict__ x, T* __restrict__ y, ovb_pool_args a) {
    pdl_enter();
    const size_t total = (size_t)a.NC * a.OH * a.OW;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int ow = int(i % a.OW);
        const int oh = int((i / a.OW) % a.OH);
        const size_t nc = i / ((size_t)a.OW * a.OH);
        const T* xp = x + nc * a.H * a.W;
        const int h0 = oh * a.sh - a.ph, w0 = ow * a.sw - a.pw;
        float acc = a.is_max ? -INFINITY : 0.f;
        int cnt = 0;
        for (int kh = 0; kh < a.kh; ++kh) {
            const int h = h0 + kh * a.dh;
            if (h < 0 || h >= a.H) continue;
            for (int kw = 0; kw < a.kw; ++kw) {
                const int w = w0 + kw * a.dw;
                if (w < 0 || w >= a.W) continue;
                const float v = to_f(xp[(size_t)h * a.W + w]);
                acc = a.is_max ? fmaxf(acc, v) : acc + v;
                ++cnt;
            }
        }
        if (!a.is_max) {
            if (a.exclude_pad) {
                acc = cnt ? acc / (float)cnt : 0.f;
            } else {
                // the divisor counts the padded cells inside the (padded) input, not the cells past its end (ceil rounding)
                const int he = min(h0 + (a.kh - 1) * a.dh + 1, a.H + a.ph_end), we = min(w0 + (a.kw - 1) * a.dw + 1, a.W + a.pw_end);
                const int nh = (he - h0 + a.dh - 1) / a.dh, nw = (we - w0 + a.dw - 1) / a.dw;
                acc /= (float)max(1, nh * nw);
            }
        }
        y[i] = from_f<T>(acc);
    }
}

static inline int grid_of(size_t work, int block) {
    size_t g = (work + block - 1) / block;
    const size_t cap = 148 * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

#define OVB_DISPATCH_DTYPE(dtype, CALL)                                   \
    switch (dtype) {                                                      \
        case OVB_DT_F32: { using T = float; CALL; break; }                \
        case OVB_DT_F16: { using T = __half; CALL; break; }               \
        case OVB_DT_BF16: { using T = __nv_bfloat16; CALL; break; }       \
        default: set_error("unsupported element type %d", dtype); return ERR_UNSUPPORTED; \
    }

}  // namespace ovb

using namespace ovb;

extern "C" {

int ovb_unary(int op, const void* x, void* y, int64_t n, int dtype, float a, float b, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(x && y && n > 0 && op >= 0 && op < OVB_UN_COUNT, "ovb_unary: bad arguments");
    OVB_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0, "ovb_unary: 16-byte aligned tensors expected");
    OVB_DISPATCH_DTYPE(dtype, OVB_CHECK_CUDA(launch_pdl(unary_kernel<T>, dim3(grid_of((size_t)n / (16 / sizeof(T)) + 1, 256)), dim3(256), 0, stream, op,
                                                        (const T*)x, (T*)y, (size_t)n, a, b)));
    return 0;
}

static int fill_dims(Dims& d, int nd, const int64_t* shape, const int64_t* sa, const int64_t* sb) {
    if (nd < 1 || nd > OVB_MAX_DIMS) return -1;
    d.nd = nd;
    for (int k = 0; k < OVB_MAX_DIMS; ++k) {
        d.shape[k] = k < nd ? (int)shape[k] : 1;
        d.sa[k] = k < nd ? sa[k] : 0;
        d.sb[k] = k < nd ? sb[k] : 0;
    }
    return 0;
}

int ovb_binary(int op, const void* a, const void* b, void* y, int nd, const int64_t* shape, const int64_t* sa, const int64_t* sb, int same, int dtype,
               ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(a && b && y && shape && op >= 0 && op < OVB_BIN_COUNT, "ovb_binary: bad arguments");
    Dims d;
    OVB_REQUIRE(fill_dims(d, nd, shape, sa, sb) == 0, "ovb_binary: 1..%d dimensions", OVB_MAX_DIMS);
    size_t n = 1;
    for (int k = 0; k < nd; ++k) n *= (size_t)shape[k];
    OVB_REQUIRE(n > 0, "ovb_binary: empty tensor");
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    if (same && aligned) {
        OVB_DISPATCH_DTYPE(dtype, OVB_CHECK_CUDA(launch_pdl(binary_same_kernel<T>, dim3(grid_of(n / (16 / sizeof(T)) + 1, 256)), dim3(256), 0, stream, op,
                                                            (const T*)a, (const T*)b, (T*)y, n)));
    } else {
        OVB_DISPATCH_DTYPE(dtype, OVB_CHECK_CUDA(launch_pdl(binary_bcast_kernel<T>, dim3(grid_of(n, 256)), dim3(256), 0, stream, op, (const T*)a, (const T*)b,
                                                            (T*)y, n, d)));
    }
    return 0;
}

int ovb_strided_copy(const void* x, void* y, int nd, const int64_t* shape, const int64_t* sx, const int64_t* sy, int elem_bytes, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(x && y && shape && sx && sy, "ovb_strided_copy: bad arguments");
    Dims d;
    OVB_REQUIRE(fill_dims(d, nd, shape, sx, sy) == 0, "ovb_strided_copy: 1..%d dimensions", OVB_MAX_DIMS);
    size_t n = 1;
    for (int k = 0; k < nd; ++k) n *= (size_t)shape[k];
    OVB_REQUIRE(n > 0, "ovb_strided_copy: empty tensor");
    const dim3 g(grid_of(n, 256)), b(256);
    switch (elem_bytes) {
        case 1: OVB_CHECK_CUDA(launch_pdl(strided_copy_kernel<uint8_t>, g, b, 0, stream, (const uint8_t*)x, (uint8_t*)y, n, d)); break;
        case 2: OVB_CHECK_CUDA(launch_pdl(strided_copy_kernel<uint16_t>, g, b, 0, stream, (const uint16_t*)x, (uint16_t*)y, n, d)); break;
        case 4: OVB_CHECK_CUDA(launch_pdl(strided_copy_kernel<uint32_t>, g, b, 0, stream, (const uint32_t*)x, (uint32_t*)y, n, d)); break;
        case 8: OVB_CHECK_CUDA(launch_pdl(strided_copy_kernel<uint64_t>, g, b, 0, stream, (const uint64_t*)x, (uint64_t*)y, n, d)); break;
        case 16:
            OVB_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0, "ovb_strided_copy: 16-byte units need 16-byte aligned tensors");
            OVB_CHECK_CUDA(launch_pdl(strided_copy_kernel<uint4>, g, b, 0, stream, (const uint4*)x, (uint4*)y, n, d));
            break;
        default: OVB_REQUIRE(false, "ovb_strided_copy: element size %d", elem_bytes);
    }
    return 0;
}

int ovb_transpose2d(const void* x, void* y, int64_t batch, int R, int C, int elem_bytes, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(x && y && batch > 0 && batch < 65536 && R > 0 && C > 0, "ovb_transpose2d: bad arguments");
    const dim3 g((C + 31) / 32, (R + 31) / 32, (unsigned)batch), b(32, 8);
    OVB_REQUIRE(g.y < 65536, "ovb_transpose2d: too many rows");
    switch (elem_bytes) {
        case 2: OVB_CHECK_CUDA(launch_pdl(transpose2d_kernel<uint16_t>, g, b, 0, stream, (const uint16_t*)x, (uint16_t*)y, R, C)); break;
        case 4: OVB_CHECK_CUDA(launch_pdl(transpose2d_kernel<uint32_t>, g, b, 0, stream, (const uint32_t*)x, (uint32_t*)y, R, C)); break;
        default: OVB_REQUIRE(false, "ovb_transpose2d: element size %d", elem_bytes);
    }
    return 0;
}

int ovb_softmax(const void* x, void* y, int64_t outer, int dim, int64_t inner, int dtype, int log_out, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(x && y && outer > 0 && dim > 0 && inner > 0, "ovb_softmax: bad arguments");
    if (inner == 1 && dim <= 8192 && outer < (1ll << 31)) {
        const int block = dim <= 1024 ? 128 : (dim <= 4096 ? 512 : 1024);
        if (dim <= block) {
            OVB_DISPATCH_DTYPE(dtype, OVB_CHECK_CUDA(launch_pdl(softmax_rows_kernel<T, 1>, dim3((unsigned)outer), dim3(block), 0, stream, (const T*)x, (T*)y, dim, log_out)));
        } else {
            OVB_DISPATCH_DTYPE(dtype, OVB_CHECK_CUDA(launch_pdl(softmax_rows_kernel<T, 8>, dim3((unsigned)outer), dim3(block), 0, stream, (const T*)x, (T*)y, dim, log_out)));
        }
    } else {
        OVB_DISPATCH_DTYPE(dtype, OVB_CHECK_CUDA(launch_pdl(softmax_strided_kernel<T>, dim3(grid_of((size_t)(outer * inner), 128)), dim3(128), 0, stream, (const T*)x,
                                                            (T*)y, (size_t)outer, dim, (size_t)inner, log_out)));
    }
    return 0;
}

int ovb_reduce(int op, const void* x, void* y, int64_t outer, int dim, int64_t inner, int dtype, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(x && y && outer > 0 && dim > 0 && inner > 0 && op >= 0 && op < OVB_RED_COUNT, "ovb_reduce: bad arguments");
    if (inner == 1) {
        const size_t blocks = ((size_t)outer + 7) / 8;
        OVB_REQUIRE(blocks < (1ull << 31), "ovb_reduce: too many rows");
        OVB_DISPATCH_DTYPE(dtype, OVB_CHECK_CUDA(launch_pdl(reduce_rows_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, op, (const T*)x, (T*)y, (size_t)outer, dim)));
    } else {
        OVB_DISPATCH_DTYPE(dtype, OVB_CHECK_CUDA(launch_pdl(reduce_strided_kernel<T>, dim3(grid_of((size_t)(outer * inner), 128)), dim3(128), 0, stream, op, (const T*)x,
                                                            (T*)y, (size_t)outer, dim, (size_t)inner)));
    }
    return 0;
}

int ovb_pool2d(const void* x, void* y, const ovb_pool_args* a, int dtype, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(x && y && a && a->NC > 0 && a->H > 0 && a->W > 0 && a->OH > 0 && a->OW > 0 && a->kh > 0 && a->kw > 0 && a->sh > 0 && a->sw > 0 && a->dh > 0 && a->dw > 0,
                "ovb_pool2d: bad arguments");
    const size_t total = (size_t)a->NC * a->OH * a->OW;
    OVB_DISPATCH_DTYPE(dtype, OVB_CHECK_CUDA(launch_pdl(pool2d_kernel<T>, dim3(grid_of(total, 256)), dim3(256), 0, stream, (const T*)x, (T*)y, *a)));
    return 0;
}

}  // extern "C"
