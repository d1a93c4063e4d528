// Bandwidth-bound kernels of the LLM / encoder paths: RMSNorm (+residual), LayerNorm, SwiGLU
// gating, embedding gather, greedy sampling (argmax), RoPE fused with the paged KV-cache write,
// int4 weight re-packing.
//
// Reference counterparts (OpenCL / JIT, Intel-only): rms_gpu_bfyx_opt.cl, rope_opt.cl,
// swiglu_gpu_opt.cl, pa_kv_cache_update_ref.cl, mvn_gpu_*.cl; math as in
// src/core/reference/include/openvino/reference/rms_norm.hpp.
#include <math_constants.h>

#include <cuda_fp8.h>

#include "common.cuh"
#include "debug_bounds.cuh"
#include "sm100_ptx.cuh"

namespace ovb {

OVB_DEBUG_LIMITS_DEFINE

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
    if (warp == 0) {
        t = warp_sum(t);
        if (lane == 0) red[0] = t;
    }
    __syncthreads();
    return red[0];
}

union Pack8 {
    uint4 u;
    __nv_bfloat16 b[8];
    __half h[8];
};

// ------------------------------------------------------------------------------------ RMSNorm
// One CTA per row; cols % 8 == 0. Row is kept in registers (up to 8 vectors per thread).
template <int THREADS, int MAXV>
__global__ void __launch_bounds__(THREADS)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
               const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ y,
               __nv_bfloat16* __restrict__ residual_out, int cols, float eps) {
    pdl_enter();
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const int nvec = cols >> 3;
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * cols);
    const uint4* rr = residual ? reinterpret_cast<const uint4*>(residual + row * cols) : nullptr;
    float vals[MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = threadIdx.x + i * THREADS;
        if (v < nvec) {
            Pack8 a;
            a.u = xr[v];
            if (rr) {
                Pack8 b;
                b.u = rr[v];
                Pack8 o;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // the residual stream is stored in bf16: round before normalising, as the stored value is
                    // what the next layer reads
                    o.b[j] = __float2bfloat16_rn(__bfloat162float(a.b[j]) + __bfloat162float(b.b[j]));
                    vals[i][j] = __bfloat162float(o.b[j]);
                }
                if (residual_out) reinterpret_cast<uint4*>(residual_out + row * cols)[v] = o.u;
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) vals[i][j] = __bfloat162float(a.b[j]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
        }
    }
    const float tot = block_sum<THREADS>(ss, red);
    const float inv = rsqrtf(tot / float(cols) + eps);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = threadIdx.x + i * THREADS;
        if (v < nvec) {
            Pack8 g, o;
            g.u = reinterpret_cast<const uint4*>(gamma)[v];
#pragma unroll
            for (int j = 0; j < 8; ++j) o.b[j] = __float2bfloat16_rn(vals[i][j] * inv * __bfloat162float(g.b[j]));
            reinterpret_cast<uint4*>(y + row * cols)[v] = o.u;
        }
    }
}

// ------------------------------------------------------------------------------------ LayerNorm
template <class E, int THREADS, int MAXV>
__global__ void __launch_bounds__(THREADS)
layernorm_kernel(const E* __restrict__ x, const E* __restrict__ residual, const E* __restrict__ gamma,
                 const E* __restrict__ beta, E* __restrict__ y, int cols, float eps) {
    pdl_enter();
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const int nvec = cols >> 3;
    float vals[MAXV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = threadIdx.x + i * THREADS;
        if (v < nvec) {
            uint4 a = reinterpret_cast<const uint4*>(x + row * cols)[v];
            const E* ae = reinterpret_cast<const E*>(&a);
            uint4 b = make_uint4(0, 0, 0, 0);
            if (residual) b = reinterpret_cast<const uint4*>(residual + row * cols)[v];
            const E* be = reinterpret_cast<const E*>(&b);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                vals[i][j] = float(ae[j]) + (residual ? float(be[j]) : 0.f);
                s += vals[i][j];
            }
        }
    }
    const float mean = block_sum<THREADS>(s, red) / float(cols);
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = threadIdx.x + i * THREADS;
        if (v < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float d = vals[i][j] - mean;
                sq += d * d;
            }
        }
    }
    const float var = block_sum<THREADS>(sq, red) / float(cols);
    const float inv = rsqrtf(var + eps);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
        const int v = threadIdx.x + i * THREADS;
        if (v < nvec) {
            uint4 g = reinterpret_cast<const uint4*>(gamma)[v];
            uint4 bt = reinterpret_cast<const uint4*>(beta)[v];
            const E* ge = reinterpret_cast<const E*>(&g);
            const E* bte = reinterpret_cast<const E*>(&bt);
            uint4 o;
            E* oe = reinterpret_cast<E*>(&o);
#pragma unroll
            for (int j = 0; j < 8; ++j) oe[j] = E((vals[i][j] - mean) * inv * float(ge[j]) + float(bte[j]));
            reinterpret_cast<uint4*>(y + row * cols)[v] = o;
        }
    }
}

// ------------------------------------------------------------------------------------ SwiGLU gate
// `nrows` (optional, device memory, written by an earlier kernel): only the first min(*nrows, rows) rows are valid.
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int rows, int F, const int* __restrict__ nrows) {
    pdl_enter();
    if (nrows != nullptr) rows = min(rows, *nrows);
    const int fv = F >> 3;
    const size_t total = (size_t)rows * fv;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / fv;
        const int c = int(i - r * fv);
        Pack8 g, u, o;
        g.u = reinterpret_cast<const uint4*>(gu + r * 2 * F)[c];
        u.u = reinterpret_cast<const uint4*>(gu + r * 2 * F + F)[c];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float gv = __bfloat162float(g.b[j]);
            const float s = gv / (1.0f + __expf(-gv));
            o.b[j] = __float2bfloat16_rn(s * __bfloat162float(u.b[j]));
        }
        reinterpret_cast<uint4*>(out + r * F)[c] = o.u;
    }
}

// ------------------------------------------------------------------------------------ mixture of experts
// Router: softmax over the E expert logits of a token, keep the top k, renormalise them to sum 1 (Mixtral rule).
// Output: dense [T, E] fp32 routing weights (0 for experts that were not selected). One thread per token, E <= 64.
__global__ void moe_route_topk_kernel(const float* __restrict__ logits, float* __restrict__ weights, int T, int E, int k) {
    pdl_enter();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    float v[64];
    float mx = -INFINITY;
    for (int e = 0; e < E; ++e) { v[e] = logits[(size_t)t * E + e]; mx = fmaxf(mx, v[e]); }
    float sum = 0.f;
    for (int e = 0; e < E; ++e) { v[e] = __expf(v[e] - mx); sum += v[e]; }
    unsigned long long picked = 0ull;
    float top_sum = 0.f;
    for (int j = 0; j < k; ++j) {
        int best = -1;
        float bv = -1.f;
        for (int e = 0; e < E; ++e)
            if (!((picked >> e) & 1ull) && v[e] > bv) { bv = v[e]; best = e; }      // first index wins ties
        picked |= 1ull << best;
        top_sum += bv;
    }
    (void)sum;   // the softmax denominator cancels in the renormalisation
    for (int e = 0; e < E; ++e) weights[(size_t)t * E + e] = ((picked >> e) & 1ull) ? v[e] / top_sum : 0.f;
}

// act[t, e*F + f] = silu(gu[t, e*2F + f]) * gu[t, e*2F + F + f] * w[t, e0 + e] for the `nloc` local experts of a rank.
// A token that is not routed to an expert gets zeros there, so the stacked down projection sums exactly the routed experts.
__global__ void moe_silu_mul_scale_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                          int rows, int F, int nloc, int E, int e0) {
    pdl_enter();
    const int fv = F >> 3;
    const size_t total = (size_t)rows * nloc * fv;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / ((size_t)nloc * fv);
        const int rem = int(i - r * (size_t)nloc * fv);
        const int e = rem / fv, c = rem - e * fv;
        const float scale = w[r * E + e0 + e];
        Pack8 o;
        if (scale == 0.f) {
            o.u = make_uint4(0u, 0u, 0u, 0u);
        } else {
            Pack8 g, u;
            const __nv_bfloat16* base = gu + (r * nloc + e) * 2 * (size_t)F;
            g.u = reinterpret_cast<const uint4*>(base)[c];
            u.u = reinterpret_cast<const uint4*>(base + F)[c];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float gv = __bfloat162float(g.b[j]);
                o.b[j] = __float2bfloat16_rn(gv / (1.0f + __expf(-gv)) * __bfloat162float(u.b[j]) * scale);
            }
        }
        reinterpret_cast<uint4*>(out + (r * nloc + e) * (size_t)F)[c] = o.u;
    }
}

__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ out, size_t nvec) {
    pdl_enter();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
        Pack8 x, y, o;
        x.u = reinterpret_cast<const uint4*>(a)[i];
        y.u = reinterpret_cast<const uint4*>(b)[i];
#pragma unroll
        for (int j = 0; j < 8; ++j) o.b[j] = __float2bfloat16_rn(__bfloat162float(x.b[j]) + __bfloat162float(y.b[j]));
        reinterpret_cast<uint4*>(out)[i] = o.u;
    }
}

// ------------------------------------------------------------------------------------ embedding
template <class IdT>
__global__ void embedding_kernel(const IdT* __restrict__ ids, const uint4* __restrict__ table,
                                 uint4* __restrict__ out, int rows, int vec_per_row, int vocab) {
    pdl_enter();
    const size_t total = (size_t)rows * vec_per_row;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / vec_per_row;
        const int c = int(i - r * vec_per_row);
        int64_t id = ids[r];
        if (id < 0 || id >= vocab) {         // out-of-range ids read row 0 instead of faulting (the debug build also reports them)
            (void)OVB_DBG_ROW(-1, 1);
            id = 0;
        }
        out[i] = table[(size_t)id * vec_per_row + c];
    }
}

// ------------------------------------------------------------------------------------ token feedback
// Steps can be chained on the device without a host round trip: a token position whose tok_src is
// >= 0 takes its id from last_token[tok_src] (the token sampled for that request by an earlier step)
// instead of the id uploaded by the host; after sampling, sequence i's token goes to
// last_token[tok_dst[i]] (tok_dst < 0: the step ended inside the prompt, nothing to record).
__global__ void resolve_ids_kernel(int* __restrict__ ids, const int* __restrict__ tok_src,
                                   const int* __restrict__ last_token, int T) {
    pdl_enter();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < T) {
        const int s = tok_src[t];
        if (s >= 0) ids[t] = last_token[s];
    }
}
__global__ void scatter_tokens_kernel(const int* __restrict__ tokens, const int* __restrict__ tok_dst,
                                      int* __restrict__ last_token, int B) {
    pdl_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < B) {
        const int d = tok_dst[i];
        if (d >= 0) last_token[d] = tokens[i];
    }
}

// ------------------------------------------------------------------------------------ argmax
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
argmax_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int vocab, void* __restrict__ out_ids, int ids_i32,
              float* __restrict__ out_max) {
    pdl_enter();
    __shared__ float sv[THREADS / 32];
    __shared__ int si[THREADS / 32];
    const size_t row = blockIdx.x;
    const __nv_bfloat16* lr = logits + row * ld;
    float best = -CUDART_INF_F;
    int bi = 0x7fffffff;
    const int nvec = vocab >> 3;
    const bool aligned = ((reinterpret_cast<uintptr_t>(lr) & 15) == 0);
    if (aligned) {
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            Pack8 a;
            a.u = reinterpret_cast<const uint4*>(lr)[v];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float f = __bfloat162float(a.b[j]);
                if (f > best) { best = f; bi = v * 8 + j; }
            }
        }
        for (int i = nvec * 8 + threadIdx.x; i < vocab; i += THREADS) {
            const float f = __bfloat162float(lr[i]);
            if (f > best) { best = f; bi = i; }
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += THREADS) {
            const float f = __bfloat162float(lr[i]);
            if (f > best) { best = f; bi = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = lane < THREADS / 32 ? sv[lane] : -CUDART_INF_F;
        bi = lane < THREADS / 32 ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (lane == 0) {
            const int res = bi == 0x7fffffff ? 0 : bi;
            if (ids_i32) reinterpret_cast<int*>(out_ids)[row] = res;
            else reinterpret_cast<int64_t*>(out_ids)[row] = res;
            if (out_max) out_max[row] = best;
        }
    }
}

// ------------------------------------------------------------------------------------ RoPE + KV write
// One CTA per token. q rotated in place; k rotated and written to the cache; v copied to the cache.
// Cache layout [num_blocks, Hkv, block_size, D].
__global__ void rope_kv_write_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ slot_map, __nv_bfloat16* __restrict__ k_cache,
                                     __nv_bfloat16* __restrict__ v_cache, int Hq, int Hkv, int D, float log2_theta,
                                     int block_size) {
    pdl_enter();
    const int t = blockIdx.x;
    const int half = D >> 1;
    const float pos = float(positions[t]);
    const int slot = OVB_DBG_SLOT(slot_map[t], block_size);
    const int blk = slot / block_size, off = slot - blk * block_size;
    __nv_bfloat16* row = qkv + (size_t)t * (Hq + 2 * Hkv) * D;
    const int pairs_q = Hq * half, pairs_k = Hkv * half;
    for (int i = threadIdx.x; i < pairs_q + pairs_k; i += blockDim.x) {
        const bool is_k = i >= pairs_q;
        const int j = is_k ? i - pairs_q : i;
        const int h = j / half, d = j - h * half;
        const float inv_freq = exp2f(-log2_theta * (2.0f * float(d) / float(D)));
        float sn, cs;
        sincosf(pos * inv_freq, &sn, &cs);
        __nv_bfloat16* p = row + (size_t)(is_k ? Hq + h : h) * D;
        const float x1 = __bfloat162float(p[d]), x2 = __bfloat162float(p[d + half]);
        const __nv_bfloat16 o1 = __float2bfloat16_rn(x1 * cs - x2 * sn);
        const __nv_bfloat16 o2 = __float2bfloat16_rn(x2 * cs + x1 * sn);
        if (is_k) {
            if (slot >= 0) {
                __nv_bfloat16* c = k_cache + (((size_t)blk * Hkv + h) * block_size + off) * D;
                c[d] = o1;
                c[d + half] = o2;
            }
        } else {
            p[d] = o1;
            p[d + half] = o2;
        }
    }
    if (slot >= 0) {
        const __nv_bfloat16* v = row + (size_t)(Hq + Hkv) * D;
        for (int i = threadIdx.x; i < Hkv * D; i += blockDim.x) {
            const int h = i / D, d = i - h * D;
            v_cache[(((size_t)blk * Hkv + h) * block_size + off) * D + d] = v[i];
        }
    }
}

// Vector form for head sizes that are multiples of 4: one warp per (token, head), a lane rotates two adjacent pairs
// (bf16x2 loads and stores); the grid covers every head of every token, so a decode step of a few dozen tokens still
// fills the machine.
__global__ void rope_kv_write_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                         const int* __restrict__ slot_map, __nv_bfloat16* __restrict__ k_cache,
                                         __nv_bfloat16* __restrict__ v_cache, int Hq, int Hkv, int D, float log2_theta,
                                         int block_size) {
    pdl_enter();
    const int t = blockIdx.x;
    const int h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (h >= Hq + 2 * Hkv) return;
    const int half = D >> 1;
    const int slot = OVB_DBG_SLOT(slot_map[t], block_size);
    const int blk = slot / block_size, off = slot - blk * block_size;
    __nv_bfloat16* p = qkv + ((size_t)t * (Hq + 2 * Hkv) + h) * D;
    if (h >= Hq + Hkv) {                       // value head: copy to the cache
        if (slot < 0) return;
        __nv_bfloat16* c = v_cache + (((size_t)blk * Hkv + (h - Hq - Hkv)) * block_size + off) * D;
        for (int d = lane * 2; d < D; d += 64) *reinterpret_cast<uint32_t*>(c + d) = *reinterpret_cast<const uint32_t*>(p + d);
        return;
    }
    const bool is_k = h >= Hq;
    if (is_k && slot < 0) return;
    __nv_bfloat16* dst = is_k ? k_cache + (((size_t)blk * Hkv + (h - Hq)) * block_size + off) * D : p;
    const float pos = float(positions[t]);
    for (int d = lane * 2; d < half; d += 64) {
        float s0, c0, s1, c1;
        sincosf(pos * exp2f(-log2_theta * (2.0f * float(d) / float(D))), &s0, &c0);
        sincosf(pos * exp2f(-log2_theta * (2.0f * float(d + 1) / float(D))), &s1, &c1);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + d));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + d + half));
        *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
        *reinterpret_cast<__nv_bfloat162*>(dst + d + half) = __floats2bfloat162_rn(b.x * c0 + a.x * s0, b.y * c1 + a.y * s1);
    }
}

// The same with a u8 KV cache (head size 128): a warp owns one (token, head), a lane four values. Key and value rows are
// quantised per row: scale = (max - min) / 255, zero point = -min / scale, byte = round(x / scale + zero point), and the
// (scale, zero point) pair is stored as fp16 beside the bytes; value = (byte - zero point) * scale. Query heads are rotated in
// place as before. Role in the reference: the by-token quantisation of the KV cache,
// src/plugins/intel_gpu/src/kernel_selector/cl_kernels/pa_kv_cache_update_ref.cl and dynamic_quantize_gpu_kv_cache.cl.
__global__ void rope_kv_write_u8_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ slot_map,
                                        uint8_t* __restrict__ k_cache, uint8_t* __restrict__ v_cache, __half2* __restrict__ k_meta,
                                        __half2* __restrict__ v_meta, int Hq, int Hkv, float log2_theta, int block_size) {
    pdl_enter();
    constexpr int D = 128, half = 64;
    const int t = blockIdx.x;
    const int h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (h >= Hq + 2 * Hkv) return;
    const int slot = OVB_DBG_SLOT(slot_map[t], block_size);
    const int blk = slot / block_size, off = slot - blk * block_size;
    __nv_bfloat16* p = qkv + ((size_t)t * (Hq + 2 * Hkv) + h) * D;
    const int d = lane * 2;
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + d));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + d + half));
    float v[4] = {a.x, a.y, b.x, b.y};
    const bool is_v = h >= Hq + Hkv;
    if (!is_v) {
        const float pos = float(positions[t]);
        float s0, c0, s1, c1;
        sincosf(pos * exp2f(-log2_theta * (2.0f * float(d) / float(D))), &s0, &c0);
        sincosf(pos * exp2f(-log2_theta * (2.0f * float(d + 1) / float(D))), &s1, &c1);
        v[0] = a.x * c0 - b.x * s0; v[1] = a.y * c1 - b.y * s1;
        v[2] = b.x * c0 + a.x * s0; v[3] = b.y * c1 + a.y * s1;
        if (h < Hq) {
            *reinterpret_cast<__nv_bfloat162*>(p + d) = __floats2bfloat162_rn(v[0], v[1]);
            *reinterpret_cast<__nv_bfloat162*>(p + d + half) = __floats2bfloat162_rn(v[2], v[3]);
            return;
        }
    }
    if (slot < 0) return;                      // uniform over the warp
    float mn = fminf(fminf(v[0], v[1]), fminf(v[2], v[3])), mx = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
    for (int o = 16; o; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    // the pair is stored as fp16: quantise with the values the reader will see
    float scale = __half2float(__float2half_rn((mx - mn) * (1.0f / 255.0f)));
    if (!(scale > 0.f)) scale = 1.0f;
    const float zp = __half2float(__float2half_rn(-mn / scale));
    uint32_t q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = (uint32_t)fminf(fmaxf(rintf(v[i] / scale + zp), 0.f), 255.f);
    const int hk = is_v ? h - Hq - Hkv : h - Hq;
    const size_t row = ((size_t)blk * Hkv + hk) * block_size + off;
    uint8_t* dst = (is_v ? v_cache : k_cache) + row * D;
    *reinterpret_cast<uint16_t*>(dst + d) = (uint16_t)(q[0] | (q[1] << 8));
    *reinterpret_cast<uint16_t*>(dst + d + half) = (uint16_t)(q[2] | (q[3] << 8));
    if (lane == 0) (is_v ? v_meta : k_meta)[row] = __floats2half2_rn(scale, zp);
}

// ------------------------------------------------------------------------------------ MoE token grouping (prefill)
// For every local expert: the indices of the tokens routed to it, in token order, and their number. One CTA per expert
// walks the tokens in chunks of its size; positions come from a ballot / prefix sum, so the order is deterministic.
__global__ void moe_group_kernel(const float* __restrict__ route, int T, int E, int e0, int* __restrict__ idx, int* __restrict__ counts, int idx_stride) {
    pdl_enter();
    const int e = blockIdx.x;
    __shared__ int warp_sums[32];
    __shared__ int base_s;
    if (threadIdx.x == 0) base_s = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int t0 = 0; t0 < T; t0 += blockDim.x) {
        const int t = t0 + threadIdx.x;
        const bool hit = t < T && route[(size_t)t * E + e0 + e] != 0.f;
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) warp_sums[warp] = __popc(m);
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; ++w) before += warp_sums[w];
        if (hit) idx[(size_t)e * idx_stride + base_s + before + __popc(m & ((1u << lane) - 1u))] = t;
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int w = 0; w < nwarps; ++w) tot += warp_sums[w];
            base_s += tot;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[e] = base_s;
}

// act[i, f] = silu(gu[i, f]) * gu[i, F + f] * route[idx[i], e]  for the gathered rows of one expert
// ---- single-launch expert path: rows of all local experts sorted by expert, no host round trip
// Per local expert (one block each, like moe_group_kernel): the position of every token inside the expert's row list
// (pos[t * nloc + e], -1 when the token is not routed to the expert) and the number of rows (counts[e]).
__global__ void moe_positions_kernel(const float* __restrict__ route, int T, int E, int e0, int nloc, int* __restrict__ pos, int* __restrict__ counts) {
    pdl_enter();
    const int e = blockIdx.x;
    __shared__ int warp_sums[32];
    __shared__ int base_s;
    if (threadIdx.x == 0) base_s = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int t0 = 0; t0 < T; t0 += blockDim.x) {
        const int t = t0 + threadIdx.x;
        const bool hit = t < T && route[(size_t)t * E + e0 + e] != 0.f;
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) warp_sums[warp] = __popc(m);
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; ++w) before += warp_sums[w];
        if (t < T) pos[(size_t)t * nloc + e] = hit ? base_s + before + __popc(m & ((1u << lane) - 1u)) : -1;
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int w = 0; w < nwarps; ++w) tot += warp_sums[w];
            base_s += tot;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[e] = base_s;
}

// Row offsets of the experts (offsets[nloc + 1], written by block 0) and the gathered activations: row offsets[e] + pos of
// the sorted buffer is a copy of token t's row. One block per token.
__global__ void moe_gather_sorted_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ pos, const int* __restrict__ counts,
                                         int* __restrict__ offsets, __nv_bfloat16* __restrict__ xg, int T, int H, int nloc, int cap) {
    pdl_enter();
    __shared__ int off_s[65];
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < nloc; ++e) { off_s[e] = acc; acc += counts[e]; }
        off_s[nloc] = acc;
        if (blockIdx.x == 0) for (int e = 0; e <= nloc; ++e) offsets[e] = min(off_s[e], cap);
    }
    __syncthreads();
    const int t = blockIdx.x;
    if (t >= T) return;
    const int hv = H >> 3;
    for (int e = 0; e < nloc; ++e) {
        const int p_ = pos[(size_t)t * nloc + e];
        if (p_ < 0) continue;
        const int r = off_s[e] + p_;
        if (r >= cap) continue;
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * H);
        uint4* dst = reinterpret_cast<uint4*>(xg + (size_t)r * H);
        for (int c = threadIdx.x; c < hv; c += blockDim.x) dst[c] = src[c];
    }
}

// dst[t] = (accumulate ? dst[t] : 0) + sum over the local experts of route[t, e0 + e] * y[offsets[e] + pos[t, e]], experts in
// index order (deterministic, no atomics: a token's row is written by one block only).
__global__ void moe_combine_sorted_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ route, const int* __restrict__ pos,
                                          const int* __restrict__ offsets, __nv_bfloat16* __restrict__ dst, int T, int H, int E, int e0, int nloc,
                                          int ld_dst, int accumulate, int cap) {
    pdl_enter();
    const int t = blockIdx.x;
    if (t >= T) return;
    const int hv = H >> 3;
    for (int c = threadIdx.x; c < hv; c += blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint4* d = reinterpret_cast<uint4*>(dst + (size_t)t * ld_dst) + c;
        if (accumulate) {
            Pack8 a;
            a.u = *d;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = __bfloat162float(a.b[j]);
        }
        for (int e = 0; e < nloc; ++e) {
            const int p_ = pos[(size_t)t * nloc + e];
            if (p_ < 0) continue;
            const int r = offsets[e] + p_;
            if (r >= cap) continue;
            const float w = route[(size_t)t * E + e0 + e];
            Pack8 v;
            v.u = reinterpret_cast<const uint4*>(y + (size_t)r * H)[c];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += w * __bfloat162float(v.b[j]);
        }
        Pack8 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.b[j] = __float2bfloat16_rn(acc[j]);
        *d = o.u;
    }
}

__global__ void moe_silu_mul_rows_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ route, const int* __restrict__ idx,
                                         __nv_bfloat16* __restrict__ out, int rows, int F, int E, int e) {
    pdl_enter();
    const int fv = F >> 3;
    const size_t total = (size_t)rows * fv;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / fv;
        const int c = int(i - r * fv);
        const float scale = route[(size_t)idx[r] * E + e];
        Pack8 g, u, o;
        const __nv_bfloat16* base = gu + r * 2 * (size_t)F;
        g.u = reinterpret_cast<const uint4*>(base)[c];
        u.u = reinterpret_cast<const uint4*>(base + F)[c];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float gv = __bfloat162float(g.b[j]);
            o.b[j] = __float2bfloat16_rn(gv / (1.0f + __expf(-gv)) * __bfloat162float(u.b[j]) * scale);
        }
        reinterpret_cast<uint4*>(out + r * (size_t)F)[c] = o.u;
    }
}

// dst[idx[i], :] += src[i, :]; the rows of one expert are distinct tokens, so no two threads touch the same element
__global__ void moe_scatter_add_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ idx, __nv_bfloat16* __restrict__ dst,
                                       int rows, int H, int ld_dst) {
    pdl_enter();
    const int hv = H >> 3;
    const size_t total = (size_t)rows * hv;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / hv;
        const int c = int(i - r * hv);
        Pack8 a, b;
        a.u = reinterpret_cast<const uint4*>(src + r * (size_t)H)[c];
        uint4* d = reinterpret_cast<uint4*>(dst + (size_t)idx[r] * ld_dst) + c;
        b.u = *d;
#pragma unroll
        for (int j = 0; j < 8; ++j) b.b[j] = __float2bfloat16_rn(__bfloat162float(a.b[j]) + __bfloat162float(b.b[j]));
        *d = b.u;
    }
}

// ------------------------------------------------------------------------------------ fp8 activation quantisation
// Per token and group of 128 channels: scale = amax / 448, q = x / scale as e4m3 (round to nearest even, saturating).
// One warp per (token, group); a lane holds four channels. Role of the reference's dynamic_quantize_gpu_opt
// (src/plugins/intel_gpu/src/kernel_selector/cl_kernels/dynamic_quantize_gpu_opt.cl:82) with fp8 instead of int8 output.
__global__ void act_quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scales, int rows, int cols) {
    pdl_enter();
    const int groups = cols / 128;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows * groups) return;
    const int r = warp / groups, g = warp - r * groups;
    const __nv_bfloat16* src = x + (size_t)r * cols + g * 128 + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float v[4] = {__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1)};
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax > 0.f ? amax / 448.0f : 1.0f;
    const float inv = 1.0f / scale;
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(v[j] * inv, __NV_SATFINITE, __NV_E4M3);
        packed |= uint32_t(b) << (8 * j);
    }
    *reinterpret_cast<uint32_t*>(q + (size_t)r * cols + g * 128 + lane * 4) = packed;
    if (lane == 0) scales[(size_t)r * groups + g] = scale;
}

// ------------------------------------------------------------------------------------ KV-cache block copy
// Copies whole cache blocks src[i] -> dst[i] for the key and the value cache (fork of a sequence, swap after a
// preemption, beam reordering). One CTA per (pair, cache); 16-byte pieces. Role of pa_kv_cache_reorder_ref.cl.
__global__ void kv_block_copy_kernel(uint4* __restrict__ k_cache, uint4* __restrict__ v_cache, const int* __restrict__ src,
                                     const int* __restrict__ dst, size_t pieces_per_block) {
    pdl_enter();
    uint4* cache = blockIdx.y == 0 ? k_cache : v_cache;
    const size_t s = (size_t)OVB_DBG_BLOCK(src[blockIdx.x]) * pieces_per_block, d = (size_t)OVB_DBG_BLOCK(dst[blockIdx.x]) * pieces_per_block;
    if (s == d) return;
    for (size_t i = threadIdx.x; i < pieces_per_block; i += blockDim.x) cache[d + i] = cache[s + i];
}

// ------------------------------------------------------------------------------------ im2col (convolution as GEMM)
// cols[t][k] for t = (b, ho, wo) and k = (c * kh + r) * kw + s is x[b][c][ho*sh - pt + r*dh][wo*sw - pl + s*dw] (zero outside
// the image and for k >= C*kh*kw): the [T, Kpad] operand of out[T, O] = cols x W[O, Kpad]^T on the tcgen05 GEMM. A thread
// fills one 16-byte piece (8 consecutive k of one output position); the 16-bit payload is copied as it is (bf16 or fp16).
__global__ void im2col_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ cols, int B, int C, int H, int W, int kh, int kw,
                              int sh, int sw, int pt, int pl, int dh, int dw, int Ho, int Wo, int Kd, int Kpad) {
    pdl_enter();
    const int pieces = Kpad >> 3;
    const size_t total = (size_t)B * Ho * Wo * pieces;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int pc = int(i % pieces);
        const size_t t = i / pieces;
        const int wo = int(t % Wo);
        const int ho = int((t / Wo) % Ho);
        const int b = int(t / ((size_t)Wo * Ho));
        uint16_t v[8];
        int k = pc * 8;
        int s_ = k % kw, r = (k / kw) % kh, c = k / (kw * kh);
#pragma unroll
        for (int j = 0; j < 8; ++j, ++k) {
            uint16_t val = 0;
            if (k < Kd) {
                const int hi = ho * sh - pt + r * dh, wi = wo * sw - pl + s_ * dw;
                if (hi >= 0 && hi < H && wi >= 0 && wi < W) val = x[(((size_t)b * C + c) * H + hi) * W + wi];
            }
            v[j] = val;
            if (++s_ == kw) { s_ = 0; if (++r == kh) { r = 0; ++c; } }
        }
        *reinterpret_cast<uint4*>(cols + t * Kpad + pc * 8) = *reinterpret_cast<const uint4*>(v);
    }
}

// ------------------------------------------------------------------------------------ int4 re-pack
// IR layout: byte b of a row holds element 2b in its low nibble and 2b+1 in its high nibble.
// Plugin layout: every aligned group of 8 elements e0..e7 becomes one u32 with nibble j (j<4) = e[2j]
// and nibble j+4 = e[2j+1], so that one mask per shifted copy yields a pair of adjacent elements.
// The words are also re-ordered so that the 128 x 64 block of one (weight tile, k-block) pair is one
// contiguous chunk of 4608 bytes: 4 KB of nibbles split in two halves of k (0..31, 32..63) with 16 bytes per row in
// each half (word (tile * KB + kb) * 1152 + khalf * 512 + row * 4 + w; a warp whose lanes are consecutive rows reads
// consecutive 16-byte pieces, no bank conflicts), followed by the 128 (scale, 16 + zero point) bf16 pairs of the
// chunk's rows for its quantisation group (word ... + 1024 + row), so that ONE bulk copy brings all a k-block needs.
__global__ void pack_u4_kernel(const uint32_t* __restrict__ w_ir, uint32_t* __restrict__ w_out, size_t nwords, int K) {
    const int wpr = K / 8;          // words per row
    const int KB = K / 64;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nwords; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t x = w_ir[i];   // nibble k = element k
        const size_t n = i / wpr;
        const int kw = int(i - n * wpr);
        const size_t dst = ((n >> 7) * KB + (kw >> 3)) * 1152 + (size_t)(((kw & 7) >> 2) * 512) + (n & 127) * 4 + (kw & 3);
        uint32_t o = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            o |= ((x >> (8 * j)) & 0xF) << (4 * j);            // e[2j]   -> nibble j
            o |= ((x >> (8 * j + 4)) & 0xF) << (4 * j + 16);   // e[2j+1] -> nibble j+4
        }
        w_out[dst] = o;
    }
}
// copies the pairs of table [G][N] into every chunk of the tiled u4 layout (see pack_u4_kernel)
__global__ void embed_pairs_kernel(const uint32_t* __restrict__ table, uint32_t* __restrict__ w_out, int N, int KB, int kb_per_group,
                                   size_t total) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int row = int(i & 127);
        const size_t chunk = i >> 7;                 // tile * KB + kb
        const int kb = int(chunk % KB);
        const size_t n = (chunk / KB) * 128 + row;
        w_out[chunk * 1152 + 1024 + row] = n < (size_t)N ? table[(size_t)(kb / kb_per_group) * N + n] : 0u;
    }
}
__global__ void pack_w16_kernel(const uint4* __restrict__ w, uint4* __restrict__ w_out, size_t npieces, int K) {
    const int ppr = K / 8;          // 16-byte pieces per row
    const int KB = K / 64;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < npieces; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / ppr;
        const int pc = int(i - n * ppr);
        const int kb = pc >> 3, c = pc & 7, r = int(n & 127);
        const size_t dst = ((((n >> 7) * KB + kb) << 7) + r) * 8 + (c ^ (r & 7));
        w_out[dst] = w[i];
    }
}
// scales_ir [N, G] fp16 + zero points -> [G, N] pairs (bf16 scale, bf16 bias + zp); zps_out (optional) [G, N]
__global__ void pack_scale_zp_kernel(const __half* __restrict__ scales_ir, const uint8_t* __restrict__ zps_ir,
                                     int zp_is_u8, __nv_bfloat16* __restrict__ scales_out,
                                     __nv_bfloat16* __restrict__ zps_out, int N, int G, float zp_bias,
                                     float zp_default) {
    const size_t total = (size_t)N * G;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / G;
        const int g = int(i - n * G);
        scales_out[((size_t)g * N + n) * 2] = __float2bfloat16_rn(__half2float(scales_ir[i]));
        float z = zp_default;
        if (zps_ir) {
            if (zp_is_u8) z = float(zps_ir[i]);
            else z = float((zps_ir[i >> 1] >> ((i & 1) * 4)) & 0xF);
        }
        scales_out[((size_t)g * N + n) * 2 + 1] = __float2bfloat16_rn(zp_bias + z);
        if (zps_out) zps_out[(size_t)g * N + n] = __float2bfloat16_rn(zp_bias + z);
    }
}

static inline int grid_for(size_t n, int threads) {
    size_t g = (n + threads - 1) / threads;
    if (g > 148 * 16) g = 148 * 16;
    if (g < 1) g = 1;
    return int(g);
}

}  // namespace ovb

#ifdef OVB_DEBUG_BOUNDS
extern "C" int ovb_debug_set_limits_elementwise(const ovb::DebugLimits* l) {
    OVB_CHECK_CUDA(cudaMemcpyToSymbol(ovb::g_dbg_limits, l, sizeof(*l)));
    return 0;
}
#endif

extern "C" {
using namespace ovb;

int ovb_rmsnorm(const void* x, const void* residual, const void* gamma, void* y, void* residual_out, int rows,
                int cols, float eps, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(x && gamma && y && rows > 0, "ovb_rmsnorm: null operand");
    OVB_REQUIRE(cols % 8 == 0 && cols <= 256 * 8 * 8, "ovb_rmsnorm: cols=%d must be a multiple of 8 and <= 16384", cols);
    auto X = (const __nv_bfloat16*)x;
    auto R = (const __nv_bfloat16*)residual;
    auto G = (const __nv_bfloat16*)gamma;
    auto Y = (__nv_bfloat16*)y;
    auto RO = (__nv_bfloat16*)residual_out;
    const int nvec = cols / 8;
    if (nvec <= 256) OVB_CHECK_CUDA(launch_pdl(rmsnorm_kernel<256, 1>, dim3(rows), dim3(256), 0, stream, X, R, G, Y, RO, cols, eps));
    else if (nvec <= 512) OVB_CHECK_CUDA(launch_pdl(rmsnorm_kernel<256, 2>, dim3(rows), dim3(256), 0, stream, X, R, G, Y, RO, cols, eps));
    else if (nvec <= 1024) OVB_CHECK_CUDA(launch_pdl(rmsnorm_kernel<256, 4>, dim3(rows), dim3(256), 0, stream, X, R, G, Y, RO, cols, eps));
    else OVB_CHECK_CUDA(launch_pdl(rmsnorm_kernel<256, 8>, dim3(rows), dim3(256), 0, stream, X, R, G, Y, RO, cols, eps));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_layernorm(const void* x, const void* residual, const void* gamma, const void* beta, void* y, int rows,
                  int cols, float eps, int is_f16, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(x && gamma && beta && y && rows > 0, "ovb_layernorm: null operand");
    OVB_REQUIRE(cols % 8 == 0 && cols <= 256 * 8 * 4, "ovb_layernorm: cols=%d must be a multiple of 8 and <= 8192", cols);
    if (is_f16)
        OVB_CHECK_CUDA(launch_pdl(layernorm_kernel<__half, 256, 4>, dim3(rows), dim3(256), 0, stream, (const __half*)x, (const __half*)residual,
                                                                  (const __half*)gamma, (const __half*)beta, (__half*)y,
                                                                  cols, eps));
    else
        OVB_CHECK_CUDA(launch_pdl(layernorm_kernel<__nv_bfloat16, 256, 4>, dim3(rows), dim3(256), 0, stream, 
            (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)gamma,
            (const __nv_bfloat16*)beta, (__nv_bfloat16*)y, cols, eps));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_silu_mul(const void* gu, void* out, int rows, int F, ovb_stream_t stream_) { return ovb_silu_mul_counted(gu, out, rows, F, nullptr, stream_); }

int ovb_silu_mul_counted(const void* gu, void* out, int rows, int F, const int* nrows, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(gu && out && rows > 0 && F % 8 == 0, "ovb_silu_mul: bad arguments");
    const size_t total = (size_t)rows * (F / 8);
    OVB_CHECK_CUDA(launch_pdl(silu_mul_kernel, dim3(grid_for(total, 256)), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, F, nrows));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_moe_route_topk(const float* logits, float* weights, int T, int E, int k, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(logits && weights && T > 0 && E > 0 && E <= 64 && k > 0 && k <= E, "ovb_moe_route_topk: need 1 <= k <= E <= 64");
    OVB_CHECK_CUDA(launch_pdl(moe_route_topk_kernel, dim3((T + 127) / 128), dim3(128), 0, stream, logits, weights, T, E, k));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_moe_silu_mul_scale(const void* gu, const float* weights, void* out, int rows, int F, int nloc, int E, int e0, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(gu && weights && out && rows > 0 && F % 8 == 0 && nloc > 0 && e0 >= 0 && e0 + nloc <= E, "ovb_moe_silu_mul_scale: bad arguments");
    const size_t total = (size_t)rows * nloc * (F / 8);
    OVB_CHECK_CUDA(launch_pdl(moe_silu_mul_scale_kernel, dim3(grid_for(total, 256)), dim3(256), 0, stream, (const __nv_bfloat16*)gu, weights, (__nv_bfloat16*)out, rows, F, nloc, E, e0));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_moe_group(const float* route, int T, int E, int e0, int nloc, int* idx, int idx_stride, int* counts, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(route && idx && counts && T > 0 && nloc > 0 && e0 >= 0 && e0 + nloc <= E && idx_stride >= T, "ovb_moe_group: bad arguments");
    OVB_CHECK_CUDA(launch_pdl(moe_group_kernel, dim3(nloc), dim3(1024), 0, stream, route, T, E, e0, idx, counts, idx_stride));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_moe_positions(const float* route, int T, int E, int e0, int nloc, int* pos, int* counts, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(route && pos && counts && T > 0 && nloc > 0 && nloc <= 64 && e0 >= 0 && e0 + nloc <= E, "ovb_moe_positions: bad arguments");
    OVB_CHECK_CUDA(launch_pdl(moe_positions_kernel, dim3(nloc), dim3(1024), 0, stream, route, T, E, e0, nloc, pos, counts));
    return 0;
}

int ovb_moe_gather_sorted(const void* x, const int* pos, const int* counts, int* offsets, void* xg, int T, int H, int nloc, int cap, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(x && pos && counts && offsets && xg && T > 0 && H % 8 == 0 && nloc > 0 && nloc <= 64 && cap > 0, "ovb_moe_gather_sorted: bad arguments");
    OVB_CHECK_CUDA(launch_pdl(moe_gather_sorted_kernel, dim3(T), dim3(256), 0, stream, (const __nv_bfloat16*)x, pos, counts, offsets, (__nv_bfloat16*)xg, T, H, nloc, cap));
    return 0;
}

int ovb_moe_combine_sorted(const void* y, const float* route, const int* pos, const int* offsets, void* dst, int T, int H, int E, int e0, int nloc,
                           int ld_dst, int accumulate, int cap, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(y && route && pos && offsets && dst && T > 0 && H % 8 == 0 && ld_dst % 8 == 0 && nloc > 0 && nloc <= 64, "ovb_moe_combine_sorted: bad arguments");
    OVB_CHECK_CUDA(launch_pdl(moe_combine_sorted_kernel, dim3(T), dim3(256), 0, stream, (const __nv_bfloat16*)y, route, pos, offsets, (__nv_bfloat16*)dst, T, H, E, e0,
                              nloc, ld_dst, accumulate, cap));
    return 0;
}

int ovb_moe_silu_mul_rows(const void* gu, const float* route, const int* idx, void* out, int rows, int F, int E, int e, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(gu && route && idx && out && rows > 0 && F % 8 == 0 && e >= 0 && e < E, "ovb_moe_silu_mul_rows: bad arguments");
    OVB_CHECK_CUDA(launch_pdl(moe_silu_mul_rows_kernel, dim3(grid_for((size_t)rows * (F / 8), 256)), dim3(256), 0, stream, (const __nv_bfloat16*)gu, route, idx, (__nv_bfloat16*)out,
                                                                                      rows, F, E, e));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_moe_scatter_add(const void* src, const int* idx, void* dst, int rows, int H, int ld_dst, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(src && idx && dst && rows > 0 && H % 8 == 0 && ld_dst % 8 == 0, "ovb_moe_scatter_add: bad arguments");
    OVB_CHECK_CUDA(launch_pdl(moe_scatter_add_kernel, dim3(grid_for((size_t)rows * (H / 8), 256)), dim3(256), 0, stream, (const __nv_bfloat16*)src, idx, (__nv_bfloat16*)dst, rows, H, ld_dst));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_add(const void* a, const void* b, void* out, int64_t n, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(a && b && out && n % 8 == 0, "ovb_add: n must be a multiple of 8");
    OVB_CHECK_CUDA(launch_pdl(add_kernel, dim3(grid_for(n / 8, 256)), dim3(256), 0, stream, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                         (__nv_bfloat16*)out, (size_t)n / 8));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_embedding(const void* ids, int ids_i32, const void* table, void* out, int rows, int cols, int vocab,
                  ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(ids && table && out && rows > 0 && cols % 8 == 0, "ovb_embedding: bad arguments");
    const size_t total = (size_t)rows * (cols / 8);
    if (ids_i32)
        OVB_CHECK_CUDA(launch_pdl(embedding_kernel<int>, dim3(grid_for(total, 256)), dim3(256), 0, stream, (const int*)ids, (const uint4*)table, (uint4*)out,
                                                                        rows, cols / 8, vocab));
    else
        OVB_CHECK_CUDA(launch_pdl(embedding_kernel<int64_t>, dim3(grid_for(total, 256)), dim3(256), 0, stream, (const int64_t*)ids, (const uint4*)table,
                                                                            (uint4*)out, rows, cols / 8, vocab));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_resolve_ids(int* ids, const int* tok_src, const int* last_token, int T, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(ids && tok_src && last_token && T > 0, "ovb_resolve_ids: bad arguments");
    OVB_CHECK_CUDA(launch_pdl(resolve_ids_kernel, dim3((T + 255) / 256), dim3(256), 0, stream, ids, tok_src, last_token, T));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_scatter_tokens(const int* tokens, const int* tok_dst, int* last_token, int B, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(tokens && tok_dst && last_token && B > 0, "ovb_scatter_tokens: bad arguments");
    OVB_CHECK_CUDA(launch_pdl(scatter_tokens_kernel, dim3((B + 255) / 256), dim3(256), 0, stream, tokens, tok_dst, last_token, B));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_argmax(const void* logits, int ld, int rows, int vocab, void* out_ids, int ids_i32, float* out_max,
               ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(logits && out_ids && rows > 0 && vocab > 0, "ovb_argmax: bad arguments");
    OVB_CHECK_CUDA(launch_pdl(argmax_kernel<1024>, dim3(rows), dim3(1024), 0, stream, (const __nv_bfloat16*)logits, ld, vocab, out_ids, ids_i32, out_max));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_rope_kv_write(void* qkv, const int* positions, const int* slot_map, void* k_cache, void* v_cache, int T,
                      int Hq, int Hkv, int D, float theta, int block_size, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(qkv && positions && slot_map && k_cache && v_cache && T > 0, "ovb_rope_kv_write: null operand");
    OVB_REQUIRE(D % 2 == 0, "ovb_rope_kv_write: head size must be even");
    if (D % 4 == 0 && (reinterpret_cast<uintptr_t>(qkv) & 3) == 0 && (reinterpret_cast<uintptr_t>(k_cache) & 3) == 0 &&
        (reinterpret_cast<uintptr_t>(v_cache) & 3) == 0) {
        const int heads = Hq + 2 * Hkv;
        OVB_CHECK_CUDA(launch_pdl(rope_kv_write_vec_kernel, dim3(T, (heads + 3) / 4), dim3(128), 0, stream, (__nv_bfloat16*)qkv, positions, slot_map, (__nv_bfloat16*)k_cache,
                                                                                (__nv_bfloat16*)v_cache, Hq, Hkv, D, log2f(theta), block_size));
    } else {
        OVB_CHECK_CUDA(launch_pdl(rope_kv_write_kernel, dim3(T), dim3(256), 0, stream, (__nv_bfloat16*)qkv, positions, slot_map, (__nv_bfloat16*)k_cache,
                                                    (__nv_bfloat16*)v_cache, Hq, Hkv, D, log2f(theta), block_size));
    }
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_rope_kv_write_u8(void* qkv, const int* positions, const int* slot_map, void* k_cache, void* v_cache, void* k_meta, void* v_meta, int T,
                         int Hq, int Hkv, int D, float theta, int block_size, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(qkv && positions && slot_map && k_cache && v_cache && k_meta && v_meta && T > 0, "ovb_rope_kv_write_u8: null operand");
    OVB_REQUIRE(D == 128, "ovb_rope_kv_write_u8: the u8 cache is served for head size 128");
    OVB_REQUIRE(((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
                  reinterpret_cast<uintptr_t>(k_meta) | reinterpret_cast<uintptr_t>(v_meta)) & 3) == 0, "ovb_rope_kv_write_u8: 4-byte aligned tensors expected");
    const int heads = Hq + 2 * Hkv;
    OVB_CHECK_CUDA(launch_pdl(rope_kv_write_u8_kernel, dim3(T, (heads + 3) / 4), dim3(128), 0, stream, (__nv_bfloat16*)qkv, positions, slot_map, (uint8_t*)k_cache,
                              (uint8_t*)v_cache, (__half2*)k_meta, (__half2*)v_meta, Hq, Hkv, log2f(theta), block_size));
    return 0;
}

int ovb_act_quant_fp8(const void* x, void* q, float* scales, int rows, int cols, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(x && q && scales && rows > 0, "ovb_act_quant_fp8: null operand");
    OVB_REQUIRE(cols % 128 == 0 && (reinterpret_cast<uintptr_t>(x) & 7) == 0 && (reinterpret_cast<uintptr_t>(q) & 3) == 0,
                "ovb_act_quant_fp8: the channel count must be a multiple of 128 and the rows 8-byte aligned");
    const size_t warps = (size_t)rows * (cols / 128);
    OVB_CHECK_CUDA(launch_pdl(act_quant_fp8_kernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), 0, stream, (const __nv_bfloat16*)x, (uint8_t*)q, scales, rows, cols));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_kv_block_copy(void* k_cache, void* v_cache, const int* src_blocks, const int* dst_blocks, int num_pairs, int64_t block_bytes,
                      ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(k_cache && v_cache && src_blocks && dst_blocks, "ovb_kv_block_copy: null operand");
    OVB_REQUIRE(block_bytes > 0 && block_bytes % 16 == 0, "ovb_kv_block_copy: a block must be a multiple of 16 bytes");
    if (num_pairs <= 0) return 0;
    OVB_CHECK_CUDA(launch_pdl(kv_block_copy_kernel, dim3(num_pairs, 2), dim3(256), 0, stream, (uint4*)k_cache, (uint4*)v_cache, src_blocks, dst_blocks, (size_t)block_bytes / 16));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_im2col(const void* x, void* cols, int B, int C, int H, int W, int kh, int kw, int sh, int sw, int pt, int pl, int dh, int dw,
               int Ho, int Wo, int Kpad, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(x && cols && B > 0 && C > 0 && Ho > 0 && Wo > 0, "ovb_im2col: null operand or empty problem");
    OVB_REQUIRE(Kpad % 8 == 0 && Kpad >= C * kh * kw, "ovb_im2col: Kpad must be a multiple of 8 that covers C*kh*kw");
    OVB_REQUIRE((reinterpret_cast<uintptr_t>(cols) & 15) == 0, "ovb_im2col: output must be 16-byte aligned");
    const size_t total = (size_t)B * Ho * Wo * (Kpad / 8);
    OVB_CHECK_CUDA(launch_pdl(im2col_kernel, dim3(grid_for(total, 256)), dim3(256), 0, stream, (const uint16_t*)x, (uint16_t*)cols, B, C, H, W, kh, kw, sh, sw, pt, pl, dh, dw,
                                                            Ho, Wo, C * kh * kw, Kpad));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_pack_w16(const void* w, void* w_out, int N, int K, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(w && w_out && N > 0 && K % 64 == 0, "ovb_pack_w16: K must be a multiple of 64");
    OVB_CHECK_CUDA(cudaMemsetAsync(w_out, 0, (size_t)((N + 127) / 128) * 128 * K * 2, stream));
    const size_t npieces = (size_t)N * K / 8;
    OVB_CHECK_CUDA(launch_serial(pack_w16_kernel, dim3(grid_for(npieces, 256)), dim3(256), 0, stream, (const uint4*)w, (uint4*)w_out, npieces, K));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_pack_u4(const void* w_ir, const void* scales_ir, const void* zps_ir, int zp_is_u8, void* w_out,
                void* scales_out, void* zps_out, int N, int K, int group_size, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(w_ir && scales_ir && w_out && scales_out, "ovb_pack_u4: null operand");
    OVB_REQUIRE(K % 64 == 0 && group_size > 0 && K % group_size == 0, "ovb_pack_u4: K must be a multiple of 64 and of group_size");
    const size_t nwords = (size_t)N * K / 8;
    // w_out holds ceil(N/128)*128 rows; rows beyond N stay zero
    OVB_REQUIRE(group_size % 64 == 0, "ovb_pack_u4: group_size must be a multiple of 64");
    const size_t chunks = (size_t)((N + 127) / 128) * (K / 64);
    OVB_CHECK_CUDA(cudaMemsetAsync(w_out, 0, chunks * 4608, stream));
    OVB_CHECK_CUDA(launch_serial(pack_u4_kernel, dim3(grid_for(nwords, 256)), dim3(256), 0, stream, (const uint32_t*)w_ir, (uint32_t*)w_out, nwords, K));
    OVB_CHECK_CUDA(cudaGetLastError());
    const int G = K / group_size;
    OVB_CHECK_CUDA(launch_serial(pack_scale_zp_kernel, dim3(grid_for((size_t)N * G, 256)), dim3(256), 0, stream, 
        (const __half*)scales_ir, (const uint8_t*)zps_ir, zp_is_u8, (__nv_bfloat16*)scales_out, (__nv_bfloat16*)zps_out,
        N, G, 16.0f, 8.0f));
    OVB_CHECK_CUDA(cudaGetLastError());
    OVB_CHECK_CUDA(launch_serial(embed_pairs_kernel, dim3(grid_for(chunks * 128, 256)), dim3(256), 0, stream, (const uint32_t*)scales_out, (uint32_t*)w_out, N, K / 64,
                                                                        group_size / 64, chunks * 128));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

}  // extern "C"
