// Stochastic sampling: temperature, top-k, top-p (nucleus), multinomial draw. One CTA per row of logits.
//
// The kept set is {v : logit[v] >= t*}: t* is found by bisection on the logit value so that the set has at most top_k
// members and the smallest probability mass >= top_p (the same rule as sorting by probability and cutting, without
// sorting 128k entries). The draw walks the kept entries in index order with a block-wide prefix sum, so a
// (seed, step, row) triple always gives the same token. The role of openvino.genai's sampler
// (multinomial / top-k / top-p transforms over logits), which the reference keeps outside its runtime repository.
#include "common.cuh"
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>

namespace ovb {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ float block_reduce(float v, float* sh, bool is_max) {
    for (int o = 16; o > 0; o >>= 1) {
        const float w = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, w) : v + w;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = lane < (blockDim.x >> 5) ? sh[lane] : (is_max ? -INFINITY : 0.f);
        for (int o = 16; o > 0; o >>= 1) {
            const float w = __shfl_xor_sync(0xffffffffu, v, o);
            v = is_max ? fmaxf(v, w) : v + w;
        }
        if (lane == 0) sh[32] = v;
    }
    __syncthreads();
    return sh[32];
}

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int V, float inv_temp,
                                                                int top_k, float top_p, uint64_t seed, const int* __restrict__ step_ptr,
                                                                int* __restrict__ out_ids) {
    pdl_enter();
    __shared__ float sh[33];
    __shared__ float scan[kSampleThreads];
    const int row = blockIdx.x;
    const __nv_bfloat16* l = logits + (size_t)row * ld;
    const int per = (V + kSampleThreads - 1) / kSampleThreads;          // contiguous chunk per thread (index order matters for the draw)
    const int v0 = threadIdx.x * per, v1 = min(V, v0 + per);
    float mx = -INFINITY, mn = INFINITY;
    for (int v = v0; v < v1; ++v) { const float x = __bfloat162float(l[v]); mx = fmaxf(mx, x); mn = fminf(mn, x); }
    mx = block_reduce(mx, sh, true);
    mn = -block_reduce(-mn, sh, true);
    float z = 0.f;
    for (int v = v0; v < v1; ++v) z += __expf((__bfloat162float(l[v]) - mx) * inv_temp);
    z = block_reduce(z, sh, false);
    // bisection on the threshold: keep(lo) is never smaller than the wanted set, keep(hi) may be
    float lo = mn, hi = mx;
    const bool restrict_k = top_k > 0 && top_k < V, restrict_p = top_p < 1.f;
    if (restrict_k || restrict_p) {
        for (int it = 0; it < 26; ++it) {
            const float mid = 0.5f * (lo + hi);
            float cnt = 0.f, mass = 0.f;
            for (int v = v0; v < v1; ++v) {
                const float x = __bfloat162float(l[v]);
                if (x >= mid) { cnt += 1.f; mass += __expf((x - mx) * inv_temp); }
            }
            cnt = block_reduce(cnt, sh, false);
            mass = block_reduce(mass, sh, false);
            // t* = max(t_k, t_p): the threshold may rise to mid while at least one active rule still holds there
            // (t_k = largest t with count(>= t) >= k, t_p = largest t with mass(>= t) >= p)
            const bool enough = (restrict_p && mass >= top_p * z) || (restrict_k && cnt >= (float)top_k);
            if (enough) lo = mid; else hi = mid;
        }
    }
    const float thr = (restrict_k || restrict_p) ? lo : -INFINITY;
    float local = 0.f;
    for (int v = v0; v < v1; ++v) {
        const float x = __bfloat162float(l[v]);
        if (x >= thr) local += __expf((x - mx) * inv_temp);
    }
    scan[threadIdx.x] = local;
    __syncthreads();
    // inclusive scan over the 1024 per-thread masses (Hillis-Steele)
    for (int o = 1; o < kSampleThreads; o <<= 1) {
        const float add = threadIdx.x >= o ? scan[threadIdx.x - o] : 0.f;
        __syncthreads();
        scan[threadIdx.x] += add;
        __syncthreads();
    }
    const float total = scan[kSampleThreads - 1];
    const uint64_t r64 = mix64(seed ^ mix64(((uint64_t)(step_ptr ? *step_ptr : 0) << 20) ^ (uint64_t)row));
    const float u = (float)((r64 >> 40) + 0.5) * (1.0f / 16777216.0f);      // (0, 1)
    const float target = u * total;
    const float before = threadIdx.x ? scan[threadIdx.x - 1] : 0.f;
    if (target > before && target <= scan[threadIdx.x] && local > 0.f) {
        float acc = before;
        int pick = -1;
        for (int v = v0; v < v1; ++v) {
            const float x = __bfloat162float(l[v]);
            if (x >= thr) {
                acc += __expf((x - mx) * inv_temp);
                pick = v;
                if (acc >= target) break;
            }
        }
        out_ids[row] = pick;
    }
}

__global__ void bump_kernel(int* p) {
    pdl_enter(); *p += 1; }

}  // namespace ovb

extern "C" {
namespace ovb {

// Uniform in the open interval (0, 1) from the top 23 bits of a hash: (k + 0.5) * 2^-23 with k < 2^23 needs 24 significant
// bits, so the fp32 sum is exact and the largest value is 1 - 2^-24 (with 24 bits of k the sum k + 0.5 would round to 2^24
// for k = 2^24 - 1, u would be exactly 1, and the Gumbel noise -log(-log(u)) would be +inf).
__host__ __device__ __forceinline__ float gumbel_uniform(uint64_t h) {
    return ((float)(h >> 41) + 0.5f) * (1.0f / 8388608.0f);
}

// Sampling over vocabulary shards without gathering the logits (Gumbel-max): argmax_i(logit_i / T + G_i) with
// G_i = -log(-log(u_i)) is a draw from softmax(logits / T) when the u_i are independent uniforms. u_i depends on the seed,
// the step word, the row and the GLOBAL token index only, so every tensor-parallel rank perturbs its own shard, reduces
// it to (best value, local index), and the usual arg-max exchange between the ranks picks the token.
__global__ void __launch_bounds__(kSampleThreads) gumbel_argmax_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int V, int vocab_offset,
                                                                       float inv_temp, uint64_t seed, const int* __restrict__ step_ptr,
                                                                       int* __restrict__ out_ids, float* __restrict__ out_max) {
    pdl_enter();
    __shared__ float sv[kSampleThreads / 32];
    __shared__ int si[kSampleThreads / 32];
    const int row = blockIdx.x;
    const __nv_bfloat16* lr = logits + (size_t)row * ld;
    const uint64_t base = mix64(seed ^ mix64(((uint64_t)(step_ptr ? *step_ptr : 0) << 20) ^ (uint64_t)row));
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += kSampleThreads) {
        const uint64_t h = mix64(base ^ ((uint64_t)(uint32_t)(vocab_offset + i) * 0xD1B54A32D192ED03ull));
        const float u = gumbel_uniform(h);
        const float g = -__logf(-__logf(u));
        const float f = __bfloat162float(lr[i]) * inv_temp + g;
        if (f > best) { best = f; bi = i; }
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
        best = lane < kSampleThreads / 32 ? sv[lane] : -INFINITY;
        bi = lane < kSampleThreads / 32 ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (lane == 0) {
            out_ids[row] = bi == 0x7fffffff ? 0 : bi;
            if (out_max) out_max[row] = best;
        }
    }
}

}  // namespace ovb

using namespace ovb;

// out_ids[row] ~ softmax(logits[row] / temperature) restricted to the top_k most likely tokens and to the smallest
// set of probability mass >= top_p. top_k <= 0 and top_p >= 1 switch the restrictions off. `step` (device int, may be
// NULL) is mixed into the random stream, so replays of a captured graph draw fresh numbers when the word is bumped.
int ovb_sample(const void* logits, int ld, int rows, int vocab, float temperature, int top_k, float top_p, uint64_t seed,
               const int* step, int* out_ids, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(logits && out_ids && rows > 0 && vocab > 0 && temperature > 0.f, "ovb_sample: bad arguments (temperature must be > 0)");
    OVB_CHECK_CUDA(launch_pdl(sample_kernel, dim3(rows), dim3(kSampleThreads), 0, stream, (const __nv_bfloat16*)logits, ld, vocab, 1.0f / temperature, top_k,
                                                       top_p <= 0.f ? 1e-6f : top_p, seed, step, out_ids));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_sample_gumbel(const void* logits, int ld, int rows, int vocab, int vocab_offset, float temperature, uint64_t seed, const int* step,
                      int* out_ids, float* out_max, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(logits && out_ids && rows > 0 && vocab > 0 && temperature > 0.f, "ovb_sample_gumbel: bad arguments (temperature must be > 0)");
    OVB_CHECK_CUDA(launch_pdl(gumbel_argmax_kernel, dim3(rows), dim3(kSampleThreads), 0, stream, (const __nv_bfloat16*)logits, ld, vocab, vocab_offset, 1.0f / temperature, seed, step,
                                                              out_ids, out_max));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// Host-side view of the hash -> uniform mapping of the Gumbel sampler (for tests of its range).
float ovb_gumbel_uniform(uint64_t h) { return gumbel_uniform(h); }

int ovb_bump(int* counter, ovb_stream_t stream_) {
    OVB_REQUIRE(counter != nullptr, "ovb_bump: null counter");
    OVB_CHECK_CUDA(launch_pdl(bump_kernel, dim3(1), dim3(1), 0, static_cast<cudaStream_t>(stream_), counter));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

}  // extern "C"
