// Paged attention (ragged prefill / mixed batches and split-KV decode) and dense SDPA.
//
// Semantics follow the PagedAttentionExtension contract
// (docs/articles_en/documentation/openvino-ir-format/operation-sets/operation-specs/internal/paged-attention.rst,
// src/core/reference/include/openvino/reference/paged_attention.hpp): a ragged batch of B
// sub-sequences described by past_lens / subsequence_begins / block_indices(_begins); every new
// token attends causally to the cached tokens of its own sequence (its own K/V row was written to
// the cache before this kernel runs) with optional sliding window; GQA by head grouping.
// The reference implementations are Intel-only (paged_attention_opt.cl, executor_pa.cpp).
//
// Layout: cache [num_blocks, Hkv, block_size, D] so that one (block, head) page is contiguous.
// Math: flash-style online softmax in the exp2 domain, bf16/fp16 tensor-core MMAs with fp32
// accumulation. All the query heads of one KV group are stacked on the M side of the MMA, so K/V
// pages are fetched once per group.
#include <cuda_fp16.h>
#include <math_constants.h>
#include <stdlib.h>

#include <atomic>

#include "attention.cuh"
#include "common.cuh"
#include "debug_bounds.cuh"
#include "sm100_ptx.cuh"

namespace ovb {

OVB_DEBUG_LIMITS_DEFINE

// ------------------------------------------------------------------------------ small PTX helpers
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
    const int sz = valid ? 16 : 0;   // src-size 0 => 16 zero bytes are written
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc, bool valid) {
    const int sz = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
template <bool F16>
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    if (F16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <bool F16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if (F16) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    return pack_bf16x2(lo, hi);
}

// Shared tiles are [rows][D] 16-bit with the 16-byte chunk index XOR-ed with (row & 7): ldmatrix of
// 8 consecutive rows at one chunk column then touches 8 different bank groups.
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return uint32_t(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}


// Address of key/value row `j` of sequence b, kv head h.
template <int D, bool PAGED>
__device__ __forceinline__ const uint8_t* kv_row_ptr(const PaKParams& p, const void* base, int b, int h, int j,
                                                     int blk_begin) {
    if (PAGED) {
        const int blk = OVB_DBG_BLOCK(p.block_indices[blk_begin + j / p.block_size]);
        const int off = j % p.block_size;
        return reinterpret_cast<const uint8_t*>(base) + ((((size_t)blk * p.Hkv + h) * p.block_size + off) * D) * 2;
    }
    return reinterpret_cast<const uint8_t*>(base) + (((size_t)b * p.dense_S + j) * p.ld_kv + (size_t)h * D) * 2;
}

// u8 cache: address of the bytes of key/value row j, and of its (scale, zero point) pair.
template <int D>
__device__ __forceinline__ const uint8_t* kv_row_ptr_u8(const PaKParams& p, const void* base, int h, int j, int blk_begin) {
    const int blk = OVB_DBG_BLOCK(p.block_indices[blk_begin + j / p.block_size]);
    const int off = j % p.block_size;
    return reinterpret_cast<const uint8_t*>(base) + (((size_t)blk * p.Hkv + h) * p.block_size + off) * D;
}
__device__ __forceinline__ const uint8_t* kv_meta_ptr(const PaKParams& p, const void* meta, int h, int j, int blk_begin) {
    const int blk = OVB_DBG_BLOCK(p.block_indices[blk_begin + j / p.block_size]);
    const int off = j % p.block_size;
    return reinterpret_cast<const uint8_t*>(meta) + (((size_t)blk * p.Hkv + h) * p.block_size + off) * 4;
}
// Eight cache bytes -> eight bf16 values (byte - zero point) * scale.
__device__ __forceinline__ uint4 dequant_u8x8(uint2 raw, float scale, float zp) {
    const float nz = -zp * scale;
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t w = i < 2 ? raw.x : raw.y;
        const int sh = (i & 1) * 16;
        o[i] = pack_bf16x2(fmaf((float)((w >> sh) & 0xFFu), scale, nz), fmaf((float)((w >> (sh + 8)) & 0xFFu), scale, nz));
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}
// A staged u8 tile ([rows][D] bytes, then one (scale, zero point) fp16 pair per row) -> the swizzled bf16 tile that the
// ldmatrix reads. `tid` / `nthreads`: the threads that share the work (a warp, or the CTA).
template <int D>
__device__ __forceinline__ void expand_u8_tile(const uint8_t* stage, const uint8_t* meta, uint8_t* tile, int rows, int tid, int nthreads) {
    constexpr int CH = D / 8;
    for (int i = tid; i < rows * CH; i += nthreads) {
        const int r = i / CH, c = i % CH;
        const __half2 sz = *reinterpret_cast<const __half2*>(meta + r * 4);
        const uint2 raw = *reinterpret_cast<const uint2*>(stage + r * D + c * 8);
        *reinterpret_cast<uint4*>(tile + tile_off<D>(r, c)) = dequant_u8x8(raw, __low2float(sz), __high2float(sz));
    }
}

// ------------------------------------------------------------------------------ prefill / mixed
// CTA = 8 warps x 16 rows = 128 stacked rows (row = token_in_tile * G + head_in_group) of one
// (sequence, kv head); K/V tiles of 64 keys double-buffered with cp.async.
// KVU8: the cache holds bytes with a (scale, zero point) pair per row; the tiles are staged as bytes (double-buffered) and
// expanded into one bf16 tile pair before the MMAs.
template <int D, int G, bool PAGED, bool F16, bool KVU8 = false>
__global__ void __launch_bounds__(256, 1) pa_prefill_kernel(PaKParams p) {
    pdl_enter_attn();
    constexpr int BM = 128, BN = 64, TOK = BM / G, CH = D / 8;   // CH = 16-byte chunks per row
    constexpr int U8_STAGE = BN * D + BN * 4;                    // bytes of one staged u8 tile (rows, then the pairs)
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint8_t* sQ = smem;
    uint8_t* sK[2] = {sQ + BM * D * 2, KVU8 ? sQ + BM * D * 2 : sQ + BM * D * 2 + 2 * BN * D * 2};
    uint8_t* sV[2] = {sK[0] + BN * D * 2, sK[1] + BN * D * 2};
    uint8_t* sU = sQ + BM * D * 2 + 2 * BN * D * 2;              // KVU8: [buf][K | V] staged byte tiles
    __shared__ int s_work[4];

    const int h = blockIdx.y;   // kv head
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // ---- find (sequence, q tile) of this CTA: tiles are numbered sequence by sequence
    if (threadIdx.x == 0) {
        int acc = 0, found = -1, tile = 0;
        for (int b = 0; b < p.B; ++b) {
            const int ql = PAGED ? p.subsequence_begins[b + 1] - p.subsequence_begins[b] : p.dense_S;
            const int nt = (ql + TOK - 1) / TOK;
            if ((int)blockIdx.x < acc + nt) { found = b; tile = blockIdx.x - acc; break; }
            acc += nt;
        }
        s_work[0] = found;
        s_work[1] = tile;
    }
    __syncthreads();
    const int b = s_work[0];
    if (b < 0) return;
    const int qtile = s_work[1];
    const int tok_begin = PAGED ? p.subsequence_begins[b] : b * p.dense_S;
    const int q_len = PAGED ? p.subsequence_begins[b + 1] - tok_begin : p.dense_S;
    const int past = PAGED ? p.past_lens[b] : 0;
    const int blk_begin = PAGED ? p.block_indices_begins[b] : 0;
    const int tq0 = qtile * TOK;                         // first query token (within the sub-sequence) of this tile
    const int tq1 = min(q_len, tq0 + TOK);               // one past the last
    const int kv_total = PAGED ? past + q_len : p.dense_S;
    int kv_end = p.causal ? min(kv_total, past + tq1) : kv_total;   // keys this tile may see
    int kv_start = 0;
    if (p.sliding_window > 0) kv_start = max(0, past + tq0 - p.sliding_window + 1);
    kv_start = (kv_start / BN) * BN;
    const int ntiles = (kv_end - kv_start + BN - 1) / BN;

    // ---- Q tile -> smem (rows beyond the sub-sequence are zero-filled)
    for (int i = threadIdx.x; i < BM * CH; i += 256) {
        const int r = i / CH, c = i % CH;
        const int tl = r / G, hg = r % G;
        const bool valid = (tq0 + tl) < q_len;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.q) +
                             ((size_t)(tok_begin + tq0 + (valid ? tl : 0)) * p.ldq + (size_t)(h * G + hg) * D) * 2 + c * 16;
        cp_async16(sQ + tile_off<D>(r, c), src, valid);
    }
    auto load_kv = [&](int tile, int buf) {
        const int j0 = kv_start + tile * BN;
        for (int i = threadIdx.x; i < BN * CH; i += 256) {
            const int r = i / CH, c = i % CH;
            const int j = j0 + r;
            const bool valid = j < kv_end;
            const int jj = valid ? j : 0;
            if (KVU8) {
                // a row is D bytes = CH / 2 chunks of 16; chunk index CH / 2 of a row carries its (scale, zero point) pair
                uint8_t* uk = sU + buf * (2 * U8_STAGE);
                uint8_t* uv = uk + U8_STAGE;
                if (c < CH / 2) {
                    cp_async16(uk + r * D + c * 16, kv_row_ptr_u8<D>(p, p.k_cache, h, jj, blk_begin) + c * 16, valid);
                    cp_async16(uv + r * D + c * 16, kv_row_ptr_u8<D>(p, p.v_cache, h, jj, blk_begin) + c * 16, valid);
                } else if (c == CH / 2) {
                    cp_async4(uk + BN * D + r * 4, kv_meta_ptr(p, p.k_meta, h, jj, blk_begin), valid);
                    cp_async4(uv + BN * D + r * 4, kv_meta_ptr(p, p.v_meta, h, jj, blk_begin), valid);
                }
                continue;
            }
            cp_async16(sK[buf] + tile_off<D>(r, c), kv_row_ptr<D, PAGED>(p, p.k_cache, b, h, jj, blk_begin) + c * 16, valid);
            cp_async16(sV[buf] + tile_off<D>(r, c), kv_row_ptr<D, PAGED>(p, p.v_cache, b, h, jj, blk_begin) + c * 16, valid);
        }
    };
    if (ntiles > 0) load_kv(0, 0);
    cp_async_commit();

    // ---- per-thread state
    float o_acc[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};
    const int row0 = warp * 16 + (lane >> 2);           // this thread's two rows: row0, row0 + 8
    int qpos[2];                                        // absolute position of the query of each row
#pragma unroll
    for (int i = 0; i < 2; ++i) qpos[i] = past + tq0 + (row0 + 8 * i) / G;

    uint32_t qf[D / 16][4];
    for (int t = 0; t < ntiles; ++t) {
        const int buf = t & 1;
        if (t + 1 < ntiles) load_kv(t + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (KVU8) {
            // (the barrier at the end of the previous iteration released the bf16 tiles)
            const uint8_t* uk = sU + buf * (2 * U8_STAGE);
            expand_u8_tile<D>(uk, uk + BN * D, sK[0], BN, threadIdx.x, 256);
            expand_u8_tile<D>(uk + U8_STAGE, uk + U8_STAGE + BN * D, sV[0], BN, threadIdx.x, 256);
            __syncthreads();
        }
        if (t == 0) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const int r = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
                const int c = ks * 2 + (lane >> 4);
                ldsm_x4(smem_u32(sQ + tile_off<D>(r, c)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
            }
        }
        // S = Q K^T : 16 x 64 per warp
        float s[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
            for (int nt = 0; nt < BN / 8; nt += 2) {
                uint32_t b0, b1, b2, b3;
                const int m = lane >> 3;
                const int kr = nt * 8 + (m >> 1) * 8 + (lane & 7);
                const int kc = ks * 2 + (m & 1);
                ldsm_x4(smem_u32(sK[buf] + tile_off<D>(kr, kc)), b0, b1, b2, b3);
                mma16816<F16>(s[nt], qf[ks], b0, b1);
                mma16816<F16>(s[nt + 1], qf[ks], b2, b3);
            }
        }
        // mask + online softmax
        const int j0 = kv_start + t * BN;
        float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                const int ri = e >> 1;
                bool ok = j < kv_end;
                if (p.causal) ok = ok && (j <= qpos[ri]);
                if (p.sliding_window > 0) ok = ok && (j > qpos[ri] - p.sliding_window);
                const float v = ok ? s[nt][e] * p.scale_log2 : -CUDART_INF_F;
                s[nt][e] = v;
                mx[ri] = fmaxf(mx[ri], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int ri = 0; ri < 2; ++ri) {
            mx[ri] = fmaxf(mx[ri], __shfl_xor_sync(0xffffffffu, mx[ri], 1));
            mx[ri] = fmaxf(mx[ri], __shfl_xor_sync(0xffffffffu, mx[ri], 2));
            const float mnew = mx[ri];
            corr[ri] = (mnew == -CUDART_INF_F) ? 1.f : exp2f(m_run[ri] - mnew);
            m_run[ri] = mnew;
            l_run[ri] *= corr[ri];
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            o_acc[i][0] *= corr[0]; o_acc[i][1] *= corr[0];
            o_acc[i][2] *= corr[1]; o_acc[i][3] *= corr[1];
        }
        uint32_t pf[BN / 16][4];
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
            float e[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int ri = k >> 1;
                e[k] = (m_run[ri] == -CUDART_INF_F) ? 0.f : exp2f(s[nt][k] - m_run[ri]);
                l_run[ri] += e[k];
            }
            pf[nt >> 1][(nt & 1) * 2 + 0] = pack2<F16>(e[0], e[1]);
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack2<F16>(e[2], e[3]);
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
            for (int dn = 0; dn < D / 8; dn += 2) {
                uint32_t b0, b1, b2, b3;
                const int m = lane >> 3;
                const int vr = kk * 16 + (m & 1) * 8 + (lane & 7);
                const int vc = dn + (m >> 1);
                ldsm_x4_t(smem_u32(sV[buf] + tile_off<D>(vr, vc)), b0, b1, b2, b3);
                mma16816<F16>(o_acc[dn], pf[kk], b0, b1);
                mma16816<F16>(o_acc[dn + 1], pf[kk], b2, b3);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    // ---- normalise and store
#pragma unroll
    for (int ri = 0; ri < 2; ++ri) {
        float l = l_run[ri];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        l_run[ri] = l > 0.f ? 1.f / l : 0.f;
    }
#pragma unroll
    for (int ri = 0; ri < 2; ++ri) {
        const int r = row0 + 8 * ri;
        const int tl = r / G, hg = r % G;
        if (tq0 + tl < q_len) {
            uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) +
                           ((size_t)(tok_begin + tq0 + tl) * p.Hq * D + (size_t)(h * G + hg) * D) * 2;
#pragma unroll
            for (int dn = 0; dn < D / 8; ++dn) {
                const int d = dn * 8 + (lane & 3) * 2;
                *reinterpret_cast<uint32_t*>(dst + d * 2) =
                    pack2<F16>(o_acc[dn][ri * 2] * l_run[ri], o_acc[dn][ri * 2 + 1] * l_run[ri]);
            }
        }
    }
}

// ------------------------------------------------------------------------------ decode (q_len == 1)
// CTA = 4 warps for one (sequence, kv head, kv split). Each warp walks pages w, w+4, ... of the
// split with its own double-buffered page stage (no CTA-wide barriers in the loop), keeping
// online-softmax state for the G query heads (padded to the 16-row MMA tile); the 4 warps merge
// through shared memory. With nsplit > 1 the partial (m, l, O) goes to scratch and
// pa_decode_combine_kernel finishes.
// KVU8: the cache holds bytes with a (scale, zero point) pair per row (half the traffic of a 16-bit cache): a page is staged
// as bytes and the warp expands it into its one bf16 page pair right before the MMAs.
template <int D, int G, int PAGE, bool KVU8 = false>
__global__ void __launch_bounds__(128) pa_decode_kernel(PaKParams p) {
    pdl_enter_attn();
    constexpr int CH = D / 8;
    constexpr int NST = 3;   // page stages per warp
    constexpr int U8_PAGE = PAGE * D + PAGE * 4;                       // bytes of one staged u8 page (rows, then the pairs)
    constexpr int STAGE = KVU8 ? 2 * U8_PAGE : 2 * PAGE * D * 2;       // K and V of one stage
    constexpr int WARP_BYTES = NST * STAGE + (KVU8 ? 2 * PAGE * D * 2 : 0);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    uint8_t* sQ = smem;                                   // 16 x D
    uint8_t* sKV = smem + 16 * D * 2 + warp * WARP_BYTES;
    uint8_t* sExp = sKV + NST * STAGE;                    // KVU8: the warp's expanded bf16 K and V pages
    float* sMerge = reinterpret_cast<float*>(smem + 16 * D * 2 + 4 * WARP_BYTES);   // [4][G][D+2]

    const int tok = p.subsequence_begins[b];
    const int ctx = p.past_lens[b] + 1;
    const int blk_begin = p.block_indices_begins[b];
    int k_lo = split * p.keys_per_split;
    int k_hi = min(ctx, k_lo + p.keys_per_split);
    if (p.sliding_window > 0) k_lo = max(k_lo, ((ctx - p.sliding_window) / PAGE) * PAGE);
    const int page_lo = k_lo / PAGE;
    const int page_hi = (k_hi + PAGE - 1) / PAGE;         // exclusive
    const int win_lo = p.sliding_window > 0 ? ctx - p.sliding_window : 0;

    // Q: G real rows, the rest zero
    for (int i = threadIdx.x; i < 16 * CH; i += 128) {
        const int r = i / CH, c = i % CH;
        const bool valid = r < G;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.q) + ((size_t)tok * p.ldq + (size_t)(h * G + (valid ? r : 0)) * D) * 2 + c * 16;
        cp_async16(sQ + tile_off<D>(r, c), src, valid);
    }
    cp_async_commit();

    auto load_page = [&](int page, int st) {
        const bool pv = page < page_hi;
        const int blk = pv ? OVB_DBG_BLOCK(p.block_indices[blk_begin + page]) : 0;
        if (KVU8) {
            // the page's bytes are contiguous (PAGE * D), so are its pairs (PAGE * 4)
            const size_t pg = (size_t)blk * p.Hkv + h;
            const uint8_t* kb = reinterpret_cast<const uint8_t*>(p.k_cache) + pg * PAGE * D;
            const uint8_t* vb = reinterpret_cast<const uint8_t*>(p.v_cache) + pg * PAGE * D;
            uint8_t* dk = sKV + st * STAGE;
            uint8_t* dv = dk + U8_PAGE;
            for (int i = lane; i < PAGE * D / 16; i += 32) {
                cp_async16(dk + i * 16, kb + i * 16, pv);
                cp_async16(dv + i * 16, vb + i * 16, pv);
            }
            if (lane < PAGE * 4 / 16) {
                cp_async16(dk + PAGE * D + lane * 16, reinterpret_cast<const uint8_t*>(p.k_meta) + pg * PAGE * 4 + lane * 16, pv);
                cp_async16(dv + PAGE * D + lane * 16, reinterpret_cast<const uint8_t*>(p.v_meta) + pg * PAGE * 4 + lane * 16, pv);
            }
            return;
        }
        const uint8_t* kb = reinterpret_cast<const uint8_t*>(p.k_cache) + (((size_t)blk * p.Hkv + h) * PAGE * D) * 2;
        const uint8_t* vb = reinterpret_cast<const uint8_t*>(p.v_cache) + (((size_t)blk * p.Hkv + h) * PAGE * D) * 2;
        uint8_t* dk = sKV + st * (2 * PAGE * D * 2);
        uint8_t* dv = dk + PAGE * D * 2;
        for (int i = lane; i < PAGE * CH; i += 32) {
            const int r = i / CH, c = i % CH;
            cp_async16(dk + tile_off<D>(r, c), kb + (size_t)r * D * 2 + c * 16, pv);
            cp_async16(dv + tile_off<D>(r, c), vb + (size_t)r * D * 2 + c * 16, pv);
        }
    };
    // prologue: NST-1 pages in flight
    int page = page_lo + warp;
#pragma unroll
    for (int s = 0; s < NST - 1; ++s) {
        load_page(page + s * 4, s);
        cp_async_commit();
    }
    cp_async_wait<NST - 1>();   // Q landed (oldest group)
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        const int r = (lane & 7) + 8 * ((lane >> 3) & 1);
        const int c = ks * 2 + (lane >> 4);
        ldsm_x4(smem_u32(sQ + tile_off<D>(r, c)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }

    float o_acc[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
    float m_run = -CUDART_INF_F, l_run = 0.f;   // rows >= 8 are padding: only row (lane>>2) state is kept

    int st = 0;
    for (; page < page_hi; page += 4) {
        load_page(page + (NST - 1) * 4, (st + NST - 1) % NST);
        cp_async_commit();
        cp_async_wait<NST - 1>();
        __syncwarp();
        const uint8_t* kS = sKV + st * (2 * PAGE * D * 2);
        const uint8_t* vS = kS + PAGE * D * 2;
        if (KVU8) {
            const uint8_t* uk = sKV + st * STAGE;
            expand_u8_tile<D>(uk, uk + PAGE * D, sExp, PAGE, lane, 32);
            expand_u8_tile<D>(uk + U8_PAGE, uk + U8_PAGE + PAGE * D, sExp + PAGE * D * 2, PAGE, lane, 32);
            __syncwarp();
            kS = sExp;
            vS = sExp + PAGE * D * 2;
        }
        float s[PAGE / 8][4];
#pragma unroll
        for (int i = 0; i < PAGE / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
            for (int nt = 0; nt < PAGE / 8; nt += 2) {
                uint32_t b0, b1, b2, b3;
                const int m = lane >> 3;
                const int kr = nt * 8 + (m >> 1) * 8 + (lane & 7);
                const int kc = ks * 2 + (m & 1);
                ldsm_x4(smem_u32(kS + tile_off<D>(kr, kc)), b0, b1, b2, b3);
                mma16816<false>(s[nt], qf[ks], b0, b1);
                mma16816<false>(s[nt + 1], qf[ks], b2, b3);
            }
        }
        const int j0 = page * PAGE;
        float mx = m_run;
#pragma unroll
        for (int nt = 0; nt < PAGE / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = j0 + nt * 8 + (lane & 3) * 2 + e;
                const bool ok = (j < k_hi) && (j >= k_lo) && (j >= win_lo);
                const float v = ok ? s[nt][e] * p.scale_log2 : -CUDART_INF_F;
                s[nt][e] = v;
                mx = fmaxf(mx, v);
            }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float corr = (mx == -CUDART_INF_F) ? 1.f : exp2f(m_run - mx);
        m_run = mx;
        l_run *= corr;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o_acc[i][0] *= corr; o_acc[i][1] *= corr; }
        uint32_t pf[PAGE / 16][4];
#pragma unroll
        for (int nt = 0; nt < PAGE / 8; ++nt) {
            const float e0 = (m_run == -CUDART_INF_F) ? 0.f : exp2f(s[nt][0] - m_run);
            const float e1 = (m_run == -CUDART_INF_F) ? 0.f : exp2f(s[nt][1] - m_run);
            l_run += e0 + e1;
            pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16x2(e0, e1);
            pf[nt >> 1][(nt & 1) * 2 + 1] = 0u;   // rows 8..15 are padding
        }
#pragma unroll
        for (int kk = 0; kk < PAGE / 16; ++kk) {
#pragma unroll
            for (int dn = 0; dn < D / 8; dn += 2) {
                uint32_t b0, b1, b2, b3;
                const int m = lane >> 3;
                const int vr = kk * 16 + (m & 1) * 8 + (lane & 7);
                const int vc = dn + (m >> 1);
                ldsm_x4_t(smem_u32(vS + tile_off<D>(vr, vc)), b0, b1, b2, b3);
                mma16816<false>(o_acc[dn], pf[kk], b0, b1);
                mma16816<false>(o_acc[dn + 1], pf[kk], b2, b3);
            }
        }
        __syncwarp();
        st = (st + 1) % NST;
    }
    cp_async_wait<0>();

    // ---- merge the 4 warps (rows 0..G-1 only)
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    const int r = lane >> 2;
    if (r < G) {
        float* dst = sMerge + ((size_t)warp * G + r) * (D + 2);
#pragma unroll
        for (int dn = 0; dn < D / 8; ++dn) {
            const int d = dn * 8 + (lane & 3) * 2;
            dst[d] = o_acc[dn][0];
            dst[d + 1] = o_acc[dn][1];
        }
        if ((lane & 3) == 0) { dst[D] = m_run; dst[D + 1] = l_run; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * D; i += 128) {
        const int rr = i / D, d = i % D;
        float m = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, sMerge[((size_t)w * G + rr) * (D + 2) + D]);
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* src = sMerge + ((size_t)w * G + rr) * (D + 2);
            const float sc = (src[D] == -CUDART_INF_F) ? 0.f : exp2f(src[D] - m);
            l += src[D + 1] * sc;
            o += src[d] * sc;
        }
        const int hq = h * G + rr;
        if (p.nsplit == 1) {
            reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)tok * p.Hq * D + (size_t)hq * D + d] =
                __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
        } else {
            float* sc = p.scratch + (((size_t)b * p.Hq + hq) * p.nsplit + split) * (D + 2);
            sc[d] = o;
            if (d == 0) { sc[D] = m; sc[D + 1] = l; }
        }
    }
}

template <int D>
__global__ void pa_decode_combine_kernel(PaKParams p) {
    pdl_enter_attn();
    const int b = blockIdx.x, hq = blockIdx.y;
    const int tok = p.subsequence_begins[b];
    const float* base = p.scratch + (((size_t)b * p.Hq + hq) * p.nsplit) * (D + 2);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float m = -CUDART_INF_F;
        for (int s = 0; s < p.nsplit; ++s) m = fmaxf(m, base[(size_t)s * (D + 2) + D]);
        float l = 0.f, o = 0.f;
        for (int s = 0; s < p.nsplit; ++s) {
            const float* src = base + (size_t)s * (D + 2);
            const float sc = (src[D] == -CUDART_INF_F) ? 0.f : exp2f(src[D] - m);
            l += src[D + 1] * sc;
            o += src[d] * sc;
        }
        reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)tok * p.Hq * D + (size_t)hq * D + d] =
            __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
}

// ------------------------------------------------------------------------------ host side
// Opt a kernel variant in to `smem` bytes of dynamic shared memory, once per device (bit `device` of `configured`).
static int set_smem_once(std::atomic<uint64_t>& configured, const void* kern, int smem) {
    int dev = 0;
    OVB_CHECK_CUDA(cudaGetDevice(&dev));
    const uint64_t bit = 1ull << (dev & 63);
    if (configured.load(std::memory_order_acquire) & bit) return 0;
    OVB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured.fetch_or(bit, std::memory_order_release);
    return 0;
}

template <int D, int G, bool PAGED, bool F16, bool KVU8 = false>
static int launch_prefill(const PaKParams& p, int num_q_tiles, cudaStream_t stream) {
    const int smem = KVU8 ? 128 * D * 2 + 2 * 64 * D * 2 + 4 * (64 * D + 64 * 4) + 128 : 128 * D * 2 + 4 * 64 * D * 2 + 128;
    auto kern = pa_prefill_kernel<D, G, PAGED, F16, KVU8>;
    static std::atomic<uint64_t> configured{0};   // one bit per device: the attribute is set on first use only
    if (int rc = set_smem_once(configured, reinterpret_cast<const void*>(kern), smem)) return rc;
    dim3 grid(num_q_tiles, p.Hkv);
    OVB_CHECK_CUDA(launch_pdl(kern, dim3(grid), dim3(256), smem, stream, p));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

template <int D, int G, bool KVU8 = false>
static int launch_decode(const PaKParams& p, cudaStream_t stream) {
    constexpr int PAGE = 16;
    const int warp_bytes = KVU8 ? 3 * 2 * (PAGE * D + PAGE * 4) + 2 * PAGE * D * 2 : 3 * 2 * PAGE * D * 2;
    const int smem = 16 * D * 2 + 4 * warp_bytes + 4 * G * (D + 2) * 4 + 128;
    auto kern = pa_decode_kernel<D, G, PAGE, KVU8>;
    static std::atomic<uint64_t> configured{0};
    if (int rc = set_smem_once(configured, reinterpret_cast<const void*>(kern), smem)) return rc;
    dim3 grid(p.B, p.Hkv, p.nsplit);
    OVB_CHECK_CUDA(launch_pdl(kern, dim3(grid), dim3(128), smem, stream, p));
    OVB_CHECK_CUDA(cudaGetLastError());
    if (p.nsplit > 1) {
        OVB_CHECK_CUDA(launch_pdl(pa_decode_combine_kernel<D>, dim3(p.B, p.Hq), dim3(128), 0, stream, p));
        OVB_CHECK_CUDA(cudaGetLastError());
    }
    return 0;
}

// OVB_ATTN_TC=0 in the environment keeps prefill and dense attention on the mma.sync kernel (for comparisons).
static bool use_tc_attention() {
    static const bool on = [] {
        const char* e = getenv("OVB_ATTN_TC");
        return !(e != nullptr && e[0] == '0');
    }();
    return on;
}

static int decode_nsplit(int B, int Hkv, int max_ctx) {
    static const int forced = [] { const char* e = getenv("OVB_PA_NSPLIT"); return e ? atoi(e) : 0; }();   // measurements only
    if (forced > 0) return forced > 32 ? 32 : forced;
    // enough CTAs to fill the machine a few times over, at least 256 keys per split
    int by_len = (max_ctx + 255) / 256;
    int want = (148 * 6 + B * Hkv - 1) / (B * Hkv);
    int n = by_len < want ? by_len : want;
    if (n < 1) n = 1;
    if (n > 32) n = 32;
    return n;
}

}  // namespace ovb

#ifdef OVB_DEBUG_BOUNDS
extern "C" int ovb_debug_set_limits_attention(const ovb::DebugLimits* l) {
    OVB_CHECK_CUDA(cudaMemcpyToSymbol(ovb::g_dbg_limits, l, sizeof(*l)));
    return 0;
}
#endif

extern "C" {
using namespace ovb;

int64_t ovb_pa_scratch_bytes(int B, int Hq, int D, int max_context_len) {
    (void)max_context_len;
    return (int64_t)B * Hq * 32 * (D + 2) * (int64_t)sizeof(float);
}

int ovb_paged_attention(const ovb_pa_args* a, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(a && a->q && a->out && a->k_cache && a->v_cache, "ovb_paged_attention: null operand");
    OVB_REQUIRE(a->past_lens && a->subsequence_begins && a->block_indices && a->block_indices_begins,
                "ovb_paged_attention: null batch descriptor");
    OVB_REQUIRE(a->B > 0 && a->T > 0 && a->Hkv > 0 && a->Hq % a->Hkv == 0, "ovb_paged_attention: bad head counts");
    OVB_REQUIRE(a->ldq % 8 == 0, "ovb_paged_attention: q row pitch must be a multiple of 8 elements");
    const int G = a->Hq / a->Hkv;
    PaKParams p;
    memset(&p, 0, sizeof(p));
    p.q = a->q; p.out = a->out; p.k_cache = a->k_cache; p.v_cache = a->v_cache;
    p.past_lens = a->past_lens; p.subsequence_begins = a->subsequence_begins;
    p.block_indices = a->block_indices; p.block_indices_begins = a->block_indices_begins;
    p.scratch = a->scratch;
    p.B = a->B; p.T = a->T; p.Hq = a->Hq; p.Hkv = a->Hkv;
    p.ldq = a->ldq; p.block_size = a->block_size; p.sliding_window = a->sliding_window;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.causal = 1;
    p.nsplit = 1;
    p.kv_u8 = a->kv_u8;
    p.k_meta = a->k_meta;
    p.v_meta = a->v_meta;
    if (a->kv_u8) {
        OVB_REQUIRE(a->k_meta && a->v_meta, "ovb_paged_attention: the u8 cache needs its (scale, zero point) tables");
        OVB_REQUIRE(a->D == 128 && a->block_size == 16 && (G == 1 || G == 2 || G == 4 || G == 8),
                    "ovb_paged_attention: the u8 cache is served for head size 128, 16-token blocks and 1, 2, 4 or 8 query heads per KV head");
    }

    if (a->max_q_len == 1 && a->D == 128 && a->block_size == 16 && (G == 1 || G == 2 || G == 4 || G == 8)) {
        OVB_REQUIRE(a->T == a->B, "ovb_paged_attention: decode batch needs one token per sequence");
        int ns = decode_nsplit(a->B, a->Hkv, a->max_context_len);
        if (!a->scratch) ns = 1;
        p.nsplit = ns;
        int kps = (a->max_context_len + ns - 1) / ns;
        p.keys_per_split = ((kps + 63) / 64) * 64;   // whole pages, and page index % 4 == warp stays aligned
        if (a->kv_u8) {
            switch (G) {
                case 1: return launch_decode<128, 1, true>(p, stream);
                case 2: return launch_decode<128, 2, true>(p, stream);
                case 4: return launch_decode<128, 4, true>(p, stream);
                case 8: return launch_decode<128, 8, true>(p, stream);
            }
        }
        switch (G) {
            case 1: return launch_decode<128, 1>(p, stream);
            case 2: return launch_decode<128, 2>(p, stream);
            case 4: return launch_decode<128, 4>(p, stream);
            case 8: return launch_decode<128, 8>(p, stream);
        }
    }
    // ragged prefill / mixed: tiles of 128/G tokens per (sequence, kv head)
    const int tok_per_tile = 128 / G;
    const int num_q_tiles = a->T / tok_per_tile + a->B;   // upper bound of sum_b ceil(q_len_b / tok_per_tile)
    if (a->kv_u8) {      // byte pages are expanded in shared memory: the mma.sync kernel (the tcgen05 kernel reads 16-bit pages by TMA)
        switch (G) {
            case 1: return launch_prefill<128, 1, true, false, true>(p, num_q_tiles, stream);
            case 2: return launch_prefill<128, 2, true, false, true>(p, num_q_tiles, stream);
            case 4: return launch_prefill<128, 4, true, false, true>(p, num_q_tiles, stream);
            case 8: return launch_prefill<128, 8, true, false, true>(p, num_q_tiles, stream);
        }
    }
    // the tcgen05 kernel serves the common shapes; everything else (and OVB_ATTN_TC=0) runs on the mma.sync kernel below
    if (use_tc_attention() && (G == 1 || G == 2 || G == 4 || G == 8)) {
        const int rc = launch_prefill_tc(p, a->D, G, /*paged=*/true, /*f16=*/false, num_q_tiles, stream);
        if (rc != ERR_UNSUPPORTED) return rc;
    }
    if (a->D == 128) {
        switch (G) {
            case 1: return launch_prefill<128, 1, true, false>(p, num_q_tiles, stream);
            case 2: return launch_prefill<128, 2, true, false>(p, num_q_tiles, stream);
            case 4: return launch_prefill<128, 4, true, false>(p, num_q_tiles, stream);
            case 8: return launch_prefill<128, 8, true, false>(p, num_q_tiles, stream);
        }
    } else if (a->D == 64) {
        switch (G) {
            case 1: return launch_prefill<64, 1, true, false>(p, num_q_tiles, stream);
            case 4: return launch_prefill<64, 4, true, false>(p, num_q_tiles, stream);
        }
    }
    set_error("ovb_paged_attention: unsupported head size %d / group %d", a->D, G);
    return ERR_UNSUPPORTED;
}

int ovb_sdpa_dense(const void* q, const void* k, const void* v, void* out, int B, int S, int H, int D, int ld,
                   float scale, int is_f16, int causal, ovb_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(q && k && v && out && B > 0 && S > 0 && H > 0, "ovb_sdpa_dense: bad arguments");
    OVB_REQUIRE(ld % 8 == 0, "ovb_sdpa_dense: row pitch must be a multiple of 8 elements");
    PaKParams p;
    memset(&p, 0, sizeof(p));
    p.q = q; p.out = out; p.k_cache = k; p.v_cache = v;
    p.B = B; p.T = B * S; p.Hq = H; p.Hkv = H;
    p.ldq = ld; p.ld_kv = ld; p.dense_S = S; p.causal = causal;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.nsplit = 1;
    const int num_q_tiles = B * ((S + 127) / 128);
    if (use_tc_attention()) {
        const int rc = launch_prefill_tc(p, D, 1, /*paged=*/false, is_f16 != 0, num_q_tiles, stream);
        if (rc != ERR_UNSUPPORTED) return rc;
    }
    if (D == 64) return is_f16 ? launch_prefill<64, 1, false, true>(p, num_q_tiles, stream)
                               : launch_prefill<64, 1, false, false>(p, num_q_tiles, stream);
    if (D == 128) return is_f16 ? launch_prefill<128, 1, false, true>(p, num_q_tiles, stream)
                                : launch_prefill<128, 1, false, false>(p, num_q_tiles, stream);
    set_error("ovb_sdpa_dense: unsupported head size %d", D);
    return ERR_UNSUPPORTED;
}

}  // extern "C"
