// Flash attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA): ragged paged prefill / mixed batches and
// dense (encoder) attention. Same semantics and parameters as pa_prefill_kernel in attention.cu, which stays as the
// fallback for shapes this kernel does not serve.
//
// Roles of the reference kernels this fills: src/plugins/intel_gpu/src/graph/impls/ocl_v2/sdpa_micro.cl:141 (prefill
// SDPA), paged_attention_opt.cl:64 (paged prefill), src/plugins/intel_cpu/src/nodes/kernels/scaled_attn/executor_pa.cpp:1470.
//
// One CTA owns 128 stacked query rows of one (sequence, KV head): row r = g * TOK + t is query head g of the group and the
// t-th token of the tile (TOK = 128 / G tokens), so that K/V pages are fetched once for the G heads that share them.
//
//   warp 4 (one lane)  : TMA. Q tile once (G boxes per 64-column half), then per 128-key tile the K and V pages of the
//                        sequence's block table, 16 keys x 64 columns per box, 128-byte swizzle, two stages.
//   warp 5 (elected)   : tcgen05.mma.  S[j] = Q K_j^T (both operands in shared memory, accumulator S in tensor memory,
//                        double buffered), then O += P_j V_j with P_j read from tensor memory (.ts form) and V_j as an
//                        MN-major shared-memory operand (V rows are keys, i.e. the reduction dimension). QK of tile j + 1
//                        is issued before PV of tile j, so the tensor core works on it while the softmax of tile j runs.
//   warps 0-3          : softmax, one thread per query row (no shuffles): tcgen05.ld of the row of S, masks, running
//                        maximum and sum in the exp2 domain, P as 16-bit pairs back into tensor memory (tcgen05.st).
//                        The running maximum is only raised when the tile's maximum exceeds it by more than 8 (a factor
//                        of 256): the accumulator O, which lives in tensor memory, then has to be rescaled only a few
//                        times per row instead of once per tile. Epilogue: O / l -> 16-bit -> global.
//
// Tensor memory (512 columns): S0 0..127, S1 128..255, O 256..256+D-1, P0 and P1 (64 columns each) behind it.
// Every wait is bounded (mbar_wait) and reports through the status word.
#include <math_constants.h>

#include <atomic>

#include "attention.cuh"
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ovb {

namespace {

constexpr int kBM = 128;   // stacked query rows per CTA
constexpr int kBK = 128;   // keys per tile
constexpr int kPage = 16;  // keys per TMA box (= the cache block size)

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// MN-major shared-memory operand with the 128-byte swizzle: 64 elements (128 bytes) of the MN dimension are contiguous, rows
// of the reduction dimension are 128 bytes apart, 8-row groups `sbo` bytes apart, 64-element MN blocks `lbo` bytes apart.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

template <bool F16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
    if (F16) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    return pack_bf16x2(lo, hi);
}

template <int D, int G, bool PAGED, bool F16>
__global__ void __launch_bounds__(192, 1)
pa_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     PaKParams p, int* status) {
    constexpr int TOK = kBM / G;               // tokens per tile
    constexpr int HALVES = D / 64;             // 64-column (128-byte) halves of a row
    constexpr int Q_BYTES = kBM * D * 2, KV_BYTES = kBK * D * 2;
    constexpr uint32_t TM_S = 0, TM_O = 256, TM_P = 256 + D;   // tensor-memory columns
    constexpr uint32_t IDESC_QK = umma_idesc_f16(kBM, kBK, !F16);
    constexpr uint32_t IDESC_PV = umma_idesc_f16(kBM, D, !F16) | (1u << 16);   // B operand MN-major

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + Q_BYTES;                // two stages
    uint8_t* sV = sK + 2 * KV_BYTES;           // two stages
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * KV_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;               // [2]
    uint64_t* v_full = bars + 3;               // [2]
    uint64_t* kv_empty = bars + 5;             // [2] PV of the tile in the stage has retired
    uint64_t* s_full = bars + 7;               // [2] QK of the tile has retired
    uint64_t* s_free = bars + 9;               // [2] the softmax threads are done with S
    uint64_t* p_full = bars + 11;              // [2] P written
    uint64_t* pv_done = bars + 13;             // [2] PV of the tile has retired (O may be touched, P may be overwritten)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* s_work = const_cast<int*>(abort_flag) + 1;   // [2]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y;
    pdl_enter_attn();

    // ---- (sequence, q tile) of this CTA: tiles are numbered sequence by sequence; the grid is walked backwards so that the
    // tiles with the longest causal context start first
    if (threadIdx.x == 0) {
        const int bx = gridDim.x - 1 - blockIdx.x;
        int acc = 0, found = -1, tile = 0;
        for (int b = 0; b < p.B; ++b) {
            const int ql = PAGED ? p.subsequence_begins[b + 1] - p.subsequence_begins[b] : p.dense_S;
            const int nt = (ql + TOK - 1) / TOK;
            if (bx < acc + nt) { found = b; tile = bx - acc; break; }
            acc += nt;
        }
        s_work[0] = found;
        s_work[1] = tile;
        *abort_flag = 0;
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&kv_empty[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&s_free[i], kBM);
            mbar_init(&p_full[i], kBM);
            mbar_init(&pv_done[i], 1);
        }
        mbar_fence_init();
    }
    // (The PV product reads whole pages only: its k-steps are 16 keys = one page, and steps past the last loaded page are
    // not issued, so stale shared memory never reaches the tensor core as V. Stale K rows only produce masked columns of S.)
    __syncthreads();
    const int b = s_work[0];
    if (b < 0) return;                          // (uniform) nothing allocated yet
    if (warp == 5) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    const int qtile = s_work[1];
    const int tok_begin = PAGED ? p.subsequence_begins[b] : b * p.dense_S;
    const int q_len = PAGED ? p.subsequence_begins[b + 1] - tok_begin : p.dense_S;
    const int past = PAGED ? p.past_lens[b] : 0;
    const int blk_begin = PAGED ? p.block_indices_begins[b] : 0;
    const int tq0 = qtile * TOK;
    const int tq1 = min(q_len, tq0 + TOK);
    const int kv_total = PAGED ? past + q_len : p.dense_S;
    const int kv_end = p.causal ? min(kv_total, past + tq1) : kv_total;
    int kv_start = 0;
    if (p.sliding_window > 0) kv_start = max(0, past + tq0 - p.sliding_window + 1);
    kv_start = (kv_start / kBK) * kBK;
    const int ntiles = (kv_end - kv_start + kBK - 1) / kBK;

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer
        // One lane posts the byte counts; then every lane issues the boxes of its own (page, half): a single thread that
        // issues the 64 small copies of a tile one after the other is slower than the tensor core consumes them.
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, Q_BYTES);
            for (int g = 0; g < G; ++g)
                for (int hf = 0; hf < HALVES; ++hf)
                    tma_load_2d(sQ + hf * (kBM * 128) + g * (TOK * 128), &tmQ, q_full, (h * G + g) * D + hf * 64, tok_begin + tq0);
        }
        for (int j = 0; j < ntiles; ++j) {
            const int st = j & 1;
            if (j >= 2 && !mbar_wait(&kv_empty[st], ((j >> 1) - 1) & 1, abort_flag, status)) break;
            const int j0 = kv_start + j * kBK;
            const int npages = (min(kv_end, j0 + kBK) - j0 + kPage - 1) / kPage;
            if (lane == 0) {
                mbar_arrive_expect_tx(&k_full[st], npages * kPage * D * 2);
                mbar_arrive_expect_tx(&v_full[st], npages * kPage * D * 2);
            }
            __syncwarp();
            for (int u = lane; u < npages * HALVES; u += 32) {
                const int pg = u / HALVES, hf = u % HALVES;
                int row, col;
                if (PAGED) {
                    const int blk = p.block_indices[blk_begin + j0 / kPage + pg];
                    row = (blk * p.Hkv + h) * kPage;
                    col = 0;
                } else {
                    row = b * p.dense_S + j0 + pg * kPage;
                    col = h * D;
                }
                tma_load_2d(sK + st * KV_BYTES + hf * (kBK * 128) + pg * (kPage * 128), &tmK, &k_full[st], col + hf * 64, row);
                tma_load_2d(sV + st * KV_BYTES + hf * (kBK * 128) + pg * (kPage * 128), &tmV, &v_full[st], col + hf * 64, row);
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer (warp-uniform flow, one elected lane issues)
        bool ok = mbar_wait(q_full, 0, abort_flag, status);
        const uint64_t dq = umma_desc_k_sw128(smem_u32(sQ), 1024);
        for (int j = 0; j <= ntiles && ok; ++j) {
            if (j < ntiles) {
                const int st = j & 1;
                ok = ok && mbar_wait(&k_full[st], (j >> 1) & 1, abort_flag, status);
                if (j >= 2) ok = ok && mbar_wait(&s_free[st], ((j >> 1) - 1) & 1, abort_flag, status);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t dk = umma_desc_k_sw128(smem_u32(sK + st * KV_BYTES), 1024);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint64_t off = (uint64_t)(((ks >> 2) * (kBM * 128) + (ks & 3) * 32) >> 4);
                    umma_f16_ss_elect(tmem + TM_S + st * kBK, dq + off, dk + off, IDESC_QK, ks > 0 ? 1u : 0u);
                }
                umma_commit_elect(&s_full[st]);
            }
            if (j >= 1) {
                const int i = j - 1, st = i & 1;
                ok = ok && mbar_wait(&v_full[st], (i >> 1) & 1, abort_flag, status);
                ok = ok && mbar_wait(&p_full[st], (i >> 1) & 1, abort_flag, status);
                if (!ok) break;
                tc_fence_after_sync();
                const int keys = min(kBK, kv_end - (kv_start + i * kBK));
                const int ksteps = (keys + 15) / 16;
                const uint64_t dv = umma_desc_mn_sw128(smem_u32(sV + st * KV_BYTES), kBK * 128, 1024);
                for (int kk = 0; kk < ksteps; ++kk)
                    umma_f16_ts_elect(tmem + TM_O, tmem + TM_P + st * 64 + kk * 8, dv + (uint64_t)((kk * 16 * 128) >> 4), IDESC_PV,
                                      (i > 0 || kk > 0) ? 1u : 0u);
                umma_commit_elect(&kv_empty[st]);
                umma_commit_elect(&pv_done[st]);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ softmax: one thread per stacked query row
        const int r = threadIdx.x;                       // 0..127 = tensor-memory lane
        const int g = r / TOK, tl = r % TOK;
        const int qpos = past + tq0 + tl;
        const bool row_valid = (tq0 + tl) < q_len;
        const uint32_t lane_base = tmem + (uint32_t(warp * 32) << 16);
        float m_used = -CUDART_INF_F, l_sum = 0.f;
        bool ok = true;
        for (int j = 0; j < ntiles && ok; ++j) {
            const int st = j & 1;
            ok = mbar_wait(&s_full[st], (j >> 1) & 1, abort_flag, status);
            if (!ok) break;
            tc_fence_after_sync();
            const int j0 = kv_start + j * kBK;
            // does any row of the tile need a mask? (uniform over the CTA)
            const bool need_mask = (j0 + kBK > kv_end) || (p.causal && (j0 + kBK - 1 > past + tq0)) ||
                                   (p.sliding_window > 0 && (j0 <= past + tq1 - 1 - p.sliding_window));
            int hi = kBK, lo = 0;                        // keys [lo, hi) of the tile are visible to this row
            if (need_mask) {
                hi = min(hi, kv_end - j0);
                if (p.causal) hi = min(hi, qpos - j0 + 1);
                if (p.sliding_window > 0) lo = max(lo, qpos - p.sliding_window + 1 - j0);
                if (!row_valid) hi = 0;
            }
            // The whole row of S goes to registers in one round trip to tensor memory (eight loads in flight, one wait);
            // S is then free for the QK product of tile j + 2 while this thread still works on the values.
            uint32_t v[kBK];
#pragma unroll
            for (int c = 0; c < kBK; c += 16) tmem_ld_x16(lane_base + TM_S + st * kBK + c, v + c);
            tmem_ld_wait();
            tc_fence_before_sync();
            mbar_arrive(&s_free[st]);
            // maximum of the visible part of the row (four independent chains)
            float mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < kBK; ++i) {
                    const bool vis = i >= lo && i < hi;
                    if (!vis) v[i] = __float_as_uint(-CUDART_INF_F);
                    mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(v[i]));
                }
            } else {
#pragma unroll
                for (int i = 0; i < kBK; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(v[i]));
            }
            float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;   // scale > 0: max commutes with scaling
            // raise the running maximum only when the tile exceeds it by a factor of 2^8; the rescale of O is warp-collective
            const bool raise = m_tile > m_used + 8.f;
            if (__any_sync(0xffffffffu, raise)) {
                const float factor = !raise ? 1.f : (m_used == -CUDART_INF_F ? 0.f : fast_exp2(m_used - m_tile));
                if (j > 0) {
                    ok = mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, status);
                    if (!ok) break;
                    tc_fence_after_sync();
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        uint32_t o[32];
                        tmem_ld_x16(lane_base + TM_O + c, o);
                        tmem_ld_x16(lane_base + TM_O + c + 16, o + 16);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                        tmem_st_x16(lane_base + TM_O + c, o);
                        tmem_st_x16(lane_base + TM_O + c + 16, o + 16);
                    }
                    tmem_st_wait();
                }
                if (raise) {
                    l_sum *= factor;
                    m_used = m_tile;
                }
            }
            // exponentials (masked entries are -inf: exp2 gives 0), row sum, P as 16-bit pairs (packed in place)
            const float neg_m = (m_used == -CUDART_INF_F) ? 0.f : -m_used;
            float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < kBK; i += 2) {
                const float e0 = fast_exp2(fmaf(__uint_as_float(v[i]), p.scale_log2, neg_m));
                const float e1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, neg_m));
                ls[(i >> 1) & 3] += e0 + e1;
                v[i >> 1] = pack16<F16>(e0, e1);
            }
            l_sum += (ls[0] + ls[1]) + (ls[2] + ls[3]);
            // P of tile j - 2 (same buffer) must have been consumed
            if (j >= 2) {
                ok = mbar_wait(&pv_done[st], ((j >> 1) - 1) & 1, abort_flag, status);
                if (!ok) break;
            }
#pragma unroll
            for (int c = 0; c < kBK / 2; c += 16) tmem_st_x16(lane_base + TM_P + st * 64 + c, v + c);
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(&p_full[st]);
        }
        // ---- epilogue: O / l
        if (ok && ntiles > 0) ok = mbar_wait(&pv_done[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1, abort_flag, status);
        if (ok) {
            tc_fence_after_sync();
            const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
            uint8_t* dst = reinterpret_cast<uint8_t*>(p.out) + ((size_t)(tok_begin + tq0 + tl) * p.Hq * D + (size_t)(h * G + g) * D) * 2;
#pragma unroll 1
            for (int c = 0; c < D; c += 16) {
                uint32_t o[16];
                if (ntiles > 0) {
                    tmem_ld_x16(lane_base + TM_O + c, o);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = 0u;
                }
                if (row_valid) {
                    uint4 w0, w1;
                    w0.x = pack16<F16>(__uint_as_float(o[0]) * inv, __uint_as_float(o[1]) * inv);
                    w0.y = pack16<F16>(__uint_as_float(o[2]) * inv, __uint_as_float(o[3]) * inv);
                    w0.z = pack16<F16>(__uint_as_float(o[4]) * inv, __uint_as_float(o[5]) * inv);
                    w0.w = pack16<F16>(__uint_as_float(o[6]) * inv, __uint_as_float(o[7]) * inv);
                    w1.x = pack16<F16>(__uint_as_float(o[8]) * inv, __uint_as_float(o[9]) * inv);
                    w1.y = pack16<F16>(__uint_as_float(o[10]) * inv, __uint_as_float(o[11]) * inv);
                    w1.z = pack16<F16>(__uint_as_float(o[12]) * inv, __uint_as_float(o[13]) * inv);
                    w1.w = pack16<F16>(__uint_as_float(o[14]) * inv, __uint_as_float(o[15]) * inv);
                    *reinterpret_cast<uint4*>(dst + c * 2) = w0;
                    *reinterpret_cast<uint4*>(dst + c * 2 + 16) = w1;
                }
            }
        }
    }

    // ---------------------------------------------------------------- tear-down
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);   // copies still in flight land before the shared memory is reused
        __syncthreads();
    }
    if (warp == 5) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

template <int D, int G, bool PAGED, bool F16>
int launch_tc(const PaKParams& p, int num_q_tiles, cudaStream_t stream) {
    constexpr int TOK = kBM / G;
    const int smem = kBM * D * 2 + 4 * kBK * D * 2 + 256 + 1024;
    auto kern = pa_prefill_tc_kernel<D, G, PAGED, F16>;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    OVB_CHECK_CUDA(cudaGetDevice(&dev));
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        OVB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured.fetch_or(bit, std::memory_order_release);
    }
    const CUtensorMapDataType dt = F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    CUtensorMap tmQ, tmK, tmV;
    // Q rows are tokens; a box is the TOK tokens of a tile x 64 columns of one head (rows past T read as zeros)
    if (int rc = make_tmap_2d(&tmQ, p.q, dt, 2, (uint64_t)p.T, (uint64_t)p.ldq, (uint64_t)p.ldq * 2, TOK, 64, true)) return rc;
    if (PAGED) {
        // the cache seen as rows of D elements: row = (block * Hkv + head) * 16 + slot; the row count only bounds coordinates
        const uint64_t rows = 1ull << 30;
        if (int rc = make_tmap_2d(&tmK, p.k_cache, dt, 2, rows, D, (uint64_t)D * 2, kPage, 64, true)) return rc;
        if (int rc = make_tmap_2d(&tmV, p.v_cache, dt, 2, rows, D, (uint64_t)D * 2, kPage, 64, true)) return rc;
    } else {
        const uint64_t rows = (uint64_t)p.B * p.dense_S;
        if (int rc = make_tmap_2d(&tmK, p.k_cache, dt, 2, rows, (uint64_t)p.ld_kv, (uint64_t)p.ld_kv * 2, kPage, 64, true)) return rc;
        if (int rc = make_tmap_2d(&tmV, p.v_cache, dt, 2, rows, (uint64_t)p.ld_kv, (uint64_t)p.ld_kv * 2, kPage, 64, true)) return rc;
    }
    OVB_CHECK_CUDA(launch_pdl(kern, dim3(num_q_tiles, p.Hkv), dim3(192), (size_t)smem, stream, tmQ, tmK, tmV, p, status_word()));
    return 0;
}

}  // namespace

int launch_prefill_tc(const PaKParams& p, int D, int G, bool paged, bool f16, int num_q_tiles, cudaStream_t stream) {
    if (paged && p.block_size != kPage) return ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(p.q) & 15) || (reinterpret_cast<uintptr_t>(p.k_cache) & 15) || (reinterpret_cast<uintptr_t>(p.v_cache) & 15) ||
        (reinterpret_cast<uintptr_t>(p.out) & 15) || p.ldq % 8 != 0 || (!paged && p.ld_kv % 8 != 0))
        return ERR_UNSUPPORTED;
    if (paged && !f16) {
        if (D == 128) {
            switch (G) {
                case 1: return launch_tc<128, 1, true, false>(p, num_q_tiles, stream);
                case 2: return launch_tc<128, 2, true, false>(p, num_q_tiles, stream);
                case 4: return launch_tc<128, 4, true, false>(p, num_q_tiles, stream);
                case 8: return launch_tc<128, 8, true, false>(p, num_q_tiles, stream);
            }
        } else if (D == 64) {
            switch (G) {
                case 1: return launch_tc<64, 1, true, false>(p, num_q_tiles, stream);
                case 4: return launch_tc<64, 4, true, false>(p, num_q_tiles, stream);
            }
        }
    } else if (!paged && G == 1) {
        if (D == 64) return f16 ? launch_tc<64, 1, false, true>(p, num_q_tiles, stream) : launch_tc<64, 1, false, false>(p, num_q_tiles, stream);
        if (D == 128) return f16 ? launch_tc<128, 1, false, true>(p, num_q_tiles, stream) : launch_tc<128, 1, false, false>(p, num_q_tiles, stream);
    }
    return ERR_UNSUPPORTED;
}

}  // namespace ovb
