// Weight-stationary tcgen05 GEMM for sm_100a:  out[T, N] = epilogue(X[T, K] * dequant(W[N, K])^T).
//
// Role of this file in the reference's terms: the FullyConnected / FullyConnectedCompressed
// primitive (src/plugins/intel_gpu/src/kernel_selector/cl_kernels/fully_connected_gpu_bf_tiled.cl,
// fully_connected_gpu_gemv.cl; CPU: src/plugins/intel_cpu/src/nodes/fullyconnected.cpp), i.e. MatMul
// with constant weights, int4/int8 group dequantisation fused, bias / activation / residual epilogue.
//
// Design (Blackwell-first, not a translation):
//  * The 128 weight rows of a tile sit on the M side of tcgen05.mma, the tokens on the N side
//    (16..256). The accumulator [128 x BT] fp32 lives in TMEM.
//  * warp 0 = TMA producer (cp.async.bulk.tensor, 128-byte swizzle), warp 1 = MMA issuer (one
//    elected lane), warps 2..9 = weight dequantisation during the main loop, then the epilogue
//    (tcgen05.ld -> registers -> global).
//  * Quantised weights are fetched packed (4 KB per 128x64 tile for u4), expanded to bf16 by the
//    dequant warps straight into the swizzled K-major layout that the MMA descriptor expects,
//    made visible to the async proxy with fence.proxy.async, and handed over through an mbarrier.
//  * Small-T problems (decode) are split along K so that every SM streams weights; the last CTA
//    to arrive at a tile reduces the fp32 partials in a fixed order (bitwise reproducible).
#include <map>
#include <mutex>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ovb {

constexpr int TILE_N = 128;      // weight rows per CTA (MMA M)
constexpr int TILE_K = 64;       // bf16 elements per k-block = one 128-byte swizzle span
constexpr int NUM_DQ_WARPS = 8;  // dequant + epilogue warps
constexpr int GEMM_THREADS = (2 + NUM_DQ_WARPS) * 32;
constexpr int MAX_STAGES = 8;

struct GemmKParams {
    void* out;
    const void* bias;
    const void* residual;
    const __nv_bfloat16* scales;
    const __nv_bfloat16* zps;
    float* ws;
    int* counters;
    int* status;
    int T, N, K;
    int ldo, ldr;
    int group_size;
    int act;
    int out_f32;
    int splits;
    int stages;
    int kblocks_per_split;
};

template <bool F16>
struct Elem {
    using type = __nv_bfloat16;
};
template <>
struct Elem<true> {
    using type = __half;
};

__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
template <class E>
__device__ __forceinline__ E from_float(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_float<__half>(float v) {
    return __float2half_rn(v);
}

__device__ __forceinline__ float apply_act(float v, int act) {
    switch (act) {
        case OVB_ACT_GELU_ERF: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
        case OVB_ACT_RELU: return v > 0.f ? v : 0.f;
        case OVB_ACT_SILU: return v / (1.0f + __expf(-v));
        case OVB_ACT_GELU_TANH: {
            float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
            return 0.5f * v * (1.0f + tanhf(u));
        }
        default: return v;
    }
}

// Expand one u32 (8 packed u4 in the plugin nibble order) to 8 bf16: (q - zp) * scale.
// A nibble placed in mantissa bits 3..6 of bf16 16.0 (0x4180) reads as 16 + q exactly.
__device__ __forceinline__ uint4 dequant_u4x8(uint32_t x, __nv_bfloat162 zz, __nv_bfloat162 ss) {
    uint32_t t[4];
    t[0] = ((x << 3) & 0x00780078u) | 0x41804180u;
    t[1] = ((x >> 1) & 0x00780078u) | 0x41804180u;
    t[2] = ((x >> 5) & 0x00780078u) | 0x41804180u;
    t[3] = ((x >> 9) & 0x00780078u) | 0x41804180u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&t[i]);
        v = __hmul2(__hsub2(v, zz), ss);
        t[i] = *reinterpret_cast<uint32_t*>(&v);
    }
    return make_uint4(t[0], t[1], t[2], t[3]);
}

template <int BT, int WMODE, bool F16>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_ws_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, GemmKParams p) {
    using E = typename Elem<F16>::type;
    constexpr bool QUANT = (WMODE == OVB_W_U4 || WMODE == OVB_W_U8);
    constexpr int X_BYTES = BT * 128;
    constexpr int W_BYTES = TILE_N * 128;
    constexpr int WQ_BYTES = (WMODE == OVB_W_U4) ? TILE_N * 32 : (WMODE == OVB_W_U8 ? TILE_N * 64 : 0);
    constexpr int STAGE_BYTES = X_BYTES + W_BYTES + ((WQ_BYTES + 1023) / 1024) * 1024;
    constexpr int TMEM_COLS = BT < 32 ? 32 : BT;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int stages = p.stages;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + stages * STAGE_BYTES);
    uint64_t* full_tma = bars;                  // [stages] TMA bytes landed
    uint64_t* full_dq = bars + MAX_STAGES;      // [stages] dequantised tile written
    uint64_t* empty = bars + 2 * MAX_STAGES;    // [stages] MMAs that read the stage retired
    uint64_t* acc_full = bars + 3 * MAX_STAGES; // accumulator complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * MAX_STAGES + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* last_flag = const_cast<int*>(abort_flag) + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TILE_N;
    const int t0 = blockIdx.y * BT;
    const int split = blockIdx.z;
    const int total_kb = (p.K + TILE_K - 1) / TILE_K;
    const int kb_begin = split * p.kblocks_per_split;
    const int kb_end = min(total_kb, kb_begin + p.kblocks_per_split);
    const int num_kb = max(0, kb_end - kb_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_tma[s], 1);
            mbar_init(&full_dq[s], NUM_DQ_WARPS);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        *last_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmW);
        tma_prefetch_desc(&tmX);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t phase = 0;
            int s = 0;
            for (int i = 0; i < num_kb; ++i) {
                if (!mbar_wait(&empty[s], phase ^ 1, abort_flag, p.status)) break;
                uint8_t* st = smem + s * STAGE_BYTES;
                const int kb = kb_begin + i;
                mbar_arrive_expect_tx(&full_tma[s], X_BYTES + (QUANT ? WQ_BYTES : W_BYTES));
                tma_load_2d(st, &tmX, &full_tma[s], kb * TILE_K, t0);
                if (WMODE == OVB_W_U4) {
                    tma_load_2d(st + X_BYTES + W_BYTES, &tmW, &full_tma[s], kb * (TILE_K / 2), n0);
                } else if (WMODE == OVB_W_U8) {
                    tma_load_2d(st + X_BYTES + W_BYTES, &tmW, &full_tma[s], kb * TILE_K, n0);
                } else {
                    tma_load_2d(st + X_BYTES, &tmW, &full_tma[s], kb * TILE_K, n0);
                }
                if (++s == stages) { s = 0; phase ^= 1; }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc = umma_idesc_f16(TILE_N, BT, !F16);
        uint32_t phase = 0;
        int s = 0;
        for (int i = 0; i < num_kb; ++i) {
            bool ok = mbar_wait(&full_tma[s], phase, abort_flag, p.status);
            if (ok && QUANT) ok = mbar_wait(&full_dq[s], phase, abort_flag, p.status);
            if (!ok) break;
            tc_fence_after_sync();
            if (lane == 0) {
                const uint32_t xa = smem_u32(smem + s * STAGE_BYTES);
                const uint32_t wa = xa + X_BYTES;
#pragma unroll
                for (int k = 0; k < TILE_K / 16; ++k) {
                    const uint64_t da = umma_desc_k_sw128(wa + k * 32, 1024);
                    const uint64_t db = umma_desc_k_sw128(xa + k * 32, 1024);
                    umma_f16_ss(tmem_base, da, db, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty[s]);
            }
            __syncwarp();
            if (++s == stages) { s = 0; phase ^= 1; }
        }
        if (lane == 0) umma_commit(acc_full);
        __syncwarp();
    } else {
        // ------------------------------------------------------------ dequant warps, then epilogue
        const int dq_tid = threadIdx.x - 64;  // 0..255
        if (QUANT) {
            const int r = dq_tid >> 1;       // weight row inside the tile
            const int half = dq_tid & 1;     // which 32-element half of the 64-wide k-block
            const int n = n0 + r;
            const int G = p.K / p.group_size;
            uint32_t phase = 0;
            int s = 0;
            int cur_g = -1;
            __nv_bfloat162 ss = __floats2bfloat162_rn(0.f, 0.f), zz = ss;
            for (int i = 0; i < num_kb; ++i) {
                const int kb = kb_begin + i;
                const int g = (kb * TILE_K) / p.group_size;
                if (g != cur_g) {
                    cur_g = g;
                    __nv_bfloat16 sv = __float2bfloat16_rn(0.f), zv = sv;
                    if (n < p.N && g < G) {
                        sv = p.scales[(size_t)g * p.N + n];
                        zv = p.zps[(size_t)g * p.N + n];
                    }
                    ss = __halves2bfloat162(sv, sv);
                    zz = __halves2bfloat162(zv, zv);
                }
                bool ok = mbar_wait(&empty[s], phase ^ 1, abort_flag, p.status);
                if (ok) ok = mbar_wait(&full_tma[s], phase, abort_flag, p.status);
                if (!ok) break;
                uint8_t* st = smem + s * STAGE_BYTES;
                uint8_t* wdst = st + X_BYTES + r * 128;
                const uint8_t* wq = st + X_BYTES + W_BYTES;
                if (WMODE == OVB_W_U4) {
                    const uint4 pk = *reinterpret_cast<const uint4*>(wq + r * 32 + half * 16);
                    const uint32_t xs[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int c = half * 4 + j;
                        *reinterpret_cast<uint4*>(wdst + ((c ^ (r & 7)) << 4)) = dequant_u4x8(xs[j], zz, ss);
                    }
                } else {
                    const float sf = __bfloat162float(__low2bfloat16(ss));
                    const float zf = __bfloat162float(__low2bfloat16(zz));
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint2 pk = *reinterpret_cast<const uint2*>(wq + r * 64 + half * 32 + j * 8);
                        const uint32_t b[2] = {pk.x, pk.y};
                        uint32_t o[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t w32 = b[e >> 1];
                            const int sh = (e & 1) * 16;
                            const float f0 = (float((w32 >> sh) & 0xFF) - zf) * sf;
                            const float f1 = (float((w32 >> (sh + 8)) & 0xFF) - zf) * sf;
                            o[e] = pack_bf16x2(f0, f1);
                        }
                        const int c = half * 4 + j;
                        *reinterpret_cast<uint4*>(wdst + ((c ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_dq[s]);
                if (++s == stages) { s = 0; phase ^= 1; }
            }
        }

        // -------- epilogue: warp (w % 4) owns TMEM lanes 32*(w%4) .. +31; two warps share a quarter
        const int q = warp & 3;
        const int colhalf = (warp - 2) >> 2;  // 0 or 1
        const int row = q * 32 + lane;
        const int oc = n0 + row;
        constexpr int COLS_PER_WARP = BT / 2;            // BT >= 32 -> multiple of 16
        constexpr int CHUNKS = (COLS_PER_WARP + 15) / 16;
        const int cbeg = (BT >= 32) ? colhalf * COLS_PER_WARP : 0;
        const bool active_warp = (BT >= 32) || (colhalf == 0);
        const bool acc_ok = (num_kb > 0) ? mbar_wait(acc_full, 0, abort_flag, p.status) : true;
        tc_fence_after_sync();

        const float bias_v = (p.bias != nullptr && oc < p.N) ? to_float(reinterpret_cast<const E*>(p.bias)[oc]) : 0.f;
        const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
        float* ws_tile = p.ws ? p.ws + ((size_t)tile_id * p.splits) * (TILE_N * BT) : nullptr;

        auto finish = [&](int col, float v) {
            const int tok = t0 + col;
            if (tok < p.T && oc < p.N) {
                v += bias_v;
                v = apply_act(v, p.act);
                if (p.residual) v += to_float(reinterpret_cast<const E*>(p.residual)[(size_t)tok * p.ldr + oc]);
                if (p.out_f32)
                    reinterpret_cast<float*>(p.out)[(size_t)tok * p.ldo + oc] = v;
                else
                    reinterpret_cast<E*>(p.out)[(size_t)tok * p.ldo + oc] = from_float<E>(v);
            }
        };

        if (acc_ok && active_warp) {
#pragma unroll 1
            for (int ch = 0; ch < CHUNKS; ++ch) {
                const int c0 = cbeg + ch * 16;
                uint32_t r[16];
                if (num_kb > 0) {
                    tmem_ld_x16(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(c0), r);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = 0;
                }
                if (p.splits == 1) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) finish(c0 + j, __uint_as_float(r[j]));
                } else {
                    float* dst = ws_tile + (size_t)split * (TILE_N * BT);
#pragma unroll
                    for (int j = 0; j < 16; ++j) dst[(c0 + j) * TILE_N + row] = __uint_as_float(r[j]);
                }
            }
        }
        if (p.splits > 1) {
            // Last CTA to arrive at this tile sums the partials in split order.
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"n"(NUM_DQ_WARPS * 32));
            if (dq_tid == 0) {
                const int prev = atomicAdd(&p.counters[tile_id], 1);
                *last_flag = (prev == p.splits - 1) ? 1 : 0;
                if (prev == p.splits - 1) p.counters[tile_id] = 0;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NUM_DQ_WARPS * 32));
            if (*last_flag && active_warp) {
                __threadfence();
                for (int c = cbeg; c < cbeg + (BT >= 32 ? COLS_PER_WARP : BT); ++c) {
                    float acc = 0.f;
                    for (int z = 0; z < p.splits; ++z) acc += __ldcg(ws_tile + (size_t)z * (TILE_N * BT) + c * TILE_N + row);
                    finish(c, acc);
                }
            }
        }
    }

    // ---------------------------------------------------------------- tear-down
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // Give copies that are still in flight time to land before the CTA's shared memory is reused.
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// --------------------------------------------------------------------------------------------- host
static int stage_bytes(int bt, int wmode) {
    int wq = wmode == OVB_W_U4 ? TILE_N * 32 : (wmode == OVB_W_U8 ? TILE_N * 64 : 0);
    return bt * 128 + TILE_N * 128 + ((wq + 1023) / 1024) * 1024;
}

constexpr int kSmemBudget = 212 * 1024;
constexpr int kNumCounters = 4096;
constexpr int kNumSMs = 148;

static int pick_block_t(int T) {
    if (T <= 16) return 16;
    if (T <= 32) return 32;
    if (T <= 64) return 64;
    if (T <= 128) return 128;
    return 256;
}

static int pick_splits(int T, int N, int K, int bt) {
    const int tiles = ceil_div(N, TILE_N) * ceil_div(T, bt);
    const int total_kb = ceil_div(K, TILE_K);
    if (tiles >= 120 || total_kb < 8) return 1;
    int s = ceil_div(kNumSMs, tiles);
    s = s < total_kb / 4 ? s : total_kb / 4;
    if (s > 16) s = 16;
    return s < 1 ? 1 : s;
}

template <int BT, int WMODE, bool F16>
static int launch(const ovb_gemm_args* a, const CUtensorMap& tmW, const CUtensorMap& tmX, GemmKParams& p,
                  cudaStream_t stream) {
    const int sb = stage_bytes(BT, WMODE);
    int stages = kSmemBudget / sb;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) stages = 2;
    p.stages = stages;
    const int smem = stages * sb + 1024 + 512;
    auto kern = gemm_ws_kernel<BT, WMODE, F16>;
    static uint64_t configured = 0;  // one bit per device
    int dev = 0;
    OVB_CHECK_CUDA(cudaGetDevice(&dev));
    if (!(configured & (1ull << dev))) {
        OVB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024));
        configured |= (1ull << dev);
    }
    dim3 grid(ceil_div(a->N, TILE_N), ceil_div(a->T, BT), p.splits);
    kern<<<grid, GEMM_THREADS, smem, stream>>>(tmW, tmX, p);
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

template <int WMODE, bool F16>
static int dispatch_bt(int bt, const ovb_gemm_args* a, const CUtensorMap& tmW, const CUtensorMap& tmX, GemmKParams& p,
                       cudaStream_t stream) {
    switch (bt) {
        case 16: return launch<16, WMODE, F16>(a, tmW, tmX, p, stream);
        case 32: return launch<32, WMODE, F16>(a, tmW, tmX, p, stream);
        case 64: return launch<64, WMODE, F16>(a, tmW, tmX, p, stream);
        case 128: return launch<128, WMODE, F16>(a, tmW, tmX, p, stream);
        case 256: return launch<256, WMODE, F16>(a, tmW, tmX, p, stream);
    }
    set_error("unsupported block_t %d", bt);
    return ERR_BAD_ARG;
}

}  // namespace ovb

extern "C" {

int ovb_gemm_num_counters(void) { return ovb::kNumCounters; }

int64_t ovb_gemm_ws_bytes(int T, int N, int K, int act) {
    (void)act;
    const int bt = ovb::pick_block_t(T);
    const int splits = ovb::pick_splits(T, N, K, bt);
    if (splits == 1) return 0;
    const int64_t tiles = (int64_t)ovb::ceil_div(N, ovb::TILE_N) * ovb::ceil_div(T, bt);
    return tiles * splits * ovb::TILE_N * bt * (int64_t)sizeof(float);
}

int ovb_gemm(const ovb_gemm_args* a, ovb_stream_t stream_) {
    using namespace ovb;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(a && a->x && a->w && a->out, "ovb_gemm: null operand");
    OVB_REQUIRE(a->T > 0 && a->N > 0 && a->K > 0, "ovb_gemm: empty problem T=%d N=%d K=%d", a->T, a->N, a->K);
    OVB_REQUIRE(a->K % 8 == 0 && a->ldx % 8 == 0, "ovb_gemm: K and ldx must be multiples of 8 (TMA 16-byte rule)");
    const bool f16 = a->wmode == OVB_W_F16;
    const bool quant = a->wmode == OVB_W_U4 || a->wmode == OVB_W_U8;
    if (quant) {
        OVB_REQUIRE(a->scales && a->zps, "ovb_gemm: quantised weights need scales and zero points");
        OVB_REQUIRE(a->group_size >= 64 && a->group_size % 64 == 0 && a->K % a->group_size == 0,
                    "ovb_gemm: group_size %d must be a multiple of 64 that divides K=%d", a->group_size, a->K);
        OVB_REQUIRE(a->K % 32 == 0, "ovb_gemm: K must be a multiple of 32 for packed weights");
    }
    OVB_REQUIRE(a->act != OVB_ACT_SWIGLU, "ovb_gemm: SWIGLU epilogue is provided by ovb_silu_mul");

    const int bt = a->block_t ? a->block_t : pick_block_t(a->T);
    int splits = a->splits ? a->splits : pick_splits(a->T, a->N, a->K, bt);
    const int total_kb = ceil_div(a->K, TILE_K);
    if (splits > total_kb) splits = total_kb;
    const int64_t tiles = (int64_t)ceil_div(a->N, TILE_N) * ceil_div(a->T, bt);
    if (splits > 1) {
        const int64_t need = tiles * splits * TILE_N * bt * (int64_t)sizeof(float);
        if (!a->ws || !a->counters || a->ws_bytes < need || tiles > kNumCounters) splits = 1;
    }

    GemmKParams p;
    memset(&p, 0, sizeof(p));
    p.out = a->out;
    p.bias = a->bias;
    p.residual = a->residual;
    p.scales = reinterpret_cast<const __nv_bfloat16*>(a->scales);
    p.zps = reinterpret_cast<const __nv_bfloat16*>(a->zps);
    p.ws = a->ws;
    p.counters = a->counters;
    p.status = status_word();
    p.T = a->T; p.N = a->N; p.K = a->K;
    p.ldo = a->ldo ? a->ldo : a->N;
    p.ldr = a->ldr ? a->ldr : a->N;
    p.group_size = quant ? a->group_size : a->K;
    p.act = a->act;
    p.out_f32 = a->out_f32;
    p.splits = splits;
    p.kblocks_per_split = ceil_div(total_kb, splits);

    CUtensorMap tmW, tmX;
    const int ldx = a->ldx ? a->ldx : a->K;
    const CUtensorMapDataType dt16 = f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    if (int rc = make_tmap_2d(&tmX, a->x, dt16, 2, a->T, a->K, (uint64_t)ldx * 2, bt, TILE_K, true)) return rc;
    int rc = 0;
    if (a->wmode == OVB_W_U4) {
        rc = make_tmap_2d(&tmW, a->w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->N, a->K / 2, (uint64_t)a->K / 2, TILE_N, 32, false);
    } else if (a->wmode == OVB_W_U8) {
        rc = make_tmap_2d(&tmW, a->w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->N, a->K, (uint64_t)a->K, TILE_N, 64, false);
    } else {
        rc = make_tmap_2d(&tmW, a->w, dt16, 2, a->N, a->K, (uint64_t)a->K * 2, TILE_N, TILE_K, true);
    }
    if (rc) return rc;

    switch (a->wmode) {
        case OVB_W_BF16: return dispatch_bt<OVB_W_BF16, false>(bt, a, tmW, tmX, p, stream);
        case OVB_W_F16: return dispatch_bt<OVB_W_BF16, true>(bt, a, tmW, tmX, p, stream);
        case OVB_W_U4: return dispatch_bt<OVB_W_U4, false>(bt, a, tmW, tmX, p, stream);
        case OVB_W_U8: return dispatch_bt<OVB_W_U8, false>(bt, a, tmW, tmX, p, stream);
    }
    set_error("ovb_gemm: unknown wmode %d", a->wmode);
    return ERR_BAD_ARG;
}

}  // extern "C"
