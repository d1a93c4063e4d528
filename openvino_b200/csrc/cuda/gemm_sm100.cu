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
//  * warp 0 = producer (one lane): TMA tensor loads of the token tile (128-byte swizzle) and 1-D bulk
//    copies of the weight chunks; warp 1 = MMA issuer (one lane); warps 2..9 = weight dequantisation
//    during the main loop, then the epilogue.
//  * Weights are constants, so the plugin stores them tile-contiguously: every (128-row tile, 64-column
//    k-block) pair is ONE chunk (u4: 4 KB packed; bf16: 16 KB already in the swizzled smem order), which
//    a single bulk copy fetches with full DRAM locality.
//  * Quantised weights use two rings: a deep ring of packed chunks that the producer fills far ahead
//    of use (HBM latency hidden), and a short ring of MMA stages (token tile + expanded bf16 weight
//    tile). Each MMA stage is owned by one or two dequant warps, so several k-blocks are expanded at the
//    same time; a stage is handed to the MMA through an mbarrier after fence.proxy.async.
//  * Small-T problems (decode) are split along K so that every SM streams weights. The splits of a tile form a
//    thread-block cluster: every CTA leaves its fp32 partial tile in its own shared memory, and after a cluster
//    barrier each CTA sums one slice of the tile over all partials through distributed shared memory, in split
//    order (bitwise reproducible), and writes that slice of the output. No partial ever goes to global memory.
//  * Epilogue: TMEM -> registers -> (bias, activation) -> 16-bit tile in shared memory -> coalesced
//    16-byte stores (residual added on the way out).
#include <stdlib.h>

#include <atomic>
#include <mutex>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ovb {

constexpr int TILE_N = 128;      // weight rows per CTA (MMA M)
constexpr int TILE_K = 64;       // bf16 elements per k-block = one 128-byte swizzle span
// Warp roles: warp 0 weight producer, warp 1 MMA issuer, warps 2 .. 2+NDQ-1 dequantisation and epilogue, the last warp
// token-tile producer (quantised modes). The kernel is written for NDQ = 8 or 16; measurements on B200 favour 8 with two
// CTAs per SM for decode-sized quantised problems: the MMA-issuing warp, not the expansion arithmetic, is what limits
// a CTA there (its instructions issue several times slower while the dequant warps run), and two CTAs bring two issuers.
constexpr int num_dq_warps(int bt, int wmode) { (void)bt; (void)wmode; return 8; }
constexpr int gemm_threads(int bt, int wmode) { return (3 + num_dq_warps(bt, wmode)) * 32; }
constexpr int MAX_STAGES = 8;    // MMA stages
constexpr int MAX_PSLOTS = 16;   // packed-weight ring slots
constexpr int kBandN = 16;       // weight tiles per rasterisation band

struct GemmKParams {
    void* out;
    const void* bias;
    const void* residual;
    const uint32_t* sz;       // [K/group, N] pairs (bf16 scale, bf16 biased zero point)
    float* ws;
    int* counters;
    int* status;
    const uint8_t* w_tiled;   // non-null: weights in the tile-contiguous plugin layout (1-D bulk copies)
    int T, N, K;
    int ldo, ldr;
    int group_size;
    int act;
    int out_f32;
    int splits;
    int stages;               // MMA stages
    int pslots;               // packed ring slots (quantised modes)
    int kblocks_per_split;
    int w_kb_stride;          // chunks between consecutive weight tiles in memory (total k-blocks unless the weight is a window)
    // Tensor-parallel all-reduce fused into the epilogue (world <= 1: off). Every rank runs the same launch;
    // heap[r] is the symmetric heap of rank r mapped into this process (heap[rank] is local memory).
    int world, rank;
    int comm_mode;            // 1: one-shot (every rank gets every partial), 2: two-shot (tile owners reduce and broadcast)
    int parity;               // one-shot staging buffer to use (consecutive fused calls alternate)
    int packets;              // 1: partials travel as flag-carrying packets; 0: plain tiles, a fence and arrival flags
    int nvls;                 // reduce inside the switch (needs `mc`)
    int twohop;               // one-shot sizes on more than two ranks: packets to the share's owner, reduced shares broadcast as packets
    int site;                 // call site number (< 256): with the step number it makes the one-shot packets' tag unique
    uint8_t* heap[8];
    long long stage_off;      // staging area of the chosen mode (one-shot: of the chosen parity), offset in the heap
    long long flags_off;      // this call site's flags: [tile][world + 1] int32, offset in the heap
    long long out_off;        // `out` as an offset in the heap (two-shot owners write it on every rank)
    const int* epoch;         // device word holding the current step number (local memory)
    long long count_off;      // one int32 in the heap: CTAs of a two-shot launch that have finished their tile
    // NVLink multicast (NVLS): multicast mapping of the symmetric heap (NULL: plain peer stores, protocols above) and this
    // call site's barrier words, [tile][kNvlsFlagStride] int32, as an offset in the heap
    uint8_t* mc;
    long long nvls_flags_off;
    // Grouped GEMM (mixture of experts): the rows of X / out are grouped, group g owns rows [group_off[g], group_off[g + 1])
    // (device array, written by an earlier kernel of the stream) and uses weight g of a stack: group_mode 1 = the weights are
    // stacked along N (tile index g * tiles_n + n_tile), 2 = stacked along K (k-block offset g * K / 64). T is the row capacity.
    uint32_t spin_limit;      // polls before a wait on a peer gives up and reports STATUS_PEER_TIMEOUT
    int nvls_reducers;        // in-switch all-reduce: the first CTAs of the grid only reduce (0: every tile CTA reduces its own tile)
    const int* group_off;
    int num_groups;
    int group_mode;
};

// polls of a peer flag (~0.25 us apart) before a wait gives up: GemmKParams::spin_limit, set per launch from peer_spin_limit()

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

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

constexpr bool is_quant(int wmode) { return wmode == OVB_W_U4 || wmode == OVB_W_U8 || wmode == OVB_W_F8; }
constexpr int wq_bytes(int wmode) { return wmode == OVB_W_U4 ? TILE_N * 32 : ((wmode == OVB_W_U8 || wmode == OVB_W_F8) ? TILE_N * 64 : 0); }

// Four fp8 e4m3 bytes -> four bf16 (two words), each scaled: an e4m3 byte placed at bits 4..10 (sign at 15) of a bf16
// reads as value * 2^-120 (sub-normals included), and the per-block scale in `ss` already carries the 2^120.
__device__ __forceinline__ void dequant_f8x4(uint32_t w, __nv_bfloat162 ss, uint32_t& lo, uint32_t& hi) {
    const uint32_t y0 = __byte_perm(w, 0u, 0x4140), y1 = __byte_perm(w, 0u, 0x4342);
    uint32_t t0 = ((y0 << 8) & 0x80008000u) | ((y0 << 4) & 0x07F007F0u);
    uint32_t t1 = ((y1 << 8) & 0x80008000u) | ((y1 << 4) & 0x07F007F0u);
    __nv_bfloat162 v0 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&t0), ss);
    __nv_bfloat162 v1 = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&t1), ss);
    lo = *reinterpret_cast<uint32_t*>(&v0);
    hi = *reinterpret_cast<uint32_t*>(&v1);
}

// Tile order of the (non-grouped) kernel: bands of kBandN weight tiles; inside a band the token tiles advance slowest, so
// the CTAs that are resident together share a few weight tiles and a few token tiles in L2.
__device__ __forceinline__ void tile_coords(int idx, int N, int T, int bt, int& n_tile, int& t_tile) {
    const int tiles_n = (N + TILE_N - 1) / TILE_N;
    const int tiles_t = (T + bt - 1) / bt;
    const int band_sz = kBandN * tiles_t;
    const int band = idx / band_sz;
    const int r = idx - band * band_sz;
    const int in_band = min(kBandN, tiles_n - band * kBandN);
    t_tile = r / in_band;
    n_tile = band * kBandN + (r - t_tile * in_band);
}

// In-switch all-reduce, the reducing half: wait until every rank has posted its partial of tile `rt` (flag words of the tile
// >= epoch), then fetch the sum over the ranks of this rank's 1/W share of the tile (multimem.ld_reduce, fp32 accumulation in
// the switch) and write it to `out` on every rank (multimem.st). Called by `nthreads` threads (thread `tid`) that meet at
// named barrier `bar_id`; `wait_s` is one shared int. Returns false when the wait ran out (status already reported).
template <int BT>
__device__ __forceinline__ bool nvls_reduce_tile(const GemmKParams& p, int rt, int epoch, int tid, int nthreads, int bar_id, volatile int* wait_s,
                                                 volatile int* abort_flag) {
    constexpr int PIECES = BT * (TILE_N / 8);
    constexpr size_t SLOT = (size_t)BT * TILE_N * 2;
    const int W = p.world;
    const int* bar_local = reinterpret_cast<const int*>(p.heap[p.rank] + p.nvls_flags_off) + (size_t)rt * kNvlsFlagStride;
    if (tid == 0) {
        bool ok = false;
        for (uint32_t it = 0; it < p.spin_limit && !ok; ++it) {
            const uint4 a = ld_relaxed_sys_v4(bar_local), b = ld_relaxed_sys_v4(bar_local + 4);
            const int w[8] = {(int)a.x, (int)a.y, (int)a.z, (int)a.w, (int)b.x, (int)b.y, (int)b.z, (int)b.w};
            ok = true;
#pragma unroll
            for (int r = 0; r < 8; ++r) ok = ok && (r >= W || w[r] >= epoch);
            if (!ok) {
                if (abort_flag != nullptr && (it & 255u) == 255u && *abort_flag) break;
                if (it > 32) __nanosleep(100);
            }
        }
        if (ok) {
            fence_sys();
        } else {
            report_status(p.status, STATUS_PEER_TIMEOUT);
        }
        *wait_s = ok ? 1 : 0;
    }
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads));
    const bool ok = *wait_s != 0;
    if (ok) {
        int rn, rtt;
        tile_coords(rt, p.N, p.T, BT, rn, rtt);
        const int r_t0 = rtt * BT, r_n0 = rn * TILE_N, r_ntok = min(BT, p.T - r_t0);
        const size_t r_slot = (size_t)p.stage_off + (size_t)rt * SLOT;
        const int per = PIECES / W;                             // PIECES is a multiple of 256, W of 2, 4 or 8
        // batches of four reducing loads in flight per thread, then their stores (a load is a round trip to the switch)
        for (int k0 = tid; k0 < per; k0 += 4 * nthreads) {
            uint4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k = k0 + j * nthreads, i = p.rank * per + k;
                if (k < per && (i >> 4) < r_ntok) v[j] = multimem_ld_reduce_bf16x8(p.mc + r_slot + (size_t)i * 16);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k = k0 + j * nthreads, i = p.rank * per + k;
                const int col = i >> 4, pc = i & 15;
                if (k < per && col < r_ntok) multimem_st_b128(p.mc + (size_t)p.out_off + ((size_t)(r_t0 + col) * p.ldo + r_n0 + pc * 8) * 2, v[j]);
            }
        }
    }
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthreads));   // wait_s may be rewritten after this point
    return ok;
}

// Quantised stages cover two k-blocks (128 elements of K) except for 256-token tiles, whose token tile alone is 32 KB
// per k-block: every barrier round trip between the producers, the dequant warps and the MMA issuer then moves twice
// the data, which halves the per-byte cost of the control chain.
constexpr int kblocks_per_stage(int bt, int wmode) { return is_quant(wmode) && bt < 256 ? 2 : 1; }

// Decode-sized quantised problems run two CTAs per SM (half the shared memory and 256 TMEM columns each): one CTA's
// control chain (barrier round trips between the producers, the dequant warps and the MMA issuer) is latency bound, a
// second resident CTA fills the gaps.
constexpr bool two_ctas(int bt, int wmode) { return bt <= 64 && is_quant(wmode) && num_dq_warps(bt, wmode) == 8; }

template <int BT, int WMODE, bool F16>
__global__ void __launch_bounds__(gemm_threads(BT, WMODE), two_ctas(BT, WMODE) ? 2 : 1)
gemm_ws_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, GemmKParams p) {
    using E = typename Elem<F16>::type;
    constexpr bool QUANT = is_quant(WMODE);
    constexpr int KPS = kblocks_per_stage(BT, WMODE);   // k-blocks per pipeline stage (see STAGE_BYTES)
    constexpr int X_BYTES = BT * 128;
    constexpr int W_BYTES = TILE_N * 128;
    constexpr int WQ_BYTES = wq_bytes(WMODE);
    constexpr int ROW_PKT = WQ_BYTES / TILE_N;          // packed bytes per row and k-block
    constexpr int SZ_BYTES = QUANT ? TILE_N * 4 : 0;    // (scale, zero point) pairs of the tile's rows for one k-block
    constexpr int WQ_SLOT = WQ_BYTES + SZ_BYTES;        // one k-block in the ring: packed chunk, then its pairs
    constexpr int RING_SLOT = KPS * WQ_SLOT;            // one ring slot = the k-blocks of one stage
    // Quantised weights never touch shared memory in expanded form: the dequant warps write the bf16 tile straight
    // into tensor memory (tcgen05.st) and the MMA takes its A operand from there, so a stage holds the token tile only.
    constexpr int STAGE_BYTES = QUANT ? KPS * X_BYTES : X_BYTES + W_BYTES;
    constexpr int ACC_COLS = BT < 32 ? 32 : BT;
    constexpr int A_COLS = KPS * 32;                             // 128 rows x 64 bf16 = 32 columns of 32 bits per k-block
    constexpr int TMEM_COLS = !QUANT ? ACC_COLS : (two_ctas(BT, WMODE) ? 256 : 512);   // accumulator + the stages of A
    constexpr int NDQ = num_dq_warps(BT, WMODE);
    constexpr int DQ_THREADS = NDQ * 32;
    constexpr int X_PRODUCER_WARP = 2 + NDQ;
    // A group of four dequant warps (one per TMEM lane quarter) expands one k-block. A stage of KPS k-blocks is served by
    // KPS groups; with more groups than that the sets of groups take alternate iterations, so that one set expands stage
    // i + 1 while the MMAs of stage i still wait for the other.
    constexpr int GPS = KPS;
    constexpr int SETS = (NDQ / 4) / GPS;
    static_assert(SETS >= 1 && SETS * GPS * 4 == NDQ, "dequant warps must form whole sets of groups");

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int stages = p.stages;
    const int pslots = p.pslots;
    uint8_t* pring = smem + stages * STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(pring + pslots * RING_SLOT);
    uint64_t* full_x = bars;                         // [stages] token tile landed and (quantised modes) weight tile expanded into TMEM
    uint64_t* empty = bars + 2 * MAX_STAGES;         // [stages] MMAs that read the stage retired
    uint64_t* p_full = bars + 3 * MAX_STAGES;        // [pslots] packed chunk landed
    uint64_t* p_empty = p_full + MAX_PSLOTS;         // [pslots] packed chunk consumed
    uint64_t* acc_full = p_empty + MAX_PSLOTS;       // accumulator complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* last_flag = const_cast<int*>(abort_flag) + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // In-switch all-reduce with reducer CTAs: the first `nvls_reducers` CTAs of the grid (dispatched first, small enough to sit
    // beside a tile CTA on an SM) do nothing but reduce: reducer r takes tiles r, r + R, ... in the order in which the tile
    // CTAs post them. The tile CTAs store their partial, post and leave, so the tensor pipe never waits for the switch.
    const int cta = (int)blockIdx.x - p.nvls_reducers;   // tile index of this CTA (negative: a reducer)
    if (cta < 0) {
        volatile int* red_wait_s = last_flag;     // a word of the dynamic shared memory (no static shared memory in this kernel: it uses the whole opt-in limit)
        pdl_wait();
        const int epoch = __ldcg(p.epoch);
        const int R = p.nvls_reducers, tiles = (int)gridDim.x - R;
        bool ok = true;
        for (int rt = (int)blockIdx.x; rt < tiles && ok; rt += R)
            ok = nvls_reduce_tile<BT>(p, rt, epoch, (int)threadIdx.x, (int)blockDim.x, 2, red_wait_s, nullptr);
        // completion: the last reducer of this rank meets the other ranks' last reducers (words 8..15 of tile 0's flags), so
        // when the kernel ends on a rank every share of every tile has landed in its `out`
        __syncthreads();
        if (threadIdx.x == 0) {
            fence_sys();
            const int done = atomicAdd(p.counters, 1);
            if (done == R - 1) {
                *p.counters = 0;
                const int* bar_local = reinterpret_cast<const int*>(p.heap[p.rank] + p.nvls_flags_off) + 8;
                int* bar_mc = reinterpret_cast<int*>(p.mc + p.nvls_flags_off) + 8;
                if (!nvls_barrier(bar_local, bar_mc, p.rank, p.world, epoch, p.spin_limit, nullptr)) report_status(p.status, STATUS_PEER_TIMEOUT);
            }
        }
        return;
    }
    int n_tile, t_tile;
    int w_tile, w_kb0 = 0;          // weight tile and first k-block inside the (possibly stacked) weight
    int t0, T_end = p.T;            // first row of the tile, one past the last valid row
    if (p.group_off != nullptr) {
        // the offsets come from an earlier kernel of the stream: nothing of this CTA may run before that kernel is done
        pdl_wait();
        const int tiles_n = (p.N + TILE_N - 1) / TILE_N;
        int g = 0, acc = 0, begin = 0, end = 0;
        for (; g < p.num_groups; ++g) {
            begin = __ldg(p.group_off + g);
            end = __ldg(p.group_off + g + 1);
            const int cnt = ((end - begin + BT - 1) / BT) * tiles_n;
            if (cta < acc + cnt) break;
            acc += cnt;
        }
        if (g == p.num_groups) return;      // more CTAs than tiles (the grid is sized for the worst case); uniform over the CTA
        // inside a group the same banded order as the plain GEMM: resident CTAs share a few weight tiles and a few row tiles
        tile_coords(cta - acc, p.N, end - begin, BT, n_tile, t_tile);
        t0 = begin + t_tile * BT;
        T_end = min(end, p.T);
        w_tile = p.group_mode == 1 ? g * tiles_n + n_tile : n_tile;
        w_kb0 = p.group_mode == 2 ? g * ((p.K + TILE_K - 1) / TILE_K) : 0;
    } else {
        tile_coords(cta, p.N, p.T, BT, n_tile, t_tile);
        w_tile = n_tile;
        t0 = t_tile * BT;
    }
    const int n0 = n_tile * TILE_N;
    const int split = p.splits > 1 ? (int)cluster_ctarank() : 0;   // the splits of a tile are one cluster along z
    const int total_kb = (p.K + TILE_K - 1) / TILE_K;
    const int kb_begin = split * p.kblocks_per_split;
    const int kb_end = min(total_kb, kb_begin + p.kblocks_per_split);
    const int num_kb = max(0, kb_end - kb_begin);
    const int num_it = (num_kb + KPS - 1) / KPS;         // stage iterations of the main loop
    // dequant warps per MMA stage: with few stages two warps share one k-block (64 rows each)

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&full_x[s], QUANT ? 1 + 4 * GPS : 1);   // producer's expect_tx arrival (+ one arrival per dequant warp of the stage)
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < pslots; ++s) {
            mbar_init(&p_full[s], 1);
            mbar_init(&p_empty[s], 4 * GPS);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        *last_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmX);
        if (!QUANT && p.w_tiled == nullptr) tma_prefetch_desc(&tmW);
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
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            if (QUANT) {
                // Weight producer: one ring slot per k-block, requested up to `pslots` k-blocks ahead of use. A u4 slot is
                // ONE bulk copy: the packed chunk and the (scale, zero point) pairs of its rows are stored together.
                // (Every instruction of this single-lane loop is on the critical path of the whole CTA: no divisions,
                // running pointers only. The token tiles have a producer lane of their own in warp X_PRODUCER_WARP.)
                int wslot = 0;
                uint32_t wpar = 1;                    // parity to wait for on the "empty" barriers
                const uint8_t* wsrc = p.w_tiled + ((size_t)w_tile * p.w_kb_stride + w_kb0 + kb_begin) * (WMODE == OVB_W_U4 ? WQ_SLOT : WQ_BYTES);
                uint32_t wdst = smem_u32(pring);
                // u8: pairs come from the [group][N] table with a second copy
                const int kpg = p.group_size / TILE_K;
                int gk = kb_begin % kpg;
                const uint32_t* zsrc = p.sz + (size_t)(kb_begin / kpg) * p.N + n0;
                int kcoord = kb_begin * TILE_K;
                for (int iw = 0; iw < num_it; ++iw) {
                    if (!mbar_wait(&p_empty[wslot], wpar, abort_flag, p.status)) break;
                    const int nk = min(KPS, num_kb - iw * KPS);
                    mbar_arrive_expect_tx(&p_full[wslot], nk * WQ_SLOT);
                    if (WMODE == OVB_W_U4) {
                        // consecutive k-blocks of a tile are consecutive chunks in memory: one copy brings the whole stage
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(wdst), "l"(wsrc), "r"(nk * WQ_SLOT), "r"(smem_u32(&p_full[wslot])) : "memory");
                        wsrc += KPS * WQ_SLOT;
                    } else {
                        for (int t = 0; t < nk; ++t) {
                            tma_load_2d(pring + wslot * RING_SLOT + t * WQ_SLOT, &tmW, &p_full[wslot], kcoord, n0);
                            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                         ::"r"(wdst + t * WQ_SLOT + WQ_BYTES), "l"(zsrc), "r"(SZ_BYTES), "r"(smem_u32(&p_full[wslot])) : "memory");
                            kcoord += TILE_K;
                            if (++gk == kpg) { gk = 0; zsrc += p.N; }
                        }
                    }
                    wdst += RING_SLOT;
                    if (++wslot == pslots) { wslot = 0; wpar ^= 1; wdst = smem_u32(pring); }
                }
            } else {
                auto load_w = [&](int s, int kb) {
                    uint8_t* st = smem + s * STAGE_BYTES;
                    if (p.w_tiled != nullptr)
                        bulk_load_1d(st + X_BYTES, p.w_tiled + ((size_t)w_tile * p.w_kb_stride + w_kb0 + kb) * W_BYTES, W_BYTES, &full_x[s]);
                    else
                        tma_load_2d(st + X_BYTES, &tmW, &full_x[s], kb * TILE_K, n0);
                };
                // Weights are constants: the first ring of weight tiles is requested before the kernel that produces
                // the activations has finished (programmatic dependent launch); the token tiles follow after the wait.
                const int pre = min(stages, num_kb);
                for (int i = 0; i < pre; ++i) {
                    mbar_arrive_expect_tx(&full_x[i], X_BYTES + W_BYTES);
                    load_w(i, kb_begin + i);
                }
                pdl_wait();
                if (OVB_PDL_GEMM == 2) pdl_trigger();
                for (int i = 0; i < pre; ++i) tma_load_2d(smem + i * STAGE_BYTES, &tmX, &full_x[i], (kb_begin + i) * TILE_K, t0);
                uint32_t phase = pre == stages ? 1 : 0;
                int s = pre == stages ? 0 : pre;
                for (int i = pre; i < num_kb; ++i) {
                    if (!mbar_wait(&empty[s], phase ^ 1, abort_flag, p.status)) break;
                    const int kb = kb_begin + i;
                    mbar_arrive_expect_tx(&full_x[s], X_BYTES + W_BYTES);
                    tma_load_2d(smem + s * STAGE_BYTES, &tmX, &full_x[s], kb * TILE_K, t0);
                    load_w(s, kb);
                    if (++s == stages) { s = 0; phase ^= 1; }
                }
                if (OVB_PDL_GEMM == 1) pdl_trigger();
            }
        }
        __syncwarp();
    } else if (warp == X_PRODUCER_WARP) {
        // ------------------------------------------------------------ token-tile producer (quantised modes only)
        if (QUANT && lane == 0) {
            uint32_t xpar = 1;
            int xs = 0;
            int xk = kb_begin * TILE_K;
            uint32_t xdst = smem_u32(smem);
            // the activations come from the kernel before this one; the weight producer (constants) does not wait
            pdl_wait();
            if (OVB_PDL_GEMM == 2) pdl_trigger();
            for (int ix = 0; ix < num_it; ++ix) {
                if (!mbar_wait(&empty[xs], xpar, abort_flag, p.status)) break;
                const int nk = min(KPS, num_kb - ix * KPS);
                mbar_arrive_expect_tx(&full_x[xs], nk * X_BYTES);
                for (int t = 0; t < nk; ++t) {
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                        ::"r"(xdst + t * X_BYTES), "l"(reinterpret_cast<uint64_t>(&tmX)), "r"(smem_u32(&full_x[xs])), "r"(xk), "r"(t0)
                        : "memory");
                    xk += TILE_K;
                }
                xdst += STAGE_BYTES;
                if (++xs == stages) { xs = 0; xpar ^= 1; xdst = smem_u32(smem); }
            }
            if (OVB_PDL_GEMM == 1) pdl_trigger();
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp runs the loop with warp-uniform control flow and elect.sync picks the lane that issues:
        // descriptors then live in uniform registers and the four MMAs of a k-block issue back to back (a loop under
        // `if (lane == 0)` costs about twice the cycles per k-block on the issuing thread).
        constexpr uint32_t idesc = umma_idesc_f16(TILE_N, BT, !F16);
        const uint64_t desc0 = umma_desc_k_sw128(smem_u32(smem), 1024);
        {
            uint32_t phase = 0;
            int s = 0;
            for (int i = 0; i < (QUANT ? num_it : num_kb); ++i) {
                // every lane polls the same barrier word (no divergence, no shuffle): one wait per stage covers both the
                // token tile and the expanded weights
                const bool ok = mbar_wait(&full_x[s], phase, abort_flag, p.status);
                if (!ok) break;
                tc_fence_after_sync();
                // descriptors differ only in the 16-byte-unit start address (low 14 bits, no carry out here)
                const uint64_t db0 = desc0 + (uint64_t)((s * STAGE_BYTES) >> 4);
                const uint32_t acc_first = i > 0 ? 1u : 0u;
                if (QUANT) {
                    const uint32_t a0 = tmem_base + uint32_t(ACC_COLS + s * A_COLS);   // 8 columns per K=16 slice
                    umma_f16_ts_elect(tmem_base, a0, db0, idesc, acc_first);
#pragma unroll
                    for (int k = 1; k < TILE_K / 16; ++k) umma_f16_ts_elect(tmem_base, a0 + 8 * k, db0 + 2 * k, idesc, 1u);
                    if (KPS == 2 && num_kb - i * KPS > 1) {                            // second k-block of the stage
                        const uint64_t db1 = db0 + (uint64_t)(X_BYTES >> 4);
#pragma unroll
                        for (int k = 0; k < TILE_K / 16; ++k) umma_f16_ts_elect(tmem_base, a0 + 32 + 8 * k, db1 + 2 * k, idesc, 1u);
                    }
                } else {
                    const uint64_t da0 = db0 + (uint64_t)(X_BYTES >> 4);
                    umma_f16_ss_elect(tmem_base, da0, db0, idesc, acc_first);
#pragma unroll
                    for (int k = 1; k < TILE_K / 16; ++k) umma_f16_ss_elect(tmem_base, da0 + 2 * k, db0 + 2 * k, idesc, 1u);
                }
                umma_commit_elect(&empty[s]);
                if (++s == stages) { s = 0; phase ^= 1; }
            }
            umma_commit_elect(acc_full);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ dequant warps, then epilogue
        const int dq_tid = threadIdx.x - 64;  // 0..255
        if (QUANT) {
            // Group g belongs to set g / GPS and expands k-block g % GPS of the stages that its set serves. Inside a group a
            // warp owns the 32 rows of its TMEM lane quarter; a thread expands the 64 values of one row and writes them to
            // tensor memory as 32 columns of bf16 pairs (two tcgen05.st).
            const int grp = (warp - 2) >> 2;
            const int set = grp / GPS, kin = grp % GPS;
            const int qd = warp & 3;                    // TMEM lane quarter this warp may access
            const int row = qd * 32 + lane;
            const bool row_ok = (n0 + row) < p.N;
            int slot = set, st = set;                   // ring lengths are multiples of SETS (host side): an entry has one owner set
            uint32_t ppar = 0, phase = 0;
            const uint32_t a_lane = tmem_base + (uint32_t(qd * 32) << 16) + uint32_t(ACC_COLS + kin * 32);
            for (int i = set; i < num_it; i += SETS) {
                // every lane polls (same word, same answer): no divergence and no shuffle on the way to the work
                bool ok = mbar_wait(&p_full[slot], ppar, abort_flag, p.status);
                ok = ok && mbar_wait(&empty[st], phase ^ 1, abort_flag, p.status);
                if (!ok) break;
                const uint32_t slot_a = smem_u32(pring + slot * RING_SLOT + kin * WQ_SLOT);
                if (i * KPS + kin < num_kb) {
                uint32_t cur;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(cur) : "r"(slot_a + WQ_BYTES + row * 4));
                if (!row_ok) cur = 0u;          // rows past N: scale 0
                const __nv_bfloat162 szp = *reinterpret_cast<const __nv_bfloat162*>(&cur);
                uint32_t r[32];
                if (WMODE == OVB_W_U4) {
                    const __nv_bfloat162 ss2 = __halves2bfloat162(__low2bfloat16(szp), __low2bfloat16(szp));
                    const __nv_bfloat162 zz2 = __halves2bfloat162(__high2bfloat16(szp), __high2bfloat16(szp));
                    const uint4 pk0 = lds128(slot_a + row * 16), pk1 = lds128(slot_a + TILE_N * 16 + row * 16);
                    const uint32_t xs[8] = {pk0.x, pk0.y, pk0.z, pk0.w, pk1.x, pk1.y, pk1.z, pk1.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint4 e = dequant_u4x8(xs[j], zz2, ss2);
                        r[4 * j] = e.x; r[4 * j + 1] = e.y; r[4 * j + 2] = e.z; r[4 * j + 3] = e.w;
                    }
                } else if (WMODE == OVB_W_F8) {
                    const __nv_bfloat162 ss2 = __halves2bfloat162(__low2bfloat16(szp), __low2bfloat16(szp));
#pragma unroll
                    for (int h = 0; h < 4; ++h) {
                        const uint4 pk = lds128(slot_a + row * ROW_PKT + h * 16);
                        dequant_f8x4(pk.x, ss2, r[h * 8 + 0], r[h * 8 + 1]);
                        dequant_f8x4(pk.y, ss2, r[h * 8 + 2], r[h * 8 + 3]);
                        dequant_f8x4(pk.z, ss2, r[h * 8 + 4], r[h * 8 + 5]);
                        dequant_f8x4(pk.w, ss2, r[h * 8 + 6], r[h * 8 + 7]);
                    }
                } else {
                    const float sf = __bfloat162float(__low2bfloat16(szp));
                    const float zf = __bfloat162float(__high2bfloat16(szp));
#pragma unroll
                    for (int h = 0; h < 4; ++h) {
                        const uint4 pk = lds128(slot_a + row * ROW_PKT + h * 16);
                        const uint32_t b[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const uint32_t w32 = b[e >> 1];
                            const int sh = (e & 1) * 16;
                            r[h * 8 + e] = pack_bf16x2((float((w32 >> sh) & 0xFF) - zf) * sf, (float((w32 >> (sh + 8)) & 0xFF) - zf) * sf);
                        }
                    }
                }
                tmem_st_x16(a_lane + uint32_t(st * A_COLS), r);
                tmem_st_x16(a_lane + uint32_t(st * A_COLS + 16), r + 16);
                tmem_st_wait();
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&full_x[st]);
                    mbar_arrive(&p_empty[slot]);
                }
                st += SETS;
                if (st >= stages) { st -= stages; phase ^= 1; }
                slot += SETS;
                if (slot >= pslots) { slot -= pslots; ppar ^= 1; }
            }
        }

        // -------- epilogue: warp (w % 4) owns TMEM lanes 32*(w%4) .. +31; two warps share a quarter
        const int q = warp & 3;
        const int colpart = (warp - 2) >> 2;  // which slice of the token columns this warp drains
        const int row = q * 32 + lane;
        const int oc = n0 + row;
        constexpr int PARTS = (NDQ / 4) < (BT / 16) ? (NDQ / 4) : (BT / 16);   // column slices, 16 columns at least
        constexpr int COLS_PER_WARP = BT / PARTS;
        constexpr int CHUNKS = COLS_PER_WARP / 16;
        const int cbeg = colpart * COLS_PER_WARP;
        const bool active_warp = colpart < PARTS;
        // one thread polls the accumulator barrier; the other 255 park at a hardware named barrier
        if (dq_tid == 0 && num_kb > 0) mbar_wait(acc_full, 0, abort_flag, p.status);
        asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
        const bool acc_ok = (*abort_flag == 0);
        tc_fence_after_sync();
        pdl_wait();   // the epilogue reads the residual and writes the output: both belong to the stream's earlier kernels until now

        const float bias_v = (p.bias != nullptr && oc < p.N) ? to_float(reinterpret_cast<const E*>(p.bias)[oc]) : 0.f;
        const int tile_id = cta;
        // Fast path: whole 128-row tile inside N, 16-bit output with 16-byte aligned rows. The tile is staged
        // in shared memory as [token][128] (the pipeline stages are free by now) and written with 16-byte
        // stores that cover 256 contiguous bytes per token row.
        const bool fast = p.world <= 1 && p.splits == 1 && !p.out_f32 && (n0 + TILE_N <= p.N) && (p.ldo % 8 == 0) &&
                          ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                          (p.residual == nullptr || ((p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0)));
        // fp32 staging keeps a single rounding (after the residual add): BT x 128 x 4 bytes <= 2 * STAGE_BYTES
        float* stage_out = reinterpret_cast<float*>(smem);

        // ---- tensor-parallel: the fp32 partial tile in stage_out is summed over the ranks (see GemmKParams)
        const bool comm = p.world > 1;
        auto comm_epilogue = [&](bool tile_ok) {
            const int ntok = min(BT, T_end - t0);
            const int epoch = __ldcg(p.epoch);
            constexpr int PIECES = BT * (TILE_N / 8);               // 16-byte pieces of the bf16 tile
            constexpr size_t SLOT = (size_t)BT * TILE_N * 2;        // bytes of one bf16 tile
            const int tiles = (int)gridDim.x - p.nvls_reducers;
            const int W = p.world;
            if (p.nvls) {
                // In-switch all-reduce (NVLS). Every rank stores its bf16 partial tile in its OWN staging slot (rank 0 adds
                // bias and residual first, so the switch's sum is the finished value and is rounded once), the ranks meet at
                // the tile's barrier, then rank r fetches the sum over all ranks of its 1/W share of the tile with
                // multimem.ld_reduce and writes it to `out` on every rank with multimem.st. A second barrier tells every
                // rank that all shares have landed. Each piece is reduced exactly once, so all ranks hold the same bits.
                // Traffic per rank and tile: one tile out (pulled by the switch), one tile in.
                if (!tile_ok) return;
                uint8_t* my_heap = p.heap[p.rank];
                const size_t slot_off = (size_t)p.stage_off + (size_t)tile_id * SLOT;
                for (int i = dq_tid; i < PIECES; i += DQ_THREADS) {
                    const int col = i >> 4, pc = i & 15;
                    if (col >= ntok) continue;
                    const float4 f0 = *reinterpret_cast<const float4*>(stage_out + col * TILE_N + pc * 8);
                    const float4 f1 = *reinterpret_cast<const float4*>(stage_out + col * TILE_N + pc * 8 + 4);
                    float f[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
                    if (p.rank == 0) {
                        const size_t tok = (size_t)(t0 + col);
                        if (p.bias) {
                            const uint4 bb = *reinterpret_cast<const uint4*>(reinterpret_cast<const E*>(p.bias) + n0 + pc * 8);
                            const E* be = reinterpret_cast<const E*>(&bb);
#pragma unroll
                            for (int j = 0; j < 8; ++j) f[j] += to_float(be[j]);
                        }
                        if (p.residual) {
                            const uint4 rr = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const E*>(p.residual) + tok * p.ldr + n0 + pc * 8));
                            const E* re = reinterpret_cast<const E*>(&rr);
#pragma unroll
                            for (int j = 0; j < 8; ++j) f[j] += to_float(re[j]);
                        }
                    }
                    *reinterpret_cast<uint4*>(my_heap + slot_off + (size_t)i * 16) =
                        make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
                }
                // Post: tell every rank that this rank's partial of the tile is in place (release: CTA barrier, then fence + flag).
                asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
                if (dq_tid == 0) {
                    fence_sys();
                    multimem_st_u32(reinterpret_cast<int*>(p.mc + p.nvls_flags_off) + (size_t)tile_id * kNvlsFlagStride + p.rank, (uint32_t)epoch);
                }
                if (p.nvls_reducers > 0) return;      // the reducer CTAs take it from here
                // No reducer CTAs (a launch of a single wave, e.g. a decode step): this CTA waits for the other ranks' copies of
                // its own tile and reduces its share.
                if (!nvls_reduce_tile<BT>(p, tile_id, epoch, dq_tid, DQ_THREADS, 1, last_flag, abort_flag)) {
                    if (dq_tid == 0) *abort_flag = 1;
                    return;
                }
                // Completion: the last CTA of this rank to get here meets the other ranks' last CTAs (words 8..15 of tile 0's
                // flags), so when the kernel ends on a rank every share of every tile has landed in its `out`, and every
                // rank is done reading the staging slots.
                if (dq_tid == 0) {
                    fence_sys();
                    const int done = atomicAdd(p.counters, 1);
                    if (done == tiles - 1) {
                        *p.counters = 0;
                        const int* bar_local = reinterpret_cast<const int*>(my_heap + p.nvls_flags_off) + 8;
                        int* bar_mc = reinterpret_cast<int*>(p.mc + p.nvls_flags_off) + 8;
                        if (!nvls_barrier(bar_local, bar_mc, p.rank, W, epoch, p.spin_limit, abort_flag)) report_status(p.status, STATUS_PEER_TIMEOUT);
                    }
                }
                return;
            }
            auto flags_of = [&](int r) { return reinterpret_cast<int*>(p.heap[r] + p.flags_off) + (size_t)tile_id * (W + 1); };
            int* my_flags = flags_of(p.rank);
            auto wait_flag = [&](const int* f) {
                for (uint32_t i = 0; i < p.spin_limit; ++i) {
                    if (ld_acquire_sys(f) >= epoch) return;
                    if ((i & 255u) == 255u && *abort_flag) return;
                    __nanosleep(200);
                }
                report_status(p.status, STATUS_PEER_TIMEOUT);
                *abort_flag = 1;
            };
            auto partial_piece = [&](int col, int pc) {
                const float4 f0 = *reinterpret_cast<const float4*>(stage_out + col * TILE_N + pc * 8);
                const float4 f1 = *reinterpret_cast<const float4*>(stage_out + col * TILE_N + pc * 8 + 4);
                return make_uint4(pack_bf16x2(f0.x, f0.y), pack_bf16x2(f0.z, f0.w), pack_bf16x2(f1.x, f1.y), pack_bf16x2(f1.z, f1.w));
            };
            // sum of the W bf16 partials of one piece (rank order, so every rank gets the same bits) + bias + residual
            auto reduced_piece = [&](const uint8_t* slots, size_t slot_stride, int col, int pc) {
                float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int r = 0; r < W; ++r) {
                    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(slots + (size_t)r * slot_stride + ((size_t)col * TILE_N + pc * 8) * 2));
                    const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
                    for (int j = 0; j < 8; ++j) f[j] += __bfloat162float(e[j]);
                }
                const size_t tok = (size_t)(t0 + col);
                if (p.bias) {
                    const uint4 bb = *reinterpret_cast<const uint4*>(reinterpret_cast<const E*>(p.bias) + n0 + pc * 8);
                    const E* be = reinterpret_cast<const E*>(&bb);
#pragma unroll
                    for (int j = 0; j < 8; ++j) f[j] += to_float(be[j]);
                }
                if (p.residual) {
                    const uint4 rr = *reinterpret_cast<const uint4*>(reinterpret_cast<const E*>(p.residual) + tok * p.ldr + n0 + pc * 8);
                    const E* re = reinterpret_cast<const E*>(&rr);
#pragma unroll
                    for (int j = 0; j < 8; ++j) f[j] += to_float(re[j]);
                }
                uint4 v;
                E* ve = reinterpret_cast<E*>(&v);
#pragma unroll
                for (int j = 0; j < 8; ++j) ve[j] = from_float<E>(f[j]);
                return v;
            };
            // Packets: sums the W partials of one piece in rank order (this rank's from shared memory, the peers' from their
            // packets in `slots`), polling until every packet carries `tag`. The packets of LLB ranks are fetched together,
            // so their loads are in flight at the same time.
            constexpr int LLB = BT > 64 ? 8 : 2;
            auto packet_sum = [&](const uint8_t* slots, size_t slot_stride, int col, int pc, uint32_t tag, float* f) -> bool {
                const size_t poff = ((size_t)col * TILE_N + pc * 8) * 4;
                for (int r0 = 0; r0 < W; r0 += LLB) {
                    uint4 a[LLB], b[LLB];
#pragma unroll
                    for (int j = 0; j < LLB; ++j) {
                        const int r = r0 + j;
                        if (r < W && r != p.rank) {
                            const uint8_t* src = slots + (size_t)r * slot_stride + poff;
                            a[j] = ld_volatile_v4(src);
                            b[j] = ld_volatile_v4(src + 16);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < LLB; ++j) {
                        const int r = r0 + j;
                        if (r < W) {
                            uint4 v;
                            if (r == p.rank) {
                                v = partial_piece(col, pc);
                            } else {
                                const uint8_t* src = slots + (size_t)r * slot_stride + poff;
                                uint32_t spins = 0;
                                while (!(a[j].y == tag && a[j].w == tag && b[j].y == tag && b[j].w == tag)) {
                                    if (++spins > p.spin_limit || ((spins & 1023u) == 0 && *abort_flag)) return false;
                                    if (spins > 64) __nanosleep(100);
                                    a[j] = ld_volatile_v4(src);
                                    b[j] = ld_volatile_v4(src + 16);
                                }
                                v = make_uint4(a[j].x, a[j].z, b[j].x, b[j].z);
                            }
                            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
                            for (int k = 0; k < 8; ++k) f[k] += __bfloat162float(e[k]);
                        }
                    }
                }
                return true;
            };
            // bias + residual on top of the summed piece, rounded once to the output type
            auto finish_piece = [&](float* f, int col, int pc) {
                const size_t tok = (size_t)(t0 + col);
                if (p.bias) {
                    const uint4 bb = *reinterpret_cast<const uint4*>(reinterpret_cast<const E*>(p.bias) + n0 + pc * 8);
                    const E* be = reinterpret_cast<const E*>(&bb);
#pragma unroll
                    for (int j = 0; j < 8; ++j) f[j] += to_float(be[j]);
                }
                if (p.residual) {
                    const uint4 rr = *reinterpret_cast<const uint4*>(reinterpret_cast<const E*>(p.residual) + tok * p.ldr + n0 + pc * 8);
                    const E* re = reinterpret_cast<const E*>(&rr);
#pragma unroll
                    for (int j = 0; j < 8; ++j) f[j] += to_float(re[j]);
                }
                uint4 o;
                E* oe = reinterpret_cast<E*>(&o);
#pragma unroll
                for (int j = 0; j < 8; ++j) oe[j] = from_float<E>(f[j]);
                return o;
            };
            constexpr size_t LL_SLOT = 2 * SLOT;
            // two call sites share a staging buffer within a step, so the tag names the site as well as the step
            const uint32_t tag = packet_tag(epoch, p.site);
            if (!tile_ok && !(p.comm_mode == 2 && p.packets)) return;
            if (p.comm_mode == 1 && p.twohop) {
                // Two hops of flag-carrying packets, no fence and no flag anywhere. Rank q owns the q-th share (PIECES / W
                // consecutive 16-byte pieces) of every tile. Hop 1: every rank sends each piece of its bf16 partial to the
                // piece's owner only. The owner polls the packets of its share, sums them in rank order, adds bias and
                // residual, and (hop 2) sends the finished piece to every rank as a packet: one multimem.st through the switch
                // when the heap has a multicast mapping, else one store per rank. Every rank then polls the finished pieces
                // of the whole tile in its own memory and writes its own copy of `out`. Per rank and tile this moves
                // (1 - 1/W) + 1 packet tiles in and, with multicast, (1 - 1/W) + 1/W out; pushing every partial to every
                // rank moves W - 1 both ways. Each piece is summed once, by its owner: all ranks get the same bits.
                const int share = PIECES / W;
                uint8_t* mine = p.heap[p.rank] + p.stage_off;
                for (int i = dq_tid; i < PIECES; i += DQ_THREADS) {
                    const int col = i >> 4, owner = twohop_owner(i, share);
                    if (col >= ntok || owner == p.rank) continue;
                    const uint4 v = partial_piece(col, i & 15);
                    uint8_t* d = p.heap[owner] + p.stage_off + twohop_hop1_offset(p.rank, tiles, tile_id, share, i - owner * share);
                    st_volatile_v4(d, v.x, tag, v.y, tag);
                    st_volatile_v4(d + 16, v.z, tag, v.w, tag);
                }
                bool ok_ll = true;
                // packet_sum() adds (col * 128 + pc * 8) * 4 = i * 32 with i = rank * share + k to this base
                const uint8_t* share_slots = mine + (ptrdiff_t)twohop_hop1_offset(0, tiles, tile_id, share, 0) - (ptrdiff_t)p.rank * share * kPacketBytes;
                for (int k = dq_tid; k < share && ok_ll; k += DQ_THREADS) {
                    const int i = p.rank * share + k, col = i >> 4, pc = i & 15;
                    if (col >= ntok) continue;
                    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    ok_ll = packet_sum(share_slots, twohop_hop1_offset(1, tiles, 0, share, 0), col, pc, tag, f);
                    if (!ok_ll) break;
                    const uint4 o = finish_piece(f, col, pc);
                    const size_t off = (size_t)p.stage_off + twohop_hop2_offset(tiles, PIECES, tile_id, i);
                    if (p.mc != nullptr) {
                        multimem_st_b128(p.mc + off, make_uint4(o.x, tag, o.y, tag));
                        multimem_st_b128(p.mc + off + 16, make_uint4(o.z, tag, o.w, tag));
                    } else {
                        for (int r = 0; r < W; ++r) {
                            st_volatile_v4(p.heap[r] + off, o.x, tag, o.y, tag);
                            st_volatile_v4(p.heap[r] + off + 16, o.z, tag, o.w, tag);
                        }
                    }
                }
                const uint8_t* done = mine + twohop_hop2_offset(tiles, PIECES, tile_id, 0);
                for (int i0 = dq_tid; i0 < PIECES && ok_ll; i0 += 2 * DQ_THREADS) {
                    // two pieces per round: their loads are in flight together
                    uint4 a[2], b[2];
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int i = i0 + j * DQ_THREADS;
                        if (i < PIECES && (i >> 4) < ntok) {
                            a[j] = ld_volatile_v4(done + (size_t)i * 32);
                            b[j] = ld_volatile_v4(done + (size_t)i * 32 + 16);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int i = i0 + j * DQ_THREADS;
                        if (i >= PIECES || (i >> 4) >= ntok) continue;
                        uint32_t spins = 0;
                        while (!(a[j].y == tag && a[j].w == tag && b[j].y == tag && b[j].w == tag)) {
                            if (++spins > p.spin_limit || ((spins & 1023u) == 0 && *abort_flag)) { ok_ll = false; break; }
                            if (spins > 64) __nanosleep(100);
                            a[j] = ld_volatile_v4(done + (size_t)i * 32);
                            b[j] = ld_volatile_v4(done + (size_t)i * 32 + 16);
                        }
                        if (!ok_ll) break;
                        *reinterpret_cast<uint4*>(reinterpret_cast<E*>(p.out) + (size_t)(t0 + (i >> 4)) * p.ldo + n0 + (i & 15) * 8) =
                            make_uint4(a[j].x, a[j].z, b[j].x, b[j].z);
                    }
                }
                if (!ok_ll) {
                    report_status(p.status, STATUS_PEER_TIMEOUT);
                    *abort_flag = 1;
                }
            } else if (p.comm_mode == 1 && p.packets) {
                // One-shot with flag-carrying packets: every 16-byte store holds two (data word, tag) pairs, so the
                // receiver sees data and "it has arrived" in the same 8-byte unit and needs neither a fence nor a flag
                // round trip. A thread pushes its pieces of the bf16 partial to every peer, then polls the same pieces
                // of every peer's partial in its own staging area and sums in rank order (identical bits on all ranks;
                // its own partial is rounded to bf16 like the copies the peers receive).
                const size_t my_slot = (size_t)p.stage_off + ((size_t)p.rank * tiles + tile_id) * LL_SLOT;
                for (int i = dq_tid; i < PIECES; i += DQ_THREADS) {
                    const int col = i >> 4, pc = i & 15;
                    if (col < ntok) {
                        const uint4 v = partial_piece(col, pc);
                        const size_t off = my_slot + ((size_t)col * TILE_N + pc * 8) * 4;
                        for (int r = 0; r < W; ++r) {
                            if (r == p.rank) continue;
                            st_volatile_v4(p.heap[r] + off, v.x, tag, v.y, tag);
                            st_volatile_v4(p.heap[r] + off + 16, v.z, tag, v.w, tag);
                        }
                    }
                }
                const uint8_t* slots = p.heap[p.rank] + p.stage_off + (size_t)tile_id * LL_SLOT;
                bool ok_ll = true;
                for (int i = dq_tid; i < PIECES && ok_ll; i += DQ_THREADS) {
                    const int col = i >> 4, pc = i & 15;
                    if (col >= ntok) continue;
                    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    ok_ll = packet_sum(slots, (size_t)tiles * LL_SLOT, col, pc, tag, f);
                    if (ok_ll)
                        *reinterpret_cast<uint4*>(reinterpret_cast<E*>(p.out) + (size_t)(t0 + col) * p.ldo + n0 + pc * 8) = finish_piece(f, col, pc);
                }
                if (!ok_ll) {
                    report_status(p.status, STATUS_PEER_TIMEOUT);
                    *abort_flag = 1;
                }
            } else if (p.comm_mode == 1) {
                    // one-shot: push the partial to every rank, then every rank reduces the tile for itself
                    const size_t slot = (size_t)p.stage_off + ((size_t)p.rank * tiles + tile_id) * SLOT;
                    for (int i = dq_tid; i < PIECES; i += DQ_THREADS) {
                        const int col = i >> 4, pc = i & 15;
                        if (col < ntok) {
                            const uint4 v = partial_piece(col, pc);
                            for (int r = 0; r < W; ++r)
                                *reinterpret_cast<uint4*>(p.heap[r] + slot + ((size_t)col * TILE_N + pc * 8) * 2) = v;
                        }
                    }
                    __threadfence_system();
                    asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
                    if (dq_tid < W) {
                        st_release_sys(flags_of(dq_tid) + p.rank, epoch);
                        wait_flag(my_flags + dq_tid);
                    }
                    asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
                    if (*abort_flag == 0) {
                        const uint8_t* slots = p.heap[p.rank] + p.stage_off + (size_t)tile_id * SLOT;
                        for (int i = dq_tid; i < PIECES; i += DQ_THREADS) {
                            const int col = i >> 4, pc = i & 15;
                            if (col < ntok)
                                *reinterpret_cast<uint4*>(reinterpret_cast<E*>(p.out) + (size_t)(t0 + col) * p.ldo + n0 + pc * 8) =
                                    reduced_piece(slots, (size_t)tiles * SLOT, col, pc);
                        }
                    }
            } else if (p.packets) {
                if (tile_ok) {
                // Two-shot: the owner of the tile (tile_id mod W) collects the partials, reduces, and writes the finished
                // tile into `out` on every rank. The partials travel as flag-carrying packets, so a CTA that does not
                // own its tile stores and leaves: no fence, no flag, no wait, and the SM goes on to the next tile. Only
                // the last CTA of the launch to get here waits (bounded) until the owners on the other ranks have
                // delivered every tile, which also tells it that they are done reading this rank's partials.
                const int owner = tile_id % W, own_idx = tile_id / W, own_cap = (tiles + W - 1) / W;
                if (p.rank != owner) {
                    uint8_t* dst = p.heap[owner] + p.stage_off + ((size_t)p.rank * own_cap + own_idx) * LL_SLOT;
                    for (int i = dq_tid; i < PIECES; i += DQ_THREADS) {
                        const int col = i >> 4, pc = i & 15;
                        if (col < ntok) {
                            const uint4 v = partial_piece(col, pc);
                            uint8_t* d = dst + ((size_t)col * TILE_N + pc * 8) * 4;
                            st_volatile_v4(d, v.x, tag, v.y, tag);
                            st_volatile_v4(d + 16, v.z, tag, v.w, tag);
                        }
                    }
                } else {
                    const uint8_t* slots = p.heap[p.rank] + p.stage_off + (size_t)own_idx * LL_SLOT;
                    bool ok_ll = true;
                    for (int i = dq_tid; i < PIECES && ok_ll; i += DQ_THREADS) {
                        const int col = i >> 4, pc = i & 15;
                        if (col >= ntok) continue;
                        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                        ok_ll = packet_sum(slots, (size_t)own_cap * LL_SLOT, col, pc, tag, f);
                        if (ok_ll) {
                            const uint4 o = finish_piece(f, col, pc);
                            const size_t off = (size_t)p.out_off + ((size_t)(t0 + col) * p.ldo + n0 + pc * 8) * 2;
                            for (int r = 0; r < W; ++r) *reinterpret_cast<uint4*>(p.heap[r] + off) = o;
                        }
                    }
                    if (!ok_ll) {
                        report_status(p.status, STATUS_PEER_TIMEOUT);
                        *abort_flag = 1;
                    }
                    __threadfence_system();
                    asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
                    if (*abort_flag == 0 && dq_tid < W && dq_tid != p.rank) st_release_sys(flags_of(dq_tid) + W, epoch);
                }
                }
                // The last CTA of this launch collects the "tile is final" flags of the tiles that peers own. Every CTA is
                // counted, also one whose tile was given up (a wait that ran out): the counter must be back at zero when the
                // launch ends, or later launches would never find their last CTA.
                int* done_count = reinterpret_cast<int*>(p.heap[p.rank] + p.count_off);
                asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
                if (dq_tid == 0) {
                    const int last = atomicAdd(done_count, 1) == tiles - 1;
                    if (last) *done_count = 0;
                    *last_flag = last;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
                if (*last_flag && *abort_flag == 0) {
                    int* base = reinterpret_cast<int*>(p.heap[p.rank] + p.flags_off);
                    for (int t = dq_tid; t < tiles; t += DQ_THREADS)
                        if (t % W != p.rank) wait_flag(base + (size_t)t * (W + 1) + W);
                }
            } else {
                    // two-shot: the owner of the tile (tile_id mod W) collects the partials, reduces, and writes the
                    // finished tile into `out` on every rank; nobody leaves before its copy of the tile is final
                    const int owner = tile_id % W, own_idx = tile_id / W, own_cap = (tiles + W - 1) / W;
                    const size_t slot = (size_t)p.stage_off + ((size_t)p.rank * own_cap + own_idx) * SLOT;
                    for (int i = dq_tid; i < PIECES; i += DQ_THREADS) {
                        const int col = i >> 4, pc = i & 15;
                        if (col < ntok)
                            *reinterpret_cast<uint4*>(p.heap[owner] + slot + ((size_t)col * TILE_N + pc * 8) * 2) = partial_piece(col, pc);
                    }
                    __threadfence_system();
                    asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
                    if (dq_tid == 0) st_release_sys(flags_of(owner) + p.rank, epoch);
                    if (p.rank == owner) {
                        if (dq_tid < W) wait_flag(my_flags + dq_tid);
                        asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
                        const bool good = (*abort_flag == 0);
                        if (good) {
                            const uint8_t* slots = p.heap[p.rank] + p.stage_off + (size_t)own_idx * SLOT;
                            for (int i = dq_tid; i < PIECES; i += DQ_THREADS) {
                                const int col = i >> 4, pc = i & 15;
                                if (col < ntok) {
                                    const uint4 v = reduced_piece(slots, (size_t)own_cap * SLOT, col, pc);
                                    const size_t off = (size_t)p.out_off + ((size_t)(t0 + col) * p.ldo + n0 + pc * 8) * 2;
                                    for (int r = 0; r < W; ++r) *reinterpret_cast<uint4*>(p.heap[r] + off) = v;
                                }
                            }
                        }
                        __threadfence_system();
                        asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
                        if (good && dq_tid < W) st_release_sys(flags_of(dq_tid) + W, epoch);
                    }
                    if (dq_tid == 0) wait_flag(my_flags + W);
                    asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
            }
        };

        auto finish = [&](int col, float v) {
            const int tok = t0 + col;
            if (tok < T_end && oc < p.N) {
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
                if (comm && p.splits == 1) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) stage_out[(c0 + j) * TILE_N + row] = __uint_as_float(r[j]);
                } else if (fast) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        stage_out[(c0 + j) * TILE_N + row] = apply_act(__uint_as_float(r[j]) + bias_v, p.act);
                } else if (p.splits == 1) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) finish(c0 + j, __uint_as_float(r[j]));
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) stage_out[(c0 + j) * TILE_N + row] = __uint_as_float(r[j]);
                }
            }
        }
        // The communication epilogue has ONE call site (below, after the split-K reduction): the compiler then inlines the
        // lambda, and its by-reference captures stay in registers instead of a stack frame.
        bool run_comm = false, comm_tile_ok = false;
        if (comm && p.splits == 1) {
            run_comm = true;
            comm_tile_ok = acc_ok;   // acc_ok is uniform over the epilogue threads
        } else if (fast && p.act == OVB_ACT_SWIGLU) {
            // Gated MLP: the tile holds 64 "gate" rows followed by the 64 "up" rows of the same channels (the packer
            // interleaves them per tile), so out[tok, 64 * tile + c] = silu(gate_c) * up_c needs this tile only.
            asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
            if (acc_ok) {
                constexpr int PIECES = BT * (TILE_N / 16);    // 16-byte pieces of the 64 output channels
                const int ntok = min(BT, T_end - t0);
                for (int i = dq_tid; i < PIECES; i += DQ_THREADS) {
                    const int col = i >> 3, pc = i & 7;
                    if (col < ntok) {
                        const float* g = stage_out + col * TILE_N + pc * 8;
                        const float* u = g + TILE_N / 2;
                        uint4 v;
                        E* ve = reinterpret_cast<E*>(&v);
#pragma unroll
                        for (int j = 0; j < 8; ++j) ve[j] = from_float<E>(g[j] / (1.0f + __expf(-g[j])) * u[j]);
                        *reinterpret_cast<uint4*>(reinterpret_cast<E*>(p.out) + (size_t)(t0 + col) * p.ldo + n_tile * (TILE_N / 2) + pc * 8) = v;
                    }
                }
            }
        } else if (fast) {
            asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
            if (acc_ok) {
                constexpr int PIECES = BT * (TILE_N / 8);     // 16-byte pieces in the tile
                const int ntok = min(BT, T_end - t0);
                for (int i = dq_tid; i < PIECES; i += DQ_THREADS) {
                    const int col = i >> 4, pc = i & 15;
                    if (col < ntok) {
                        const float4 f0 = *reinterpret_cast<const float4*>(stage_out + col * TILE_N + pc * 8);
                        const float4 f1 = *reinterpret_cast<const float4*>(stage_out + col * TILE_N + pc * 8 + 4);
                        float f[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
                        const size_t tok = (size_t)(t0 + col);
                        if (p.residual) {
                            const uint4 rr = *reinterpret_cast<const uint4*>(reinterpret_cast<const E*>(p.residual) + tok * p.ldr + n0 + pc * 8);
                            const E* re = reinterpret_cast<const E*>(&rr);
#pragma unroll
                            for (int j = 0; j < 8; ++j) f[j] += to_float(re[j]);
                        }
                        uint4 v;
                        E* ve = reinterpret_cast<E*>(&v);
#pragma unroll
                        for (int j = 0; j < 8; ++j) ve[j] = from_float<E>(f[j]);
                        *reinterpret_cast<uint4*>(reinterpret_cast<E*>(p.out) + tok * p.ldo + n0 + pc * 8) = v;
                    }
                }
            }
        }
        if (p.splits > 1) {
            // Every CTA of the cluster (one per split) holds its fp32 partial tile in `stage_out`. After the first cluster
            // barrier CTA r sums slice r of the tile over all partials (split order) and writes that part of the output;
            // the second barrier keeps every partial alive until all peers have read it. With the fused all-reduce the
            // whole tile is summed by CTA 0 (in place), which then runs the communication epilogue on it.
            cluster_arrive();
            cluster_wait();
            constexpr int TOTAL4 = TILE_N * BT / 4;
            const uint32_t S = (uint32_t)p.splits;
            const uint32_t base = smem_u32(stage_out);
            const bool ok_all = (*abort_flag == 0);
            if (ok_all && comm) {
                if (split == 0) {
                    for (int i4 = dq_tid; i4 < TOTAL4; i4 += DQ_THREADS) {
                        float4 acc = reinterpret_cast<float4*>(stage_out)[i4];
#pragma unroll 4
                        for (uint32_t z = 1; z < S; ++z) {
                            const float4 v = ld_dsmem_f4(dsmem_addr(base + (uint32_t)i4 * 16u, z));
                            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                        }
                        reinterpret_cast<float4*>(stage_out)[i4] = acc;
                    }
                }
            } else if (ok_all) {
                const int per = (TOTAL4 + (int)S - 1) / (int)S;
                const int i_end = min(TOTAL4, (split + 1) * per);
                for (int i4 = split * per + dq_tid; i4 < i_end; i4 += DQ_THREADS) {
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                    for (uint32_t z = 0; z < S; ++z) {
                        const float4 v = ld_dsmem_f4(dsmem_addr(base + (uint32_t)i4 * 16u, z));
                        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                    }
                    const int e = i4 * 4;
                    const int col = e / TILE_N, r4 = e % TILE_N;
                    const int tok = t0 + col, oc4 = n0 + r4;
                    if (tok < T_end) {
                        float vv[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (oc4 + j < p.N) {
                                float v = vv[j];
                                if (p.bias) v += to_float(reinterpret_cast<const E*>(p.bias)[oc4 + j]);
                                v = apply_act(v, p.act);
                                if (p.residual) v += to_float(reinterpret_cast<const E*>(p.residual)[(size_t)tok * p.ldr + oc4 + j]);
                                vv[j] = v;
                            }
                        }
                        if (p.out_f32) {
                            float* o = reinterpret_cast<float*>(p.out) + (size_t)tok * p.ldo + oc4;
#pragma unroll
                            for (int j = 0; j < 4; ++j) if (oc4 + j < p.N) o[j] = vv[j];
                        } else {
                            E* o = reinterpret_cast<E*>(p.out) + (size_t)tok * p.ldo + oc4;
                            if (oc4 + 3 < p.N && ((reinterpret_cast<uintptr_t>(o) & 7) == 0)) {
                                E t4[4] = {from_float<E>(vv[0]), from_float<E>(vv[1]), from_float<E>(vv[2]), from_float<E>(vv[3])};
                                *reinterpret_cast<uint2*>(o) = *reinterpret_cast<uint2*>(t4);
                            } else {
#pragma unroll
                                for (int j = 0; j < 4; ++j) if (oc4 + j < p.N) o[j] = from_float<E>(vv[j]);
                            }
                        }
                    }
                }
            }
            cluster_arrive();
            cluster_wait();
            if (comm && split == 0) {
                run_comm = true;
                comm_tile_ok = (*abort_flag == 0);
            }
        }
        if (run_comm) {
            asm volatile("bar.sync 1, %0;" ::"n"(DQ_THREADS));
            comm_epilogue(comm_tile_ok);
        }
    }
    // The producer and MMA warps take part in the two cluster barriers of the split-K reduction (a cluster barrier
    // counts every thread of every CTA).
    if (p.splits > 1 && (warp < 2 || warp == X_PRODUCER_WARP)) {
        cluster_arrive();
        cluster_wait();
        cluster_arrive();
        cluster_wait();
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
constexpr int kSmemLimit = 227 * 1024;          // opt-in dynamic shared memory per CTA
constexpr int kSmemBudget = kSmemLimit - 2560;  // minus alignment slack and the barrier block
constexpr int kNumCounters = 4096;
constexpr int kNumSMs = 148;

static int pick_block_t(int T) {
    if (T <= 16) return 16;
    if (T <= 32) return 32;
    if (T <= 64) return 64;
    if (T <= 128) return 128;
    return 256;
}

static int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return e ? atoi(e) : dflt;
}

constexpr int kMaxSplits = 8;   // portable cluster size
static std::mutex g_launch_mu;   // first-use set-up of a kernel variant (function attributes, occupancy table)

// Split-K trades idle SMs against the cost of the cluster reduction (two cluster barriers and one pass over the partial
// tiles through distributed shared memory). Estimate the time of every candidate with a small model (all constants in
// microseconds, measured on B200 with the decode shapes of an 8B model) and take the cheapest. `resident[s]` is the
// number of CTAs of a launch with clusters of s that the device holds at a time (clusters are placed inside one GPC, so
// it is not simply a multiple of the SM count).
static int pick_splits(int T, int N, int K, int bt, int wmode, const int* resident) {
    const int tiles = ceil_div(N, TILE_N) * ceil_div(T, bt);
    const int total_kb = ceil_div(K, TILE_K);
    if (tiles >= resident[1] || total_kb < 8) return 1;
    const double t_kb = is_quant(wmode) ? 0.36 : 0.12 + 0.0028 * bt;   // one k-block in one CTA
    const double t_cta = 6.0;                                              // set-up, pipeline fill, epilogue of a CTA
    int best = 1;
    double best_t = 1e30;
    const int max_s = total_kb / 4 < kMaxSplits ? total_kb / 4 : kMaxSplits;
    for (int s = 1; s <= max_s; ++s) {
        if (resident[s] <= 0) continue;
        const int ctas = tiles * s;
        const int waves = ceil_div(ctas, resident[s]);
        const bool shared_sm = two_ctas(bt, wmode) && s == 1 && ctas > kNumSMs;   // two CTAs on an SM slow each other down
        double t = waves * (ceil_div(total_kb, s) * t_kb * (shared_sm ? 1.25 : 1.0) + t_cta);
        if (s > 1) t += 2.5;                                               // cluster barriers + the slice reduction
        if (t < best_t - 0.25) { best_t = t; best = s; }
    }
    return best;
}

// MMA stages and packed-ring slots that fit the shared-memory budget.
static void pick_rings(int bt, int wmode, int* stages, int* pslots) {
    const int stage = bt * 128 + TILE_N * 128;
    const int wq = wq_bytes(wmode);
    if (wq == 0) {
        int s = kSmemBudget / stage;
        *stages = s > MAX_STAGES ? MAX_STAGES : (s < 2 ? 2 : s);
        *pslots = 0;
        return;
    }
    // quantised: a stage is the token tile only (the expanded weights live in tensor memory); four stages, the rest of
    // the budget goes to the packed ring so that weight chunks are requested far ahead of use
    // a quantised stage covers kps k-blocks: token tiles of kps x 64 K-elements, ring slots of kps chunks, kps x 32 TMEM columns of A
    const int kps = kblocks_per_stage(bt, wmode);
    const int xstage = kps * bt * 128;
    const int slot = kps * (wq + TILE_N * 4);  // packed chunks + (scale, zero point) pairs
    // Large token tiles come from L2 with a latency of a microsecond or two under load: the token ring has to cover it
    // (a 256-token stage is consumed in ~0.3 us); decode-sized tiles take seven stages so that the dequant sets run well
    // ahead of the MMAs. The packed-weight ring keeps what is left. The accumulator and s x 32 (64 for two-k-block
    // stages) columns of A fit the 512 TMEM columns.
    // Both rings are walked by `sets` sets of dequant groups that take alternate iterations: their lengths are multiples
    // of `sets`, so that a ring entry always belongs to the same set (a waiter on an mbarrier phase parity must never be
    // two phases ahead of the barrier, which a set that sees only every other use of an entry could be).
    const int sets = (num_dq_warps(bt, wmode) / 4) / kps;
    int s = bt >= 256 ? 6 : (bt >= 128 ? 5 : 6);
    int budget = kSmemBudget;
    if (two_ctas(bt, wmode)) {               // two CTAs share the SM: half the shared memory, 256 TMEM columns each
        s = 3;                               // accumulator (<= 64 columns) + 3 x 64 columns of A
        budget = (kSmemLimit - 2 * 1024) / 2 - 2560;
    }
    s -= s % sets;
    int pmax = (budget - s * xstage) / slot;
    if (pmax > MAX_PSLOTS) pmax = MAX_PSLOTS;
    pmax -= pmax % sets;
    *stages = s;
    *pslots = pmax;
}

template <int BT, int WMODE, bool F16>
static int launch(const ovb_gemm_args* a, const CUtensorMap& tmW, const CUtensorMap& tmX, GemmKParams& p,
                  cudaStream_t stream) {
    int stages = 2, pslots = 0;
    pick_rings(BT, WMODE, &stages, &pslots);
    p.stages = stages;
    p.pslots = pslots;
    const int wq = wq_bytes(WMODE);
    const int kps = kblocks_per_stage(BT, WMODE);
    const int smem = stages * (wq ? kps * BT * 128 : BT * 128 + TILE_N * 128) + pslots * (wq ? kps * (wq + TILE_N * 4) : 0) + 1024 + 1024;
    auto kern = gemm_ws_kernel<BT, WMODE, F16>;
    static uint64_t configured = 0;  // one bit per device, guarded by g_launch_mu
    int dev = 0;
    OVB_CHECK_CUDA(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lk(g_launch_mu);
        if (!(configured & (1ull << (dev & 63)))) {
            OVB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
            OVB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
            configured |= (1ull << (dev & 63));
        }
    }
    if (smem > kSmemLimit) {
        set_error("ovb_gemm: internal error, %d bytes of shared memory requested", smem);
        return ERR_TOO_LARGE;
    }
    // the splits of a tile are one thread-block cluster (reduction through distributed shared memory)
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.blockDim = dim3(gemm_threads(BT, WMODE), 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // CTAs resident at a time for every cluster size, asked of the driver once per kernel variant
    static int resident[kMaxSplits + 1] = {-1};
    {
        std::lock_guard<std::mutex> lk(g_launch_mu);
        if (resident[0] < 0) {
            resident[1] = (two_ctas(BT, WMODE) ? 2 : 1) * kNumSMs;
            for (int sz = 2; sz <= kMaxSplits; ++sz) {
                int n = 0;
                cfg.gridDim = dim3(sz * 64, 1, sz);
                attr[0].val.clusterDim.z = sz;
                resident[sz] = cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess ? n * sz : 0;
            }
            (void)cudaGetLastError();
            resident[0] = 0;
        }
    }
    // reducer CTAs when the tiles take more than one wave (set below with the grid)
    if (p.splits == 0) p.splits = pick_splits(a->T, a->N, a->K, BT, WMODE, resident);
    const int total_kb = ceil_div(a->K, TILE_K);
    if (p.splits > total_kb) p.splits = total_kb;
    if (p.splits > kMaxSplits) p.splits = kMaxSplits;
    p.kblocks_per_split = ceil_div(total_kb, p.splits);
    cfg.gridDim = dim3(ceil_div(a->N, TILE_N) * ceil_div(a->T, BT), 1, p.splits);
    if (p.group_off != nullptr)     // every group may end with a partial row tile: num_groups extra tiles cover the worst case
        cfg.gridDim = dim3(ceil_div(a->N, TILE_N) * (ceil_div(a->T, BT) + p.num_groups), 1, 1);
    p.nvls_reducers = 0;
    if (p.nvls && p.splits == 1 && p.group_off == nullptr && (int)cfg.gridDim.x > resident[1]) {
        // dedicated reducer CTAs are an option, off by default: at 8 ranks (T 8192, N 4096) 32 / 64 of them gave 360 / 320 us
        // against 334 us with every tile CTA reducing its own share after the last tile, and the serving pass was 4 % slower
        static const int want = env_int("OVB_NVLS_REDUCERS", 0);
        p.nvls_reducers = want < 0 ? 0 : (want > 128 ? 128 : want);
        cfg.gridDim.x += p.nvls_reducers;
    }
    attr[0].val.clusterDim.z = p.splits;
    // programmatic dependent launch: set-up, tensor-memory allocation and the first weight fetches run under the tail of
    // the kernel before this one (the kernel waits before it reads activations or writes anything)
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    OVB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

// ---- conditional compilation (selective build). The analysing run records which (token tile, weight format) variants
// were launched (ovb_cc_used_gemm); a selective build is compiled with -DOVB_CC_SELECTIVE and a generated "cc_selected.h"
// whose cc_gemm_selected(bt, wmode, f16) names the variants to keep. A variant that is not selected is never instantiated,
// so it costs neither build time nor binary size; launching it reports an error. Role in the reference:
// src/common/conditional_compilation (OV_CC_COLLECT / OV_CC_SELECTIVE scopes around kernels and passes).
#ifdef OVB_CC_SELECTIVE
#include "cc_selected.h"
#else
constexpr bool cc_gemm_selected(int, int, bool) { return true; }
#endif

static std::atomic<uint32_t> g_cc_gemm_used[16];      // [wmode * 2 + f16]: bit log2(bt) - 4

static int bt_bit(int bt) { return bt == 16 ? 0 : bt == 32 ? 1 : bt == 64 ? 2 : bt == 128 ? 3 : 4; }

template <int BT, int WMODE, bool F16>
static int launch_selected(const ovb_gemm_args* a, const CUtensorMap& tmW, const CUtensorMap& tmX, GemmKParams& p, cudaStream_t stream) {
    if constexpr (cc_gemm_selected(BT, WMODE, F16)) {
        g_cc_gemm_used[(WMODE * 2 + (F16 ? 1 : 0)) & 15].fetch_or(1u << bt_bit(BT), std::memory_order_relaxed);
        return launch<BT, WMODE, F16>(a, tmW, tmX, p, stream);
    } else {
        set_error("ovb_gemm: the variant (token tile %d, weight format %d%s) was left out of this selective build", BT, WMODE, F16 ? ", fp16" : "");
        return ERR_UNSUPPORTED;
    }
}

template <int WMODE, bool F16>
static int dispatch_bt(int bt, const ovb_gemm_args* a, const CUtensorMap& tmW, const CUtensorMap& tmX, GemmKParams& p,
                       cudaStream_t stream) {
    switch (bt) {
        case 16: return launch_selected<16, WMODE, F16>(a, tmW, tmX, p, stream);
        case 32: return launch_selected<32, WMODE, F16>(a, tmW, tmX, p, stream);
        case 64: return launch_selected<64, WMODE, F16>(a, tmW, tmX, p, stream);
        case 128: return launch_selected<128, WMODE, F16>(a, tmW, tmX, p, stream);
        case 256: return launch_selected<256, WMODE, F16>(a, tmW, tmX, p, stream);
    }
    set_error("unsupported block_t %d", bt);
    return ERR_BAD_ARG;
}

}  // namespace ovb

extern "C" {

int ovb_gemm_num_counters(void) { return ovb::kNumCounters; }

unsigned ovb_cc_used_gemm(int wmode, int is_f16) { return ovb::g_cc_gemm_used[(wmode * 2 + (is_f16 ? 1 : 0)) & 15].load(std::memory_order_relaxed); }

int ovb_cc_is_selective(void) {
#ifdef OVB_CC_SELECTIVE
    return 1;
#else
    return 0;
#endif
}

int64_t ovb_gemm_ws_bytes(int T, int N, int K, int act) {
    // split-K partials stay in shared memory (cluster reduction): no global workspace is needed any more
    (void)T; (void)N; (void)K; (void)act;
    return 0;
}

// Which protocol carries the partials of the fused all-reduce: flag-carrying packets (twice the bytes, no fence and no
// flag round trip) or plain tiles with a fence and arrival flags. Every rank must choose alike, so the choice depends
// on the world size and the mode only; OVB_COMM_PACKETS (bit 0: one-shot, bit 1: two-shot) overrides it for measurements.
// Environment overrides for measurements (every rank must set them alike): OVB_COMM_TWOHOP = 0 / 1 forces the two-hop packet
// protocol of the one-shot sizes off / on; OVB_COMM_NVLS_MODES is a bit mask of the modes (bit 0: T <= 128, bit 1: larger) that
// reduce inside the switch when the heap has a multicast mapping.
static int comm_twohop(int world) {
    static const int env = ovb::env_int("OVB_COMM_TWOHOP", -1);
    return env >= 0 ? env : (world > 2);
}
// Bit (mode - 1) set: the all-reduce of that mode runs inside the switch (multimem.ld_reduce / multimem.st) when the heap has a
// multicast mapping. Measured (T=8192, N=4096, per-rank K=512/1792): with 8 ranks in-switch takes 378/423 us against 475/531 us
// for the two-shot packets and 425/474 us for GEMM then NCCL; with 2 ranks the packets win (362/533 us against 499/683 us).
// At T=64 the two-hop packets (28.7/31.7 us with 8 ranks) beat in-switch (37.8/43.0 us) at every world size.
static int comm_nvls_modes(int world) {
    static const int env = ovb::env_int("OVB_COMM_NVLS_MODES", -1);
    return env >= 0 ? env : (world >= 4 ? 2 : 0);
}

static int comm_packets(int world, int mode) {
    static const int env = [] {
        const char* e = getenv("OVB_COMM_PACKETS");
        return e ? atoi(e) : -1;
    }();
    if (env >= 0) return (env >> (mode - 1)) & 1;
    // measured: with 2 ranks packets win in both modes (28.5 vs 39 us at T=64, 347 vs 441 us at T=8192); with 8 ranks the
    // doubled bytes and the longer per-thread polling chains cost more than the fence and the flags
    return world <= 2;
}

int ovb_gemm(const ovb_gemm_args* a, ovb_stream_t stream_) {
    using namespace ovb;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    OVB_REQUIRE(a && a->x && a->w && a->out, "ovb_gemm: null operand");
    OVB_REQUIRE(a->T > 0 && a->N > 0 && a->K > 0, "ovb_gemm: empty problem T=%d N=%d K=%d", a->T, a->N, a->K);
    OVB_REQUIRE(a->K % 8 == 0 && a->ldx % 8 == 0, "ovb_gemm: K and ldx must be multiples of 8 (TMA 16-byte rule)");
    const bool f16 = a->wmode == OVB_W_F16;
    const bool quant = is_quant(a->wmode);
    if (quant) {
        OVB_REQUIRE(a->scales, "ovb_gemm: quantised weights need the (scale, zero point) table");
        OVB_REQUIRE(a->group_size >= 64 && a->group_size % 64 == 0 && a->K % a->group_size == 0,
                    "ovb_gemm: group_size %d must be a multiple of 64 that divides K=%d", a->group_size, a->K);
        OVB_REQUIRE(a->K % 32 == 0, "ovb_gemm: K must be a multiple of 32 for packed weights");
        OVB_REQUIRE(a->N % 4 == 0 && (reinterpret_cast<uintptr_t>(a->scales) & 15) == 0,
                    "ovb_gemm: quantised weights need N %% 4 == 0 and a 16-byte aligned (scale, zero point) table");
    }
    const bool swiglu = a->act == OVB_ACT_SWIGLU;
    if (swiglu) {
        // fused gated MLP: W rows are interleaved per 128-row tile (64 gate rows, then the 64 up rows of the same channels)
        OVB_REQUIRE(a->N % TILE_N == 0 && !a->out_f32 && a->residual == nullptr && a->comm == nullptr && a->bias == nullptr,
                    "ovb_gemm: the SWIGLU epilogue needs N %% 128 == 0, a 16-bit output and no bias / residual / communicator");
        OVB_REQUIRE((reinterpret_cast<uintptr_t>(a->out) & 15) == 0 && (a->ldo ? a->ldo : a->N / 2) % 8 == 0,
                    "ovb_gemm: the SWIGLU epilogue needs a 16-byte aligned output with a row pitch that is a multiple of 8");
    }

    const bool grouped = a->group_offsets != nullptr;
    if (grouped) {
        OVB_REQUIRE(a->num_groups >= 1 && a->num_groups <= 256 && (a->group_mode == 1 || a->group_mode == 2), "ovb_gemm: grouped GEMM needs 1..256 groups and group_mode 1 or 2");
        OVB_REQUIRE((a->wmode == OVB_W_U4 || (a->w_tiled && !quant)) && a->comm == nullptr && a->N % TILE_N == 0 && a->K % TILE_K == 0,
                    "ovb_gemm: grouped GEMM needs tile-packed weights (u4 or 16-bit), N %% 128 == 0, K %% 64 == 0 and no communicator");
    }
    const int bt = a->block_t ? a->block_t : pick_block_t(a->T);
    const int splits = (swiglu || grouped) ? 1 : a->splits;   // 0: chosen at launch, where the kernel variant and its cluster occupancy are known
    const int64_t tiles = (int64_t)ceil_div(a->N, TILE_N) * ceil_div(a->T, bt);

    GemmKParams p;
    memset(&p, 0, sizeof(p));
    p.out = a->out;
    p.bias = a->bias;
    p.residual = a->residual;
    p.sz = reinterpret_cast<const uint32_t*>(a->scales);
    p.ws = a->ws;
    p.counters = a->counters;
    p.status = status_word();
    p.T = a->T; p.N = a->N; p.K = a->K;
    p.ldo = a->ldo ? a->ldo : (swiglu ? a->N / 2 : a->N);
    p.ldr = a->ldr ? a->ldr : a->N;
    p.group_size = quant ? a->group_size : a->K;
    p.act = a->act;
    p.out_f32 = a->out_f32;
    p.splits = splits;
    p.w_kb_stride = a->w_kb_stride > 0 ? a->w_kb_stride : ceil_div(a->K, TILE_K) * (grouped && a->group_mode == 2 ? a->num_groups : 1);
    p.spin_limit = peer_spin_limit();
    p.group_off = a->group_offsets;
    p.num_groups = a->num_groups;
    p.group_mode = a->group_mode;
    if (a->comm != nullptr && static_cast<const ovb_comm*>(a->comm)->world > 1) {
        const ovb_comm* c = static_cast<const ovb_comm*>(a->comm);
        OVB_REQUIRE(c->world <= 8 && c->rank >= 0 && c->rank < c->world, "ovb_gemm: bad communicator (rank %d of %d)", c->rank, c->world);
        OVB_REQUIRE(!f16 && !a->out_f32 && a->act == OVB_ACT_NONE, "ovb_gemm: the fused all-reduce needs a bf16 output and no activation");
        OVB_REQUIRE(a->N % TILE_N == 0 && p.ldo % 8 == 0 && p.ldr % 8 == 0 && (reinterpret_cast<uintptr_t>(a->out) & 15) == 0 &&
                        (reinterpret_cast<uintptr_t>(a->residual) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->bias) & 15) == 0,
                    "ovb_gemm: the fused all-reduce needs N %% 128 == 0 and 16-byte aligned rows");
        const int mode = c->mode ? c->mode : (a->T <= 128 ? 1 : 2);
        const int64_t slot = (int64_t)bt * TILE_N * 2;
        // the staging areas hold flag-carrying packets: twice the bytes of the bf16 tiles
        const int64_t need = mode == 1 ? 2 * c->world * tiles * slot : 2 * c->world * ((tiles + c->world - 1) / c->world) * slot;
        OVB_REQUIRE(need <= (mode == 1 ? c->stage1_bytes : c->stage2_bytes),
                    "ovb_gemm: the communicator's staging area (%lld bytes) is too small for T=%d N=%d (%lld bytes)",
                    (long long)(mode == 1 ? c->stage1_bytes : c->stage2_bytes), a->T, a->N, (long long)need);
        OVB_REQUIRE(tiles * (c->world + 1) <= c->flags_per_site && c->site >= 0 && c->site < c->num_sites,
                    "ovb_gemm: communicator flag area too small (%lld tiles) or bad call site %d", (long long)tiles, c->site);
        OVB_REQUIRE(mode != 1 || c->num_sites <= 256, "ovb_gemm: the one-shot all-reduce tags packets with an 8-bit call site (%d sites)", c->num_sites);
        p.world = c->world;
        p.rank = c->rank;
        p.comm_mode = mode;
        p.parity = c->site & 1;
        p.site = c->site;
        p.packets = comm_packets(c->world, mode);
        for (int r = 0; r < c->world; ++r) {
            OVB_REQUIRE(c->heap[r] != nullptr, "ovb_gemm: communicator heap of rank %d is not mapped", r);
            p.heap[r] = static_cast<uint8_t*>(c->heap[r]);
        }
        p.stage_off = mode == 1 ? c->stage1_off + (int64_t)p.parity * c->stage1_bytes : c->stage2_off;
        p.flags_off = c->flags_off + (int64_t)c->site * c->flags_per_site * 4;
        p.epoch = reinterpret_cast<const int*>(p.heap[c->rank] + c->epoch_off);
        p.count_off = c->epoch_off + 64;   // the first 256 bytes of the heap are reserved for such words
        const int64_t out_heap_off = static_cast<uint8_t*>(a->out) - p.heap[c->rank];
        const bool out_in_heap = out_heap_off >= 0 && out_heap_off + ((int64_t)(a->T - 1) * p.ldo + a->N) * 2 <= c->heap_bytes;
        if (mode == 2) {
            OVB_REQUIRE(out_in_heap, "ovb_gemm: with the two-shot all-reduce the output must live in the communicator's symmetric heap");
            p.out_off = out_heap_off;
        }
        // In-switch reduction when the heap has a multicast mapping: plain bf16 tiles in the staging area of the mode (half of
        // what the packets need), barrier words of the call site, output in the heap, 2, 4 or 8 ranks.
        if (mode == 1 && comm_twohop(c->world) && (bt * 16) % c->world == 0 && 2 * tiles * bt * 16 * 32 <= c->stage1_bytes) {
            p.twohop = 1;
            p.mc = static_cast<uint8_t*>(c->mc_base);   // NULL: hop 2 stores to every rank in turn
        } else if (c->mc_base != nullptr && ((comm_nvls_modes(c->world) >> (mode - 1)) & 1) && out_in_heap && (c->world == 2 || c->world == 4 || c->world == 8) &&
            tiles * kNvlsFlagStride <= c->nvls_flags_per_site && tiles * slot <= (mode == 1 ? c->stage1_bytes : c->stage2_bytes)) {
            p.mc = static_cast<uint8_t*>(c->mc_base);
            p.nvls = 1;
            p.nvls_flags_off = c->nvls_flags_off + (int64_t)c->site * c->nvls_flags_per_site * 4;
            p.out_off = out_heap_off;
        }
    }

    CUtensorMap tmW, tmX;
    const int ldx = a->ldx ? a->ldx : a->K;
    const CUtensorMapDataType dt16 = f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    if (int rc = make_tmap_2d(&tmX, a->x, dt16, 2, a->T, a->K, (uint64_t)ldx * 2, bt, TILE_K, true)) return rc;
    int rc = 0;
    if (a->wmode == OVB_W_U4 || (a->w_tiled && !quant)) {
        OVB_REQUIRE(a->K % TILE_K == 0, "ovb_gemm: tile-packed weights need K to be a multiple of 64");
        OVB_REQUIRE((reinterpret_cast<uintptr_t>(a->w) & 15) == 0, "ovb_gemm: packed weights must be 16-byte aligned");
        p.w_tiled = reinterpret_cast<const uint8_t*>(a->w);
        tmW = tmX;   // unused by the kernel in this mode
    } else if (a->wmode == OVB_W_U8 || a->wmode == OVB_W_F8) {
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
        case OVB_W_F8: return dispatch_bt<OVB_W_F8, false>(bt, a, tmW, tmX, p, stream);
    }
    set_error("ovb_gemm: unknown wmode %d", a->wmode);
    return ERR_BAD_ARG;
}

}  // extern "C"
