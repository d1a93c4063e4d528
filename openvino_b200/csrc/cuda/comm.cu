// Tensor-parallel communication over NVLink peer memory: symmetric-heap plumbing (CUDA IPC), the step counter,
// the cross-rank argmax of sharded logits and a small-tensor all-reduce. The GEMM with the all-reduce fused into
// its epilogue lives in gemm_sm100.cu; this file holds what is not a GEMM.
//
// Protocol shared by all of it: a rank writes data into a peer's heap with plain stores, fences at system scope,
// and then stores the current step number into a flag word of that peer (st.release.sys). The peer polls the flag
// (ld.acquire.sys, bounded) until it holds at least the current step number and reads the data with L1 bypassed.
// Flags are never reset: the step number only grows. A wait that runs out reports STATUS_PEER_TIMEOUT through the
// status word and the kernel returns; nothing here spins without a limit.
//
// Reference counterpart: tensor-parallel FullyConnected across sockets, selected with
// ov::hint::model_distribution_policy(TENSOR_PARALLEL) (src/inference/include/openvino/runtime/properties.hpp:484-488),
// where ranks exchange partial results through shared memory guarded by flags
// (src/plugins/intel_cpu/src/nodes/fullyconnected.cpp:226-330, src/plugins/intel_cpu/src/sub_memory_manager.hpp).
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ovb {

constexpr int kArgmaxRowsCap = 1024;
constexpr int kArgmaxDataOff = 64;   // ints: flags first, then two (value, index) buffers

__device__ __forceinline__ bool wait_flag_ge(const int* f, int epoch, int* status, uint32_t spin_limit) {
    for (uint32_t i = 0; i < spin_limit; ++i) {
        if (ld_acquire_sys(f) >= epoch) return true;
        __nanosleep(200);
    }
    report_status(status, STATUS_PEER_TIMEOUT);
    return false;
}

__global__ void step_begin_kernel(int* epoch) {
    pdl_enter(); *epoch = *epoch + 1; }

// One thread waits for *flag >= value with a caller-chosen poll budget; when the budget runs out the kernel records
// STATUS_PEER_TIMEOUT in the status word and returns, so the context stays usable. The building block of the
// failure-detection tests: a flag that nobody sets makes the wait run out.
__global__ void wait_flag_kernel(const int* flag, int value, unsigned max_polls, int* status, int* result) {
    pdl_enter();
    bool ok = false;
    for (unsigned i = 0; i < max_polls; ++i) {
        if (ld_acquire_sys(flag) >= value) { ok = true; break; }
        __nanosleep(200);
    }
    if (!ok) report_status(status, STATUS_PEER_TIMEOUT);
    if (result) *result = ok ? 1 : 0;
}

struct CommK {
    int rank, world;
    uint8_t* heap[8];
    long long flags_off;     // of the call site
    long long stage_off;
    const int* epoch;
    int* status;
    uint8_t* mc;             // multicast mapping of the heap (NVLS) or NULL
    long long nvls_flags_off;   // of the call site
    uint32_t spin_limit;        // polls before a wait on a peer gives up (peer_spin_limit())
};

// One CTA; thread = row. Every rank pushes (max value, global index) of its shard to every rank, then picks.
__global__ void argmax_combine_kernel(CommK c, int* ids, const float* max_vals, int rows, int shard_size) {
    pdl_enter();
    const int epoch = __ldcg(c.epoch);
    const int W = c.world;
    const int row = threadIdx.x;
    const int buf = epoch & 1;
    const size_t data_off = (size_t)c.flags_off + ((size_t)kArgmaxDataOff + (size_t)buf * W * kArgmaxRowsCap * 2) * 4;
    if (row < rows) {
        const int2 mine = make_int2(__float_as_int(max_vals[row]), ids[row] + c.rank * shard_size);
        for (int r = 0; r < W; ++r)
            reinterpret_cast<int2*>(c.heap[r] + data_off)[(size_t)c.rank * kArgmaxRowsCap + row] = mine;
    }
    __threadfence_system();
    __syncthreads();
    __shared__ int ok_s;
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    if (threadIdx.x < W) {
        st_release_sys(reinterpret_cast<int*>(c.heap[threadIdx.x] + c.flags_off) + c.rank, epoch);
        if (!wait_flag_ge(reinterpret_cast<const int*>(c.heap[c.rank] + c.flags_off) + threadIdx.x, epoch, c.status, c.spin_limit)) ok_s = 0;
    }
    __syncthreads();
    if (ok_s && row < rows) {
        const int2* all = reinterpret_cast<const int2*>(c.heap[c.rank] + data_off);
        float best = -INFINITY;
        int best_id = 0x7fffffff;
        for (int r = 0; r < W; ++r) {
            const int2 v = __ldcg(all + (size_t)r * kArgmaxRowsCap + row);
            const float f = __int_as_float(v.x);
            if (f > best || (f == best && v.y < best_id)) { best = f; best_id = v.y; }
        }
        ids[row] = best_id;
    }
}

// Small-tensor all-reduce (one-shot): CTA b owns pieces b, b + grid, ...; flags: one per (CTA, source rank).
// DT: 0 = fp32 (4 values per 16-byte piece), 1 = fp16, 2 = bf16 (8 values); sums in fp32, ranks in index order.
template <int DT>
__device__ __forceinline__ void piece_add(float* f, const uint4& v) {
    if (DT == OVB_DT_F32) {
        f[0] += __uint_as_float(v.x); f[1] += __uint_as_float(v.y); f[2] += __uint_as_float(v.z); f[3] += __uint_as_float(v.w);
    } else if (DT == OVB_DT_F16) {
        const __half* e = reinterpret_cast<const __half*>(&v);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += __half2float(e[j]);
    } else {
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += __bfloat162float(e[j]);
    }
}
template <int DT>
__device__ __forceinline__ uint4 piece_pack(const float* f) {
    uint4 o;
    if (DT == OVB_DT_F32) {
        o = make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    } else if (DT == OVB_DT_F16) {
        __half* oe = reinterpret_cast<__half*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) oe[j] = __float2half_rn(f[j]);
    } else {
        __nv_bfloat16* oe = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) oe[j] = __float2bfloat16_rn(f[j]);
    }
    return o;
}

template <int DT>
__global__ void allreduce_kernel(CommK c, long long data_off, long long npieces, long long rank_stride) {
    pdl_enter();
    const int epoch = __ldcg(c.epoch);
    const int W = c.world;
    const uint4* mine = reinterpret_cast<const uint4*>(c.heap[c.rank] + data_off);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < npieces; i += (long long)gridDim.x * blockDim.x) {
        const uint4 v = mine[i];
        for (int r = 0; r < W; ++r)
            reinterpret_cast<uint4*>(c.heap[r] + c.stage_off + (size_t)c.rank * rank_stride)[i] = v;
    }
    __threadfence_system();
    __syncthreads();
    __shared__ int ok_s;
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    if (threadIdx.x < W) {
        st_release_sys(reinterpret_cast<int*>(c.heap[threadIdx.x] + c.flags_off) + (size_t)blockIdx.x * W + c.rank, epoch);
        if (!wait_flag_ge(reinterpret_cast<const int*>(c.heap[c.rank] + c.flags_off) + (size_t)blockIdx.x * W + threadIdx.x, epoch, c.status, c.spin_limit))
            ok_s = 0;
    }
    __syncthreads();
    if (!ok_s) return;
    uint4* out = reinterpret_cast<uint4*>(c.heap[c.rank] + data_off);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < npieces; i += (long long)gridDim.x * blockDim.x) {
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < W; ++r) {
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(c.heap[c.rank] + c.stage_off + (size_t)r * rank_stride) + i);
            piece_add<DT>(f, v);
        }
        out[i] = piece_pack<DT>(f);
    }
}

// In-place all-reduce through the switch (NVLS): the ranks meet at a barrier (every rank's tensor is complete), rank r
// fetches the sum over the ranks of its 1/W share of the 16-byte pieces (multimem.ld_reduce, fp32 accumulation) and writes
// it back to every rank (multimem.st), and a second barrier tells every rank that all shares have landed. No staging: a
// piece is read and rewritten by its one owner only. CTA b uses barrier b of the call site.
template <int DT>
__global__ void allreduce_nvls_kernel(CommK c, long long data_off, long long npieces) {
    pdl_enter();
    const int epoch = __ldcg(c.epoch);
    const int W = c.world;
    const int* bar_local = reinterpret_cast<const int*>(c.heap[c.rank] + c.nvls_flags_off) + (size_t)blockIdx.x * kNvlsFlagStride;
    int* bar_mc = reinterpret_cast<int*>(c.mc + c.nvls_flags_off) + (size_t)blockIdx.x * kNvlsFlagStride;
    __shared__ int ok_s;
    if (threadIdx.x == 0) ok_s = nvls_barrier(bar_local, bar_mc, c.rank, W, epoch, c.spin_limit, nullptr) ? 1 : 0;
    __syncthreads();
    if (!ok_s) {
        if (threadIdx.x == 0) report_status(c.status, STATUS_PEER_TIMEOUT);
        return;
    }
    const long long per = (npieces + W - 1) / W;
    const long long begin = (long long)c.rank * per;
    const long long end = begin + per < npieces ? begin + per : npieces;
    uint8_t* base = c.mc + data_off;
    for (long long i = begin + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < end; i += (long long)gridDim.x * blockDim.x)
        multimem_st_b128(base + i * 16, DT == OVB_DT_F32 ? multimem_ld_reduce_f32x4(base + i * 16)
                                                           : (DT == OVB_DT_F16 ? multimem_ld_reduce_f16x8(base + i * 16) : multimem_ld_reduce_bf16x8(base + i * 16)));
    fence_sys();
    __syncthreads();
    if (threadIdx.x == 0 && !nvls_barrier(bar_local + 8, bar_mc + 8, c.rank, W, epoch, c.spin_limit, nullptr)) report_status(c.status, STATUS_PEER_TIMEOUT);
}

static int fill(const ovb_comm* c, CommK* k, int site) {
    OVB_REQUIRE(c != nullptr && c->world >= 1 && c->world <= 8 && c->rank >= 0 && c->rank < c->world, "bad communicator");
    OVB_REQUIRE(site >= 0 && site < c->num_sites, "communicator call site %d out of range (%d sites)", site, c->num_sites);
    k->rank = c->rank;
    k->world = c->world;
    for (int r = 0; r < c->world; ++r) {
        OVB_REQUIRE(c->heap[r] != nullptr, "communicator heap of rank %d is not mapped", r);
        k->heap[r] = static_cast<uint8_t*>(c->heap[r]);
    }
    k->flags_off = c->flags_off + (int64_t)site * c->flags_per_site * 4;
    k->stage_off = c->stage3_bytes > 0 ? c->stage3_off + (int64_t)(site & 1) * c->stage3_bytes
                                       : c->stage1_off + (int64_t)(site & 1) * c->stage1_bytes;
    k->epoch = reinterpret_cast<const int*>(k->heap[c->rank] + c->epoch_off);
    k->status = status_word();
    k->mc = static_cast<uint8_t*>(c->mc_base);
    k->nvls_flags_off = c->nvls_flags_off + (int64_t)site * c->nvls_flags_per_site * 4;
    k->spin_limit = peer_spin_limit();
    return 0;
}

}  // namespace ovb

extern "C" {
using namespace ovb;

int ovb_comm_alloc(int64_t bytes, void** ptr) {
    OVB_REQUIRE(ptr != nullptr && bytes > 0, "ovb_comm_alloc: bad arguments");
    OVB_CHECK_CUDA(cudaMalloc(ptr, (size_t)bytes));
    OVB_CHECK_CUDA(cudaMemset(*ptr, 0, (size_t)bytes));
    OVB_CHECK_CUDA(cudaDeviceSynchronize());
    return 0;
}

int ovb_comm_free(void* ptr) {
    OVB_CHECK_CUDA(cudaFree(ptr));
    return 0;
}

int ovb_comm_export(void* ptr, void* handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    OVB_REQUIRE(ptr != nullptr && handle64 != nullptr, "ovb_comm_export: bad arguments");
    cudaIpcMemHandle_t h;
    OVB_CHECK_CUDA(cudaIpcGetMemHandle(&h, ptr));
    memcpy(handle64, &h, sizeof(h));
    return 0;
}

int ovb_comm_open(const void* handle64, void** ptr) {
    OVB_REQUIRE(ptr != nullptr && handle64 != nullptr, "ovb_comm_open: bad arguments");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    OVB_CHECK_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}

int ovb_comm_close(void* ptr) {
    OVB_CHECK_CUDA(cudaIpcCloseMemHandle(ptr));
    return 0;
}

int ovb_comm_step_begin(const ovb_comm* c, ovb_stream_t stream) {
    OVB_REQUIRE(c != nullptr && c->heap[c->rank] != nullptr, "ovb_comm_step_begin: bad communicator");
    OVB_CHECK_CUDA(launch_pdl(step_begin_kernel, dim3(1), dim3(1), 0, static_cast<cudaStream_t>(stream), 
        reinterpret_cast<int*>(static_cast<uint8_t*>(c->heap[c->rank]) + c->epoch_off)));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_comm_wait_flag(const int* flag, int value, unsigned max_polls, int* result, ovb_stream_t stream) {
    OVB_REQUIRE(flag != nullptr && max_polls > 0 && max_polls <= (1u << 24), "ovb_comm_wait_flag: need a flag and 1 .. 2^24 polls");
    wait_flag_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(flag, value, max_polls, status_word(), result);
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_comm_argmax_combine(const ovb_comm* c, int* ids, const float* max_vals, int rows, int shard_size, ovb_stream_t stream) {
    OVB_REQUIRE(ids != nullptr && max_vals != nullptr && rows > 0 && rows <= kArgmaxRowsCap, "ovb_comm_argmax_combine: rows must be 1..%d", kArgmaxRowsCap);
    CommK k;
    if (int rc = fill(c, &k, c ? c->site : 0)) return rc;
    OVB_REQUIRE(c->flags_per_site >= kArgmaxDataOff + 2 * c->world * kArgmaxRowsCap * 2, "ovb_comm_argmax_combine: flag area of a site is too small");
    const int threads = ((rows > c->world ? rows : c->world) + 31) / 32 * 32;
    OVB_CHECK_CUDA(launch_pdl(argmax_combine_kernel, dim3(1), dim3(threads), 0, static_cast<cudaStream_t>(stream), k, ids, max_vals, rows, shard_size));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

int ovb_comm_allreduce_bf16(const ovb_comm* c, void* data, int64_t n, ovb_stream_t stream) { return ovb_comm_allreduce(c, data, n, OVB_DT_BF16, stream); }

#define OVB_COMM_DISPATCH(dtype, CALL)                          \
    switch (dtype) {                                            \
        case OVB_DT_F32: { constexpr int DT = OVB_DT_F32; CALL; break; }   \
        case OVB_DT_F16: { constexpr int DT = OVB_DT_F16; CALL; break; }   \
        default: { constexpr int DT = OVB_DT_BF16; CALL; break; }          \
    }

int ovb_comm_allreduce(const ovb_comm* c, void* data, int64_t n, int dtype, ovb_stream_t stream) {
    OVB_REQUIRE(dtype == OVB_DT_F32 || dtype == OVB_DT_F16 || dtype == OVB_DT_BF16, "ovb_comm_allreduce: fp32, fp16 or bf16");
    const int esz = dtype == OVB_DT_F32 ? 4 : 2, per_piece = 16 / esz;
    OVB_REQUIRE(data != nullptr && n > 0 && n % per_piece == 0, "ovb_comm_allreduce: the size must be a positive multiple of 16 bytes");
    CommK k;
    if (int rc = fill(c, &k, c ? c->site : 0)) return rc;
    const int64_t off = static_cast<uint8_t*>(data) - k.heap[c->rank];
    OVB_REQUIRE(off >= 0 && off + n * esz <= c->heap_bytes && off % 16 == 0, "ovb_comm_allreduce: the tensor must live in the symmetric heap, 16-byte aligned");
    const int64_t npieces = n / per_piece;
    if (k.mc != nullptr && (c->world == 2 || c->world == 4 || c->world == 8)) {
        int grid = (int)((npieces / c->world + 255) / 256);
        if (grid < 1) grid = 1;
        if (grid > 148) grid = 148;
        if ((int64_t)grid * kNvlsFlagStride > c->nvls_flags_per_site) grid = (int)(c->nvls_flags_per_site / kNvlsFlagStride);
        OVB_REQUIRE(grid >= 1, "ovb_comm_allreduce: no barrier words for the call site");
        OVB_COMM_DISPATCH(dtype, OVB_CHECK_CUDA(launch_pdl(allreduce_nvls_kernel<DT>, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), k, (long long)off,
                                                           (long long)npieces)));
        return 0;
    }
    const int64_t rank_stride = ((c->stage3_bytes > 0 ? c->stage3_bytes : c->stage1_bytes) / c->world) & ~int64_t(15);
    OVB_REQUIRE(n * esz <= rank_stride, "ovb_comm_allreduce: %lld bytes exceed the staging share of a rank (%lld)", (long long)(n * esz), (long long)rank_stride);
    int grid = (int)((npieces + 255) / 256);
    if (grid > 148) grid = 148;
    OVB_REQUIRE((int64_t)grid * c->world <= c->flags_per_site, "ovb_comm_allreduce: flag area of a site is too small");
    OVB_COMM_DISPATCH(dtype, OVB_CHECK_CUDA(launch_pdl(allreduce_kernel<DT>, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), k, (long long)off,
                                                       (long long)npieces, (long long)rank_stride)));
    OVB_CHECK_CUDA(cudaGetLastError());
    return 0;
}

}  // extern "C"
