#include <cudaTypedefs.h>
#include <stdarg.h>
#include <stdlib.h>

#include <mutex>

#include <atomic>

#include "common.cuh"
#include "debug_bounds.cuh"

namespace ovb {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

static int* g_status[64] = {nullptr};
static std::mutex g_status_mu;

int* status_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_status_mu);
    if (g_status[dev] == nullptr) {
        int* p = nullptr;
        if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
        cudaMemset(p, 0, 256);
        g_status[dev] = p;
    }
    return g_status[dev];
}

static int g_pdl = -1;   // -1: not decided yet (environment), 0 / 1

bool pdl_enabled() {
    if (g_pdl < 0) {
        const char* e = getenv("OVB_PDL");
        g_pdl = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return g_pdl != 0;
}

static std::atomic<uint32_t> g_spin_limit{0};
uint32_t peer_spin_limit() {
    uint32_t v = g_spin_limit.load(std::memory_order_relaxed);
    if (v == 0) {
        const char* e = getenv("OVB_PEER_SPIN_LIMIT");
        const long long want = e ? atoll(e) : 0;
        v = want > 0 && want < (1ll << 31) ? (uint32_t)want : (1u << 22);
        g_spin_limit.store(v, std::memory_order_relaxed);
    }
    return v;
}

static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

static int load_encode() {
    if (g_encode) return 0;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || fn == nullptr) {
        set_error("cuTensorMapEncodeTiled entry point not available: %s", cudaGetErrorString(e));
        return ERR_TMAP;
    }
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    return 0;
}

int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t rows,
                 uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
    if (int rc = load_encode()) return rc;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (pitch_bytes & 15) != 0) {
        set_error("TMA operand must be 16-byte aligned with a 16-byte multiple row pitch (base %p pitch %llu)", base,
                  (unsigned long long)pitch_bytes);
        return ERR_BAD_ARG;
    }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with %d (rows %llu cols %llu pitch %llu box %ux%u elem %d)", (int)r,
                  (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)pitch_bytes, box_rows, box_cols,
                  elem_bytes);
        return ERR_TMAP;
    }
    return 0;
}

}  // namespace ovb

extern "C" {

int ovb_version(void) { return 100; }

int ovb_set_pdl(int on) {
    const int before = ovb::pdl_enabled() ? 1 : 0;
    ovb::g_pdl = on ? 1 : 0;
    return before;
}

unsigned ovb_set_peer_spin_limit(unsigned polls) {
    const unsigned before = ovb::peer_spin_limit();
    ovb::g_spin_limit.store(polls ? polls : (1u << 22), std::memory_order_relaxed);
    return before;
}

#ifdef OVB_DEBUG_BOUNDS
int ovb_debug_set_limits_attention(const ovb::DebugLimits* l);
int ovb_debug_set_limits_elementwise(const ovb::DebugLimits* l);
#endif

int ovb_debug_bounds_enabled(void) {
#ifdef OVB_DEBUG_BOUNDS
    return 1;
#else
    return 0;
#endif
}

int ovb_debug_set_limits(int kv_blocks, int vocab) {
#ifdef OVB_DEBUG_BOUNDS
    ovb::DebugLimits l;
    l.kv_blocks = kv_blocks;
    l.vocab = vocab;
    l.status = ovb::status_word();
    if (int rc = ovb_debug_set_limits_attention(&l)) return rc;
    return ovb_debug_set_limits_elementwise(&l);
#else
    (void)kv_blocks; (void)vocab;
    return 0;
#endif
}

const char* ovb_last_error(void) { return ovb::g_err; }

int* ovb_status_ptr(void) { return ovb::status_word(); }

int ovb_status_read(ovb_stream_t stream) {
    int* p = ovb::status_word();
    if (!p) return -1;
    int v = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&v, p, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(s) != cudaSuccess) return -1;
    if (v != 0) cudaMemsetAsync(p, 0, sizeof(int), s);
    return v;
}
}
