// Host-side helpers shared by the kernel translation units: error reporting, the per-device
// status word, and TMA tensor-map creation through the driver entry point (no link-time
// dependency on libcuda, so the library also loads on machines without a driver).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "ovb_cuda.h"

namespace ovb {

enum : int {
    ERR_BAD_ARG = -1,
    ERR_CUDA = -2,
    ERR_TMAP = -3,
    ERR_TOO_LARGE = -4,
    ERR_UNSUPPORTED = -5,
};

void set_error(const char* fmt, ...);
int* status_word();   // device pointer of the current device's status word (NULL on failure)

#define OVB_CHECK_CUDA(expr)                                                                       \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess) {                                                                   \
            ovb::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
            return ovb::ERR_CUDA;                                                                  \
        }                                                                                          \
    } while (0)

#define OVB_REQUIRE(cond, ...)            \
    do {                                  \
        if (!(cond)) {                    \
            ovb::set_error(__VA_ARGS__);  \
            return ovb::ERR_BAD_ARG;      \
        }                                 \
    } while (0)

// 2-D row-major tensor map: `rows` x `cols` elements of `elem_bytes`, row pitch `pitch_bytes`,
// box `box_cols` x `box_rows`. swizzle128: 128-byte swizzle (box_cols * elem_bytes must be 128).
int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t rows,
                 uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, bool swizzle128);

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Programmatic dependent launch: kernels of a stream that call pdl_wait() (sm100_ptx.cuh) are launched with the
// programmatic-stream-serialization attribute, so that the preamble of a kernel (barrier set-up, tensor-memory allocation,
// the first weight fetches) runs under the tail of the kernel before it. Works inside stream capture (the edge becomes a
// programmatic dependency of the graph). OVB_PDL=0 in the environment, or ovb_set_pdl(0), turns the attribute off.
bool pdl_enabled();

// Polls (about 0.25 us apart) that a kernel spends waiting for a peer GPU before it gives up, records STATUS_PEER_TIMEOUT in
// the status word and returns. About one second by default; OVB_PEER_SPIN_LIMIT in the environment or
// ovb_set_peer_spin_limit() change it (failure-detection tests use a few milliseconds).
uint32_t peer_spin_limit();

// Launch `kern` with the attribute (when enabled). Only for kernels whose every thread passes pdl_wait() before it touches
// memory that an earlier kernel of the stream may write or still read.
template <class... P, class... A>
inline cudaError_t launch_pdl(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<P>(args)...);
}

// Plain launch (fully ordered after the stream's earlier work). Kernels that write what a later GEMM reads as its
// WEIGHT operand (the re-packing kernels) use this and never call pdl_trigger(): a GEMM fetches weights before its own
// pdl_wait(), which is only sound while no kernel that may still be running writes them.
template <class... P, class... A>
inline cudaError_t launch_serial(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<P>(args)...);
}

}  // namespace ovb
