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

}  // namespace ovb
