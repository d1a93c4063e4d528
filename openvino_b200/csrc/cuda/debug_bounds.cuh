// Debug build of the kernels (-DOVB_DEBUG_BOUNDS): indices that kernels read from device memory (KV-cache block ids, cache
// slots, token ids, expert row offsets) are checked against the limits that the host declared with
// ovb_debug_set_limits(); an index out of range records STATUS_BAD_INDEX in the status word and is replaced by 0, so the
// kernel finishes without touching memory outside its tensors and the host reads the status. The release build compiles
// the checks away. Every translation unit that checks indices keeps its own copy of the limits (there is no relocatable
// device code in this library); the host entry point updates all copies.
// Role in the reference: the bounds-checking debug builds of the plugins' kernels (ENABLE_DEBUG_CAPS, OV_GPU_* dumps) and
// the sanitizer builds of cmake/developer_package/compile_flags/sanitizer.cmake.
#pragma once
#include "sm100_ptx.cuh"

namespace ovb {

struct DebugLimits {
    int kv_blocks;      // blocks of the paged KV cache (0: unknown, no check)
    int vocab;          // rows of the embedding table
    int* status;        // device status word
};

#ifdef OVB_DEBUG_BOUNDS
#define OVB_DEBUG_LIMITS_DEFINE static __device__ ovb::DebugLimits g_dbg_limits;
#define OVB_DBG_BLOCK(blk) ovb::dbg_check((blk), g_dbg_limits.kv_blocks, g_dbg_limits.status)
#define OVB_DBG_SLOT(slot, block_size) ovb::dbg_check_slot((slot), g_dbg_limits.kv_blocks, (block_size), g_dbg_limits.status)
#define OVB_DBG_ROW(row, limit) ovb::dbg_check((row), (limit), g_dbg_limits.status)
__device__ __forceinline__ int dbg_check(int idx, int limit, int* status) {
    if (limit > 0 && (unsigned)idx >= (unsigned)limit) {
        report_status(status, STATUS_BAD_INDEX);
        return 0;
    }
    return idx;
}
// a slot may be negative ("do not write"); otherwise it must fall inside the cache
__device__ __forceinline__ int dbg_check_slot(int slot, int blocks, int block_size, int* status) {
    if (slot >= 0 && blocks > 0 && slot >= blocks * block_size) {
        report_status(status, STATUS_BAD_INDEX);
        return -1;
    }
    return slot;
}
#else
#define OVB_DEBUG_LIMITS_DEFINE
#define OVB_DBG_BLOCK(blk) (blk)
#define OVB_DBG_SLOT(slot, block_size) (slot)
#define OVB_DBG_ROW(row, limit) (row)
#endif

}  // namespace ovb
