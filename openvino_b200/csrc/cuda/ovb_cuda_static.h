// Allocation-free decode attention: one extra entry point of libovb_cuda.so.
//
// This entry point has no counterpart in the reference; it exists for users of this library's C ABI.
//
// Who needs it. ovb_paged_attention() splits long contexts over several thread blocks and merges their
// partial results through a scratch buffer that the caller allocates (ovb_pa_scratch_bytes tells how much).
// Some callers have no good way to allocate device memory:
//   * a C, C++ or ctypes client that links only this library and carries no tensor allocator;
//   * a serving loop that has already handed every free byte of the device to the KV cache;
//   * a latency-critical thread that must not call cudaMalloc/cudaFree, because those calls may wait for
//     all work on the device.
// For them ovb_paged_attention_decode_static() keeps the scratch inside the library: a fixed array in
// device global memory, OVB_PA_STATIC_SCRATCH_BYTES large, that comes into being when the library's code
// is loaded onto a device. The function calls no allocating routine of the CUDA runtime, of any library
// or of PyTorch, on any call.
//
// Contract.
//   * Decode batches only: one query token per sequence (a->max_q_len == 1, a->T == a->B); a->scratch is
//     ignored. Everything else in ovb_pa_args means what it means for ovb_paged_attention(), and the result
//     is the same.
//   * Shapes: what the split-KV decode kernel serves, i.e. head size 128, cache block size 16 and 1, 2, 4 or 8
//     query heads per KV head. Other shapes are refused with an error (ovb_paged_attention() runs them through
//     a kernel that needs no scratch, so they need no entry point of their own).
//   * Size limit: the call needs ovb_pa_scratch_bytes(B, Hq, D, max_context_len) bytes, which today is
//     B * Hq * 32 * (D + 2) * 4. If that exceeds OVB_PA_STATIC_SCRATCH_BYTES the call launches nothing and
//     returns a negative code; ovb_last_error() then names both numbers. With D = 128 the limit admits
//     B * Hq <= 504, e.g. 15 sequences of a 32-head model, or 126 sequences of a 4-head tensor-parallel shard.
//   * First call on a device: it looks up the device address of the array (cudaGetSymbolAddress, with that
//     device current) and remembers it per device. The look-up may make the runtime load this library's
//     device code. Make that first call during start-up, before any stream capture begins on that device.
//     The remembered address belongs to the device's current context: after cudaDeviceReset() on that device
//     it is stale, and the library has no way to notice. A process that resets a device must not call this
//     entry point on it again.
//   * Every call on a device shares the one array, and the array keeps whatever the previous call left
//     in it. No part of it has to start at zero: each call first writes every slot that it later reads.
//     Two calls that can overlap on the device (different streams, or different host threads on the same
//     device) would overwrite each other's partial results: run such calls one after another, or use
//     ovb_paged_attention() with separate scratch buffers instead.
#pragma once
#include "ovb_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

#define OVB_PA_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)

// Returns 0 on success, a negative code otherwise (see ovb_last_error()).
int ovb_paged_attention_decode_static(const ovb_pa_args* a, ovb_stream_t stream);

#ifdef __cplusplus
}
#endif
