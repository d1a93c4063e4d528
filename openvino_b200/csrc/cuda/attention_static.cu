// ovb_paged_attention_decode_static: decode attention whose split-KV scratch is a fixed array in device
// global memory, so that the call allocates nothing. The contract is written out in ovb_cuda_static.h.
#include <mutex>

#include "common.cuh"
#include "ovb_cuda_static.h"

namespace {

// The scratch itself. Lives in this library's device image; one copy per device that loads the image.
static __device__ __align__(256) unsigned char g_pa_static_scratch[OVB_PA_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
float* g_scratch_of_device[kMaxDevices] = {nullptr};   // device address of the array, per device, set once
std::mutex g_setup_mu;

// Device address of the array on the current device. The first call per device asks the runtime for it.
int static_scratch(float** out) {
    int dev = -1;
    OVB_CHECK_CUDA(cudaGetDevice(&dev));
    OVB_REQUIRE(dev >= 0 && dev < kMaxDevices, "ovb_paged_attention_decode_static: device index %d is out of range", dev);
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (g_scratch_of_device[dev] == nullptr) {
        void* ptr = nullptr;
        OVB_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_pa_static_scratch));
        OVB_REQUIRE(ptr != nullptr, "ovb_paged_attention_decode_static: the static scratch has no device address");
        g_scratch_of_device[dev] = static_cast<float*>(ptr);
    }
    *out = g_scratch_of_device[dev];
    return 0;
}

}  // namespace

extern "C" int ovb_paged_attention_decode_static(const ovb_pa_args* a, ovb_stream_t stream) {
    OVB_REQUIRE(a != nullptr, "ovb_paged_attention_decode_static: null argument block");
    OVB_REQUIRE(a->max_q_len == 1 && a->T == a->B,
                "ovb_paged_attention_decode_static: decode batches only (one query token per sequence), got max_q_len %d, T %d, B %d",
                a->max_q_len, a->T, a->B);
    OVB_REQUIRE(a->B > 0 && a->Hq > 0 && a->D > 0 && a->Hkv > 0 && a->Hq % a->Hkv == 0, "ovb_paged_attention_decode_static: bad sizes");
    // Only the split-KV decode kernel uses the scratch; other shapes would be served by the ragged kernel, which needs none.
    // Refuse them here, so that a caller never believes it runs the split path when it does not.
    const int group = a->Hq / a->Hkv;
    OVB_REQUIRE(a->D == 128 && a->block_size == 16 && (group == 1 || group == 2 || group == 4 || group == 8),
                "ovb_paged_attention_decode_static: the split-KV decode kernel serves head size 128, block size 16 and 1, 2, 4 or 8 query "
                "heads per KV head (got D %d, block size %d, %d heads per KV head); use ovb_paged_attention for other shapes",
                a->D, a->block_size, group);
    const int64_t need = ovb_pa_scratch_bytes(a->B, a->Hq, a->D, a->max_context_len);
    if (need > (int64_t)OVB_PA_STATIC_SCRATCH_BYTES) {
        ovb::set_error("ovb_paged_attention_decode_static: this batch needs %lld bytes of scratch (B %d x Hq %d x D %d) but the static "
                       "scratch holds %lld; use ovb_paged_attention with a caller-allocated buffer",
                       (long long)need, a->B, a->Hq, a->D, (long long)OVB_PA_STATIC_SCRATCH_BYTES);
        return ovb::ERR_TOO_LARGE;
    }
    float* scratch = nullptr;
    if (int rc = static_scratch(&scratch)) return rc;
    ovb_pa_args args = *a;
    args.scratch = scratch;   // every slot that the merge step reads is written first by the same call: no clearing needed
    return ovb_paged_attention(&args, stream);
}
