// Kernel parameters shared by the attention kernels (attention.cu: mma.sync prefill fallback, split-KV decode;
// attention_sm100.cu: tcgen05 prefill).
#pragma once
#include <cuda_runtime.h>

namespace ovb {

struct PaKParams {
    const void* q;
    void* out;
    const void* k_cache;
    const void* v_cache;
    const int* past_lens;
    const int* subsequence_begins;
    const int* block_indices;
    const int* block_indices_begins;
    float* scratch;
    int B, T, Hq, Hkv;
    int ldq;
    int block_size;
    int sliding_window;
    int nsplit;
    int keys_per_split;
    float scale_log2;
    // dense mode (no paging): k/v are [B, S, H, D] with token pitch ld_kv elements
    int dense_S;
    int ld_kv;
    int causal;
    // u8 KV cache (kv_u8 != 0): k_cache / v_cache hold bytes [block, kv head, slot, D]; k_meta / v_meta hold one fp16 pair
    // (scale, zero point) per (block, kv head, slot): value = (byte - zero point) * scale
    int kv_u8;
    const void* k_meta;
    const void* v_meta;
};

// tcgen05 / TMA prefill and dense attention (attention_sm100.cu). Returns a negative code when the shape is not one it
// serves (the caller then uses the mma.sync kernel): head size 64 or 128, 16-key pages, 1, 2, 4 or 8 query heads per KV head.
int launch_prefill_tc(const PaKParams& p, int D, int G, bool paged, bool f16, int num_q_tiles, cudaStream_t stream);

}  // namespace ovb
