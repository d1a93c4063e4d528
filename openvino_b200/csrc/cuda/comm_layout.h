// Index arithmetic of the fused all-reduce protocols, shared by the kernels (gemm_sm100.cu) and by the host-side thread
// model of the protocols (tests/native/comm_protocol_model.cpp): where a piece of a tile goes, who owns it, where a
// rank's barrier words are. A "piece" is 16 bytes (eight bf16) of a [BT tokens x 128 columns] tile; piece i covers
// token i / 16, columns (i % 16) * 8 ... + 7. A packet is a piece with a tag word after every data word (32 bytes).
#pragma once
#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define OVB_HD __host__ __device__ __forceinline__
#else
#define OVB_HD inline
#endif

namespace ovb {

constexpr int kPieceBytes = 16;
constexpr int kPacketBytes = 32;

// Tag of a packet: the step number and the call site, so that a stale packet of an earlier step or of the other call
// site that shares the staging buffer is never taken for the awaited one.
OVB_HD uint32_t packet_tag(int epoch, int site) { return ((uint32_t)epoch << 8) | (uint32_t)(site & 255); }

// ---- two-hop protocol (one-shot sizes on more than two ranks)
// Owner of piece i when every rank owns `share` = pieces / world consecutive pieces.
OVB_HD int twohop_owner(int i, int share) { return i / share; }
// Hop 1, in the OWNER's staging buffer: packet k of the owner's share of tile `tile`, sent by rank `src`.
OVB_HD size_t twohop_hop1_offset(int src, int tiles, int tile, int share, int k) {
    return (((size_t)src * tiles + tile) * share + (size_t)k) * kPacketBytes;
}
// Bytes of the hop-1 area (all ranks' packets of all tiles); the hop-2 area follows it.
OVB_HD size_t twohop_hop1_bytes(int tiles, int pieces) { return (size_t)tiles * pieces * kPacketBytes; }
// Hop 2, in EVERY rank's staging buffer: finished piece i of tile `tile`.
OVB_HD size_t twohop_hop2_offset(int tiles, int pieces, int tile, int i) {
    return twohop_hop1_bytes(tiles, pieces) + ((size_t)tile * pieces + (size_t)i) * kPacketBytes;
}

// ---- one-shot packets: every rank's partial tile goes to every rank
OVB_HD size_t oneshot_slot_offset(int src, int tiles, int tile, int pieces) {
    return ((size_t)src * tiles + tile) * (size_t)pieces * kPacketBytes;
}

// ---- in-switch protocol: barrier words of a tile (int32 index): 8 "arrived" words, then 8 "done" words
constexpr int kNvlsFlagStride = 16;
OVB_HD size_t nvls_barrier_word(int tile, int phase, int rank) { return (size_t)tile * kNvlsFlagStride + (size_t)phase * 8 + rank; }

}  // namespace ovb
