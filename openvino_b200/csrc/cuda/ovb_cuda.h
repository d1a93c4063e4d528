// C ABI of the sm_100a kernel library (libovb_cuda.so). Every entry point takes raw device
// pointers plus a CUDA stream and returns 0 on success or a negative error code; device-side
// problems (a wait that ran out, a failed argument check) are reported through the status
// word returned by ovb_status_ptr()/ovb_status_read().
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* ovb_stream_t;

// ---------------------------------------------------------------------------------------------
// Library / device
int ovb_version(void);
// Device status word of the current device (allocated on first use, 4 bytes of device memory).
int* ovb_status_ptr(void);
// Copy the status word to the host (synchronises the stream) and reset it to 0.
int ovb_status_read(ovb_stream_t stream);
const char* ovb_last_error(void);
// Programmatic dependent launch of the library's kernels (on by default; OVB_PDL=0 in the environment turns it off):
// a kernel's preamble overlaps the tail of the kernel before it in the stream. Returns the previous setting.
int ovb_set_pdl(int on);
/* Polls (about 0.25 us apart) that a kernel waits for a peer GPU before it records OVB status 2 (peer timeout) and returns;
   0 restores the default (about one second). Returns the previous value. */
unsigned ovb_set_peer_spin_limit(unsigned polls);
/* Debug build of the kernels (compiled with -DOVB_DEBUG_BOUNDS, libovb_cuda_dbg.so): block ids, cache slots and token ids
   that kernels read from device memory are checked against these limits; an index out of range records status 5 and the
   access is skipped. In the release build ovb_debug_bounds_enabled() returns 0 and the limits are ignored. */
int ovb_debug_bounds_enabled(void);
int ovb_debug_set_limits(int kv_blocks, int vocab);

// ---------------------------------------------------------------------------------------------
// GEMM family:  out[T, N] = epilogue( X[T, K] * dequant(W[N, K])^T )
// Weights sit on the 128-row M side of tcgen05.mma (weight-stationary "swap-AB"), tokens on
// the N side, so the same kernel serves decode (T <= 64) and prefill (T in the thousands).
enum {
    OVB_W_BF16 = 0,   // W is bf16 [N, K]
    OVB_W_U4 = 1,     // W is packed u4 in the plugin layout made by ovb_pack_u4 (4608-byte chunks, see below)
    OVB_W_U8 = 2,     // W is u8 [N, K]
    OVB_W_F16 = 3,    // W and X are fp16 (BERT path)
    OVB_W_F8 = 4,     // W is fp8 e4m3 [N, K]; the (scale, -) pair table carries the block scale of every (k-group, row) times 2^120
};
enum {
    OVB_ACT_NONE = 0,
    OVB_ACT_GELU_ERF = 1,
    OVB_ACT_RELU = 2,
    OVB_ACT_SILU = 3,
    OVB_ACT_SWIGLU = 4,   // gated MLP: every 128-row tile of W holds 64 "gate" rows, then the 64 "up" rows of the same channels;
                          // out [T, N/2] = silu(gate) * up
    OVB_ACT_GELU_TANH = 5,
};

typedef struct {
    const void* x;        // [T, K] bf16/fp16, row pitch ldx elements
    const void* w;        // see OVB_W_*
    void* out;            // [T, N] bf16/fp16 (or fp32 when out_f32), row pitch ldo elements
    const void* bias;     // [N] same type as x, or NULL
    const void* residual; // [T, N] same type as out (16-bit only), row pitch ldr, or NULL
    const void* scales;   // u4/u8: [K/group, N] pairs of bf16 (scale, zero point); u4 zero points are stored as 16+zp
    const void* zps;      // unused (kept for layout compatibility)
    float* ws;            // split-K workspace (fp32), may be NULL when splits == 1
    int* counters;        // split-K tile counters (zero-initialised, self-resetting), may be NULL
    int64_t ws_bytes;     // capacity of ws
    int T, N, K;
    int ldx, ldo, ldr;
    int group_size;       // quantisation group along K (multiple of 64)
    int wmode;            // OVB_W_*
    int act;              // OVB_ACT_*
    int out_f32;          // 1: fp32 output
    int splits;           // 0 = choose automatically
    int block_t;          // 0 = choose automatically (16/32/64/128/256)
    int w_tiled;          // 16-bit weights are in the tile-contiguous layout made by ovb_pack_w16
    // Tensor-parallel: out = residual + sum over ranks of (x * W^T), reduced inside the epilogue (see ovb_comm below).
    void* comm;           // const ovb_comm* or NULL
    // Window into a larger tile-contiguous weight (experts stacked along N or K): chunks of one 128-row weight tile are
    // w_kb_stride apart from the next tile's (0 = K / 64, the weight is exactly [N, K]); `w` points at the window's first chunk.
    int w_kb_stride;
    // Grouped GEMM (mixture of experts, one launch for all experts of a rank). The rows of x / out are sorted by group: group
    // g owns rows [group_offsets[g], group_offsets[g + 1]) (int32 device array of num_groups + 1 entries that an earlier
    // kernel of the stream wrote; no host copy is needed) and multiplies them with weight g of a tile-packed stack:
    // group_mode 1 = stacked along N (w is [num_groups * N, K]), 2 = stacked along K (w is [N, num_groups * K]); N and K
    // describe ONE group's weight. T is the row capacity of x / out. NULL: ordinary GEMM.
    const int* group_offsets;
    int num_groups;
    int group_mode;
} ovb_gemm_args;

int ovb_gemm(const ovb_gemm_args* a, ovb_stream_t stream);
// Bytes of split-K workspace / number of counters that ovb_gemm may need for the given problem.
int64_t ovb_gemm_ws_bytes(int T, int N, int K, int act);
int ovb_gemm_num_counters(void);
/* Conditional compilation: bit (log2(token tile) - 4) of the result is set when the GEMM variant (tile, wmode, fp16) has been
   launched in this process; ovb_cc_is_selective tells whether the library is a selective build. */
unsigned ovb_cc_used_gemm(int wmode, int is_f16);
int ovb_cc_is_selective(void);

// Re-pack IR-layout u4 weights (LSB-first nibbles, [N, K]) into the plugin layout read by the
// dequantising GEMM, and build the transposed table of (bf16 scale, bf16 16+zero point) pairs.
//   w_ir    : [N, K/2] bytes         scales_ir: [N, G] fp16     zps_ir: [N, G/2..] packed u4 or NULL (zp = 8)
//   w_out      : ceil(N/128) * (K/64) chunks of 4608 bytes (4 KB of nibbles + the 128 rows' bf16 pairs)
//   scales_out : [G, N, 2] bf16      zps_out: optional [G, N] bf16 (may be NULL)
int ovb_pack_u4(const void* w_ir, const void* scales_ir, const void* zps_ir, int zp_is_u8, void* w_out,
                void* scales_out, void* zps_out, int N, int K, int group_size, ovb_stream_t stream);

// Re-pack a 16-bit [N, K] row-major weight into the tile-contiguous layout: for every 128-row tile and
// 64-column k-block one 16 KB chunk whose 16-byte pieces are already placed in the 128-byte swizzle
// ((tile * K/64 + kb) * 128 + row) * 8 + (piece ^ (row & 7)). w_out holds ceil(N/128)*128 * K elements.
int ovb_pack_w16(const void* w, void* w_out, int N, int K, ovb_stream_t stream);

// ---------------------------------------------------------------------------------------------
// Normalisation / elementwise
// y = rmsnorm(x (+ residual)) * gamma ;  if residual_out != NULL it receives x + residual.
int ovb_rmsnorm(const void* x, const void* residual, const void* gamma, void* y, void* residual_out, int rows,
                int cols, float eps, ovb_stream_t stream);
int ovb_layernorm(const void* x, const void* residual, const void* gamma, const void* beta, void* y, int rows,
                  int cols, float eps, int is_f16, ovb_stream_t stream);
// Linear recurrences (fp32, contiguous). `state` is read, advanced over the L tokens of every sequence and written back.
// Selective state-space scan: A [H], dt [B, L, H], Bm / Cm [B, L, G, S], x / y [B, L, H, P], state [B, H, P, S]; S <= 256.
int ovb_selective_ssm(const float* A, const float* dt, const float* Bm, const float* x, const float* Cm, float* state, float* y, int B, int L, int H, int P,
                      int G, int S, ovb_stream_t stream);
// Gated delta rule: q / k [B, L, Hq, Dk] (q scaled, both normalised by the caller where the layer asks for it), v / y [B, L, Hv, Dv],
// gate / beta [B, L, Hv], state [B, Hv, Dk, Dv]; Dk <= 256.
int ovb_gated_delta_rule(const float* q, const float* k, const float* v, const float* gate, const float* beta, float* state, float* y, int B, int L, int Hq,
                         int Hv, int Dk, int Dv, ovb_stream_t stream);
// out[t, :] = silu(gu[t, :F]) * gu[t, F:2F]
int ovb_silu_mul(const void* gu, void* out, int rows, int F, ovb_stream_t stream);
/* The same over the first min(*nrows, rows) rows; nrows is device memory written by an earlier kernel of the stream. */
int ovb_silu_mul_counted(const void* gu, void* out, int rows, int F, const int* nrows, ovb_stream_t stream);
/* MoE prefill: token lists per local expert (idx[e * idx_stride + i], counts[e]) from the dense routing matrix route [T, E];
   SwiGLU of an expert's gathered rows scaled by the routing weight; dst[idx[i]] += src[i]. */
int ovb_moe_group(const float* route, int T, int E, int e0, int nloc, int* idx, int idx_stride, int* counts, ovb_stream_t stream);
int ovb_moe_silu_mul_rows(const void* gu, const float* route, const int* idx, void* out, int rows, int F, int E, int e, ovb_stream_t stream);
int ovb_moe_scatter_add(const void* src, const int* idx, void* dst, int rows, int H, int ld_dst, ovb_stream_t stream);
/* Single-launch expert path (no host round trip). ovb_moe_positions: pos[t * nloc + e] = position of token t in local expert
   e's row list or -1, counts[e] rows. ovb_moe_gather_sorted: offsets[nloc + 1] = row offsets of the experts in the sorted
   buffer (capped at cap rows) and xg[offsets[e] + pos] = x[t]. ovb_moe_combine_sorted: dst[t] (+)= sum over the local
   experts, in index order, of route[t, e0 + e] * y[offsets[e] + pos[t, e]]. The grouped ovb_gemm runs in between. */
int ovb_moe_positions(const float* route, int T, int E, int e0, int nloc, int* pos, int* counts, ovb_stream_t stream);
int ovb_moe_gather_sorted(const void* x, const int* pos, const int* counts, int* offsets, void* xg, int T, int H, int nloc, int cap, ovb_stream_t stream);
int ovb_moe_combine_sorted(const void* y, const float* route, const int* pos, const int* offsets, void* dst, int T, int H, int E, int e0, int nloc,
                           int ld_dst, int accumulate, int cap, ovb_stream_t stream);
/* ---- generic primitives of the graph executor (fp32 / fp16 / bf16 storage, fp32 arithmetic) ---- */
enum { OVB_DT_F32 = 0, OVB_DT_F16 = 1, OVB_DT_BF16 = 2 };
enum {
    OVB_UN_RELU = 0, OVB_UN_SIGMOID, OVB_UN_TANH, OVB_UN_GELU_ERF, OVB_UN_GELU_TANH, OVB_UN_SWISH /* a = beta */, OVB_UN_EXP, OVB_UN_LOG,
    OVB_UN_SQRT, OVB_UN_ABS, OVB_UN_NEG, OVB_UN_HSWISH, OVB_UN_HSIGMOID, OVB_UN_MISH, OVB_UN_SOFTPLUS, OVB_UN_ERF, OVB_UN_FLOOR, OVB_UN_CEIL,
    OVB_UN_SIGN, OVB_UN_CLAMP /* a = min, b = max */, OVB_UN_ELU /* a = alpha */, OVB_UN_SIN, OVB_UN_COS, OVB_UN_RSQRT, OVB_UN_SOFTSIGN,
    OVB_UN_ROUND_EVEN, OVB_UN_ROUND_AWAY, OVB_UN_SCALE_SHIFT /* x * a + b */, OVB_UN_COUNT
};
enum { OVB_BIN_ADD = 0, OVB_BIN_SUB, OVB_BIN_MUL, OVB_BIN_DIV, OVB_BIN_MAX, OVB_BIN_MIN, OVB_BIN_POW, OVB_BIN_SQDIFF, OVB_BIN_PRELU, OVB_BIN_COUNT };
enum { OVB_RED_SUM = 0, OVB_RED_MEAN, OVB_RED_MAX, OVB_RED_MIN, OVB_RED_PROD, OVB_RED_L2, OVB_RED_L1, OVB_RED_COUNT };
#define OVB_MAX_DIMS 6
int ovb_unary(int op, const void* x, void* y, int64_t n, int dtype, float a, float b, ovb_stream_t stream);
/* y (contiguous, `shape`) = op(a, b); sa / sb are element strides of the operands (0 on a broadcast axis); same != 0: both
   operands are contiguous and of the output's shape (16-byte vector path). */
int ovb_binary(int op, const void* a, const void* b, void* y, int nd, const int64_t* shape, const int64_t* sa, const int64_t* sb, int same, int dtype,
               ovb_stream_t stream);
/* y[sum c_k * sy_k] = x[sum c_k * sx_k] over `shape`: transposes, slices, broadcasts, pieces of a concat. */
int ovb_strided_copy(const void* x, void* y, int nd, const int64_t* shape, const int64_t* sx, const int64_t* sy, int elem_bytes, ovb_stream_t stream);
/* [batch, R, C] -> [batch, C, R] through shared memory (2- and 4-byte elements). */
int ovb_transpose2d(const void* x, void* y, int64_t batch, int R, int C, int elem_bytes, ovb_stream_t stream);
/* softmax / log-softmax over the middle axis of [outer, dim, inner]. */
int ovb_softmax(const void* x, void* y, int64_t outer, int dim, int64_t inner, int dtype, int log_out, ovb_stream_t stream);
/* y[outer, inner] = reduction over the middle axis of x[outer, dim, inner]. */
int ovb_reduce(int op, const void* x, void* y, int64_t outer, int dim, int64_t inner, int dtype, ovb_stream_t stream);
typedef struct ovb_pool_args {
    int64_t NC;               /* batch * channels */
    int H, W, OH, OW, kh, kw, sh, sw, ph, pw, ph_end, pw_end, dh, dw;
    int is_max, exclude_pad;
} ovb_pool_args;
int ovb_pool2d(const void* x, void* y, const ovb_pool_args* a, int dtype, ovb_stream_t stream);

/* bf16 [rows, cols] -> fp8 e4m3 bytes with one fp32 scale per row and group of 128 channels (scales [rows, cols/128]). */
int ovb_act_quant_fp8(const void* x, void* q, float* scales, int rows, int cols, ovb_stream_t stream);
/* Copy cache blocks src_blocks[i] -> dst_blocks[i] in the key and the value cache (block_bytes per block and cache). */
int ovb_kv_block_copy(void* k_cache, void* v_cache, const int* src_blocks, const int* dst_blocks, int num_pairs, int64_t block_bytes,
                      ovb_stream_t stream);
/* Convolution operand for the GEMM: 16-bit NCHW image -> cols [B*Ho*Wo, Kpad], k = (c*kh + r)*kw + s, zero padded. */
int ovb_im2col(const void* x, void* cols, int B, int C, int H, int W, int kh, int kw, int sh, int sw, int pt, int pl, int dh, int dw,
               int Ho, int Wo, int Kpad, ovb_stream_t stream);
// ids are int64 (ids_i32 == 0) or int32; ids outside [0, vocab) read row 0.
int ovb_embedding(const void* ids, int ids_i32, const void* table, void* out, int rows, int cols, int vocab,
                  ovb_stream_t stream);
// Greedy sampling: out_ids[r] = argmax_v logits[r, v] (first index on ties); optional out_max.
int ovb_argmax(const void* logits, int ld, int rows, int vocab, void* out_ids, int ids_i32, float* out_max,
               ovb_stream_t stream);
// Stochastic sampling (sampling.cu): temperature, top-k, top-p; deterministic for a (seed, *step, row) triple.
int ovb_sample(const void* logits, int ld, int rows, int vocab, float temperature, int top_k, float top_p, uint64_t seed,
               const int* step, int* out_ids, ovb_stream_t stream);
/* Temperature sampling over a vocabulary shard: perturbed arg-max (Gumbel-max) of logits[:, 0..vocab) whose tokens have the
   global indices vocab_offset + i; out_ids are local indices, out_max the perturbed maxima (for the arg-max exchange of
   tensor-parallel ranks). With vocab_offset = 0 and the whole vocabulary it is a complete sampler. */
int ovb_sample_gumbel(const void* logits, int ld, int rows, int vocab, int vocab_offset, float temperature, uint64_t seed, const int* step,
                      int* out_ids, float* out_max, ovb_stream_t stream);
/* The uniform in (0, 1) that the perturbed arg-max derives from a 64-bit hash (runs on the host; largest value 1 - 2^-24). */
float ovb_gumbel_uniform(uint64_t h);
int ovb_bump(int* counter, ovb_stream_t stream);     // *counter += 1 on the device
int ovb_add(const void* a, const void* b, void* out, int64_t n, ovb_stream_t stream);
// Mixture of experts. Router: softmax over E logits per token, top-k kept and renormalised; weights is dense [T, E] fp32.
int ovb_moe_route_topk(const float* logits, float* weights, int T, int E, int k, ovb_stream_t stream);
// SwiGLU of the `nloc` local experts [e0, e0 + nloc) stacked along the feature axis, scaled by the routing weight:
// gu [rows, nloc * 2F] (gate block then up block per expert) -> out [rows, nloc * F]; rows not routed to an expert get zeros.
int ovb_moe_silu_mul_scale(const void* gu, const float* weights, void* out, int rows, int F, int nloc, int E, int e0, ovb_stream_t stream);
// Device-side token feedback between chained steps (see elementwise.cu).
int ovb_resolve_ids(int* ids, const int* tok_src, const int* last_token, int T, ovb_stream_t stream);
int ovb_scatter_tokens(const int* tokens, const int* tok_dst, int* last_token, int B, ovb_stream_t stream);

// RoPE (half-rotate, LLaMA style) applied in place to q and k inside a fused qkv buffer, then
// k/v rows are scattered into the paged cache.
//   qkv       : [T, (Hq + 2*Hkv) * D] bf16
//   positions : [T] int32 absolute position of each token
//   slot_map  : [T] int32 physical slot (block * block_size + offset) of each token
//   k_cache/v_cache : [num_blocks, Hkv, block_size, D] bf16
int ovb_rope_kv_write(void* qkv, const int* positions, const int* slot_map, void* k_cache, void* v_cache, int T,
                      int Hq, int Hkv, int D, float theta, int block_size, ovb_stream_t stream);
/* The same into a u8 cache: key / value rows are quantised per (token, head) row and their (scale, zero point) pairs go
   to k_meta / v_meta (see ovb_pa_args). */
int ovb_rope_kv_write_u8(void* qkv, const int* positions, const int* slot_map, void* k_cache, void* v_cache, void* k_meta, void* v_meta, int T,
                         int Hq, int Hkv, int D, float theta, int block_size, ovb_stream_t stream);

// ---------------------------------------------------------------------------------------------
// Paged attention. Cache layout [num_blocks, Hkv, block_size, D]; ragged batch described like the
// PagedAttentionExtension op: past_lens[B], subsequence_begins[B+1], block_indices[...],
// block_indices_begins[B+1].
typedef struct {
    const void* q;            // [T, Hq*D] (row pitch ldq elements)
    void* out;                // [T, Hq*D] contiguous
    const void* k_cache;
    const void* v_cache;
    const int* past_lens;
    const int* subsequence_begins;
    const int* block_indices;
    const int* block_indices_begins;
    float* scratch;           // decode split-KV partials (see ovb_pa_scratch_bytes) or NULL
    int B, T, Hq, Hkv, D;
    int ldq;
    int block_size;
    int max_context_len;
    int max_q_len;            // longest subsequence in the batch (1 = pure decode)
    int sliding_window;       // 0 = off
    float scale;
    /* u8 KV cache (kv_u8 != 0): the caches hold bytes [num_blocks, Hkv, block_size, D], k_meta / v_meta one fp16 pair
       (scale, zero point) per (block, kv head, slot): value = (byte - zero point) * scale. Head size 128, 16-token blocks. */
    int kv_u8;
    const void* k_meta;
    const void* v_meta;
} ovb_pa_args;
int ovb_paged_attention(const ovb_pa_args* a, ovb_stream_t stream);
int64_t ovb_pa_scratch_bytes(int B, int Hq, int D, int max_context_len);

// Dense (non-paged) bidirectional attention for encoder models: q,k,v [B, S, H, D] fp16/bf16.
int ovb_sdpa_dense(const void* q, const void* k, const void* v, void* out, int B, int S, int H, int D, int ld,
                   float scale, int is_f16, int causal, ovb_stream_t stream);

// ---------------------------------------------------------------------------------------------
// Tensor-parallel communicator over NVLink peer memory: one process per GPU; every rank owns a "symmetric heap"
// (one device allocation with the same layout on every rank) that all ranks map through CUDA IPC handles.
// The Python side (openvino_b200/parallel/comm.py) allocates, exchanges and maps the heaps and fills this struct.
//
// Layout inside the heap (byte offsets, identical on every rank):
//   epoch_off    one int32: the step number, bumped by ovb_comm_step_begin at the start of every step
//   flags_off    num_sites x flags_per_site int32, zero at start; a flag holds the step number of its last signal
//   stage1_off   2 x stage1_bytes: one-shot staging (two buffers used alternately by consecutive fused calls); sized for
//                packets, i.e. twice the bytes of the bf16 tiles, like stage2
//   stage2_off   stage2_bytes: two-shot staging
//   the rest     tensors handed out by the Python side (residual streams that peers write into)
typedef struct {
    int rank, world;
    void* heap[8];
    int64_t heap_bytes;
    int64_t epoch_off, flags_off, flags_per_site, stage1_off, stage1_bytes, stage2_off, stage2_bytes;
    int num_sites;
    int site;      // call site of this collective inside the step (every site has its own flags)
    int mode;      // 0: choose by size, 1: one-shot, 2: two-shot. How the partials travel (flag-carrying packets, or plain tiles with
                   // a fence and arrival flags) is chosen from the world size; the environment variable OVB_COMM_PACKETS (bit 0:
                   // one-shot, bit 1: two-shot) overrides it and must be the same on every rank.
    // NVLink multicast (NVLS). mc_base: the heap's multicast mapping (a store through it lands at the same offset of every
    // rank's heap, multimem.ld_reduce through it returns the sum over the ranks), or NULL when the heap has none; then the
    // peer-store protocols above are used. With a mapping the fused all-reduce and ovb_comm_allreduce_bf16 reduce inside the
    // switch. nvls_flags_off: num_sites x nvls_flags_per_site int32 of barrier words (16 per tile / CTA), zero at start.
    void* mc_base;
    int64_t nvls_flags_off, nvls_flags_per_site;
    // 2 x stage3_bytes of staging that only ovb_comm_allreduce_bf16 uses (alternating by call site), so that a rank running
    // ahead into the next fused GEMM never writes a buffer that a peer's all-reduce still reads. 0: share the one-shot staging.
    int64_t stage3_off, stage3_bytes;
} ovb_comm;

// Symmetric-heap plumbing (no kernels): allocate zeroed device memory, export / open / close CUDA IPC handles.
int ovb_comm_alloc(int64_t bytes, void** ptr);
int ovb_comm_free(void* ptr);
int ovb_comm_export(void* ptr, void* handle64);          // writes the 64-byte IPC handle
int ovb_comm_open(const void* handle64, void** ptr);     // maps a peer's heap
int ovb_comm_close(void* ptr);
// epoch += 1 on this rank (a one-thread kernel; first kernel of every step, also inside CUDA graphs).
int ovb_comm_step_begin(const ovb_comm* c, ovb_stream_t stream);
// Greedy sampling over vocabulary shards: every rank holds its shard's best (value, local index) per row;
// afterwards ids[row] is the global argmax on every rank (lowest index on ties). rows <= 1024.
/* Wait on the device until *flag >= value, at most max_polls polls (~0.25 us apart); on time-out the status word gets the
   peer-time-out code and *result (may be NULL) 0. Never blocks longer than max_polls allows. */
int ovb_comm_wait_flag(const int* flag, int value, unsigned max_polls, int* result, ovb_stream_t stream);
int ovb_comm_argmax_combine(const ovb_comm* c, int* ids, const float* max_vals, int rows, int shard_size, ovb_stream_t stream);
// In-place sum of a bf16 tensor of n elements that lives at the same heap offset on every rank (n % 8 == 0).
int ovb_comm_allreduce_bf16(const ovb_comm* c, void* data, int64_t n, ovb_stream_t stream);
/* The same for fp32 / fp16 / bf16 tensors (dtype: OVB_DT_*); n elements, a multiple of 16 bytes. */
int ovb_comm_allreduce(const ovb_comm* c, void* data, int64_t n, int dtype, ovb_stream_t stream);

#ifdef __cplusplus
}
#endif
