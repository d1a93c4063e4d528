// Continuous-batching scheduler and paged KV block manager (host side, native).
//
// The reference keeps only the device contract in tree (PagedAttentionExtension inputs, the reference
// PagedCacheManager src/core/reference/include/openvino/reference/utils/paged_cache_manager.hpp:33-313);
// the scheduler itself ships in openvino.genai. This one produces exactly the ragged-batch inputs of the
// stateless PagedAttention model (input_ids, position_ids, past_lens, subsequence_begins, block_indices,
// block_indices_begins, max_context_len) plus the physical slot of every new token.
//
// Policy: prompt chunks first (FIFO, at most max_num_batched_tokens per step, a prompt may be split over
// steps), otherwise one decode token for every running sequence; with dynamic_split_fuse both kinds share
// a step. Blocks come from a free list; when it runs dry the youngest running sequence is preempted
// (blocks released, recomputed later). Token values are not needed to schedule: a step is committed with
// placeholders and patched when the device results arrive, so the host can run one step ahead.
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <list>
#include <string>
#include <unordered_map>
#include <vector>

namespace ovc {

struct SchedulerConfig {
    int64_t max_num_batched_tokens = 8192;
    int64_t max_num_seqs = 64;
    int64_t num_kv_blocks = 0;
    int64_t block_size = 16;
    bool dynamic_split_fuse = false;
    // Prefix caching: full blocks of prompt tokens are remembered by a hash of everything up to and including the block;
    // a new request whose prompt starts with the same tokens shares those blocks and skips their computation.
    bool enable_prefix_caching = false;
};

struct SeqState {
    int64_t request_id = 0;
    std::vector<int32_t> prompt;
    std::vector<int32_t> generated;     // -1 = value not yet known
    int64_t max_new_tokens = 0;
    int32_t eos_token_id = -1;
    bool ignore_eos = true;
    int64_t num_computed = 0;
    std::vector<int32_t> blocks;
    bool finished = false;
    int64_t slot = -1;
    std::vector<uint64_t> block_hashes;   // chain hash of every full prompt block (prefix caching)
    int64_t num_cached_tokens = 0;        // prompt tokens whose KV came from shared blocks at the last admission
    int64_t total_len() const { return (int64_t)prompt.size() + (int64_t)generated.size(); }
    int32_t token_at(int64_t i) const { return i < (int64_t)prompt.size() ? prompt[(size_t)i] : generated[(size_t)(i - (int64_t)prompt.size())]; }
};
using SeqPtr = std::shared_ptr<SeqState>;

struct Produced {
    SeqPtr seq;
    int64_t gen_index;
    int64_t row;
};

struct ScheduledStep {
    std::vector<SeqPtr> seqs;
    std::vector<int64_t> num_new;
    int64_t T = 0, max_q_len = 0, max_ctx = 0;
};

// Offsets (in int32 words) of the descriptor fields inside one packed step buffer.
struct DescLayout {
    int64_t ids = 0, positions = 0, slot_map = 0, tok_src = 0, tok_dst = 0, logit_idx = 0, past_lens = 0, subsequence_begins = 0,
            block_indices_begins = 0, block_indices = 0;
    int64_t Tcap = 0, Bcap = 0, blocks_cap = 0;
};

class Scheduler {
public:
    explicit Scheduler(const SchedulerConfig& cfg);
    SeqPtr add(int64_t request_id, std::vector<int32_t> prompt, int64_t max_new_tokens, int32_t eos_token_id, bool ignore_eos);
    bool has_unfinished() const { return !waiting_.empty() || !running_.empty(); }
    bool schedule(ScheduledStep& out);
    // write the step descriptor; host_ids_for_generated: upload generated ids instead of using the device table
    void fill(const ScheduledStep& st, int32_t* desc, const DescLayout& lay, bool host_ids_for_generated = false) const;
    std::vector<Produced> commit(const ScheduledStep& st, const int32_t* tokens /* may be null */);
    void patch(const std::vector<Produced>& produced, const int32_t* tokens);
    // blocks that a sequence could be given right now: never used or invalidated ones plus cached ones that nobody holds
    int64_t num_free_blocks() const { return (int64_t)free_.size() + (int64_t)evictable_.size(); }
    int64_t num_cached_blocks() const { return (int64_t)by_hash_.size(); }
    int64_t prefix_hit_tokens() const { return prefix_hit_tokens_; }
    int64_t num_preemptions() const { return preemptions_; }
    int64_t num_running() const { return (int64_t)running_.size(); }
    int64_t num_waiting() const { return (int64_t)waiting_.size(); }
    const SchedulerConfig& config() const { return cfg_; }
private:
    bool grow(SeqState& s, int64_t new_len);
    void release(SeqState& s);
    bool preempt_one(const SeqState* keep, const std::vector<SeqPtr>& scheduled);
    void finish(const SeqPtr& s);
    void check_eos(const std::vector<Produced>& produced);
    bool take_block(int32_t& out);
    void match_prefix(SeqState& s);
    void register_full_blocks(SeqState& s, int64_t before, int64_t after);
    struct BlockMeta { int32_t ref = 0; bool hashed = false; uint64_t hash = 0; std::list<int32_t>::iterator lru; };
    SchedulerConfig cfg_;
    std::vector<BlockMeta> meta_;
    std::unordered_map<uint64_t, int32_t> by_hash_;   // chain hash -> block holding those tokens' KV
    std::list<int32_t> evictable_;                     // cached blocks that no sequence holds, least recently released first
    int64_t prefix_hit_tokens_ = 0;
    std::deque<int32_t> free_;
    std::deque<SeqPtr> waiting_;
    std::vector<SeqPtr> running_;
    std::deque<int64_t> free_slots_;
    int64_t preemptions_ = 0;
};

}  // namespace ovc
