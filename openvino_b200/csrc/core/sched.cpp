#include "sched.hpp"

#include <algorithm>
#include <stdexcept>

namespace ovc {

Scheduler::Scheduler(const SchedulerConfig& cfg) : cfg_(cfg) {
    for (int64_t i = 0; i < cfg.num_kv_blocks; ++i) free_.push_back((int32_t)i);
    for (int64_t i = 0; i < cfg.max_num_seqs * 4; ++i) free_slots_.push_back(i);
    meta_.resize((size_t)std::max<int64_t>(cfg.num_kv_blocks, 0));
}

static uint64_t mix_hash(uint64_t h, uint64_t v) {
    h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h *= 0xBF58476D1CE4E5B9ull;
    return h ^ (h >> 31);
}

SeqPtr Scheduler::add(int64_t request_id, std::vector<int32_t> prompt, int64_t max_new_tokens, int32_t eos, bool ignore_eos) {
    if (prompt.empty()) throw std::invalid_argument("a request needs at least one prompt token");
    auto s = std::make_shared<SeqState>();
    s->request_id = request_id;
    s->prompt = std::move(prompt);
    s->max_new_tokens = max_new_tokens;
    s->eos_token_id = eos;
    s->ignore_eos = ignore_eos;
    if (cfg_.enable_prefix_caching) {
        // hash of block i covers tokens [0, (i + 1) * block_size): equal hashes mean equal prefixes (up to collisions of a
        // 64-bit hash), so the KV of the block is the same whatever request computed it
        const int64_t bs = cfg_.block_size, full = (int64_t)s->prompt.size() / bs;
        uint64_t h = 0x243F6A8885A308D3ull;
        for (int64_t b = 0; b < full; ++b) {
            for (int64_t j = 0; j < bs; ++j) h = mix_hash(h, (uint64_t)(uint32_t)s->prompt[(size_t)(b * bs + j)]);
            s->block_hashes.push_back(h);
        }
    }
    waiting_.push_back(s);
    return s;
}

bool Scheduler::take_block(int32_t& out) {
    if (!free_.empty()) {
        out = free_.front();
        free_.pop_front();
    } else if (!evictable_.empty()) {
        out = evictable_.front();          // least recently released cached block: forget what it held
        evictable_.pop_front();
        BlockMeta& m = meta_[(size_t)out];
        auto it = by_hash_.find(m.hash);
        if (it != by_hash_.end() && it->second == out) by_hash_.erase(it);
        m.hashed = false;
    } else {
        return false;
    }
    meta_[(size_t)out].ref = 1;
    return true;
}

bool Scheduler::grow(SeqState& s, int64_t new_len) {
    const int64_t need = (new_len + cfg_.block_size - 1) / cfg_.block_size - (int64_t)s.blocks.size();
    if (need <= 0) return true;
    if (need > num_free_blocks()) return false;
    for (int64_t i = 0; i < need; ++i) {
        int32_t b = -1;
        take_block(b);
        s.blocks.push_back(b);
    }
    return true;
}

void Scheduler::release(SeqState& s) {
    for (auto b : s.blocks) {
        BlockMeta& m = meta_[(size_t)b];
        if (--m.ref > 0) continue;         // another sequence still shares the block
        m.ref = 0;
        if (m.hashed) {
            evictable_.push_back(b);
            m.lru = std::prev(evictable_.end());
        } else {
            free_.push_back(b);
        }
    }
    s.blocks.clear();
}

// A sequence that starts (or restarts) with no blocks takes over the cached blocks of its longest known prompt prefix. The
// last prompt token is always computed, so that the step that finishes the prompt has logits to sample from.
void Scheduler::match_prefix(SeqState& s) {
    s.num_cached_tokens = 0;
    if (!cfg_.enable_prefix_caching || !s.blocks.empty() || s.num_computed != 0) return;
    const int64_t bs = cfg_.block_size;
    const int64_t usable = std::min<int64_t>((int64_t)s.block_hashes.size(), ((int64_t)s.prompt.size() - 1) / bs);
    for (int64_t b = 0; b < usable; ++b) {
        auto it = by_hash_.find(s.block_hashes[(size_t)b]);
        if (it == by_hash_.end()) break;
        BlockMeta& m = meta_[(size_t)it->second];
        if (m.ref == 0) evictable_.erase(m.lru);
        ++m.ref;
        s.blocks.push_back(it->second);
    }
    s.num_computed = (int64_t)s.blocks.size() * bs;
    s.num_cached_tokens = s.num_computed;
    prefix_hit_tokens_ += s.num_computed;
}

// Prompt blocks that became complete between `before` and `after` computed tokens are entered into the cache.
void Scheduler::register_full_blocks(SeqState& s, int64_t before, int64_t after) {
    if (!cfg_.enable_prefix_caching) return;
    const int64_t bs = cfg_.block_size;
    const int64_t last = std::min<int64_t>(after / bs, (int64_t)s.block_hashes.size());
    for (int64_t b = before / bs; b < last; ++b) {
        if ((size_t)b >= s.blocks.size()) break;
        const int32_t blk = s.blocks[(size_t)b];
        BlockMeta& m = meta_[(size_t)blk];
        const uint64_t h = s.block_hashes[(size_t)b];
        if (m.hashed || by_hash_.count(h)) continue;     // already cached (possibly under another block)
        m.hashed = true;
        m.hash = h;
        by_hash_[h] = blk;
    }
}

bool Scheduler::preempt_one(const SeqState* keep, const std::vector<SeqPtr>& scheduled) {
    // youngest running sequence that is neither `keep` nor part of the step being built (its block table is in use)
    for (auto it = running_.rbegin(); it != running_.rend(); ++it) {
        SeqPtr v = *it;
        if (v.get() == keep || v->blocks.empty()) continue;
        if (std::find(scheduled.begin(), scheduled.end(), v) != scheduled.end()) continue;
        release(*v);
        v->num_computed = 0;
        running_.erase(std::next(it).base());
        waiting_.push_front(v);
        ++preemptions_;
        return true;
    }
    return false;
}
void Scheduler::finish(const SeqPtr& s) {
    if (s->finished) return;
    s->finished = true;
    release(*s);
    running_.erase(std::remove(running_.begin(), running_.end(), s), running_.end());
    if (s->slot >= 0) { free_slots_.push_back(s->slot); s->slot = -1; }
}

bool Scheduler::schedule(ScheduledStep& out) {
    out = ScheduledStep();
    int64_t budget = cfg_.max_num_batched_tokens;
    auto pending = [](const SeqState& s) { return s.total_len() - s.num_computed; };
    auto in_running = [&](const SeqPtr& s) { return std::find(running_.begin(), running_.end(), s) != running_.end(); };
    auto want_prefill = [&]() {
        if (!waiting_.empty()) return true;
        for (auto& s : running_) if (pending(*s) > 1) return true;
        return false;
    };
    auto decode_phase = [&]() {
        std::vector<SeqPtr> decode_running;
        for (auto& s : running_) if (pending(*s) == 1) decode_running.push_back(s);
        for (auto& s : decode_running) {
            if (budget <= 0 || (int64_t)out.seqs.size() >= cfg_.max_num_seqs) break;
            if (!in_running(s)) continue;   // preempted on behalf of an earlier sequence of this loop
            while (!grow(*s, s->total_len())) if (!preempt_one(s.get(), out.seqs)) break;
            if ((s->total_len() + cfg_.block_size - 1) / cfg_.block_size > (int64_t)s->blocks.size()) continue;
            out.seqs.push_back(s);
            out.num_new.push_back(1);
            --budget;
        }
    };
    auto prefill_phase = [&](bool may_preempt) {
        // taken after the decode phase: a preemption there moves a mid-prefill sequence from running_ to waiting_
        std::vector<SeqPtr> cands;
        for (auto& s : running_) if (pending(*s) > 1) cands.push_back(s);
        const size_t n_running_cands = cands.size();
        while (!waiting_.empty() && (int64_t)running_.size() + (int64_t)(cands.size() - n_running_cands) < cfg_.max_num_seqs) {
            cands.push_back(waiting_.front());
            waiting_.pop_front();
        }
        std::vector<SeqPtr> back;
        for (auto& s : cands) {
            const bool was_running = in_running(s);
            if (budget <= 0 || (int64_t)out.seqs.size() >= cfg_.max_num_seqs) { if (!was_running) back.push_back(s); continue; }
            if (!was_running) match_prefix(*s);
            const int64_t n = std::min(budget, s->total_len() - s->num_computed);
            bool ok = n > 0 && grow(*s, s->num_computed + n);
            // last resort: the oldest candidate evicts younger sequences
            while (n > 0 && !ok && may_preempt && out.seqs.empty() && preempt_one(s.get(), out.seqs)) ok = grow(*s, s->num_computed + n);
            if (!ok) {
                if (!was_running) {
                    if (!s->blocks.empty()) { release(*s); s->num_computed = 0; }   // shared prefix blocks taken a moment ago
                    back.push_back(s);
                }
                continue;
            }
            if (!was_running) {
                running_.push_back(s);
                if (s->slot < 0) { s->slot = free_slots_.front(); free_slots_.pop_front(); }
            }
            out.seqs.push_back(s);
            out.num_new.push_back(n);
            budget -= n;
        }
        for (auto it = back.rbegin(); it != back.rend(); ++it) waiting_.push_front(*it);
    };
    if (cfg_.dynamic_split_fuse) {
        decode_phase();
        if (want_prefill()) prefill_phase(false);
    } else {
        if (want_prefill()) prefill_phase(false);
        if (out.seqs.empty()) decode_phase();   // no prompt chunk fits: keep the running sequences going (they may preempt)
    }
    if (out.seqs.empty() && want_prefill()) prefill_phase(true);
    if (out.seqs.empty()) return false;
    for (size_t i = 0; i < out.seqs.size(); ++i) {
        out.T += out.num_new[i];
        out.max_q_len = std::max(out.max_q_len, out.num_new[i]);
        out.max_ctx = std::max(out.max_ctx, out.seqs[i]->num_computed + out.num_new[i]);
    }
    return true;
}

void Scheduler::fill(const ScheduledStep& st, int32_t* d, const DescLayout& lay, bool host_ids) const {
    const int64_t bs = cfg_.block_size;
    int64_t t = 0, nb = 0;
    if ((int64_t)st.seqs.size() > lay.Bcap || st.T > lay.Tcap) throw std::length_error("step does not fit the descriptor buffer");
    d[lay.subsequence_begins] = 0;
    d[lay.block_indices_begins] = 0;
    for (size_t i = 0; i < st.seqs.size(); ++i) {
        const SeqState& s = *st.seqs[i];
        const int64_t n = st.num_new[i], c0 = s.num_computed;
        for (int64_t j = 0; j < n; ++j) {
            const int64_t pos = c0 + j;
            d[lay.ids + t + j] = s.token_at(pos);
            d[lay.positions + t + j] = (int32_t)pos;
            d[lay.slot_map + t + j] = s.blocks[(size_t)(pos / bs)] * (int32_t)bs + (int32_t)(pos % bs);
            d[lay.tok_src + t + j] = -1;
        }
        const bool ends_on_last = c0 + n == s.total_len();
        if (!host_ids && !s.generated.empty() && ends_on_last) d[lay.tok_src + t + n - 1] = (int32_t)s.slot;
        d[lay.tok_dst + (int64_t)i] = ends_on_last ? (int32_t)s.slot : -1;
        d[lay.past_lens + (int64_t)i] = (int32_t)c0;
        d[lay.logit_idx + (int64_t)i] = (int32_t)(t + n - 1);
        const int64_t k = (c0 + n + bs - 1) / bs;
        if (nb + k > lay.blocks_cap) throw std::length_error("block table does not fit the descriptor buffer");
        for (int64_t j = 0; j < k; ++j) d[lay.block_indices + nb + j] = s.blocks[(size_t)j];
        nb += k;
        t += n;
        d[lay.subsequence_begins + (int64_t)i + 1] = (int32_t)t;
        d[lay.block_indices_begins + (int64_t)i + 1] = (int32_t)nb;
    }
}

std::vector<Produced> Scheduler::commit(const ScheduledStep& st, const int32_t* tokens) {
    std::vector<Produced> produced;
    for (size_t i = 0; i < st.seqs.size(); ++i) {
        const SeqPtr& s = st.seqs[i];
        const int64_t before = s->num_computed;
        s->num_computed += st.num_new[i];
        register_full_blocks(*s, before, s->num_computed);
        if (s->num_computed >= s->total_len() && !s->finished) {
            s->generated.push_back(tokens ? tokens[i] : -1);
            produced.push_back({s, (int64_t)s->generated.size() - 1, (int64_t)i});
            if ((int64_t)s->generated.size() >= s->max_new_tokens) finish(s);
        }
    }
    if (tokens) check_eos(produced);
    return produced;
}

void Scheduler::patch(const std::vector<Produced>& produced, const int32_t* tokens) {
    for (auto& p : produced)
        if (p.gen_index < (int64_t)p.seq->generated.size()) p.seq->generated[(size_t)p.gen_index] = tokens[p.row];
    check_eos(produced);
}

void Scheduler::check_eos(const std::vector<Produced>& produced) {
    for (auto& p : produced) {
        SeqState& s = *p.seq;
        if (s.ignore_eos || p.gen_index >= (int64_t)s.generated.size() || s.generated[(size_t)p.gen_index] != s.eos_token_id) continue;
        s.generated.resize((size_t)p.gen_index + 1);   // tokens sampled by steps launched before the EOS was seen are dropped
        s.num_computed = std::min(s.num_computed, s.total_len());
        finish(p.seq);
    }
}

}  // namespace ovc
