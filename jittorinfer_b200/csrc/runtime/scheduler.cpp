#include "scheduler.h"

#include <algorithm>
#include <cstring>

namespace jib {

Scheduler::Scheduler(PagedKv * kv, int n_slots, int n_batch, int n_ctx_slot, int eos_id, int n_keep, bool cont_batching)
    : kv_(kv), slots_(n_slots), n_batch_(n_batch), n_ctx_slot_(n_ctx_slot), eos_id_(eos_id), n_keep_(n_keep),
      cont_batching_(cont_batching) {
    for (int i = 0; i < n_slots; ++i) slots_[i].id = i;
}

bool Scheduler::idle() const {
    if (!waiting_.empty()) return false;
    for (const auto & s : slots_)
        if (s.state != SLOT_IDLE) return false;
    return true;
}

int Scheduler::n_running() const {
    int n = 0;
    for (const auto & s : slots_) n += s.state != SLOT_IDLE;
    return n;
}

static int common_prefix(const std::vector<int32_t> & a, const std::vector<int32_t> & b) {
    size_t n = std::min(a.size(), b.size()), i = 0;
    while (i < n && a[i] == b[i]) ++i;
    return (int) i;
}

// Idle slot with the longest cached prefix of the prompt; ties and "no prefix" fall back to the
// least recently used idle slot.
int Scheduler::pick_slot(const Request & r, int * lcp_out) {
    int best = -1, best_lcp = 0;
    int lru = -1;
    int64_t lru_t = INT64_MAX;
    for (auto & s : slots_) {
        if (s.state != SLOT_IDLE) continue;
        int cached = std::min<int>((int) s.tokens.size(), kv_->seq_len(s.id));
        int lcp = 0;
        if (cached > 0) {
            lcp = common_prefix(s.tokens, r.prompt);
            lcp = std::min(lcp, cached);
        }
        if (lcp > best_lcp) { best_lcp = lcp; best = s.id; }
        if (s.t_last_used < lru_t) { lru_t = s.t_last_used; lru = s.id; }
    }
    if (best < 0) { best = lru; best_lcp = 0; }
    *lcp_out = best_lcp;
    return best;
}

void Scheduler::launch(Slot & s, const Request & r, int lcp) {
    s.req_id = r.id;
    s.max_new = r.max_new;
    s.ignore_eos = r.ignore_eos;
    s.n_decoded = r.n_decoded_before;
    s.n_prompt_orig = r.n_prompt_orig > 0 ? r.n_prompt_orig : (int) r.prompt.size();
    s.truncated = false;
    s.n_keep = r.n_keep;
    std::vector<int32_t> prompt = r.prompt;
    // A prompt that does not fit the slot loses blocks from its middle, keeping n_keep head tokens
    // (same policy as the reference, examples/server/server.cpp:1395-1415).
    if ((int) prompt.size() >= n_ctx_slot_ && n_ctx_slot_ > 4) {
        int n_keep = r.n_keep == KEEP_DEFAULT ? n_keep_ : r.n_keep;
        if (n_keep < 0) n_keep = (int) prompt.size();          // "keep the prompt": as much of its head as fits
        n_keep = std::min(n_keep, n_ctx_slot_ - 4);
        int n_left = n_ctx_slot_ - n_keep;
        int n_block = std::max(1, n_left / 2);
        int erased = ((int) prompt.size() - n_keep - n_block) / n_block;
        std::vector<int32_t> np(prompt.begin(), prompt.begin() + n_keep);
        np.insert(np.end(), prompt.begin() + n_keep + erased * n_block, prompt.end());
        prompt.swap(np);
        s.truncated = true;
        lcp = std::min(lcp, common_prefix(s.tokens, prompt));
    }
    s.n_prompt = (int) prompt.size();
    // at least one prompt token must be evaluated to obtain logits
    int n_past = std::min(lcp, s.n_prompt - 1);
    if (n_past < 0) n_past = 0;
    kv_->seq_rm(s.id, n_past, -1);
    if (n_past > 0) ++stats_.prefix_hits;
    s.tokens.swap(prompt);
    s.n_past = n_past;
    s.n_cached = n_past;
    s.pending_token = -1;
    s.state = SLOT_STARTED;
    s.t_started = ++clock_;
    s.t_last_used = clock_;
}

void Scheduler::release(Slot & s, bool keep_cache) {
    s.state = SLOT_IDLE;
    s.req_id = -1;
    s.pending_token = -1;
    s.out_row = -1;
    s.t_last_used = ++clock_;
    if (!keep_cache) {
        kv_->seq_rm(s.id, 0, -1);
        s.tokens.clear();
        s.n_past = 0;
    } else {
        // only tokens already evaluated are reusable
        s.tokens.resize(std::min<size_t>(s.tokens.size(), (size_t) kv_->seq_len(s.id)));
    }
}

void Scheduler::preempt(Slot & s) {
    Request r;
    r.id = s.req_id;
    r.prompt = s.tokens;                  // prompt + generated so far: recomputed on resume
    if (s.pending_token >= 0 && (int) r.prompt.size() == kv_->seq_len(s.id)) r.prompt.push_back(s.pending_token);
    r.max_new = s.max_new;
    r.ignore_eos = s.ignore_eos;
    r.n_decoded_before = s.n_decoded;
    r.n_prompt_orig = s.n_prompt_orig;
    r.n_keep = s.n_keep;
    waiting_.push_front(r);
    release(s, false);
    ++stats_.preemptions;
}

// Makes room for n_tokens more tokens in `slot`: first drops cached blocks of idle slots (LRU
// first), then preempts the youngest running slot other than `slot` / `protect_slot`.
bool Scheduler::ensure_blocks(int slot, int n_tokens, int protect_slot) {
    while (kv_->blocks_needed(slot, n_tokens) > kv_->free_blocks()) {
        int victim = -1;
        int64_t t = INT64_MAX;
        for (auto & s : slots_)
            if (s.state == SLOT_IDLE && kv_->seq_len(s.id) > 0 && s.t_last_used < t) { t = s.t_last_used; victim = s.id; }
        if (victim >= 0) {
            kv_->seq_rm(victim, 0, -1);
            slots_[victim].tokens.clear();
            continue;
        }
        int64_t newest = -1;
        for (auto & s : slots_)
            if (s.state != SLOT_IDLE && s.id != slot && s.id != protect_slot && !s.in_batch && s.t_started > newest) {
                newest = s.t_started;
                victim = s.id;
            }
        if (victim < 0) return false;
        preempt(slots_[victim]);
    }
    return true;
}

bool Scheduler::cancel(int64_t req_id, std::vector<StepEvent> * events) {
    for (auto it = waiting_.begin(); it != waiting_.end(); ++it)
        if (it->id == req_id) {
            if (events) events->push_back({req_id, -1, -1, FINISH_CANCELLED, (int32_t) it->prompt.size(), 0});
            waiting_.erase(it);
            return true;
        }
    for (auto & s : slots_)
        if (s.state != SLOT_IDLE && s.req_id == req_id) {
            if (events) events->push_back({req_id, s.id, -1, FINISH_CANCELLED, s.n_prompt_orig, s.n_decoded});
            release(s, true);
            return true;
        }
    return false;
}

StepInfo Scheduler::step(StepArrays & out) {
    StepInfo info;
    // 1. waiting requests -> idle slots
    while (!waiting_.empty()) {
        int lcp = 0;
        int sid = pick_slot(waiting_.front(), &lcp);
        if (sid < 0) break;
        Request r = std::move(waiting_.front());
        waiting_.pop_front();
        if (r.prompt.empty()) r.prompt.push_back(eos_id_);
        // A longer prefix may sit in another slot's sequence (idle or running): share its full blocks by reference.
        // Whole blocks only, so that neither sequence ever has to copy one on its next write.
        {
            const int bs = kv_->block_size();
            int donor = -1, best = lcp;
            for (const auto & o : slots_) {
                if (o.id == sid) continue;
                const int cached = std::min<int>((int) o.tokens.size(), kv_->seq_len(o.id));
                if (cached < best + bs) continue;
                const int l = std::min(common_prefix(o.tokens, r.prompt), cached) / bs * bs;
                if (l >= best + bs) { best = l; donor = o.id; }
            }
            if (donor >= 0 && kv_->seq_cp(donor, sid, 0, best)) {
                slots_[sid].tokens.assign(r.prompt.begin(), r.prompt.begin() + best);
                lcp = best;
                ++stats_.prefix_shared;
            }
        }
        launch(slots_[sid], r, lcp);
    }
    for (auto & s : slots_) { s.out_row = -1; s.in_batch = false; }
    last_out_slots_.clear();

    int n_tok = 0, n_seq = 0, n_outp = 0;
    const int budget = std::min(n_batch_, out.cap_tokens);
    auto emit_seq = [&](Slot & s, int n_new, bool want_logits) {
        // tokens s.tokens[n_past .. n_past+n_new) enter the cache now
        out.q_start[n_seq] = n_tok;
        for (int i = 0; i < n_new; ++i) {
            out.tokens[n_tok + i] = s.tokens[s.n_past + i];
            out.positions[n_tok + i] = s.n_past + i;
        }
        kv_->append(s.id, n_new, out.slot_mapping + n_tok);
        n_tok += n_new;
        s.n_past += n_new;
        out.seq_lens[n_seq] = s.n_past;
        out.seq_slots[n_seq] = s.id;
        const auto & bl = kv_->seq_blocks(s.id);
        int32_t * row = out.block_tables + (size_t) n_seq * out.max_blocks_per_seq;
        int nb = std::min<int>((int) bl.size(), out.max_blocks_per_seq);
        std::memcpy(row, bl.data(), nb * sizeof(int32_t));
        for (int i = nb; i < out.max_blocks_per_seq; ++i) row[i] = 0;
        if (want_logits) {
            out.out_rows[n_outp] = n_tok - 1;
            out.out_slots[n_outp] = s.id;
            s.out_row = n_outp;
            last_out_slots_.push_back(s.id);
            ++n_outp;
        }
        info.max_q_len = std::max(info.max_q_len, n_new);
        ++n_seq;
        s.in_batch = true;
        s.t_last_used = ++clock_;
    };

    // 2. one token per generating slot (oldest first so that preemption hits the youngest)
    std::vector<int> order;
    for (auto & s : slots_)
        if (s.state == SLOT_GENERATING) order.push_back(s.id);
    std::sort(order.begin(), order.end(), [&](int a, int b) { return slots_[a].t_started < slots_[b].t_started; });
    for (int sid : order) {
        Slot & s = slots_[sid];
        if (s.state != SLOT_GENERATING) continue;        // preempted meanwhile
        if (n_tok >= budget || n_seq >= out.cap_seqs) break;
        if (!ensure_blocks(sid, 1, -1)) {
            // nothing left to evict: this request cannot continue
            preempt(s);
            ++info.n_preempted;
            continue;
        }
        if ((int) s.tokens.size() == s.n_past) s.tokens.push_back(s.pending_token);
        s.pending_token = -1;
        emit_seq(s, 1, true);
        ++info.n_decode_seqs;
    }
    // 3. prompt chunks until the token budget is used (a smaller budget while sequences are generating, if configured)
    const int prompt_budget = (mixed_prompt_budget_ > 0 && n_tok > 0) ? std::min(budget, n_tok + mixed_prompt_budget_) : budget;
    if (cont_batching_ || n_tok == 0) {
        order.clear();
        for (auto & s : slots_)
            if (s.state == SLOT_STARTED || s.state == SLOT_PROCESSING_PROMPT) order.push_back(s.id);
        std::sort(order.begin(), order.end(), [&](int a, int b) { return slots_[a].t_started < slots_[b].t_started; });
        for (int sid : order) {
            Slot & s = slots_[sid];
            if (s.state != SLOT_STARTED && s.state != SLOT_PROCESSING_PROMPT) continue;
            if (n_tok >= prompt_budget || n_seq >= out.cap_seqs) break;
            int remaining = (int) s.tokens.size() - s.n_past;
            int chunk = std::min(remaining, prompt_budget - n_tok);
            if (chunk <= 0) continue;
            if (!ensure_blocks(sid, chunk, -1)) {
                // shrink the chunk to what fits right now; if nothing fits, wait for a later step
                int fit = kv_->free_blocks() * kv_->block_size() +
                          (kv_->block_size() - kv_->seq_len(sid) % kv_->block_size()) % kv_->block_size();
                chunk = std::min(chunk, fit);
                if (chunk <= 0 || kv_->blocks_needed(sid, chunk) > kv_->free_blocks()) continue;
            }
            s.state = SLOT_PROCESSING_PROMPT;
            bool last = chunk == remaining;
            emit_seq(s, chunk, last);
            stats_.prompt_tokens += chunk;
            if (last) s.state = SLOT_DONE_PROMPT;
        }
    }
    out.q_start[n_seq] = n_tok;
    info.n_tokens = n_tok;
    info.n_seqs = n_seq;
    info.n_out = n_outp;
    info.n_copies = (int) kv_->pending_copies().size();
    info.n_preempted += 0;
    if (n_tok > 0) ++stats_.steps;
    return info;
}

void Scheduler::commit(const int32_t * sampled, int n_out, std::vector<StepEvent> * events) {
    for (int i = 0; i < n_out && i < (int) last_out_slots_.size(); ++i) {
        Slot & s = slots_[last_out_slots_[i]];
        if (s.state == SLOT_IDLE) continue;
        int tok = sampled[i];
        ++s.n_decoded;
        ++stats_.decode_tokens;
        s.state = SLOT_GENERATING;
        s.pending_token = tok;
        int finish = FINISH_NONE;
        if (!s.ignore_eos && tok == eos_id_) finish = FINISH_STOP;
        else if (s.max_new >= 0 && s.n_decoded >= s.max_new) finish = FINISH_LENGTH;
        else if (s.n_past + 1 >= n_ctx_slot_) finish = FINISH_LENGTH;
        if (events) events->push_back({s.req_id, s.id, tok, finish, s.n_prompt_orig, s.n_decoded});
        if (finish != FINISH_NONE) {
            ++stats_.finished;
            release(s, true);
        }
    }
    last_out_slots_.clear();
}

bool Scheduler::can_run_ahead() const {
    if (!waiting_.empty() || !deferred_.empty()) return false;
    int active = 0, new_blocks = 0;
    for (const auto & s : slots_) {
        if (s.state == SLOT_IDLE) continue;
        if (s.out_row < 0) return false;                   // still inside its prompt: the next step is not a pure decode step
        ++active;
        new_blocks += kv_->blocks_needed(s.id, 1);         // incl. a copy-on-write block
    }
    // every block the next step can ask for is free now: nothing is evicted, nobody is preempted
    return active > 0 && active == (int) last_out_slots_.size() && new_blocks <= kv_->free_blocks();
}

void Scheduler::commit_deferred(int n_out) {
    deferred_.clear();
    for (int i = 0; i < n_out && i < (int) last_out_slots_.size(); ++i) {
        Slot & s = slots_[last_out_slots_[i]];
        Deferred d{s.id, s.req_id, FINISH_NONE, s.n_prompt_orig, 0, s.n_past, s.ignore_eos};
        if (s.state == SLOT_IDLE) {                        // cancelled since the step was assembled: nothing to resolve
            d.req_id = -1;
            deferred_.push_back(d);
            continue;
        }
        ++s.n_decoded;
        ++stats_.decode_tokens;
        s.state = SLOT_GENERATING;
        s.pending_token = TOKEN_UNKNOWN;
        d.n_decoded = s.n_decoded;
        if (s.max_new >= 0 && s.n_decoded >= s.max_new) d.finish = FINISH_LENGTH;
        else if (s.n_past + 1 >= n_ctx_slot_) d.finish = FINISH_LENGTH;
        if (d.finish != FINISH_NONE) {
            ++stats_.finished;
            release(s, true);
        }
        deferred_.push_back(d);
    }
    last_out_slots_.clear();
}

void Scheduler::resolve(const int32_t * sampled, int n_out, std::vector<StepEvent> * events) {
    for (int i = 0; i < n_out && i < (int) deferred_.size(); ++i) {
        const Deferred & d = deferred_[i];
        if (d.req_id < 0) continue;
        const int32_t tok = sampled[i];
        if (d.finish != FINISH_NONE) {                     // ended by a length limit: the slot is free already
            // the end-of-sequence token on the very step of the limit reads "stop", as commit() reports it
            const int32_t fin = (!d.ignore_eos && tok == eos_id_) ? FINISH_STOP : d.finish;
            if (events) events->push_back({d.req_id, d.slot, tok, fin, d.n_prompt, d.n_decoded});
            continue;
        }
        Slot & s = slots_[d.slot];
        if (s.state == SLOT_IDLE || s.req_id != d.req_id) continue;       // cancelled meanwhile (its event is out already)
        if (s.pending_token == TOKEN_UNKNOWN) s.pending_token = tok;
        else if (d.token_index < (int) s.tokens.size() && s.tokens[d.token_index] == TOKEN_UNKNOWN) s.tokens[d.token_index] = tok;
        int finish = FINISH_NONE;
        if (!s.ignore_eos && tok == eos_id_) finish = FINISH_STOP;
        if (events) events->push_back({d.req_id, d.slot, tok, finish, d.n_prompt, d.n_decoded});
        if (finish != FINISH_NONE) {
            ++stats_.finished;
            release(s, true);                              // a step that already carries this slot's next token drops its output
        }
    }
    deferred_.clear();
}

}  // namespace jib
