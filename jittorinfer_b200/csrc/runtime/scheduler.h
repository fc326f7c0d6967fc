// Continuous-batching scheduler with chunked prefill over the paged KV allocator.
//
// Plays the role of server_context::update_slots / process_single_task in the reference's servers
// (examples/server/server.cpp:995-1062 slot pick and launch, 1304-1564 batch assembly, 1070-1131 stop
// rules) but as a library object that both the OpenAI server and the C API drive.  State names
// follow the reference's slot state machine (server.cpp:41-47).  Deliberate differences: request
// `max_tokens` / `ignore_eos` are honoured; when the cache is full the *youngest* running request is
// preempted and re-queued (the reference releases every slot, server.cpp:1493-1500); idle slots keep
// their blocks for prefix reuse only until someone else needs them; a new request whose prompt starts like the tokens
// of ANOTHER slot's sequence (idle or running, e.g. a common system prompt) shares that sequence's full blocks by
// reference instead of recomputing them.
#pragma once
#include <cstdint>
#include <deque>
#include <vector>

#include "kv_paged.h"

namespace jib {

enum SlotState : int32_t { SLOT_IDLE = 0, SLOT_STARTED, SLOT_PROCESSING_PROMPT, SLOT_DONE_PROMPT, SLOT_GENERATING };

enum FinishReason : int32_t { FINISH_NONE = 0, FINISH_STOP = 1, FINISH_LENGTH = 2, FINISH_CANCELLED = 3, FINISH_ERROR = 4 };

constexpr int32_t KEEP_DEFAULT = INT32_MIN;

struct Request {
    int64_t id = 0;
    std::vector<int32_t> prompt;
    int32_t max_new = -1;          // <0: until EOS / context limit
    bool ignore_eos = false;
    int32_t n_decoded_before = 0;  // >0 when re-queued after preemption
    int32_t n_prompt_orig = 0;
    int32_t n_keep = KEEP_DEFAULT; // head tokens kept when the prompt is cut to fit; <0: the whole prompt; KEEP_DEFAULT: the scheduler's
};

struct Slot {
    int32_t id = 0;
    SlotState state = SLOT_IDLE;
    int64_t req_id = -1;
    std::vector<int32_t> tokens;   // tokens whose KV is cached or scheduled (prompt + generated)
    int32_t n_prompt = 0;          // prompt length after truncation
    int32_t n_keep = KEEP_DEFAULT; // the request's n_keep (carried over a preemption)
    int32_t n_prompt_orig = 0;
    int32_t n_past = 0;            // tokens already evaluated into the cache
    int32_t n_cached = 0;          // prompt tokens found in the cache when the request was (last) launched
    int32_t n_decoded = 0;
    int32_t max_new = -1;
    bool ignore_eos = false;
    int32_t pending_token = -1;    // sampled but not yet evaluated
    int64_t t_last_used = 0;
    int64_t t_started = 0;
    int32_t out_row = -1;
    bool truncated = false;
    bool in_batch = false;         // already part of the batch being assembled (not preemptible)
};

struct StepEvent {
    int64_t req_id;
    int32_t slot;
    int32_t token;
    int32_t finish;    // FinishReason
    int32_t n_prompt;
    int32_t n_decoded;
};

// Caller-owned arrays the scheduler fills for one engine step (pinned host memory in the engine).
struct StepArrays {
    int32_t * tokens;        // [cap_tokens]
    int32_t * positions;     // [cap_tokens]
    int32_t * slot_mapping;  // [cap_tokens]
    int32_t * q_start;       // [cap_seqs + 1]
    int32_t * seq_lens;      // [cap_seqs]
    int32_t * seq_slots;     // [cap_seqs]   slot id of each batch sequence
    int32_t * block_tables;  // [cap_seqs * max_blocks_per_seq]
    int32_t * out_rows;      // [cap_seqs]   token row whose logits are sampled
    int32_t * out_slots;     // [cap_seqs]   slot each output row belongs to
    int32_t cap_tokens, cap_seqs, max_blocks_per_seq;
};

struct StepInfo {
    int32_t n_tokens = 0, n_seqs = 0, n_out = 0, n_decode_seqs = 0, max_q_len = 0, n_preempted = 0, n_copies = 0;
};

struct SchedStats {
    int64_t steps = 0, prompt_tokens = 0, decode_tokens = 0, preemptions = 0, finished = 0, prefix_hits = 0;
    int64_t prefix_shared = 0;     // requests that started from blocks shared with another slot's sequence
};

class Scheduler {
  public:
    Scheduler(PagedKv * kv, int n_slots, int n_batch, int n_ctx_slot, int eos_id, int n_keep = 0, bool cont_batching = true);

    void add_request(const Request & r) { waiting_.push_back(r); }
    bool cancel(int64_t req_id, std::vector<StepEvent> * events);

    // Assigns waiting requests to idle slots and assembles the next batch. Returns StepInfo with
    // n_tokens == 0 when there is nothing to run.
    StepInfo step(StepArrays & out);
    // Feeds the sampled token of every output row of the last step() back; appends events.
    void commit(const int32_t * sampled, int n_out, std::vector<StepEvent> * events);

    // ---- running one step ahead of the sampled ids ------------------------------------------------------------------
    // With greedy sampling on the device the ids of a step are not needed on the host to launch the next decode step:
    // the device feeds them forward itself.  commit_deferred() does what commit() does for a step whose ids are still
    // on their way (counts, length limits, slot release), marking the tokens TOKEN_UNKNOWN; resolve() later supplies
    // the ids in the same order, patches the token histories, applies the end-of-sequence rule (a sequence that ended
    // has then been fed one token too many, whose output is dropped) and appends the events.  At most one deferred
    // commit may be outstanding.  can_run_ahead() tells whether the next step() can be assembled without knowing the
    // ids of the last step: every active slot produced an output in it, nothing waits for a slot, and no step() can
    // run out of blocks (so nothing with an unknown token is ever preempted or re-queued).
    static constexpr int32_t TOKEN_UNKNOWN = -2;
    bool can_run_ahead() const;
    void commit_deferred(int n_out);
    void resolve(const int32_t * sampled, int n_out, std::vector<StepEvent> * events);
    int n_deferred() const { return (int) deferred_.size(); }

    bool idle() const;
    int n_waiting() const { return (int) waiting_.size(); }
    int n_running() const;
    const std::vector<Slot> & slots() const { return slots_; }
    const SchedStats & stats() const { return stats_; }
    const std::vector<int32_t> & last_out_slots() const { return last_out_slots_; }
    int n_batch() const { return n_batch_; }
    void set_n_batch(int n) { n_batch_ = n; }
    // Most prompt tokens a step may carry while sequences are generating (0 = no extra limit).  A long prompt chunk makes
    // every running sequence wait for it; a smaller share keeps their token-to-token latency bounded at the price of more
    // steps for the prompt.
    void set_mixed_prompt_budget(int n) { mixed_prompt_budget_ = n; }

  private:
    int pick_slot(const Request & r, int * lcp_out);
    void launch(Slot & s, const Request & r, int lcp);
    bool ensure_blocks(int slot, int n_tokens, int protect_slot);
    void release(Slot & s, bool keep_cache);
    void preempt(Slot & s);

    PagedKv * kv_;
    std::vector<Slot> slots_;
    std::deque<Request> waiting_;
    int n_batch_, n_ctx_slot_, eos_id_, n_keep_;
    int mixed_prompt_budget_ = 0;
    bool cont_batching_;
    int64_t clock_ = 0;
    std::vector<int32_t> last_out_slots_;
    SchedStats stats_;
    struct Deferred {
        int32_t slot;
        int64_t req_id;
        int32_t finish;        // decided at commit time (length limits) or FINISH_NONE
        int32_t n_prompt, n_decoded;
        int32_t token_index;   // where the token lands in the slot's history once it is scheduled
        bool ignore_eos;
    };
    std::vector<Deferred> deferred_;
};

}  // namespace jib
