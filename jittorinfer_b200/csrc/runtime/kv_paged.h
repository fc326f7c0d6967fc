// Paged latent-KV block allocator with per-sequence block tables.
//
// Replaces the reference's cell ring buffer (src/llama-kv-cache.h:12-25, src/llama-kv-cache.cpp:347-476):
// there every cell carries {pos, seq_id bitset<32>} and attention spans the high-water mark of the whole
// pool; here a sequence owns an ordered list of fixed-size blocks, so attention cost follows the
// sequence's own length, more than 32 sequences can be live, and sharing a prefix (llama_kv_cache_seq_cp)
// is a reference-count bump with copy-on-write of the one partially filled block.
#pragma once
#include <cstdint>
#include <utility>
#include <vector>

namespace jib {

struct KvSeq {
    std::vector<int32_t> blocks;   // block ids in position order
    int32_t len = 0;               // tokens stored (positions 0..len-1)
    bool live = false;
};

class PagedKv {
  public:
    PagedKv(int n_blocks, int block_size, int max_seqs);

    int n_blocks() const { return n_blocks_; }
    int block_size() const { return block_size_; }
    int max_seqs() const { return (int) seqs_.size(); }
    int free_blocks() const { return (int) free_.size(); }
    int used_blocks() const { return n_blocks_ - (int) free_.size(); }

    // Blocks that appending `n` tokens to `seq` would newly allocate (incl. a copy-on-write block).
    int blocks_needed(int seq, int n) const;
    // Append n tokens; writes the flat slot index (block*block_size+offset) of each. false = out of blocks
    // (nothing changed).
    bool append(int seq, int n, int32_t * slots_out);
    // Drop positions [p0, p1) (negative = open end). Only tail ranges and whole sequences are
    // representable in a paged layout; returns false for a hole in the middle.
    bool seq_rm(int seq, int p0, int p1);
    // Make positions [p0,p1) of dst alias src. Supported: p0<=0 (prefix share). dst is cleared first.
    bool seq_cp(int src, int dst, int p0, int p1);
    void seq_keep(int seq);
    void clear();

    int seq_len(int seq) const { return seqs_[seq].len; }
    const std::vector<int32_t> & seq_blocks(int seq) const { return seqs_[seq].blocks; }
    int refcount(int block) const { return ref_[block]; }

    // Copy-on-write block copies queued by append(); the engine runs them on the device before the
    // next forward and then clears the list.
    std::vector<std::pair<int32_t, int32_t>> & pending_copies() { return pending_; }

    // (highest used block id + 1 - used) / (highest + 1): share of holes below the high-water mark.
    float fragmentation() const;
    // Hole-filling plan: move the highest used blocks into the lowest free ids, at most max_moves.
    // Tables are rewritten immediately; returns (src,dst) pairs for the device copy.
    // (reference planner: src/llama-execute-kvupdate.cpp:12-149)
    std::vector<std::pair<int32_t, int32_t>> defrag(int max_moves);

    // Memory-pressure injection for host-side fault tests: takes up to n free blocks out of circulation (returns how
    // many) until unreserve() puts them back.  Reserved blocks count as used.
    int reserve(int n);
    void unreserve();

    // Debug aid ("poison freed blocks"): with tracking on, every block whose reference count drops to zero is remembered;
    // take_freed() returns those that are still free (not handed out again since) and forgets them.  The engine fills
    // them with NaN so that a read through a stale block table shows up in the logits.
    void track_freed(bool on) { track_freed_ = on; if (!on) freed_.clear(); }
    std::vector<int32_t> take_freed();

    // Consistency check used by tests and the bounds-check build: every block's refcount equals the
    // number of tables naming it, and free blocks have refcount 0.
    bool check() const;

  private:
    int alloc_block();
    void release_block(int b);

    int n_blocks_, block_size_;
    std::vector<KvSeq> seqs_;
    std::vector<int32_t> ref_;
    std::vector<int32_t> free_;    // min-heap (std::greater): alloc_block() hands out the lowest free id
    std::vector<std::pair<int32_t, int32_t>> pending_;
    std::vector<int32_t> reserved_;
    std::vector<int32_t> freed_;
    bool track_freed_ = false;
};

}  // namespace jib
