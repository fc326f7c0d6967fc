#include "kv_paged.h"

#include <algorithm>
#include <functional>

namespace jib {

PagedKv::PagedKv(int n_blocks, int block_size, int max_seqs)
    : n_blocks_(n_blocks), block_size_(block_size), seqs_(max_seqs), ref_(n_blocks, 0) {
    clear();
}

void PagedKv::clear() {
    for (auto & s : seqs_) { s.blocks.clear(); s.len = 0; s.live = false; }
    std::fill(ref_.begin(), ref_.end(), 0);
    free_.resize(n_blocks_);
    for (int i = 0; i < n_blocks_; ++i) free_[i] = i;
    std::make_heap(free_.begin(), free_.end(), std::greater<int32_t>());   // min-heap: lowest id first
    pending_.clear();
}

int PagedKv::alloc_block() {
    if (free_.empty()) return -1;
    std::pop_heap(free_.begin(), free_.end(), std::greater<int32_t>());
    int b = free_.back();
    free_.pop_back();
    ref_[b] = 1;
    return b;
}

void PagedKv::release_block(int b) {
    if (--ref_[b] == 0) {
        free_.push_back(b);
        std::push_heap(free_.begin(), free_.end(), std::greater<int32_t>());
        if (track_freed_) freed_.push_back(b);
    }
}

std::vector<int32_t> PagedKv::take_freed() {
    std::vector<int32_t> out;
    for (int32_t b : freed_)
        if (ref_[b] == 0 && std::find(out.begin(), out.end(), b) == out.end()) out.push_back(b);      // still free: not handed out again
    freed_.clear();
    return out;
}

int PagedKv::blocks_needed(int seq, int n) const {
    const KvSeq & s = seqs_[seq];
    if (n <= 0) return 0;
    int have = (int) s.blocks.size();
    int want = (s.len + n + block_size_ - 1) / block_size_;
    int need = want - have;
    // a shared, partially filled tail block must be copied before it is written
    if (s.len % block_size_ != 0 && have > 0 && ref_[s.blocks.back()] > 1) need += 1;
    return need;
}

bool PagedKv::append(int seq, int n, int32_t * slots_out) {
    KvSeq & s = seqs_[seq];
    if (n <= 0) return true;
    if (blocks_needed(seq, n) > (int) free_.size()) return false;
    s.live = true;
    if (s.len % block_size_ != 0 && !s.blocks.empty() && ref_[s.blocks.back()] > 1) {
        int old = s.blocks.back();
        int nb = alloc_block();
        pending_.emplace_back(old, nb);
        release_block(old);
        s.blocks.back() = nb;
    }
    for (int i = 0; i < n; ++i) {
        int pos = s.len + i;
        int bi = pos / block_size_;
        if (bi >= (int) s.blocks.size()) s.blocks.push_back(alloc_block());
        if (slots_out) slots_out[i] = s.blocks[bi] * block_size_ + pos % block_size_;
    }
    s.len += n;
    return true;
}

bool PagedKv::seq_rm(int seq, int p0, int p1) {
    if (seq < 0) {   // all sequences
        bool ok = true;
        for (int i = 0; i < (int) seqs_.size(); ++i) ok = seq_rm(i, p0, p1) && ok;
        return ok;
    }
    KvSeq & s = seqs_[seq];
    if (p0 < 0) p0 = 0;
    if (p1 < 0 || p1 > s.len) p1 = s.len;
    if (p0 >= p1) return true;
    if (p1 != s.len) return false;            // hole in the middle: not representable
    int keep_blocks = (p0 + block_size_ - 1) / block_size_;
    while ((int) s.blocks.size() > keep_blocks) {
        release_block(s.blocks.back());
        s.blocks.pop_back();
    }
    s.len = p0;
    if (p0 == 0) s.live = false;
    return true;
}

bool PagedKv::seq_cp(int src, int dst, int p0, int p1) {
    if (src == dst) return true;
    if (p0 > 0) return false;
    const KvSeq & a = seqs_[src];
    if (p1 < 0 || p1 > a.len) p1 = a.len;
    seq_rm(dst, 0, -1);
    KvSeq & d = seqs_[dst];
    int nb = (p1 + block_size_ - 1) / block_size_;
    for (int i = 0; i < nb; ++i) {
        d.blocks.push_back(a.blocks[i]);
        ++ref_[a.blocks[i]];
    }
    d.len = p1;
    d.live = p1 > 0;
    return true;
}

void PagedKv::seq_keep(int seq) {
    for (int i = 0; i < (int) seqs_.size(); ++i)
        if (i != seq) seq_rm(i, 0, -1);
}

float PagedKv::fragmentation() const {
    int hi = -1;
    for (int b = n_blocks_ - 1; b >= 0; --b)
        if (ref_[b] > 0) { hi = b; break; }
    if (hi < 0) return 0.f;
    int used = used_blocks();
    return float(hi + 1 - used) / float(hi + 1);
}

std::vector<std::pair<int32_t, int32_t>> PagedKv::defrag(int max_moves) {
    std::vector<std::pair<int32_t, int32_t>> moves;
    if (max_moves <= 0) return moves;
    // free ids ascending, used ids descending; move while src > dst
    std::vector<int32_t> holes(free_.begin(), free_.end());
    std::sort(holes.begin(), holes.end());
    std::vector<int32_t> remap(n_blocks_, -1);
    size_t hi = 0;
    int src = n_blocks_ - 1;
    while ((int) moves.size() < max_moves && hi < holes.size()) {
        while (src >= 0 && ref_[src] == 0) --src;
        if (src < 0 || holes[hi] >= src) break;
        int dst = holes[hi++];
        remap[src] = dst;
        ref_[dst] = ref_[src];
        ref_[src] = 0;
        if (track_freed_) freed_.push_back(src);
        moves.emplace_back(src, dst);
        --src;
    }
    if (moves.empty()) return moves;
    for (auto & s : seqs_)
        for (auto & b : s.blocks)
            if (remap[b] >= 0) b = remap[b];
    for (auto & pc : pending_) {
        if (remap[pc.first] >= 0) pc.first = remap[pc.first];
        if (remap[pc.second] >= 0) pc.second = remap[pc.second];
    }
    free_.clear();
    for (int b = 0; b < n_blocks_; ++b)
        if (ref_[b] == 0 && std::find(reserved_.begin(), reserved_.end(), b) == reserved_.end()) free_.push_back(b);
    std::make_heap(free_.begin(), free_.end(), std::greater<int32_t>());
    return moves;
}

int PagedKv::reserve(int n) {
    int got = 0;
    while (got < n && !free_.empty()) {
        reserved_.push_back(free_.back());
        free_.pop_back();
        ++got;
    }
    return got;
}

void PagedKv::unreserve() {
    for (int32_t b : reserved_) free_.push_back(b);
    reserved_.clear();
    std::make_heap(free_.begin(), free_.end(), std::greater<int32_t>());      // the same min-heap order alloc_block() relies on
}

bool PagedKv::check() const {
    std::vector<int32_t> cnt(n_blocks_, 0);
    for (const auto & s : seqs_) {
        if ((int) s.blocks.size() != (s.len + block_size_ - 1) / block_size_) return false;
        for (int b : s.blocks) {
            if (b < 0 || b >= n_blocks_) return false;
            ++cnt[b];
        }
    }
    for (int b = 0; b < n_blocks_; ++b)
        if (cnt[b] != ref_[b]) return false;
    std::vector<char> is_free(n_blocks_, 0);
    for (int b : free_) {
        if (ref_[b] != 0 || is_free[b]) return false;
        is_free[b] = 1;
    }
    for (int b : reserved_) {
        if (ref_[b] != 0 || is_free[b]) return false;
        is_free[b] = 1;
    }
    for (int b = 0; b < n_blocks_; ++b)
        if (ref_[b] == 0 && !is_free[b]) return false;
    return true;
}

}  // namespace jib
