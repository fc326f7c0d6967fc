#include "tokenizer.h"

#include <algorithm>
#include <cstring>
#include <queue>

namespace jib {

#include "unicode_tables.inc"

namespace {

bool in_ranges(const uint32_t (*tab)[2], int n, uint32_t cp) {
    int lo = 0, hi = n - 1;
    while (lo <= hi) {
        const int mid = (lo + hi) >> 1;
        if (cp < tab[mid][0]) hi = mid - 1;
        else if (cp > tab[mid][1]) lo = mid + 1;
        else return true;
    }
    return false;
}
bool is_space(uint32_t c) { return in_ranges(kSpaceRanges, kSpaceRanges_n, c); }
bool is_number(uint32_t c) { return in_ranges(kNumberRanges, kNumberRanges_n, c); }
bool is_cased(uint32_t c) { return in_ranges(kCasedRanges, kCasedRanges_n, c); }
// rule 3 class: [!-/:-~ U+FF01-FF0F U+FF1A-FF5E U+2018-201F U+3000-3002]
bool is_punct3(uint32_t c) {
    return (c >= 0x21 && c <= 0x2F) || (c >= 0x3A && c <= 0x7E) || (c >= 0xFF01 && c <= 0xFF0F) || (c >= 0xFF1A && c <= 0xFF5E) ||
           (c >= 0x2018 && c <= 0x201F) || (c >= 0x3000 && c <= 0x3002);
}
// rule 5 class: U+4E00-9FA5, U+0800-4E00, U+AC00-D7FF
bool is_cjk5(uint32_t c) { return (c >= 0x0800 && c <= 0x9FA5) || (c >= 0xAC00 && c <= 0xD7FF); }

std::vector<uint32_t> utf8_to_cps(const std::string & s) {
    std::vector<uint32_t> out;
    out.reserve(s.size());
    size_t i = 0;
    while (i < s.size()) {
        const unsigned char c = s[i];
        uint32_t cp;
        int n;
        if (c < 0x80) { cp = c; n = 1; }
        else if ((c >> 5) == 6) { cp = c & 0x1F; n = 2; }
        else if ((c >> 4) == 14) { cp = c & 0x0F; n = 3; }
        else if ((c >> 3) == 30) { cp = c & 0x07; n = 4; }
        else { out.push_back(0xFFFD); ++i; continue; }
        if (i + n > s.size()) { out.push_back(0xFFFD); break; }
        bool ok = true;
        for (int k = 1; k < n; ++k) {
            const unsigned char cc = s[i + k];
            if ((cc >> 6) != 2) { ok = false; break; }
            cp = (cp << 6) | (cc & 0x3F);
        }
        if (!ok) { out.push_back(0xFFFD); ++i; continue; }
        out.push_back(cp);
        i += n;
    }
    return out;
}
void append_utf8(std::string & s, uint32_t cp) {
    if (cp < 0x80) s += (char) cp;
    else if (cp < 0x800) { s += (char) (0xC0 | (cp >> 6)); s += (char) (0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { s += (char) (0xE0 | (cp >> 12)); s += (char) (0x80 | ((cp >> 6) & 0x3F)); s += (char) (0x80 | (cp & 0x3F)); }
    else { s += (char) (0xF0 | (cp >> 18)); s += (char) (0x80 | ((cp >> 12) & 0x3F)); s += (char) (0x80 | ((cp >> 6) & 0x3F)); s += (char) (0x80 | (cp & 0x3F)); }
}

// GPT-2 byte <-> printable code point map.
struct ByteMap {
    uint32_t to_cp[256];
    std::unordered_map<uint32_t, uint8_t> to_byte;
    ByteMap() {
        bool direct[256] = {false};
        for (int b = '!'; b <= '~'; ++b) direct[b] = true;
        for (int b = 0xA1; b <= 0xAC; ++b) direct[b] = true;
        for (int b = 0xAE; b <= 0xFF; ++b) direct[b] = true;
        int n = 0;
        for (int b = 0; b < 256; ++b) {
            to_cp[b] = direct[b] ? (uint32_t) b : (uint32_t) (256 + n++);
            to_byte[to_cp[b]] = (uint8_t) b;
        }
    }
};
const ByteMap & byte_map() {
    static const ByteMap m;
    return m;
}

typedef std::pair<size_t, size_t> Span;     // [begin, end) in code points

// One pre-split rule: `match(cps, i, end)` returns the length of a match starting at i (0 = none).
template <typename F>
std::vector<Span> refine(const std::vector<uint32_t> & cps, const std::vector<Span> & spans, F match) {
    std::vector<Span> out;
    for (const Span & sp : spans) {
        size_t gap = sp.first, i = sp.first;
        while (i < sp.second) {
            const size_t len = match(cps, i, sp.second);
            if (len > 0) {
                if (i > gap) out.emplace_back(gap, i);
                out.emplace_back(i, i + len);
                i += len;
                gap = i;
            } else {
                ++i;
            }
        }
        if (sp.second > gap) out.emplace_back(gap, sp.second);
    }
    return out;
}

template <typename P>
size_t opt_space_then_run(const std::vector<uint32_t> & c, size_t i, size_t end, P pred) {
    size_t j = i;
    if (j < end && is_space(c[j]) && j + 1 < end && pred(c[j + 1])) ++j;       // \s? is taken only when a run follows
    size_t k = j;
    while (k < end && pred(c[k])) ++k;
    return k > j ? k - i : 0;
}

}  // namespace

// The six deepseek-llm rules, applied in sequence; each refines the spans left by the previous ones.
std::vector<std::string> Tokenizer::pre_split(const std::string & text) {
    const std::vector<uint32_t> cps = utf8_to_cps(text);
    std::vector<Span> spans;
    if (!cps.empty()) spans.emplace_back(0, cps.size());
    spans = refine(cps, spans, [](const std::vector<uint32_t> & c, size_t i, size_t) -> size_t { return (c[i] == '\r' || c[i] == '\n') ? 1 : 0; });
    spans = refine(cps, spans, [](const std::vector<uint32_t> & c, size_t i, size_t e) { return opt_space_then_run(c, i, e, is_cased); });
    spans = refine(cps, spans, [](const std::vector<uint32_t> & c, size_t i, size_t e) { return opt_space_then_run(c, i, e, is_punct3); });
    spans = refine(cps, spans, [](const std::vector<uint32_t> & c, size_t i, size_t e) -> size_t {      // \s+$
        size_t k = i;
        while (k < e && is_space(c[k])) ++k;
        return (k == e && k > i) ? k - i : 0;
    });
    spans = refine(cps, spans, [](const std::vector<uint32_t> & c, size_t i, size_t e) -> size_t {
        size_t k = i;
        while (k < e && is_cjk5(c[k])) ++k;
        return k - i;
    });
    spans = refine(cps, spans, [](const std::vector<uint32_t> & c, size_t i, size_t e) -> size_t {
        size_t k = i;
        while (k < e && is_number(c[k])) ++k;
        return k - i;
    });
    std::vector<std::string> words;
    words.reserve(spans.size());
    for (const Span & sp : spans) {
        std::string w;
        for (size_t i = sp.first; i < sp.second; ++i) append_utf8(w, cps[i]);
        words.push_back(std::move(w));
    }
    return words;
}

// ---------------------------------------------------------------------------------------------
Tokenizer::Tokenizer(std::vector<std::string> tokens, std::vector<int32_t> types, const std::vector<std::string> & merges,
                     TokenizerConfig cfg)
    : tokens_(std::move(tokens)), types_(std::move(types)), cfg_(cfg) {
    types_.resize(tokens_.size(), TOK_NORMAL);
    token_id_.reserve(tokens_.size() * 2);
    for (size_t i = 0; i < tokens_.size(); ++i) token_id_.emplace(tokens_[i], (int32_t) i);
    rank_.reserve(merges.size() * 2);
    for (size_t i = 0; i < merges.size(); ++i) {
        // "left right": split at the first space after index 1 (a merge may start with a space-like symbol)
        const std::string & m = merges[i];
        const size_t pos = m.find(' ', 1);
        if (pos == std::string::npos) continue;
        rank_.emplace(m, (int32_t) i);
    }
    for (size_t i = 0; i < tokens_.size(); ++i)
        if (types_[i] == TOK_CONTROL || types_[i] == TOK_USER_DEFINED || types_[i] == TOK_UNKNOWN) special_ids_.push_back((int32_t) i);
    std::sort(special_ids_.begin(), special_ids_.end(),
              [&](int32_t a, int32_t b) { return tokens_[a].size() > tokens_[b].size(); });
    // end-of-generation set: eos, eot, plus well-known end markers found by text
    static const char * eog_texts[] = {"<|eot_id|>", "<|im_end|>", "<|end|>", "<end_of_turn>", "<|endoftext|>", "<|eom_id|>", "<EOT>",
                                       "<\xef\xbd\x9c" "end\xe2\x96\x81of\xe2\x96\x81sentence\xef\xbd\x9c>"};
    auto add_eog = [&](int32_t id) {
        if (id >= 0 && id < (int32_t) tokens_.size() && std::find(eog_.begin(), eog_.end(), id) == eog_.end()) eog_.push_back(id);
    };
    add_eog(cfg_.eos);
    add_eog(cfg_.eot);
    for (const char * t : eog_texts) {
        auto it = token_id_.find(t);
        if (it != token_id_.end()) {
            add_eog(it->second);
            if (cfg_.eot < 0) cfg_.eot = it->second;
        }
    }
    // piece cache: byte-level decode of every token
    const ByteMap & bm = byte_map();
    piece_cache_.resize(tokens_.size());
    for (size_t i = 0; i < tokens_.size(); ++i) {
        if (types_[i] == TOK_CONTROL || types_[i] == TOK_USER_DEFINED || types_[i] == TOK_UNKNOWN || types_[i] == TOK_UNUSED) {
            piece_cache_[i] = tokens_[i];
            continue;
        }
        std::string bytes;
        for (uint32_t cp : utf8_to_cps(tokens_[i])) {
            auto it = bm.to_byte.find(cp);
            if (it != bm.to_byte.end()) bytes += (char) it->second;
            else append_utf8(bytes, cp);          // not a byte symbol: keep as is
        }
        piece_cache_[i] = std::move(bytes);
    }
}

bool Tokenizer::is_eog(int32_t id) const { return std::find(eog_.begin(), eog_.end(), id) != eog_.end(); }

// BPE over one pre-split word whose bytes were already mapped to the printable alphabet.
void Tokenizer::bpe_word(const std::string & word, std::vector<int32_t> & out) const {
    struct Sym { int prev, next; size_t pos, len; };
    std::vector<Sym> syms;
    {
        size_t i = 0;
        while (i < word.size()) {
            const unsigned char c = word[i];
            const size_t n = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : 4;
            syms.push_back({(int) syms.size() - 1, (int) syms.size() + 1, i, std::min(n, word.size() - i)});
            i += n;
        }
        if (!syms.empty()) syms.back().next = -1;
    }
    struct Bigram { int left, right, rank; size_t size; };
    auto cmp = [](const Bigram & a, const Bigram & b) { return a.rank > b.rank || (a.rank == b.rank && a.left > b.left); };
    std::priority_queue<Bigram, std::vector<Bigram>, decltype(cmp)> queue(cmp);
    auto try_add = [&](int l, int r) {
        if (l < 0 || r < 0) return;
        const std::string key = word.substr(syms[l].pos, syms[l].len) + " " + word.substr(syms[r].pos, syms[r].len);
        auto it = rank_.find(key);
        if (it == rank_.end()) return;
        queue.push({l, r, it->second, syms[l].len + syms[r].len});
    };
    for (int i = 0; i + 1 < (int) syms.size(); ++i) try_add(i, i + 1);
    while (!queue.empty()) {
        const Bigram b = queue.top();
        queue.pop();
        Sym & L = syms[b.left];
        Sym & Rr = syms[b.right];
        if (L.len == 0 || Rr.len == 0 || L.len + Rr.len != b.size || L.next != b.right) continue;     // stale entry
        L.len += Rr.len;
        Rr.len = 0;
        L.next = Rr.next;
        if (Rr.next >= 0) syms[Rr.next].prev = b.left;
        try_add(L.prev, b.left);
        try_add(b.left, L.next);
    }
    for (int i = 0; i >= 0 && i < (int) syms.size(); i = syms[i].next) {
        if (syms[i].len == 0) continue;
        const std::string piece = word.substr(syms[i].pos, syms[i].len);
        auto it = token_id_.find(piece);
        if (it != token_id_.end()) {
            out.push_back(it->second);
        } else {
            // unknown piece: fall back to its single symbols (byte tokens)
            size_t p = 0;
            while (p < piece.size()) {
                const unsigned char c = piece[p];
                const size_t n = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : 4;
                auto jt = token_id_.find(piece.substr(p, n));
                if (jt != token_id_.end()) out.push_back(jt->second);
                p += n;
            }
        }
        if (syms[i].next < 0) break;
    }
}

std::vector<int32_t> Tokenizer::encode(const std::string & text, bool add_special, bool parse_special) const {
    std::vector<int32_t> out;
    if (add_special && cfg_.add_bos && cfg_.bos >= 0) out.push_back(cfg_.bos);
    // 1. partition around special tokens (longest first); control/unknown ones only when parse_special
    struct Frag { bool is_token; int32_t id; size_t pos, len; };
    std::vector<Frag> frags{{false, -1, 0, text.size()}};
    for (int32_t sid : special_ids_) {
        if (!parse_special && (types_[sid] == TOK_CONTROL || types_[sid] == TOK_UNKNOWN)) continue;
        const std::string & st = tokens_[sid];
        if (st.empty()) continue;
        std::vector<Frag> next;
        for (const Frag & f : frags) {
            if (f.is_token) { next.push_back(f); continue; }
            size_t cur = f.pos;
            const size_t end = f.pos + f.len;
            while (cur < end) {
                const size_t hit = text.find(st, cur);
                if (hit == std::string::npos || hit + st.size() > end) break;
                if (hit > cur) next.push_back({false, -1, cur, hit - cur});
                next.push_back({true, sid, hit, st.size()});
                cur = hit + st.size();
            }
            if (cur < end) next.push_back({false, -1, cur, end - cur});
        }
        frags.swap(next);
    }
    // 2. pre-split + byte mapping + BPE per raw fragment
    const ByteMap & bm = byte_map();
    for (const Frag & f : frags) {
        if (f.is_token) { out.push_back(f.id); continue; }
        for (const std::string & w : pre_split(text.substr(f.pos, f.len))) {
            std::string mapped;
            for (unsigned char c : w) append_utf8(mapped, bm.to_cp[c]);
            bpe_word(mapped, out);
        }
    }
    if (add_special && cfg_.add_eos && cfg_.eos >= 0) out.push_back(cfg_.eos);
    return out;
}

std::string Tokenizer::token_to_piece(int32_t id, bool special) const {
    if (id < 0 || id >= n_tokens()) return "";
    if ((types_[id] == TOK_CONTROL || types_[id] == TOK_UNKNOWN) && !special) return "";
    return piece_cache_[id];
}

std::string Tokenizer::decode(const std::vector<int32_t> & ids, bool remove_special, bool unparse_special) const {
    std::string s;
    for (size_t i = 0; i < ids.size(); ++i) {
        const int32_t id = ids[i];
        if (remove_special && ((i == 0 && id == cfg_.bos && cfg_.add_bos) || (i + 1 == ids.size() && id == cfg_.eos && cfg_.add_eos))) continue;
        s += token_to_piece(id, unparse_special);
    }
    return s;
}

size_t utf8_incomplete_tail(const std::string & s) {
    // number of bytes at the end that start a multi-byte sequence which is not complete yet
    for (size_t back = 1; back <= 4 && back <= s.size(); ++back) {
        const unsigned char c = s[s.size() - back];
        if ((c & 0xC0) == 0x80) continue;                       // continuation byte: keep looking for the lead
        const size_t need = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 1;
        return need > back ? back : 0;
    }
    return 0;
}

bool utf8_valid(const std::string & s) {
    size_t i = 0;
    while (i < s.size()) {
        const unsigned char c = s[i];
        const size_t n = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 0;
        if (n == 0 || i + n > s.size()) return false;
        for (size_t k = 1; k < n; ++k)
            if ((((unsigned char) s[i + k]) >> 6) != 2) return false;
        i += n;
    }
    return true;
}

}  // namespace jib
