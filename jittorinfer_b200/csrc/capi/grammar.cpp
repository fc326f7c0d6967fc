#include "grammar.h"

#include <algorithm>
#include <cstring>

namespace jib {

size_t utf8_to_codepoints(const std::string & s, std::vector<uint32_t> & out) {
    Utf8Tail tail;
    return utf8_decode(s, out, tail);
}

// Strict decoder: continuation bytes are checked.  An incomplete sequence at the end is not consumed; `tail` then holds
// the range of code points it can still become.  tail.invalid is set (and decoding stops) at a malformed sequence.
size_t utf8_decode(const std::string & s, std::vector<uint32_t> & out, Utf8Tail & tail) {
    tail = Utf8Tail();
    size_t i = 0;
    while (i < s.size()) {
        const unsigned char c = (unsigned char) s[i];
        const int n = c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 0;
        if (n == 0) { tail.invalid = true; return i; }
        uint32_t cp = n == 1 ? c : c & (0xFF >> (n + 1));
        int have = 1;
        for (; have < n && i + have < s.size(); ++have) {
            const unsigned char cc = (unsigned char) s[i + have];
            if ((cc & 0xC0) != 0x80) { tail.invalid = true; return i; }
            cp = (cp << 6) | (cc & 0x3F);
        }
        if (have < n) {                    // incomplete sequence at the end: what it can still become
            const int missing = n - have;
            tail.pending = true;
            tail.lo = cp << (6 * missing);
            tail.hi = tail.lo | ((1u << (6 * missing)) - 1);
            static const uint32_t min_cp[5] = {0, 0, 0x80, 0x800, 0x10000};     // overlong forms are not characters
            if (tail.lo < min_cp[n]) tail.lo = min_cp[n];
            if (tail.hi < tail.lo) { tail.invalid = true; tail.pending = false; }
            return i;
        }
        out.push_back(cp);
        i += (size_t) n;
    }
    return i;
}

namespace {

struct Parser {
    const std::string & src;
    size_t p = 0;
    Grammar & g;
    std::string err;
    int anon = 0;

    Parser(const std::string & s, Grammar & gr) : src(s), g(gr) {}

    bool eof() const { return p >= src.size(); }
    static bool name_char(char c) { return isalnum((unsigned char) c) || c == '-' || c == '_'; }

    // skips blanks and comments; newlines only when `newlines`
    void skip(bool newlines) {
        while (!eof()) {
            const char c = src[p];
            if (c == '#') {
                while (!eof() && src[p] != '\n') ++p;
            } else if (c == ' ' || c == '\t' || c == '\r' || (newlines && c == '\n')) {
                ++p;
            } else {
                break;
            }
        }
    }

    int rule_id(const std::string & name) {
        auto it = g.names.find(name);
        if (it != g.names.end()) return it->second;
        const int id = (int) g.rules.size();
        g.names[name] = id;
        g.rules.emplace_back();
        return id;
    }
    int fresh_rule() { return rule_id("_" + std::to_string(anon++)); }

    bool parse_hex(int digits, uint32_t & v) {
        v = 0;
        for (int i = 0; i < digits; ++i) {
            if (eof()) return false;
            const char c = src[p++];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else return false;
        }
        return true;
    }

    // one (possibly escaped, possibly multi-byte) character of a literal or class
    bool parse_char(uint32_t & cp) {
        if (eof()) { err = "unexpected end inside a literal"; return false; }
        if (src[p] == '\\') {
            ++p;
            if (eof()) { err = "dangling escape"; return false; }
            const char e = src[p++];
            switch (e) {
                case 'n': cp = '\n'; return true;
                case 'r': cp = '\r'; return true;
                case 't': cp = '\t'; return true;
                case 'x': if (!parse_hex(2, cp)) { err = "bad \\x escape"; return false; } return true;
                case 'u': if (!parse_hex(4, cp)) { err = "bad \\u escape"; return false; } return true;
                case 'U': if (!parse_hex(8, cp)) { err = "bad \\U escape"; return false; } return true;
                default: cp = (unsigned char) e; return true;       // \\ \" \[ \] \- ...
            }
        }
        std::vector<uint32_t> one;
        const unsigned char c = (unsigned char) src[p];
        const int n = c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 1;
        utf8_to_codepoints(src.substr(p, (size_t) n), one);
        if (one.empty()) { err = "bad UTF-8 in grammar"; return false; }
        cp = one[0];
        p += (size_t) n;
        return true;
    }

    // wraps `seq[from..]` into a fresh rule and returns a reference to it
    GrammarElem wrap(std::vector<GrammarElem> & seq, size_t from) {
        GrammarElem ref;
        ref.kind = GrammarElem::RULE_REF;
        if (seq.size() - from == 1 && seq[from].kind == GrammarElem::RULE_REF) {
            ref = seq[from];
        } else {
            const int r = fresh_rule();
            g.rules[r].push_back(std::vector<GrammarElem>(seq.begin() + (long) from, seq.end()));
            ref.rule = r;
        }
        seq.resize(from);
        return ref;
    }

    GrammarElem ref_to(int rule) {
        GrammarElem e;
        e.kind = GrammarElem::RULE_REF;
        e.rule = rule;
        return e;
    }

    // item* as a rule: S ::= item S | (empty)
    int star_rule(const GrammarElem & item) {
        const int r = fresh_rule();
        g.rules[r].push_back({item, ref_to(r)});
        g.rules[r].push_back({});
        return r;
    }

    void apply_repeat(std::vector<GrammarElem> & seq, size_t from, int lo, int hi /* -1 = unbounded */) {
        const GrammarElem item = wrap(seq, from);
        for (int i = 0; i < lo; ++i) seq.push_back(item);
        if (hi < 0) {
            seq.push_back(ref_to(star_rule(item)));
        } else if (hi > lo) {
            // nested optionals: O_k ::= item O_{k-1} | (empty)
            int prev = -1;
            for (int i = 0; i < hi - lo; ++i) {
                const int r = fresh_rule();
                std::vector<GrammarElem> alt{item};
                if (prev >= 0) alt.push_back(ref_to(prev));
                g.rules[r].push_back(alt);
                g.rules[r].push_back({});
                prev = r;
            }
            seq.push_back(ref_to(prev));
        }
    }

    bool parse_sequence(std::vector<GrammarElem> & seq, bool nested) {
        for (;;) {
            skip(nested);
            if (eof()) return true;
            const char c = src[p];
            size_t from = seq.size();
            if (c == '"') {
                ++p;
                while (!eof() && src[p] != '"') {
                    uint32_t cp;
                    if (!parse_char(cp)) return false;
                    GrammarElem e;
                    e.ranges.push_back({cp, cp});
                    seq.push_back(e);
                }
                if (eof()) { err = "unterminated literal"; return false; }
                ++p;
            } else if (c == '[') {
                ++p;
                GrammarElem e;
                if (!eof() && src[p] == '^') { e.negated = true; ++p; }
                while (!eof() && src[p] != ']') {
                    uint32_t lo, hi;
                    if (!parse_char(lo)) return false;
                    hi = lo;
                    if (p + 1 < src.size() && src[p] == '-' && src[p + 1] != ']') {
                        ++p;
                        if (!parse_char(hi)) return false;
                    }
                    e.ranges.push_back({lo, hi});
                }
                if (eof()) { err = "unterminated character class"; return false; }
                ++p;
                seq.push_back(e);
            } else if (c == '.') {
                ++p;
                GrammarElem e;
                e.negated = true;              // "not in the empty set" = any character
                seq.push_back(e);
            } else if (c == '(') {
                ++p;
                const int r = fresh_rule();
                if (!parse_alternates(r, true)) return false;
                skip(true);
                if (eof() || src[p] != ')') { err = "missing ')'"; return false; }
                ++p;
                seq.push_back(ref_to(r));
            } else if (name_char(c)) {
                // a rule reference -- unless this name starts the next rule ("name ::=")
                size_t q = p;
                while (q < src.size() && name_char(src[q])) ++q;
                size_t t = q;
                while (t < src.size() && (src[t] == ' ' || src[t] == '\t')) ++t;
                if (!nested && src.compare(t, 3, "::=") == 0) return true;
                seq.push_back(ref_to(rule_id(src.substr(p, q - p))));
                p = q;
            } else {
                return true;                   // '|', ')', newline: the caller decides
            }
            // repetition suffixes
            for (;;) {
                if (eof()) break;
                const char r = src[p];
                if (r == '*') { ++p; apply_repeat(seq, from, 0, -1); }
                else if (r == '+') { ++p; apply_repeat(seq, from, 1, -1); }
                else if (r == '?') { ++p; apply_repeat(seq, from, 0, 1); }
                else if (r == '{') {
                    ++p;
                    int lo = 0, hi = -2;
                    bool any = false;
                    while (!eof() && isdigit((unsigned char) src[p])) { lo = lo * 10 + (src[p++] - '0'); any = true; }
                    if (!eof() && src[p] == ',') {
                        ++p;
                        if (!eof() && isdigit((unsigned char) src[p])) {
                            hi = 0;
                            while (!eof() && isdigit((unsigned char) src[p])) hi = hi * 10 + (src[p++] - '0');
                        } else {
                            hi = -1;
                        }
                    } else {
                        hi = lo;
                    }
                    if (eof() || src[p] != '}' || (!any && hi == lo)) { err = "bad repetition {m,n}"; return false; }
                    ++p;
                    if (hi >= 0 && hi < lo) { err = "repetition with max < min"; return false; }
                    if (lo > 4096 || hi > 4096) { err = "repetition count too large"; return false; }
                    apply_repeat(seq, from, lo, hi);
                } else {
                    break;
                }
            }
        }
    }

    bool parse_alternates(int rule, bool nested) {
        for (;;) {
            std::vector<GrammarElem> seq;
            if (!parse_sequence(seq, nested)) return false;
            g.rules[rule].push_back(seq);
            // a '|' may follow on this line or, for top-level rules, at the start of a following line
            size_t save = p;
            skip(true);
            if (!eof() && src[p] == '|') { ++p; continue; }
            p = nested ? p : save;
            return true;
        }
    }

    bool parse_all() {
        for (;;) {
            skip(true);
            if (eof()) return true;
            size_t q = p;
            while (q < src.size() && name_char(src[q])) ++q;
            if (q == p) { err = "expected a rule name at offset " + std::to_string(p); return false; }
            const std::string name = src.substr(p, q - p);
            p = q;
            skip(false);
            if (src.compare(p, 3, "::=") != 0) { err = "expected ::= after " + name; return false; }
            p += 3;
            const int r = rule_id(name);
            if (!g.rules[r].empty()) { err = "rule " + name + " defined twice"; return false; }
            if (!parse_alternates(r, false)) return false;
        }
    }
};

}  // namespace

std::string Grammar::parse(const std::string & text, const std::string & root_name) {
    rules.clear();
    names.clear();
    Parser ps(text, *this);
    if (!ps.parse_all()) return ps.err.empty() ? "syntax error" : ps.err;
    for (const auto & kv : names)
        if (rules[kv.second].empty()) return "rule " + kv.first + " is used but never defined";
    auto it = names.find(root_name);
    if (it == names.end()) return "no rule named " + root_name;
    root = it->second;
    return "";
}

// ---- matcher ----------------------------------------------------------------------------------------------------
GrammarMatcher::GrammarMatcher(const Grammar * g) : g_(g) { reset(); }

void GrammarMatcher::reset() {
    stacks_.clear();
    for (int a = 0; a < (int) g_->rules[g_->root].size(); ++a) expand({GrammarPos{g_->root, a, 0}}, stacks_, 0);
    std::sort(stacks_.begin(), stacks_.end());
    stacks_.erase(std::unique(stacks_.begin(), stacks_.end()), stacks_.end());
}

// Rewrites `stack` until its innermost frame points at a terminal (or the stack is empty) and appends the results.
void GrammarMatcher::expand(GrammarStack stack, std::vector<GrammarStack> & out, int depth) const {
    if (depth > 256) return;                   // left recursion or absurd nesting: give up on this branch
    while (!stack.empty()) {
        const GrammarPos top = stack.back();
        const std::vector<GrammarElem> & alt = g_->rules[top.rule][top.alt];
        if (top.elem >= (int) alt.size()) {     // end of this alternative: return to the caller's frame
            stack.pop_back();
            continue;
        }
        const GrammarElem & e = alt[top.elem];
        if (e.kind == GrammarElem::CHARS) {
            out.push_back(std::move(stack));
            return;
        }
        stack.back().elem = top.elem + 1;       // where to continue after the call
        const int callee = e.rule;
        for (int a = 0; a < (int) g_->rules[callee].size(); ++a) {
            GrammarStack next = stack;
            next.push_back(GrammarPos{callee, a, 0});
            expand(std::move(next), out, depth + 1);
        }
        return;
    }
    out.emplace_back();                        // everything returned: the sentence may end here
}

static bool elem_admits(const GrammarElem & e, uint32_t cp) {
    bool in = false;
    for (const auto & r : e.ranges)
        if (cp >= r.first && cp <= r.second) { in = true; break; }
    return in != e.negated;
}

bool GrammarMatcher::step(const Grammar & g, const std::vector<GrammarStack> & in, uint32_t cp, std::vector<GrammarStack> & out,
                          const GrammarMatcher * self) {
    out.clear();
    for (const GrammarStack & s : in) {
        if (s.empty()) continue;
        const GrammarPos top = s.back();
        if (!elem_admits(g.rules[top.rule][top.alt][top.elem], cp)) continue;
        GrammarStack next = s;
        next.back().elem = top.elem + 1;
        self->expand(std::move(next), out, 0);
    }
    std::sort(out.begin(), out.end());
    out.erase(std::unique(out.begin(), out.end()), out.end());
    return !out.empty();
}

bool GrammarMatcher::accept(uint32_t cp) {
    std::vector<GrammarStack> next;
    if (!step(*g_, stacks_, cp, next, this)) return false;
    stacks_.swap(next);
    return true;
}

bool GrammarMatcher::would_accept(const std::vector<uint32_t> & cps) const {
    if (cps.empty()) return true;
    std::vector<GrammarStack> cur = stacks_, next;
    for (uint32_t cp : cps) {
        if (!step(*g_, cur, cp, next, this)) return false;
        cur.swap(next);
    }
    return true;
}

static bool elem_admits_range(const GrammarElem & e, uint32_t lo, uint32_t hi) {
    if (!e.negated) {
        for (const auto & r : e.ranges)
            if (r.first <= hi && r.second >= lo) return true;
        return false;
    }
    // negated: some code point of [lo, hi] lies outside every listed range.  Candidates: lo, and the first code point after
    // each range that starts inside [lo, hi].
    auto listed = [&](uint32_t cp) {
        for (const auto & r : e.ranges)
            if (cp >= r.first && cp <= r.second) return true;
        return false;
    };
    if (!listed(lo)) return true;
    for (const auto & r : e.ranges)
        if (r.second >= lo && r.second < hi && !listed(r.second + 1)) return true;
    return false;
}

bool GrammarMatcher::would_accept_tail(const std::vector<uint32_t> & cps, uint32_t lo, uint32_t hi) const {
    std::vector<GrammarStack> cur = stacks_, next;
    for (uint32_t cp : cps) {
        if (!step(*g_, cur, cp, next, this)) return false;
        cur.swap(next);
    }
    for (const GrammarStack & s : cur) {
        if (s.empty()) continue;
        const GrammarPos top = s.back();
        if (elem_admits_range(g_->rules[top.rule][top.alt][top.elem], lo, hi)) return true;
    }
    return false;
}

bool GrammarMatcher::complete() const {
    for (const GrammarStack & s : stacks_)
        if (s.empty()) return true;
    return false;
}

bool GrammarMatcher::dead_end() const {
    for (const GrammarStack & s : stacks_)
        if (!s.empty()) return false;
    return true;
}

}  // namespace jib
