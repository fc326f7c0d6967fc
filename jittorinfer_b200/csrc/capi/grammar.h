// GBNF grammars and incremental matching for grammar-constrained sampling.
//
// The reference declares llama_sampler_init_grammar but its implementation asserts on a non-empty grammar
// (src/llama-sampling.cpp:313-389), so nothing there can enforce a response_format.  This is a working engine for the
// GBNF dialect that common/json-schema-to-grammar_local.cpp (and server/json_schema.py here) emit:
//   rule ::= alternatives of sequences of  "literal"  [char-class]  rule-name  ( group )  with  * + ? {m} {m,} {m,n}.
// Matching is over Unicode code points.  The matcher keeps a set of stacks of positions inside rules (the classic
// pushdown-automaton simulation); accepting a code point advances every stack whose next terminal admits it.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

namespace jib {

struct GrammarElem {
    enum Kind : uint8_t { CHARS, RULE_REF } kind = CHARS;
    bool negated = false;                               // CHARS: [^...]
    std::vector<std::pair<uint32_t, uint32_t>> ranges;  // CHARS: inclusive code-point ranges
    int rule = -1;                                      // RULE_REF
};

struct Grammar {
    // rules[r] = alternatives; an alternative = sequence of elements (possibly empty)
    std::vector<std::vector<std::vector<GrammarElem>>> rules;
    std::map<std::string, int> names;
    int root = -1;

    // Parses GBNF text.  Returns "" on success, else a message.
    std::string parse(const std::string & text, const std::string & root_name);
};

// A position: element `elem` of alternative `alt` of rule `rule`.
struct GrammarPos {
    int rule, alt, elem;
    bool operator<(const GrammarPos & o) const { return rule != o.rule ? rule < o.rule : alt != o.alt ? alt < o.alt : elem < o.elem; }
    bool operator==(const GrammarPos & o) const { return rule == o.rule && alt == o.alt && elem == o.elem; }
};
typedef std::vector<GrammarPos> GrammarStack;           // back() = innermost frame; every frame points at a terminal
                                                        // (innermost) or at the element after a rule call (outer frames)

class GrammarMatcher {
  public:
    explicit GrammarMatcher(const Grammar * g);
    void reset();
    // Feeds one code point.  False (state unchanged) if no stack admits it.
    bool accept(uint32_t cp);
    // True if the code points could be fed from the current state (state unchanged).
    bool would_accept(const std::vector<uint32_t> & cps) const;
    // As would_accept, and additionally some character in [lo, hi] (what an unfinished UTF-8 sequence can still become)
    // must be admissible afterwards.
    bool would_accept_tail(const std::vector<uint32_t> & cps, uint32_t lo, uint32_t hi) const;
    // The text so far is a complete sentence of the grammar.
    bool complete() const;
    // No continuation exists (only completion).
    bool dead_end() const;
    size_t n_stacks() const { return stacks_.size(); }

  private:
    void expand(GrammarStack stack, std::vector<GrammarStack> & out, int depth) const;
    static bool step(const Grammar & g, const std::vector<GrammarStack> & in, uint32_t cp, std::vector<GrammarStack> & out,
                     const GrammarMatcher * self);
    const Grammar * g_;
    std::vector<GrammarStack> stacks_;                  // an empty stack = "may end here"
};

// UTF-8 -> code points; returns the number of bytes consumed (an incomplete tail sequence is left unconsumed).
size_t utf8_to_codepoints(const std::string & s, std::vector<uint32_t> & out);
struct Utf8Tail {
    bool pending = false;      // the input ends inside a multi-byte sequence ...
    uint32_t lo = 0, hi = 0;   // ... which can still become a code point in [lo, hi]
    bool invalid = false;      // malformed input (decoding stopped there)
};
size_t utf8_decode(const std::string & s, std::vector<uint32_t> & out, Utf8Tail & tail);

}  // namespace jib
