// Sampler chain of the C API (section 8 of llama.h).
//
// Same sampler set and parameter meanings as the reference's src/llama-sampling.cpp (top-k 146-220, softmax 222-244,
// dist 270-312, top-p 432-496, min-p 498-590, XTC 592-677, typical 679-774, dynamic temperature 776-885, DRY 887-1245,
// penalties 1247-1357, logit bias 1424-1498, chain 1500-1629), written for the way this engine uses them: the candidate
// array is normally the GPU's top-k (64 entries, already sorted), so every sampler works on a short, usually sorted
// array and none needs a bucket sort over the whole vocabulary.
#include "capi_internal.h"
#include "grammar.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <numeric>
#include <random>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

using arr_t = llama_token_data_array;

double now_us() {
    return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

uint32_t resolve_seed(uint32_t seed) {
    if (seed != LLAMA_DEFAULT_SEED) return seed;
    std::random_device rd;
    return rd();
}

void sort_desc(arr_t * a) {
    if (a->sorted) return;
    std::sort(a->data, a->data + a->size, [](const llama_token_data & x, const llama_token_data & y) { return x.logit > y.logit; });
    a->sorted = true;
}

// probabilities from logits; keeps order (sorts first so that later prefix cuts are meaningful)
void softmax(arr_t * a) {
    if (a->size == 0) return;
    sort_desc(a);
    const float mx = a->data[0].logit;
    double sum = 0;
    for (size_t i = 0; i < a->size; ++i) {
        const float p = std::exp(a->data[i].logit - mx);
        a->data[i].p = p;
        sum += p;
    }
    const float inv = (float) (1.0 / sum);
    for (size_t i = 0; i < a->size; ++i) a->data[i].p *= inv;
}

template <typename Ctx>
llama_sampler * make(const llama_sampler_i * iface, Ctx * ctx) { return llama_sampler_init(iface, ctx); }

template <typename Ctx>
void free_ctx(llama_sampler * s) { delete (Ctx *) s->ctx; }

// ---- greedy ---------------------------------------------------------------------------------------------------------
const char * greedy_name(const llama_sampler *) { return "greedy"; }
void greedy_apply(llama_sampler *, arr_t * a) {
    a->selected = 0;
    for (size_t i = 1; i < a->size; ++i)
        if (a->data[i].logit > a->data[a->selected].logit) a->selected = (int64_t) i;
}
const llama_sampler_i greedy_i = {greedy_name, nullptr, greedy_apply, nullptr, nullptr, nullptr};

// ---- dist -----------------------------------------------------------------------------------------------------------
struct DistCtx {
    uint32_t seed, seed_cur;
    std::mt19937 rng;
};
const char * dist_name(const llama_sampler *) { return "dist"; }
void dist_apply(llama_sampler * s, arr_t * a) {
    auto * c = (DistCtx *) s->ctx;
    if (a->size == 0) { a->selected = -1; return; }
    softmax(a);
    // inverse-CDF draw: one uniform number, no per-call distribution object
    const double u = std::generate_canonical<double, 53>(c->rng);
    double cum = 0;
    a->selected = (int64_t) a->size - 1;
    for (size_t i = 0; i < a->size; ++i) {
        cum += a->data[i].p;
        if (u < cum) { a->selected = (int64_t) i; break; }
    }
}
void dist_reset(llama_sampler * s) {
    auto * c = (DistCtx *) s->ctx;
    c->seed_cur = resolve_seed(c->seed);
    c->rng.seed(c->seed_cur);
}
llama_sampler * dist_clone(const llama_sampler * s) {
    auto * c = (const DistCtx *) s->ctx;
    llama_sampler * r = llama_sampler_init_dist(c->seed);
    ((DistCtx *) r->ctx)->rng = c->rng;       // the clone continues the same random stream
    ((DistCtx *) r->ctx)->seed_cur = c->seed_cur;
    return r;
}
const llama_sampler_i dist_i = {dist_name, nullptr, dist_apply, dist_reset, dist_clone, free_ctx<DistCtx>};

// ---- top-k ----------------------------------------------------------------------------------------------------------
struct TopKCtx { int32_t k; };
const char * top_k_name(const llama_sampler *) { return "top-k"; }
void top_k_apply(llama_sampler * s, arr_t * a) {
    int32_t k = ((TopKCtx *) s->ctx)->k;
    if (k <= 0) k = (int32_t) a->size;
    k = std::min<int32_t>(k, (int32_t) a->size);
    if (!a->sorted) {
        auto cmp = [](const llama_token_data & x, const llama_token_data & y) { return x.logit > y.logit; };
        std::partial_sort(a->data, a->data + k, a->data + a->size, cmp);
        a->sorted = true;
    }
    a->size = (size_t) k;
}
llama_sampler * top_k_clone(const llama_sampler * s) { return llama_sampler_init_top_k(((TopKCtx *) s->ctx)->k); }
const llama_sampler_i top_k_i = {top_k_name, nullptr, top_k_apply, nullptr, top_k_clone, free_ctx<TopKCtx>};

// ---- top-p ----------------------------------------------------------------------------------------------------------
struct PCtx { float p; size_t min_keep; };
const char * top_p_name(const llama_sampler *) { return "top-p"; }
void top_p_apply(llama_sampler * s, arr_t * a) {
    auto * c = (PCtx *) s->ctx;
    if (c->p >= 1.0f) return;
    softmax(a);
    double cum = 0;
    size_t keep = a->size;
    for (size_t i = 0; i < a->size; ++i) {
        cum += a->data[i].p;
        if (cum >= c->p && i + 1 >= c->min_keep) { keep = i + 1; break; }
    }
    a->size = keep;
}
llama_sampler * top_p_clone(const llama_sampler * s) {
    auto * c = (PCtx *) s->ctx;
    return llama_sampler_init_top_p(c->p, c->min_keep);
}
const llama_sampler_i top_p_i = {top_p_name, nullptr, top_p_apply, nullptr, top_p_clone, free_ctx<PCtx>};

// ---- min-p ----------------------------------------------------------------------------------------------------------
const char * min_p_name(const llama_sampler *) { return "min-p"; }
void min_p_apply(llama_sampler * s, arr_t * a) {
    auto * c = (PCtx *) s->ctx;
    if (c->p <= 0.0f || a->size == 0) return;
    // p_i >= p * p_max  <=>  logit_i >= logit_max + log(p): no softmax needed
    sort_desc(a);
    const float cut = a->data[0].logit + std::log(c->p);
    size_t keep = 0;
    while (keep < a->size && (a->data[keep].logit >= cut || keep < c->min_keep)) ++keep;
    a->size = std::max<size_t>(keep, 1);
}
llama_sampler * min_p_clone(const llama_sampler * s) {
    auto * c = (PCtx *) s->ctx;
    return llama_sampler_init_min_p(c->p, c->min_keep);
}
const llama_sampler_i min_p_i = {min_p_name, nullptr, min_p_apply, nullptr, min_p_clone, free_ctx<PCtx>};

// ---- locally typical ------------------------------------------------------------------------------------------------
const char * typical_name(const llama_sampler *) { return "typical"; }
void typical_apply(llama_sampler * s, arr_t * a) {
    auto * c = (PCtx *) s->ctx;
    if (c->p >= 1.0f || a->size == 0) return;
    softmax(a);
    double entropy = 0;
    for (size_t i = 0; i < a->size; ++i)
        if (a->data[i].p > 0) entropy -= (double) a->data[i].p * std::log((double) a->data[i].p);
    // distance of each token's surprise from the entropy; keep the closest ones until their mass reaches p
    std::vector<std::pair<float, size_t>> dist(a->size);
    for (size_t i = 0; i < a->size; ++i) {
        const double surprise = a->data[i].p > 0 ? -std::log((double) a->data[i].p) : 1e30;
        dist[i] = {(float) std::fabs(surprise - entropy), i};
    }
    std::stable_sort(dist.begin(), dist.end(), [](const auto & x, const auto & y) { return x.first < y.first; });
    double cum = 0;
    size_t keep = a->size;
    for (size_t i = 0; i < dist.size(); ++i) {
        cum += a->data[dist[i].second].p;
        if (cum > c->p && i + 1 >= c->min_keep) { keep = i + 1; break; }
    }
    std::vector<llama_token_data> kept(keep);
    for (size_t i = 0; i < keep; ++i) kept[i] = a->data[dist[i].second];
    std::copy(kept.begin(), kept.end(), a->data);
    a->size = keep;
    a->sorted = false;
}
llama_sampler * typical_clone(const llama_sampler * s) {
    auto * c = (PCtx *) s->ctx;
    return llama_sampler_init_typical(c->p, c->min_keep);
}
const llama_sampler_i typical_i = {typical_name, nullptr, typical_apply, nullptr, typical_clone, free_ctx<PCtx>};

// ---- temperature (plain and entropy-scaled) -------------------------------------------------------------------------
struct TempCtx { float t, delta, exponent; bool ext; };
void scale_by_temp(arr_t * a, float t) {
    if (t <= 0.0f) {          // keep the arg-max only
        size_t best = 0;
        for (size_t i = 1; i < a->size; ++i)
            if (a->data[i].logit > a->data[best].logit) best = i;
        for (size_t i = 0; i < a->size; ++i)
            if (i != best) a->data[i].logit = -INFINITY;
        return;
    }
    for (size_t i = 0; i < a->size; ++i) a->data[i].logit /= t;
}
const char * temp_name(const llama_sampler * s) { return ((TempCtx *) s->ctx)->ext ? "temp-ext" : "temp"; }
void temp_apply(llama_sampler * s, arr_t * a) {
    auto * c = (TempCtx *) s->ctx;
    if (!c->ext || c->delta <= 0.0f) { scale_by_temp(a, c->t); return; }
    if (a->size <= 1) return;
    const float t_lo = std::max(0.0f, c->t - c->delta), t_hi = c->t + c->delta;
    softmax(a);
    double entropy = 0;
    for (size_t i = 0; i < a->size; ++i)
        if (a->data[i].p > 0) entropy -= (double) a->data[i].p * std::log((double) a->data[i].p);
    const double h_max = std::log((double) a->size);
    const double h_norm = h_max > 0 ? entropy / h_max : 0;
    const float t_dyn = t_lo + (t_hi - t_lo) * (float) std::pow(h_norm, (double) c->exponent);
    scale_by_temp(a, t_dyn);
    a->sorted = a->sorted && t_dyn > 0;
    softmax(a);              // probabilities follow the rescaled logits
}
llama_sampler * temp_clone(const llama_sampler * s) {
    auto * c = (TempCtx *) s->ctx;
    return c->ext ? llama_sampler_init_temp_ext(c->t, c->delta, c->exponent) : llama_sampler_init_temp(c->t);
}
const llama_sampler_i temp_i = {temp_name, nullptr, temp_apply, nullptr, temp_clone, free_ctx<TempCtx>};

// ---- XTC (exclude top choices) --------------------------------------------------------------------------------------
struct XtcCtx {
    float p, t;
    size_t min_keep;
    uint32_t seed, seed_cur;
    std::mt19937 rng;
};
const char * xtc_name(const llama_sampler *) { return "xtc"; }
void xtc_apply(llama_sampler * s, arr_t * a) {
    auto * c = (XtcCtx *) s->ctx;
    if (c->p <= 0.0f || c->t > 0.5f || a->size < 2) return;
    if (std::generate_canonical<double, 53>(c->rng) >= c->p) return;
    softmax(a);
    // candidates are sorted: [0, last] are at or above the threshold; all but the last of them go
    int64_t last = -1;
    for (size_t i = 0; i < a->size && a->data[i].p >= c->t; ++i) last = (int64_t) i;
    if (last < 1) return;
    if (a->size - (size_t) last < c->min_keep) return;
    a->data += last;
    a->size -= (size_t) last;
}
void xtc_reset(llama_sampler * s) {
    auto * c = (XtcCtx *) s->ctx;
    c->seed_cur = resolve_seed(c->seed);
    c->rng.seed(c->seed_cur);
}
llama_sampler * xtc_clone(const llama_sampler * s) {
    auto * c = (XtcCtx *) s->ctx;
    llama_sampler * r = llama_sampler_init_xtc(c->p, c->t, c->min_keep, c->seed);
    ((XtcCtx *) r->ctx)->rng = c->rng;                 // the clone continues the same random stream ...
    ((XtcCtx *) r->ctx)->seed_cur = c->seed_cur;       // ... and reports the seed that stream started from
    return r;
}
const llama_sampler_i xtc_i = {xtc_name, nullptr, xtc_apply, xtc_reset, xtc_clone, free_ctx<XtcCtx>};

// ---- repetition / frequency / presence penalties --------------------------------------------------------------------
struct PenCtx {
    int32_t last_n;
    float repeat, freq, present;
    std::vector<llama_token> ring;      // the last_n most recent tokens, oldest first
    std::unordered_map<llama_token, int> count;
};
const char * pen_name(const llama_sampler *) { return "penalties"; }
void pen_accept(llama_sampler * s, llama_token tok) {
    auto * c = (PenCtx *) s->ctx;
    if (c->last_n == 0) return;
    c->ring.push_back(tok);
    c->count[tok]++;
    if (c->last_n > 0 && (int32_t) c->ring.size() > c->last_n) {
        const llama_token old = c->ring.front();
        c->ring.erase(c->ring.begin());
        if (--c->count[old] == 0) c->count.erase(old);
    }
}
void pen_apply(llama_sampler * s, arr_t * a) {
    auto * c = (PenCtx *) s->ctx;
    if (c->last_n == 0 || (c->repeat == 1.0f && c->freq == 0.0f && c->present == 0.0f) || c->count.empty()) return;
    for (size_t i = 0; i < a->size; ++i) {
        auto it = c->count.find(a->data[i].id);
        if (it == c->count.end()) continue;
        float & l = a->data[i].logit;
        // dividing a negative logit would make the token more likely, so the sign picks the direction
        l = l <= 0 ? l * c->repeat : l / c->repeat;
        l -= (float) it->second * c->freq + c->present;
    }
    a->sorted = false;
}
void pen_reset(llama_sampler * s) {
    auto * c = (PenCtx *) s->ctx;
    c->ring.clear();
    c->count.clear();
}
llama_sampler * pen_clone(const llama_sampler * s) {
    auto * c = (PenCtx *) s->ctx;
    llama_sampler * r = llama_sampler_init_penalties(c->last_n, c->repeat, c->freq, c->present);
    ((PenCtx *) r->ctx)->ring = c->ring;
    ((PenCtx *) r->ctx)->count = c->count;
    return r;
}
const llama_sampler_i pen_i = {pen_name, pen_accept, pen_apply, pen_reset, pen_clone, free_ctx<PenCtx>};

// ---- DRY ------------------------------------------------------------------------------------------------------------
struct DryCtx {
    int32_t n_ctx_train;
    float multiplier, base;
    int32_t allowed_length, last_n;
    std::vector<uint8_t> is_breaker;    // per token id: the token's text contains a breaker string
    std::vector<std::vector<llama_token>> multi;   // breakers spelled with several tokens, as token sequences
    std::unordered_map<llama_token, std::vector<int32_t>> by_last;     // last token of a sequence -> indices into multi
    std::vector<llama_token> hist;      // most recent last, capped at the effective window
    int32_t window() const { return last_n < 0 ? n_ctx_train : last_n; }
};
const char * dry_name(const llama_sampler *) { return "dry"; }
void dry_accept(llama_sampler * s, llama_token tok) {
    auto * c = (DryCtx *) s->ctx;
    if (c->multiplier == 0.0f || c->base < 1.0f || c->last_n == 0) return;
    c->hist.push_back(tok);
    const size_t w = (size_t) std::max(1, c->window());
    if (c->hist.size() > 2 * w) c->hist.erase(c->hist.begin(), c->hist.end() - w);   // amortised trim
}
void dry_apply(llama_sampler * s, arr_t * a) {
    auto * c = (DryCtx *) s->ctx;
    if (c->multiplier == 0.0f || c->base < 1.0f || c->last_n == 0) return;
    const size_t w = (size_t) std::max(1, c->window());
    const size_t n = std::min(c->hist.size(), w);
    if (n < 2) return;
    const llama_token * h = c->hist.data() + (c->hist.size() - n);
    auto breaker = [&](llama_token t) { return t >= 0 && (size_t) t < c->is_breaker.size() && c->is_breaker[t]; };
    // a match cannot reach back across a breaker: cap = number of trailing non-breaker tokens
    size_t cap = 0;
    while (cap < n && !breaker(h[n - 1 - cap])) ++cap;
    // ... nor across a breaker that is spelled with several tokens: the most recent place where such a sequence ends
    if (!c->multi.empty()) {
        for (size_t back = 0; back < cap; ++back) {                        // a sequence that ends `back` tokens before the end
            auto it = c->by_last.find(h[n - 1 - back]);
            if (it == c->by_last.end()) continue;
            bool hit = false;
            for (int32_t idx : it->second) {
                const std::vector<llama_token> & seq = c->multi[(size_t) idx];
                const size_t L = seq.size();
                if (back + L <= n && std::equal(seq.begin(), seq.end(), h + (n - back - L))) { hit = true; break; }
            }
            if (hit) { cap = back; break; }
        }
    }
    if (cap == 0) return;
    // Z-function of the reversed history: z[i] = length of the match between the text ending at the end and the
    // text ending at position n-1-i
    std::vector<int32_t> z(n, 0);
    auto rv = [&](size_t i) { return h[n - 1 - i]; };
    for (size_t i = 1, l = 0, r = 0; i < n; ++i) {
        if (i < r) z[i] = (int32_t) std::min(r - i, (size_t) z[i - l]);
        while (i + z[i] < n && rv(z[i]) == rv(i + z[i])) ++z[i];
        if (i + z[i] > r) { l = i; r = i + z[i]; }
    }
    std::unordered_map<llama_token, int32_t> longest;     // token that would extend a repeat -> repeat length
    for (size_t i = 1; i < n; ++i) {
        const int32_t len = (int32_t) std::min((size_t) z[i], cap);
        if (len < c->allowed_length || len == 0) continue;
        const llama_token next = h[n - i];               // the token that followed the earlier occurrence
        auto it = longest.find(next);
        if (it == longest.end() || it->second < len) longest[next] = len;
    }
    if (longest.empty()) return;
    const float max_exp = c->base > 1.000001f ? std::log(3.0e38f / std::max(c->multiplier, 1e-30f)) / std::log(c->base) : 0.0f;
    for (size_t i = 0; i < a->size; ++i) {
        auto it = longest.find(a->data[i].id);
        if (it == longest.end()) continue;
        float e = (float) (it->second - c->allowed_length);
        if (max_exp > 0 && e > max_exp) e = max_exp;
        a->data[i].logit -= c->multiplier * std::pow(c->base, e);
    }
    a->sorted = false;
}
void dry_reset(llama_sampler * s) { ((DryCtx *) s->ctx)->hist.clear(); }
extern const llama_sampler_i dry_i;
llama_sampler * dry_clone(const llama_sampler * s) { return llama_sampler_init(&dry_i, new DryCtx(*(DryCtx *) s->ctx)); }
extern const llama_sampler_i dry_i = {dry_name, dry_accept, dry_apply, dry_reset, dry_clone, free_ctx<DryCtx>};

// ---- logit bias -----------------------------------------------------------------------------------------------------
struct BiasCtx {
    int32_t n_vocab;
    std::vector<llama_logit_bias> bias;
};
const char * bias_name(const llama_sampler *) { return "logit-bias"; }
void bias_apply(llama_sampler * s, arr_t * a) {
    auto * c = (BiasCtx *) s->ctx;
    if (c->bias.empty()) return;
    // full-vocabulary arrays are indexed by token id; candidate lists need a search
    const bool dense = a->size == (size_t) c->n_vocab && a->size > 0 && a->data[0].id == 0 && a->data[a->size - 1].id == c->n_vocab - 1;
    bool touched = false;
    for (const llama_logit_bias & b : c->bias) {
        if (dense) {
            if (b.token >= 0 && b.token < c->n_vocab && a->data[b.token].id == b.token) {
                a->data[b.token].logit += b.bias;
                touched = true;
                continue;
            }
        }
        for (size_t i = 0; i < a->size; ++i)
            if (a->data[i].id == b.token) { a->data[i].logit += b.bias; touched = true; break; }
    }
    if (touched) a->sorted = false;
}
llama_sampler * bias_clone(const llama_sampler * s) {
    auto * c = (BiasCtx *) s->ctx;
    return llama_sampler_init_logit_bias(c->n_vocab, (int32_t) c->bias.size(), c->bias.data());
}
const llama_sampler_i bias_i = {bias_name, nullptr, bias_apply, nullptr, bias_clone, free_ctx<BiasCtx>};

// ---- grammar ----------------------------------------------------------------------------------------------------------
// Keeps only the candidates whose text can continue the grammar (end-of-generation tokens only where the text so far is a
// complete sentence).  If none of the candidates can, one token that can is put in their place, so that generation
// always stays inside the grammar even when the candidate list is a short device top-k.
struct GrammarCtx {
    std::string text, root;
    jib::Grammar grammar;
    std::unique_ptr<jib::GrammarMatcher> matcher;
    std::vector<std::string> pieces;          // bytes of every token ("" = never allowed: control tokens)
    std::vector<uint8_t> is_eog;
    llama_token eos = -1;
    std::string pending;                      // bytes of an incomplete UTF-8 sequence carried between tokens
    std::vector<llama_token> history;         // accepted tokens (replayed by clone)
    bool empty_grammar = false;

    bool allows(llama_token t) const {
        if (t < 0 || (size_t) t >= pieces.size()) return false;
        if (is_eog[(size_t) t]) return matcher->complete() && pending.empty();
        const std::string & piece = pieces[(size_t) t];
        if (piece.empty()) return false;
        std::vector<uint32_t> cps;
        jib::Utf8Tail tail;
        jib::utf8_decode(pending + piece, cps, tail);
        if (tail.invalid) return false;               // would break a multi-byte character
        return tail.pending ? matcher->would_accept_tail(cps, tail.lo, tail.hi) : matcher->would_accept(cps);
    }
};
const char * grammar_name(const llama_sampler *) { return "grammar"; }
void grammar_apply(llama_sampler * s, arr_t * a) {
    auto * c = (GrammarCtx *) s->ctx;
    if (c == nullptr || c->empty_grammar) return;
    size_t keep = 0;
    for (size_t i = 0; i < a->size; ++i)
        if (c->allows(a->data[i].id)) a->data[keep++] = a->data[i];
    if (keep == 0 && a->size > 0) {
        llama_token pick = -1;
        if (c->matcher->complete() && c->pending.empty() && c->eos >= 0) {
            pick = c->eos;
        } else {
            for (size_t t = 0; t < c->pieces.size(); ++t)
                if (!c->is_eog[t] && c->allows((llama_token) t)) { pick = (llama_token) t; break; }
        }
        if (pick >= 0) {
            a->data[0] = llama_token_data{pick, 0.0f, 1.0f};
            keep = 1;
        }
    }
    if (keep > 0) a->size = keep;             // keep == 0: nothing in the whole vocabulary fits; leave the list alone
    if (a->selected >= (int64_t) a->size) a->selected = -1;
}
void grammar_accept(llama_sampler * s, llama_token tok) {
    auto * c = (GrammarCtx *) s->ctx;
    if (c == nullptr || c->empty_grammar || tok < 0 || (size_t) tok >= c->pieces.size()) return;
    c->history.push_back(tok);
    if (c->is_eog[(size_t) tok]) return;
    std::string bytes = c->pending + c->pieces[(size_t) tok];
    std::vector<uint32_t> cps;
    jib::Utf8Tail tail;
    const size_t used = jib::utf8_decode(bytes, cps, tail);
    for (uint32_t cp : cps)
        if (!c->matcher->accept(cp)) break;   // a token the grammar rejects (sampled without apply): state stays put
    c->pending = tail.invalid ? std::string() : bytes.substr(used);
}
void grammar_reset(llama_sampler * s) {
    auto * c = (GrammarCtx *) s->ctx;
    if (c == nullptr || c->empty_grammar) return;
    c->matcher->reset();
    c->pending.clear();
    c->history.clear();
}
llama_sampler * grammar_clone(const llama_sampler * s);
void grammar_free(llama_sampler * s) { delete (GrammarCtx *) s->ctx; }
const llama_sampler_i grammar_i = {grammar_name, grammar_accept, grammar_apply, grammar_reset, grammar_clone, grammar_free};

llama_sampler * grammar_make(std::vector<std::string> pieces, std::vector<uint8_t> is_eog, llama_token eos, const char * text,
                             const char * root) {
    auto * c = new GrammarCtx();
    c->text = text ? text : "";
    c->root = root && root[0] ? root : "root";
    c->empty_grammar = c->text.find_first_not_of(" \t\r\n") == std::string::npos;
    c->pieces = std::move(pieces);
    c->is_eog = std::move(is_eog);
    c->eos = eos;
    if (!c->empty_grammar) {
        const std::string err = c->grammar.parse(c->text, c->root);
        if (!err.empty()) {
            fprintf(stderr, "llama_sampler_init_grammar: %s\n", err.c_str());
            delete c;
            return nullptr;
        }
        c->matcher.reset(new jib::GrammarMatcher(&c->grammar));
    }
    return llama_sampler_init(&grammar_i, c);
}
llama_sampler * grammar_clone(const llama_sampler * s) {
    auto * c = (const GrammarCtx *) s->ctx;
    llama_sampler * r = grammar_make(c->pieces, c->is_eog, c->eos, c->text.c_str(), c->root.c_str());
    if (r != nullptr)
        for (llama_token t : c->history) grammar_accept(r, t);
    return r;
}

// ---- chain ----------------------------------------------------------------------------------------------------------
struct ChainCtx {
    llama_sampler_chain_params params;
    std::vector<llama_sampler *> members;
    double t_sample_us = 0;
    int32_t n_sample = 0;
};
const char * chain_name(const llama_sampler *) { return "chain"; }
void chain_accept(llama_sampler * s, llama_token tok) {
    auto * c = (ChainCtx *) s->ctx;
    const double t0 = c->params.no_perf ? 0 : now_us();
    for (llama_sampler * m : c->members) llama_sampler_accept(m, tok);
    c->n_sample++;
    if (!c->params.no_perf) c->t_sample_us += now_us() - t0;
}
void chain_apply(llama_sampler * s, arr_t * a) {
    auto * c = (ChainCtx *) s->ctx;
    const double t0 = c->params.no_perf ? 0 : now_us();
    for (llama_sampler * m : c->members) llama_sampler_apply(m, a);
    if (!c->params.no_perf) c->t_sample_us += now_us() - t0;
}
void chain_reset(llama_sampler * s) {
    auto * c = (ChainCtx *) s->ctx;
    for (llama_sampler * m : c->members) llama_sampler_reset(m);
    c->t_sample_us = 0;
    c->n_sample = 0;
}
llama_sampler * chain_clone(const llama_sampler * s) {
    auto * c = (const ChainCtx *) s->ctx;
    llama_sampler * r = llama_sampler_chain_init(c->params);
    for (llama_sampler * m : c->members) llama_sampler_chain_add(r, llama_sampler_clone(m));
    return r;
}
void chain_free(llama_sampler * s) {
    auto * c = (ChainCtx *) s->ctx;
    for (llama_sampler * m : c->members) llama_sampler_free(m);
    delete c;
}
const llama_sampler_i chain_i = {chain_name, chain_accept, chain_apply, chain_reset, chain_clone, chain_free};

}  // namespace

// =====================================================================================================================
extern "C" {

llama_sampler * llama_sampler_init(const llama_sampler_i * iface, llama_sampler_context_t ctx) {
    return new llama_sampler{iface, ctx};
}
const char * llama_sampler_name(const llama_sampler * s) { return s->iface->name ? s->iface->name(s) : "(unnamed)"; }
void llama_sampler_accept(llama_sampler * s, llama_token tok) {
    if (s->iface->accept) s->iface->accept(s, tok);
}
void llama_sampler_apply(llama_sampler * s, llama_token_data_array * cur_p) { s->iface->apply(s, cur_p); }
void llama_sampler_reset(llama_sampler * s) {
    if (s->iface->reset) s->iface->reset(s);
}
llama_sampler * llama_sampler_clone(const llama_sampler * s) {
    if (s->iface->clone) return s->iface->clone(s);
    return s->ctx == nullptr ? llama_sampler_init(s->iface, nullptr) : nullptr;
}
void llama_sampler_free(llama_sampler * s) {
    if (s == nullptr) return;
    if (s->iface->free) s->iface->free(s);
    delete s;
}

llama_sampler_chain_params llama_sampler_chain_default_params(void) { return llama_sampler_chain_params{/*no_perf=*/true}; }
llama_sampler * llama_sampler_chain_init(llama_sampler_chain_params params) {
    auto * c = new ChainCtx();
    c->params = params;
    return llama_sampler_init(&chain_i, c);
}
void llama_sampler_chain_add(llama_sampler * chain, llama_sampler * smpl) {
    if (smpl != nullptr) ((ChainCtx *) chain->ctx)->members.push_back(smpl);
}
llama_sampler * llama_sampler_chain_get(const llama_sampler * chain, int32_t i) {
    auto * c = (const ChainCtx *) chain->ctx;
    return i >= 0 && (size_t) i < c->members.size() ? c->members[i] : nullptr;
}
int llama_sampler_chain_n(const llama_sampler * chain) { return (int) ((const ChainCtx *) chain->ctx)->members.size(); }

llama_sampler * llama_sampler_init_greedy(void) { return llama_sampler_init(&greedy_i, nullptr); }
llama_sampler * llama_sampler_init_dist(uint32_t seed) {
    auto * c = new DistCtx();
    c->seed = seed;
    c->seed_cur = resolve_seed(seed);
    c->rng.seed(c->seed_cur);
    return make(&dist_i, c);
}
llama_sampler * llama_sampler_init_top_k(int32_t k) { return make(&top_k_i, new TopKCtx{k}); }
llama_sampler * llama_sampler_init_top_p(float p, size_t min_keep) { return make(&top_p_i, new PCtx{p, min_keep}); }
llama_sampler * llama_sampler_init_min_p(float p, size_t min_keep) { return make(&min_p_i, new PCtx{p, min_keep}); }
llama_sampler * llama_sampler_init_typical(float p, size_t min_keep) { return make(&typical_i, new PCtx{p, min_keep}); }
llama_sampler * llama_sampler_init_temp(float t) { return make(&temp_i, new TempCtx{t, 0.0f, 1.0f, false}); }
llama_sampler * llama_sampler_init_temp_ext(float t, float delta, float exponent) {
    return make(&temp_i, new TempCtx{t, delta, exponent, true});
}
llama_sampler * llama_sampler_init_xtc(float p, float t, size_t min_keep, uint32_t seed) {
    auto * c = new XtcCtx();
    c->p = p; c->t = t; c->min_keep = min_keep; c->seed = seed;
    c->seed_cur = resolve_seed(seed);
    c->rng.seed(c->seed_cur);
    return make(&xtc_i, c);
}
llama_sampler * llama_sampler_init_penalties(int32_t last_n, float repeat, float freq, float present) {
    auto * c = new PenCtx();
    c->last_n = last_n; c->repeat = repeat; c->freq = freq; c->present = present;
    return make(&pen_i, c);
}
llama_sampler * llama_sampler_init_dry(const llama_vocab * vocab, int32_t n_ctx_train, float multiplier, float base,
                                       int32_t allowed_length, int32_t last_n, const char ** seq_breakers, size_t num_breakers) {
    auto * c = new DryCtx();
    c->n_ctx_train = n_ctx_train; c->multiplier = multiplier; c->base = base;
    c->allowed_length = std::max(allowed_length, 1); c->last_n = last_n;
    if (vocab != nullptr && num_breakers > 0 && multiplier != 0.0f) {
        const int32_t V = llama_vocab_n_tokens(vocab);
        c->is_breaker.assign((size_t) V, 0);
        std::vector<std::string> brk;
        for (size_t i = 0; i < num_breakers; ++i)
            if (seq_breakers[i] != nullptr && seq_breakers[i][0] != 0) brk.emplace_back(seq_breakers[i]);
        char buf[256];
        std::vector<uint8_t> found(brk.size(), 0);
        llama_token ids[64];
        for (int32_t t = 0; t < V && !brk.empty(); ++t) {
            const int32_t len = llama_token_to_piece(vocab, t, buf, (int32_t) sizeof(buf), 0, true);
            if (len <= 0) continue;
            const std::string piece(buf, (size_t) len);
            for (size_t i = 0; i < brk.size(); ++i) {
                const std::string & b = brk[i];
                if (piece.find(b) != std::string::npos) { c->is_breaker[(size_t) t] = 1; found[i] = 1; continue; }
                // the breaker may begin inside this token: the token's last characters are the breaker's first ones, the rest
                // follows as the tokens the remainder tokenises to (the reference's head-token table, src/llama-sampling.cpp:895)
                for (size_t ov = std::min(piece.size(), b.size() - 1); ov >= 1; --ov) {
                    if (piece.compare(piece.size() - ov, ov, b, 0, ov) != 0) continue;
                    const std::string rest = b.substr(ov);
                    const int32_t n = llama_tokenize(vocab, rest.c_str(), (int32_t) rest.size(), ids, 63, false, false);
                    if (n >= 1 && c->multi.size() < 4096) {
                        std::vector<llama_token> seq;
                        seq.push_back(t);
                        seq.insert(seq.end(), ids, ids + n);
                        c->multi.push_back(std::move(seq));
                    }
                    break;                                 // the longest overlap only
                }
            }
        }
        // a breaker that only ever appears spread over several tokens is matched as the token sequence it tokenises to
        // (the reference keeps head token -> tail sequences for the same purpose, src/llama-sampling.cpp:895)
        for (size_t i = 0; i < brk.size(); ++i) {
            if (found[i]) continue;
            const int32_t n = llama_tokenize(vocab, brk[i].c_str(), (int32_t) brk[i].size(), ids, 64, false, false);
            if (n >= 2) c->multi.emplace_back(ids, ids + n);
        }
        for (size_t i = 0; i < c->multi.size(); ++i) c->by_last[c->multi[i].back()].push_back((int32_t) i);
    }
    return llama_sampler_init(&dry_i, c);
}
llama_sampler * llama_sampler_init_logit_bias(int32_t n_vocab, int32_t n_logit_bias, const llama_logit_bias * logit_bias) {
    auto * c = new BiasCtx();
    c->n_vocab = n_vocab;
    if (n_logit_bias > 0 && logit_bias != nullptr) c->bias.assign(logit_bias, logit_bias + n_logit_bias);
    return make(&bias_i, c);
}
llama_sampler * llama_sampler_init_grammar(const llama_vocab * vocab, const char * grammar_str, const char * grammar_root) {
    std::vector<std::string> pieces;
    std::vector<uint8_t> eog;
    llama_token eos = -1;
    const bool has_text = grammar_str != nullptr && std::string(grammar_str).find_first_not_of(" \t\r\n") != std::string::npos;
    if (has_text) {
        if (vocab == nullptr || llama_vocab_n_tokens(vocab) <= 0) {
            fprintf(stderr, "llama_sampler_init_grammar: a grammar needs a vocabulary with token texts\n");
            return nullptr;
        }
        const int32_t V = llama_vocab_n_tokens(vocab);
        pieces.resize((size_t) V);
        eog.assign((size_t) V, 0);
        std::vector<char> buf(512);
        for (int32_t t = 0; t < V; ++t) {
            eog[(size_t) t] = llama_vocab_is_eog(vocab, t) ? 1 : 0;
            int32_t n = llama_token_to_piece(vocab, t, buf.data(), (int32_t) buf.size(), 0, false);
            if (n < 0) {
                buf.resize((size_t) -n);
                n = llama_token_to_piece(vocab, t, buf.data(), (int32_t) buf.size(), 0, false);
            }
            if (n > 0) pieces[(size_t) t].assign(buf.data(), (size_t) n);
        }
        eos = llama_vocab_eos(vocab);
    }
    return grammar_make(std::move(pieces), std::move(eog), eos, grammar_str, grammar_root);
}

// The same sampler from a table of token texts instead of a llama_vocab (used by the Python engine, whose tokenizer is
// not a llama_vocab).  pieces[i] / lens[i]: bytes of token i (length 0 = never allowed); eog: ids that end generation.
MINI_API llama_sampler * jib_sampler_init_grammar_pieces(const char * const * pieces, const int32_t * lens, int32_t n_tokens,
                                                         const llama_token * eog, int32_t n_eog, llama_token eos, const char * grammar_str,
                                                         const char * grammar_root) {
    std::vector<std::string> p((size_t) std::max(n_tokens, 0));
    std::vector<uint8_t> e((size_t) std::max(n_tokens, 0), 0);
    for (int32_t i = 0; i < n_tokens; ++i)
        if (lens[i] > 0) p[(size_t) i].assign(pieces[i], (size_t) lens[i]);
    for (int32_t i = 0; i < n_eog; ++i)
        if (eog[i] >= 0 && eog[i] < n_tokens) e[(size_t) eog[i]] = 1;
    return grammar_make(std::move(p), std::move(e), eos, grammar_str, grammar_root);
}

llama_perf_sampler_data llama_perf_sampler(const llama_sampler * chain) {
    llama_perf_sampler_data d{0.0, 0};
    if (chain == nullptr || chain->iface != &chain_i) return d;
    auto * c = (const ChainCtx *) chain->ctx;
    d.t_sample_ms = c->t_sample_us * 1e-3;
    d.n_sample = c->n_sample;
    return d;
}
void llama_perf_sampler_print(const llama_sampler * chain) {
    const llama_perf_sampler_data d = llama_perf_sampler(chain);
    fprintf(stderr, "sampling time = %10.2f ms / %5d runs (%8.3f ms per token)\n", d.t_sample_ms, d.n_sample,
            d.n_sample ? d.t_sample_ms / d.n_sample : 0.0);
}
void llama_perf_sampler_reset(llama_sampler * chain) {
    if (chain == nullptr || chain->iface != &chain_i) return;
    auto * c = (ChainCtx *) chain->ctx;
    c->t_sample_us = 0;
    c->n_sample = 0;
}

}  // extern "C"
