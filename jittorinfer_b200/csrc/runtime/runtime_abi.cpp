// C ABI over the host runtime (paged KV allocator + scheduler) for the Python engine (ctypes) and
// the llama.h layer.  Handles are opaque pointers; every array is caller-owned.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

#include "kv_paged.h"
#include "scheduler.h"

using namespace jib;

#define JIB_API extern "C" __attribute__((visibility("default")))

struct jib_sched {
    Scheduler sched;
    std::vector<StepEvent> events;
    jib_sched(PagedKv * kv, int n_slots, int n_batch, int n_ctx_slot, int eos, int n_keep, bool cb)
        : sched(kv, n_slots, n_batch, n_ctx_slot, eos, n_keep, cb) {}
};

// ---- paged KV -------------------------------------------------------------------------------
JIB_API PagedKv * jib_kv_create(int n_blocks, int block_size, int max_seqs) { return new PagedKv(n_blocks, block_size, max_seqs); }
JIB_API void jib_kv_destroy(PagedKv * kv) { delete kv; }
JIB_API int jib_kv_append(PagedKv * kv, int seq, int n, int32_t * slots) { return kv->append(seq, n, slots) ? 0 : 1; }
JIB_API int jib_kv_blocks_needed(PagedKv * kv, int seq, int n) { return kv->blocks_needed(seq, n); }
JIB_API int jib_kv_seq_rm(PagedKv * kv, int seq, int p0, int p1) { return kv->seq_rm(seq, p0, p1) ? 1 : 0; }
JIB_API int jib_kv_seq_cp(PagedKv * kv, int src, int dst, int p0, int p1) { return kv->seq_cp(src, dst, p0, p1) ? 1 : 0; }
JIB_API void jib_kv_seq_keep(PagedKv * kv, int seq) { kv->seq_keep(seq); }
JIB_API void jib_kv_clear(PagedKv * kv) { kv->clear(); }
JIB_API int jib_kv_seq_len(PagedKv * kv, int seq) { return kv->seq_len(seq); }
JIB_API int jib_kv_seq_blocks(PagedKv * kv, int seq, int32_t * out, int cap) {
    const auto & b = kv->seq_blocks(seq);
    int n = std::min<int>((int) b.size(), cap);
    if (out) std::memcpy(out, b.data(), n * sizeof(int32_t));
    return (int) b.size();
}
JIB_API int jib_kv_free_blocks(PagedKv * kv) { return kv->free_blocks(); }
JIB_API int jib_kv_used_blocks(PagedKv * kv) { return kv->used_blocks(); }
JIB_API int jib_kv_n_blocks(PagedKv * kv) { return kv->n_blocks(); }
JIB_API int jib_kv_block_size(PagedKv * kv) { return kv->block_size(); }
JIB_API int jib_kv_refcount(PagedKv * kv, int block) { return kv->refcount(block); }
JIB_API float jib_kv_fragmentation(PagedKv * kv) { return kv->fragmentation(); }
JIB_API int jib_kv_check(PagedKv * kv) { return kv->check() ? 1 : 0; }
JIB_API int jib_kv_reserve(PagedKv * kv, int n) { return kv->reserve(n); }
JIB_API void jib_kv_unreserve(PagedKv * kv) { kv->unreserve(); }
JIB_API void jib_kv_track_freed(PagedKv * kv, int on) { kv->track_freed(on != 0); }
// Blocks freed since the last call that are still free; returns the count (at most cap are written).
JIB_API int jib_kv_take_freed(PagedKv * kv, int32_t * out, int cap) {
    const std::vector<int32_t> f = kv->take_freed();
    const int n = std::min<int>((int) f.size(), cap);
    for (int i = 0; i < n; ++i) out[i] = f[i];
    return n;
}
// Pops up to cap queued copy-on-write copies.
JIB_API int jib_kv_take_copies(PagedKv * kv, int32_t * src, int32_t * dst, int cap) {
    auto & p = kv->pending_copies();
    int n = std::min<int>((int) p.size(), cap);
    for (int i = 0; i < n; ++i) { src[i] = p[i].first; dst[i] = p[i].second; }
    p.erase(p.begin(), p.begin() + n);
    return n;
}
JIB_API int jib_kv_defrag(PagedKv * kv, int max_moves, int32_t * src, int32_t * dst) {
    auto m = kv->defrag(max_moves);
    for (size_t i = 0; i < m.size(); ++i) { src[i] = m[i].first; dst[i] = m[i].second; }
    return (int) m.size();
}

// ---- scheduler ------------------------------------------------------------------------------
JIB_API jib_sched * jib_sched_create(PagedKv * kv, int n_slots, int n_batch, int n_ctx_slot, int eos_id, int n_keep,
                                     int cont_batching) {
    return new jib_sched(kv, n_slots, n_batch, n_ctx_slot, eos_id, n_keep, cont_batching != 0);
}
JIB_API void jib_sched_destroy(jib_sched * s) { delete s; }
JIB_API void jib_sched_add(jib_sched * s, int64_t req_id, const int32_t * prompt, int n_prompt, int max_new, int ignore_eos) {
    Request r;
    r.id = req_id;
    r.prompt.assign(prompt, prompt + n_prompt);
    r.max_new = max_new;
    r.ignore_eos = ignore_eos != 0;
    s->sched.add_request(r);
}
// As jib_sched_add, with the request's own n_keep (<0: keep the whole prompt's head when it must be cut).
JIB_API void jib_sched_add_keep(jib_sched * s, int64_t req_id, const int32_t * prompt, int n_prompt, int max_new, int ignore_eos,
                                int n_keep) {
    Request r;
    r.id = req_id;
    r.prompt.assign(prompt, prompt + n_prompt);
    r.max_new = max_new;
    r.ignore_eos = ignore_eos != 0;
    r.n_keep = n_keep;
    s->sched.add_request(r);
}
JIB_API int jib_sched_cancel(jib_sched * s, int64_t req_id) { return s->sched.cancel(req_id, &s->events) ? 1 : 0; }
// info_out: n_tokens, n_seqs, n_out, n_decode_seqs, max_q_len, n_preempted, n_copies
JIB_API int jib_sched_step(jib_sched * s, StepArrays * arrays, int32_t * info_out) {
    StepInfo i = s->sched.step(*arrays);
    info_out[0] = i.n_tokens; info_out[1] = i.n_seqs; info_out[2] = i.n_out; info_out[3] = i.n_decode_seqs;
    info_out[4] = i.max_q_len; info_out[5] = i.n_preempted; info_out[6] = i.n_copies;
    return i.n_tokens;
}
JIB_API void jib_sched_commit(jib_sched * s, const int32_t * sampled, int n_out) { s->sched.commit(sampled, n_out, &s->events); }
JIB_API int jib_sched_can_run_ahead(jib_sched * s) { return s->sched.can_run_ahead() ? 1 : 0; }
JIB_API void jib_sched_commit_deferred(jib_sched * s, int n_out) { s->sched.commit_deferred(n_out); }
JIB_API void jib_sched_resolve(jib_sched * s, const int32_t * sampled, int n_out) { s->sched.resolve(sampled, n_out, &s->events); }
// Pops queued events; each is 6 x int64: req_id, slot, token, finish, n_prompt, n_decoded.
JIB_API int jib_sched_take_events(jib_sched * s, int64_t * out, int cap) {
    int n = std::min<int>((int) s->events.size(), cap);
    for (int i = 0; i < n; ++i) {
        const StepEvent & e = s->events[i];
        int64_t * o = out + 6 * i;
        o[0] = e.req_id; o[1] = e.slot; o[2] = e.token; o[3] = e.finish; o[4] = e.n_prompt; o[5] = e.n_decoded;
    }
    s->events.erase(s->events.begin(), s->events.begin() + n);
    return n;
}
// Request id owning each output row of the last step().
JIB_API int jib_sched_out_reqs(jib_sched * s, int64_t * out, int cap) {
    const auto & v = s->sched.last_out_slots();
    int n = std::min<int>((int) v.size(), cap);
    for (int i = 0; i < n; ++i) out[i] = s->sched.slots()[v[i]].req_id;
    return n;
}
JIB_API int64_t jib_sched_slot_req(jib_sched * s, int slot) { return s->sched.slots()[slot].req_id; }
JIB_API int jib_sched_slot_cached(jib_sched * s, int slot) { return s->sched.slots()[slot].n_cached; }
JIB_API int jib_sched_idle(jib_sched * s) { return s->sched.idle() ? 1 : 0; }
JIB_API int jib_sched_n_waiting(jib_sched * s) { return s->sched.n_waiting(); }
JIB_API int jib_sched_n_running(jib_sched * s) { return s->sched.n_running(); }
JIB_API void jib_sched_set_n_batch(jib_sched * s, int n) { s->sched.set_n_batch(n); }
JIB_API void jib_sched_set_mixed_prompt_budget(jib_sched * s, int n) { s->sched.set_mixed_prompt_budget(n); }
JIB_API int jib_sched_slot_state(jib_sched * s, int slot) { return s->sched.slots()[slot].state; }
// stats_out (7 values): steps, prompt_tokens, decode_tokens, preemptions, finished, prefix_hits, prefix_shared
JIB_API void jib_sched_stats(jib_sched * s, int64_t * o) {
    const SchedStats & st = s->sched.stats();
    o[0] = st.steps; o[1] = st.prompt_tokens; o[2] = st.decode_tokens; o[3] = st.preemptions; o[4] = st.finished; o[5] = st.prefix_hits;
    o[6] = st.prefix_shared;
}

// ---- tokenizer ------------------------------------------------------------------------------
#include "tokenizer.h"

JIB_API Tokenizer * jib_tok_create(const char ** tokens, const int32_t * token_lens, const int32_t * types, int n_tokens,
                                   const char ** merges, const int32_t * merge_lens, int n_merges, int bos, int eos, int eot,
                                   int add_bos, int add_eos) {
    std::vector<std::string> toks(n_tokens), mg(n_merges);
    for (int i = 0; i < n_tokens; ++i) toks[i].assign(tokens[i], token_lens[i]);
    for (int i = 0; i < n_merges; ++i) mg[i].assign(merges[i], merge_lens[i]);
    std::vector<int32_t> ty(types ? types : nullptr, types ? types + n_tokens : nullptr);
    TokenizerConfig cfg;
    cfg.bos = bos; cfg.eos = eos; cfg.eot = eot; cfg.add_bos = add_bos != 0; cfg.add_eos = add_eos != 0;
    return new Tokenizer(std::move(toks), std::move(ty), mg, cfg);
}
JIB_API void jib_tok_destroy(Tokenizer * t) { delete t; }
// Returns the token count; writes at most cap ids (call again with a larger buffer if the count exceeds cap).
JIB_API int jib_tok_encode(Tokenizer * t, const char * text, int len, int add_special, int parse_special, int32_t * out, int cap) {
    const std::vector<int32_t> ids = t->encode(std::string(text, len), add_special != 0, parse_special != 0);
    const int n = std::min<int>((int) ids.size(), cap);
    if (out && n > 0) std::memcpy(out, ids.data(), n * sizeof(int32_t));
    return (int) ids.size();
}
JIB_API int jib_tok_piece(Tokenizer * t, int32_t id, int special, char * buf, int cap) {
    const std::string s = t->token_to_piece(id, special != 0);
    const int n = std::min<int>((int) s.size(), cap);
    if (buf && n > 0) std::memcpy(buf, s.data(), n);
    return (int) s.size();
}
JIB_API int jib_tok_decode(Tokenizer * t, const int32_t * ids, int n_ids, int remove_special, int unparse_special, char * buf, int cap) {
    const std::string s = t->decode(std::vector<int32_t>(ids, ids + n_ids), remove_special != 0, unparse_special != 0);
    const int n = std::min<int>((int) s.size(), cap);
    if (buf && n > 0) std::memcpy(buf, s.data(), n);
    return (int) s.size();
}
JIB_API int jib_tok_is_eog(Tokenizer * t, int32_t id) { return t->is_eog(id) ? 1 : 0; }
JIB_API int jib_tok_n_tokens(Tokenizer * t) { return t->n_tokens(); }
JIB_API int jib_tok_bos(Tokenizer * t) { return t->config().bos; }
JIB_API int jib_tok_eos(Tokenizer * t) { return t->config().eos; }
JIB_API int jib_tok_eot(Tokenizer * t) { return t->config().eot; }
JIB_API int jib_utf8_incomplete_tail(const char * s, int len) { return (int) utf8_incomplete_tail(std::string(s, len)); }

// ---- GGUF reader ------------------------------------------------------------------------------
#include "dequant.h"
#include "gguf.h"

#include <cmath>
#include <cstdio>
#include <string>

namespace {

void json_escape(const std::string & in, std::string & out) {
    out.push_back('"');
    for (unsigned char c : in) {
        switch (c) {
            case '"': out += "\\\""; break;
            case '\\': out += "\\\\"; break;
            case '\n': out += "\\n"; break;
            case '\r': out += "\\r"; break;
            case '\t': out += "\\t"; break;
            default:
                if (c < 0x20) {
                    char buf[8];
                    snprintf(buf, sizeof(buf), "\\u%04x", c);
                    out += buf;
                } else {
                    out.push_back((char) c);
                }
        }
    }
    out.push_back('"');
}

void json_number(double v, bool is_float, std::string & out) {
    char buf[40];
    if (!is_float) {
        snprintf(buf, sizeof(buf), "%lld", (long long) v);
    } else if (std::isfinite(v)) {
        snprintf(buf, sizeof(buf), "%.17g", v);
    } else {
        snprintf(buf, sizeof(buf), "null");
    }
    out += buf;
}

template <typename T>
void json_array(const uint8_t * p, uint64_t n, bool is_float, std::string & out) {
    out.push_back('[');
    for (uint64_t i = 0; i < n; ++i) {
        T v;
        memcpy(&v, p + i * sizeof(T), sizeof(T));
        if (i) out.push_back(',');
        json_number((double) v, is_float, out);
    }
    out.push_back(']');
}

std::string kv_to_json(const GgufFile & f) {
    std::string out = "{";
    bool first = true;
    for (const auto & it : f.kv()) {
        if (!first) out.push_back(',');
        first = false;
        json_escape(it.first, out);
        out.push_back(':');
        const GgufValue & v = it.second;
        if (v.type == GT_STR) {
            json_escape(v.s, out);
        } else if (v.type == GT_ARR) {
            if (v.arr_type == GT_STR) {
                out.push_back('[');
                for (size_t i = 0; i < v.arr_s.size(); ++i) {
                    if (i) out.push_back(',');
                    json_escape(v.arr_s[i], out);
                }
                out.push_back(']');
            } else {
                switch (v.arr_type) {
                    case GT_U8: case GT_BOOL: json_array<uint8_t>(v.arr_data, v.arr_n, false, out); break;
                    case GT_I8: json_array<int8_t>(v.arr_data, v.arr_n, false, out); break;
                    case GT_U16: json_array<uint16_t>(v.arr_data, v.arr_n, false, out); break;
                    case GT_I16: json_array<int16_t>(v.arr_data, v.arr_n, false, out); break;
                    case GT_U32: json_array<uint32_t>(v.arr_data, v.arr_n, false, out); break;
                    case GT_I32: json_array<int32_t>(v.arr_data, v.arr_n, false, out); break;
                    case GT_U64: json_array<uint64_t>(v.arr_data, v.arr_n, false, out); break;
                    case GT_I64: json_array<int64_t>(v.arr_data, v.arr_n, false, out); break;
                    case GT_F32: json_array<float>(v.arr_data, v.arr_n, true, out); break;
                    case GT_F64: json_array<double>(v.arr_data, v.arr_n, true, out); break;
                    default: out += "null";
                }
            }
        } else if (v.type == GT_BOOL) {
            out += v.u ? "true" : "false";
        } else if (v.type == GT_F32 || v.type == GT_F64) {
            json_number(v.f, true, out);
        } else {
            json_number((double) (int64_t) v.u, false, out);
        }
    }
    out.push_back('}');
    return out;
}

}  // namespace

struct jib_gguf {
    GgufFile file;
    std::string kv_json;
};

// Opens and parses a GGUF file.  On failure returns NULL and writes the reason (NUL-terminated) into err.
JIB_API jib_gguf * jib_gguf_open(const char * path, int populate, char * err, int err_cap) {
    jib_gguf * g = new jib_gguf();
    const std::string e = g->file.open(path ? path : "", populate != 0);
    if (!e.empty()) {
        if (err != nullptr && err_cap > 0) snprintf(err, (size_t) err_cap, "%s", e.c_str());
        delete g;
        return nullptr;
    }
    return g;
}
JIB_API void jib_gguf_close(jib_gguf * g) { delete g; }

// Expands block-quantised tensor data to float (dst_bf16 == 0) or bf16.  0 ok, -1 type not handled, -2 partial block.
JIB_API int jib_dequantize(uint32_t ggml_type, const void * src, uint64_t n_elements, void * dst, int dst_bf16, int n_threads) {
    if ((src == nullptr || dst == nullptr) && n_elements != 0) return -3;
    return jib::dequantize(ggml_type, src, n_elements, dst, dst_bf16 != 0, n_threads);
}
JIB_API int jib_dequantize_elementwise(uint32_t ggml_type, const void * src, uint64_t n_elements, float * dst) {
    if ((src == nullptr || dst == nullptr) && n_elements != 0) return -3;
    return jib::dequantize_elementwise(ggml_type, src, n_elements, dst);
}
JIB_API uint64_t jib_quant_block_elems(uint32_t ggml_type) { return jib::quant_block_elems(ggml_type); }
JIB_API uint64_t jib_quant_block_bytes(uint32_t ggml_type) { return jib::quant_block_bytes(ggml_type); }
JIB_API int jib_gguf_version(jib_gguf * g) { return (int) g->file.version(); }
JIB_API int jib_gguf_alignment(jib_gguf * g) { return (int) g->file.alignment(); }
JIB_API int64_t jib_gguf_n_tensors(jib_gguf * g) { return (int64_t) g->file.tensors().size(); }
// Tensor i: name (NUL-terminated, truncated to name_cap), ne[0..nd) in ggml order, ggml type, byte size, data pointer
// into the read-only mapping (valid until close).  Returns the number of dimensions, or -1.
JIB_API int jib_gguf_tensor_info(jib_gguf * g, int64_t i, char * name, int name_cap, uint64_t * ne, uint32_t * type, uint64_t * nbytes,
                                 const void ** data) {
    if (i < 0 || (size_t) i >= g->file.tensors().size()) return -1;
    const GgufTensor & t = g->file.tensors()[(size_t) i];
    if (name != nullptr && name_cap > 0) snprintf(name, (size_t) name_cap, "%s", t.name.c_str());
    for (size_t d = 0; d < t.ne.size() && d < 8; ++d) ne[d] = t.ne[d];
    *type = t.type;
    *nbytes = t.nbytes;
    *data = g->file.tensor_data(t);
    return (int) t.ne.size();
}
// All key/value pairs as one JSON object (UTF-8).  Returns the byte length; copies min(length, cap) bytes.
JIB_API int64_t jib_gguf_kv_json(jib_gguf * g, char * buf, int64_t cap) {
    if (g->kv_json.empty()) g->kv_json = kv_to_json(g->file);
    if (buf != nullptr && cap > 0) memcpy(buf, g->kv_json.data(), (size_t) std::min<int64_t>(cap, (int64_t) g->kv_json.size()));
    return (int64_t) g->kv_json.size();
}
