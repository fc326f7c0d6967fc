// libllama.so: sections 2-7 and 9 of llama.h (parameters, model, context, batch/decode, KV, vocabulary, chat, timings).
//
// Mapping onto the reference: llama_model_load_from_file (src/llama-model-load-utils.cpp:13-73) reads the GGUF
// natively (metadata, vocabulary, chat templates) and asks the Python backend to put the weights on the GPU;
// llama_init_from_model (src/llama-context-load-utils.cpp:32-190) creates the paged latent cache; llama_decode
// (src/llama-execute-decode.cpp:156-344) turns the batch into per-sequence appends on the block allocator and packs
// one step descriptor per n_ubatch chunk; the KV functions (src/llama-kv-cache.cpp:182-345) act on block tables.
#include "capi_internal.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <numeric>

namespace {

double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

void log_err(const char * where, const std::string & msg) { fprintf(stderr, "%s: %s\n", where, msg.c_str()); }

int64_t kv_i64(const jib::GgufFile & g, const std::string & key, int64_t dflt) {
    const jib::GgufValue * v = g.find(key);
    return v != nullptr && v->type != jib::GT_STR && v->type != jib::GT_ARR ? v->as_i64() : dflt;
}

std::string kv_str(const jib::GgufFile & g, const std::string & key, const std::string & dflt) {
    const jib::GgufValue * v = g.find(key);
    return v != nullptr && v->type == jib::GT_STR ? v->s : dflt;
}

// vocabulary from tokenizer.ggml.* (reference: llama_vocab::impl::load, src/llama-vocab.cpp:430-560)
std::string load_vocab(const jib::GgufFile & g, llama_vocab & v, int32_t n_vocab_hparam) {
    const jib::GgufValue * toks = g.find("tokenizer.ggml.tokens");
    v.bos = (int32_t) kv_i64(g, "tokenizer.ggml.bos_token_id", 11);
    v.eos = (int32_t) kv_i64(g, "tokenizer.ggml.eos_token_id", 11);
    v.sep = (int32_t) kv_i64(g, "tokenizer.ggml.seperator_token_id", -1);
    v.add_bos = kv_i64(g, "tokenizer.ggml.add_bos_token", 0) != 0;
    v.add_eos = kv_i64(g, "tokenizer.ggml.add_eos_token", 0) != 0;
    if (toks == nullptr || toks->type != jib::GT_ARR || toks->arr_type != jib::GT_STR) {
        v.n_tokens = n_vocab_hparam;          // token ids only
        return "";
    }
    const std::string model = kv_str(g, "tokenizer.ggml.model", "gpt2");
    const std::string pre = kv_str(g, "tokenizer.ggml.pre", "deepseek-llm");
    if (model != "gpt2" || pre != "deepseek-llm")
        return "unsupported tokenizer " + model + "/" + pre + " (only gpt2 BPE with the deepseek-llm pre-tokenizer)";
    std::vector<int32_t> types;
    if (const jib::GgufValue * tt = g.find("tokenizer.ggml.token_type")) {
        if (tt->type == jib::GT_ARR && (tt->arr_type == jib::GT_I32 || tt->arr_type == jib::GT_U32)) {
            types.resize(tt->arr_n);
            memcpy(types.data(), tt->arr_data, tt->arr_n * 4);
        }
    }
    types.resize(toks->arr_s.size(), jib::TOK_NORMAL);
    std::vector<std::string> merges;
    if (const jib::GgufValue * m = g.find("tokenizer.ggml.merges"))
        if (m->type == jib::GT_ARR && m->arr_type == jib::GT_STR) merges = m->arr_s;
    jib::TokenizerConfig cfg;
    cfg.bos = v.bos;
    cfg.eos = v.eos;
    cfg.eot = (int32_t) kv_i64(g, "tokenizer.ggml.eot_token_id", -1);
    cfg.pad = (int32_t) kv_i64(g, "tokenizer.ggml.padding_token_id", -1);
    cfg.add_bos = v.add_bos;
    cfg.add_eos = v.add_eos;
    v.tok.reset(new jib::Tokenizer(toks->arr_s, types, merges, cfg));
    v.n_tokens = v.tok->n_tokens();
    return "";
}

int copy_out(const std::string & s, char * buf, int32_t cap) {
    if ((int64_t) s.size() > (int64_t) cap) return -(int) s.size();
    if (!s.empty()) memcpy(buf, s.data(), s.size());
    return (int) s.size();
}

}  // namespace

extern "C" {

// ---- 2. parameters ----------------------------------------------------------------------------------------------------
llama_model_params llama_model_default_params(void) {
    llama_model_params p;
    memset(&p, 0, sizeof(p));
    p.n_gpu_layers = 999;
    p.split_mode = LLAMA_SPLIT_MODE_NONE;
    p.enable_mla = true;
    p.enable_fused_moe = true;
    p.num_parallel = 1;
    p.use_mmap = true;
    return p;
}

llama_context_params llama_context_default_params(void) {
    llama_context_params p;
    memset(&p, 0, sizeof(p));
    p.n_ctx = 4096;
    p.n_batch = 2048;
    p.n_ubatch = 2048;
    p.n_seq_max = 8;
    p.n_threads = 1;
    p.n_threads_batch = 1;
    p.rope_scaling_type = LLAMA_ROPE_SCALING_TYPE_UNSPECIFIED;
    p.pooling_type = LLAMA_POOLING_TYPE_UNSPECIFIED;
    p.attention_type = LLAMA_ATTENTION_TYPE_UNSPECIFIED;
    p.yarn_ext_factor = -1.0f;
    p.yarn_attn_factor = 1.0f;
    p.yarn_beta_fast = 32.0f;
    p.yarn_beta_slow = 1.0f;
    p.defrag_thold = -1.0f;
    p.type_k = GGML_TYPE_BF16;
    p.type_v = GGML_TYPE_BF16;
    p.offload_kqv = true;
    p.flash_attn = true;
    p.no_perf = false;
    p.presample_count = -1;
    return p;
}

// ---- 3. backend, model, context -------------------------------------------------------------------------------------------
void llama_backend_init(void) {}
void llama_backend_free(void) { jib::PyBridge::shutdown(); }
bool llama_supports_gpu_offload(void) { return true; }
bool llama_supports_rpc(void) { return false; }

llama_model * llama_model_load_from_file(const char * path_model, llama_model_params params) {
    const double t0 = now_ms();
    std::unique_ptr<llama_model> m(new llama_model());
    m->path = path_model ? path_model : "";
    m->params = params;
    const std::string err = m->gguf.open(m->path, false);
    if (!err.empty()) { log_err("llama_model_load_from_file", err); return nullptr; }
    const std::string arch = kv_str(m->gguf, "general.architecture", "");
    if (arch != "deepseek2") { log_err("llama_model_load_from_file", "unsupported architecture '" + arch + "' (deepseek2 only)"); return nullptr; }
    m->n_layer = (int32_t) kv_i64(m->gguf, "deepseek2.block_count", 0);
    m->n_ctx_train = (int32_t) kv_i64(m->gguf, "deepseek2.context_length", 0);
    m->n_embd = (int32_t) kv_i64(m->gguf, "deepseek2.embedding_length", 0);
    m->kv_row = (int32_t) (kv_i64(m->gguf, "deepseek2.attention.kv_lora_rank", 0) + kv_i64(m->gguf, "deepseek2.rope.dimension_count", 0));
    int32_t n_vocab = (int32_t) kv_i64(m->gguf, "deepseek2.vocab_size", 0);
    if (n_vocab == 0)
        if (const jib::GgufTensor * te = m->gguf.tensor("token_embd.weight"))
            if (te->ne.size() == 2) n_vocab = (int32_t) te->ne[1];
    const std::string verr = load_vocab(m->gguf, m->vocab, n_vocab);
    if (!verr.empty()) { log_err("llama_model_load_from_file", verr); return nullptr; }
    for (const auto & kv : m->gguf.kv()) {
        static const std::string key = "tokenizer.chat_template";
        if (kv.second.type != jib::GT_STR || kv.first.compare(0, key.size(), key) != 0) continue;
        m->templates[kv.first.size() > key.size() ? kv.first.substr(key.size() + 1) : ""] = kv.second.s;
    }
    if (!params.vocab_only) {
        if (params.progress_callback && !params.progress_callback(0.0f, params.progress_callback_user_data)) return nullptr;
        std::string perr;
        const bool tp = params.enable_tensor_parallel || params.split_mode == LLAMA_SPLIT_MODE_ROW;
        // LLAMA_SPLIT_MODE_LAYER in a single process: consecutive layer ranges over the visible GPUs, in the proportions of
        // tensor_split (up to 8 entries; NULL = even).  Passed as a comma-separated string.
        std::string split;
        if (!tp && params.split_mode == LLAMA_SPLIT_MODE_LAYER) {
            split = "even";
            if (params.tensor_split != nullptr) {
                split.clear();
                for (int i = 0; i < 8; ++i) split += (i ? "," : "") + std::to_string(params.tensor_split[i]);
            }
        }
        // metadata overrides (the list ends at an empty key), as a JSON object for the loader
        std::string ov = "{";
        for (const llama_model_kv_override * o = params.kv_overrides; o != nullptr && o->key[0] != 0; ++o) {
            if (ov.size() > 1) ov += ",";
            ov += "\"" + std::string(o->key, strnlen(o->key, sizeof(o->key))) + "\":";
            switch (o->tag) {
                case LLAMA_KV_OVERRIDE_TYPE_INT: ov += std::to_string((long long) o->val_i64); break;
                case LLAMA_KV_OVERRIDE_TYPE_FLOAT: { char b[40]; snprintf(b, sizeof(b), "%.17g", o->val_f64); ov += b; break; }
                case LLAMA_KV_OVERRIDE_TYPE_BOOL: ov += o->val_bool ? "true" : "false"; break;
                case LLAMA_KV_OVERRIDE_TYPE_STR: {
                    ov += "\"";
                    for (size_t i = 0; i < strnlen(o->val_str, sizeof(o->val_str)); ++i) {
                        const char ch = o->val_str[i];
                        if (ch == '"' || ch == '\\') ov += '\\';
                        if ((unsigned char) ch >= 0x20) ov += ch;
                    }
                    ov += "\"";
                    break;
                }
            }
        }
        ov += "}";
        if (!jib::PyBridge::call("load_model", &m->py, &perr, "(siiiiiiiss)", m->path.c_str(), params.n_gpu_layers > 0 ? 1 : 0,
                                 params.main_gpu, tp ? params.tp_id : 0, tp ? std::max(params.num_parallel, 1) : 1,
                                 params.enable_expert_parallel ? 1 : 0, params.check_tensors ? 1 : 0,
                                 params.enable_data_parallel ? 1 : 0, split.c_str(), ov.c_str())) {
            log_err("llama_model_load_from_file", perr);
            return nullptr;
        }
        if (params.progress_callback) params.progress_callback(1.0f, params.progress_callback_user_data);
    }
    m->t_load_ms = now_ms() - t0;
    return m.release();
}

void llama_model_free(llama_model * model) {
    if (model == nullptr) return;
    if (model->py != 0) jib::PyBridge::call("free_model", nullptr, nullptr, "(L)", model->py);
    delete model;
}

const llama_vocab * llama_model_get_vocab(const llama_model * model) { return &model->vocab; }
llama_rope_type llama_model_rope_type(const llama_model *) { return LLAMA_ROPE_TYPE_NORM; }   // adjacent pairs
int32_t llama_model_n_ctx_train(const llama_model * model) { return model->n_ctx_train; }
bool llama_model_is_recurrent(const llama_model *) { return false; }
bool llama_model_has_encoder(const llama_model *) { return false; }
bool llama_model_has_decoder(const llama_model *) { return true; }
llama_token llama_model_decoder_start_token(const llama_model *) { return LLAMA_TOKEN_NULL; }
const char * llama_model_chat_template(const llama_model * model, const char * name) {
    auto it = model->templates.find(name ? name : "");
    return it == model->templates.end() ? nullptr : it->second.c_str();
}

llama_context * llama_init_from_model(llama_model * model, llama_context_params params) {
    if (model == nullptr || model->py == 0) {
        log_err("llama_init_from_model", "the model was loaded with vocab_only or failed to load");
        return nullptr;
    }
    std::unique_ptr<llama_context> c(new llama_context());
    c->model = model;
    c->params = params;
    if (c->params.n_ctx == 0) c->params.n_ctx = (uint32_t) model->n_ctx_train;
    if (c->params.n_seq_max == 0) c->params.n_seq_max = 1;
    if (c->params.n_batch == 0) c->params.n_batch = 2048;
    if (c->params.n_ubatch == 0 || c->params.n_ubatch > c->params.n_batch) c->params.n_ubatch = c->params.n_batch;
    // every sequence may end in a partially filled block, so n_ctx tokens need up to n_seq_max extra blocks
    const int n_blocks = (int) ((c->params.n_ctx + c->block_size - 1) / c->block_size + c->params.n_seq_max);
    c->kv.reset(new jib::PagedKv(n_blocks, c->block_size, (int) c->params.n_seq_max));
    std::string err;
    // RoPE overrides of the context parameters (0 / negative = keep the model's values)
    char rope[160];
    snprintf(rope, sizeof(rope), "{\"freq_base\":%.9g,\"freq_scale\":%.9g,\"attn_factor\":%.9g,\"orig_ctx\":%u,\"scaling_type\":%d}",
             (double) params.rope_freq_base, (double) params.rope_freq_scale, (double) params.yarn_attn_factor, params.yarn_orig_ctx,
             (int) params.rope_scaling_type);
    if (!jib::PyBridge::call("create_context", &c->py, &err, "(Liiiis)", model->py, n_blocks, c->block_size,
                             c->params.presample_count, (int) c->params.n_ctx, rope)) {
        log_err("llama_init_from_model", err);
        return nullptr;
    }
    c->abort_cb = params.abort_callback;
    c->abort_data = params.abort_callback_data;
    c->t_start_ms = now_ms();
    return c.release();
}

void llama_free(llama_context * ctx) {
    if (ctx == nullptr) return;
    if (ctx->py != 0) jib::PyBridge::call("free_context", nullptr, nullptr, "(L)", ctx->py);
    delete ctx;
}

const llama_model * llama_get_model(const llama_context * ctx) { return ctx->model; }
uint32_t llama_n_ctx(const llama_context * ctx) { return ctx->params.n_ctx; }
uint32_t llama_n_batch(const llama_context * ctx) { return ctx->params.n_batch; }
enum llama_pooling_type llama_pooling_type(const llama_context *) { return LLAMA_POOLING_TYPE_NONE; }
void llama_set_embeddings(llama_context * ctx, bool embeddings) { ctx->params.embeddings = embeddings; }
void llama_set_abort_callback(llama_context * ctx, ggml_abort_callback cb, void * data) {
    ctx->abort_cb = cb;
    ctx->abort_data = data;
}
void llama_attach_threadpool(llama_context *, ggml_threadpool_t, ggml_threadpool_t) {}
void llama_clear_adapter_lora(llama_context *) {}
int32_t llama_set_adapter_lora(llama_context *, llama_adapter_lora *, float) { return -1; }

// ---- 4. batch, decode, logits ---------------------------------------------------------------------------------------------
llama_batch llama_batch_get_one(llama_token * tokens, int32_t n_tokens) {
    llama_batch b;
    memset(&b, 0, sizeof(b));
    b.n_tokens = n_tokens;
    b.token = tokens;
    return b;
}

llama_batch llama_batch_init(int32_t n_tokens, int32_t embd, int32_t n_seq_max) {
    llama_batch b;
    memset(&b, 0, sizeof(b));
    if (embd != 0) {
        b.embd = (float *) calloc((size_t) n_tokens * embd, sizeof(float));
    } else {
        b.token = (llama_token *) calloc((size_t) n_tokens, sizeof(llama_token));
    }
    b.pos = (llama_pos *) calloc((size_t) n_tokens, sizeof(llama_pos));
    b.n_seq_id = (int32_t *) calloc((size_t) n_tokens, sizeof(int32_t));
    b.seq_id = (llama_seq_id **) calloc((size_t) n_tokens + 1, sizeof(llama_seq_id *));      // NULL-terminated
    for (int32_t i = 0; i < n_tokens; ++i) b.seq_id[i] = (llama_seq_id *) calloc((size_t) std::max(n_seq_max, 1), sizeof(llama_seq_id));
    b.logits = (int8_t *) calloc((size_t) n_tokens, sizeof(int8_t));
    return b;
}

void llama_batch_free(llama_batch b) {
    free(b.token);
    free(b.embd);
    free(b.pos);
    free(b.n_seq_id);
    if (b.seq_id != nullptr) {
        for (int32_t i = 0; b.seq_id[i] != nullptr; ++i) free(b.seq_id[i]);
        free(b.seq_id);
    }
    free(b.logits);
}

static bool flush_block_copies(llama_context * ctx) {
    auto & pend = ctx->kv->pending_copies();
    if (pend.empty()) return true;
    std::vector<int32_t> flat;
    for (const auto & pr : pend) { flat.push_back(pr.first); flat.push_back(pr.second); }
    pend.clear();
    std::string err;
    if (!jib::PyBridge::call("copy_blocks", nullptr, &err, "(LLi)", ctx->py, (long long) (intptr_t) flat.data(), (int) flat.size() / 2)) {
        log_err("kv block copy", err);
        return false;
    }
    return true;
}

int32_t llama_decode(llama_context * ctx, llama_batch batch, bool sync_all_servers) {
    const int n = batch.n_tokens;
    if (ctx == nullptr || n <= 0 || batch.token == nullptr) { log_err("llama_decode", "empty batch or embeddings input (token ids only)"); return -1; }
    if ((uint32_t) n > ctx->params.n_batch) { log_err("llama_decode", "batch larger than n_batch"); return -1; }
    jib::PagedKv & kv = *ctx->kv;
    const int n_vocab = ctx->model->vocab.n_tokens;
    std::vector<int> seq(n, 0), want(n, 0);
    for (int i = 0; i < n; ++i) {
        if (batch.token[i] < 0 || batch.token[i] >= n_vocab) { log_err("llama_decode", "token id out of range"); return -1; }
        if (batch.n_seq_id != nullptr && batch.seq_id != nullptr) {
            if (batch.n_seq_id[i] != 1) { log_err("llama_decode", "a token must belong to exactly one sequence (share prefixes with llama_kv_cache_seq_cp)"); return -1; }
            seq[i] = batch.seq_id[i][0];
        }
        if (seq[i] < 0 || seq[i] >= kv.max_seqs()) { log_err("llama_decode", "sequence id out of range (n_seq_max)"); return -1; }
        want[i] = batch.logits != nullptr ? batch.logits[i] != 0 : (ctx->params.logits_all || i == n - 1);
    }
    std::vector<int> order(n);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return seq[a] < seq[b]; });
    // positions: every sequence continues where it ends; a batch that restarts earlier first drops the tail
    std::vector<int> pos(n);
    for (int a = 0; a < n;) {
        int b = a;
        while (b < n && seq[order[b]] == seq[order[a]]) ++b;
        const int s = seq[order[a]];
        int base = kv.seq_len(s);
        if (batch.pos != nullptr) {
            const int p0 = batch.pos[order[a]];
            if (p0 < 0 || p0 > base) { log_err("llama_decode", "positions leave a gap after the cached tokens of a sequence"); return -1; }
            if (p0 < base) { kv.seq_rm(s, p0, -1); base = p0; }
            for (int j = a; j < b; ++j)
                if (batch.pos[order[j]] != base + (j - a)) { log_err("llama_decode", "positions of a sequence must be consecutive"); return -1; }
        }
        for (int j = a; j < b; ++j) pos[order[j]] = base + (j - a);
        a = b;
    }
    // capacity: all or nothing for the appends (a tail that the batch's positions dropped above stays dropped)
    {
        int need = 0;
        for (int a = 0; a < n;) {
            int b = a;
            while (b < n && seq[order[b]] == seq[order[a]]) ++b;
            need += kv.blocks_needed(seq[order[a]], b - a);
            a = b;
        }
        if (need > kv.free_blocks()) return 1;
    }
    const bool topk = ctx->params.presample_count > 0;
    const int64_t len = topk ? std::min<int64_t>(ctx->params.presample_count, n_vocab) : n_vocab;
    const int64_t n_out = std::accumulate(want.begin(), want.end(), (int64_t) 0);
    ctx->out_len = len;
    ctx->n_out = n_out;
    ctx->out_values.resize((size_t) (n_out * len));
    ctx->out_indices.resize(topk ? (size_t) (n_out * len) : 0);
    ctx->row_of_token.assign(n, -1);

    const int n_ub = (int) ctx->params.n_ubatch;
    int64_t row = 0;
    std::vector<int32_t> buf, slots;
    for (int c0 = 0; c0 < n; c0 += n_ub) {
        if (ctx->abort_cb != nullptr && ctx->abort_cb(ctx->abort_data)) return 2;
        const int c1 = std::min(n, c0 + n_ub), T = c1 - c0;
        // segments of this chunk
        struct Seg { int s, a, b; };
        std::vector<Seg> segs;
        for (int a = c0; a < c1;) {
            int b = a;
            while (b < c1 && seq[order[b]] == seq[order[a]]) ++b;
            segs.push_back({seq[order[a]], a, b});
            a = b;
        }
        const int B = (int) segs.size();
        slots.assign(T, -1);
        int max_q = 1;
        for (const Seg & g : segs) {
            if (!kv.append(g.s, g.b - g.a, slots.data() + (g.a - c0))) { log_err("llama_decode", "KV append failed after the capacity check"); return -3; }
            max_q = std::max(max_q, g.b - g.a);
        }
        int max_blocks = 1;
        for (const Seg & g : segs) max_blocks = std::max(max_blocks, (int) kv.seq_blocks(g.s).size());
        int n_out_c = 0;
        for (int j = c0; j < c1; ++j) n_out_c += want[order[j]];
        // [tokens T | positions T | slot_mapping T | out_rows n_out_c | seq_lens B | q_start B+1 | block_tables B*max_blocks]
        buf.assign((size_t) (3 * T + n_out_c + B + B + 1 + B * max_blocks), 0);
        int32_t * p_tok = buf.data(), * p_pos = p_tok + T, * p_slot = p_pos + T, * p_out = p_slot + T;
        int32_t * p_len = p_out + n_out_c, * p_qs = p_len + B, * p_bt = p_qs + B + 1;
        int k = 0;
        for (int j = c0; j < c1; ++j) {
            const int i = order[j];
            p_tok[j - c0] = batch.token[i];
            p_pos[j - c0] = pos[i];
            p_slot[j - c0] = slots[j - c0];
            if (want[i]) { p_out[k] = j - c0; ctx->row_of_token[i] = (int32_t) (row + k); ++k; }
        }
        for (int g = 0; g < B; ++g) {
            p_len[g] = kv.seq_len(segs[g].s);
            p_qs[g] = segs[g].a - c0;
            const std::vector<int32_t> & bl = kv.seq_blocks(segs[g].s);
            std::copy(bl.begin(), bl.end(), p_bt + (size_t) g * max_blocks);
        }
        p_qs[B] = T;
        if (!flush_block_copies(ctx)) return -4;
        const double t0 = now_ms();
        std::string err;
        long long rc = 0;
        float * out_v = ctx->out_values.data() + row * len;
        int64_t * out_i = topk ? ctx->out_indices.data() + row * len : nullptr;
        if (!jib::PyBridge::call("forward", &rc, &err, "(LLiiiiiLLi)", ctx->py, (long long) (intptr_t) buf.data(), T, B, max_blocks, n_out_c,
                                 max_q, (long long) (intptr_t) out_v, (long long) (intptr_t) out_i, sync_all_servers ? 1 : 0)) {
            log_err("llama_decode", err);
            return -2;
        }
        if (sync_all_servers) ctx->all_processed = (int) rc;
        const double dt = now_ms() - t0;
        if (max_q > 1) { ctx->t_p_eval_ms += dt; ctx->n_p_eval += T; } else { ctx->t_eval_ms += dt; ctx->n_eval += T; }
        row += n_out_c;
    }
    return 0;
}

int32_t llama_encode(llama_context *, llama_batch) { return -1; }

bool llama_empty_run(llama_context * ctx) {
    long long rc = 0;
    std::string err;
    if (!jib::PyBridge::call("empty_run", &rc, &err, "(L)", ctx->py)) { log_err("llama_empty_run", err); return false; }
    ctx->all_processed = (int) rc;
    return true;
}

int llama_all_processed_tokens(const llama_context * ctx) { return ctx->all_processed; }

void llama_synchronize(llama_context * ctx) { jib::PyBridge::call("synchronize", nullptr, nullptr, "(L)", ctx->py); }

llama_logits llama_get_logits_ith(llama_context * ctx, int32_t i) {
    llama_logits r;
    r.type = ctx->params.presample_count > 0 ? LLAMA_LOGITS_TYPE_TOPK : LLAMA_LOGITS_TYPE_RAW;
    r.values = nullptr;
    r.indices = nullptr;
    r.len = -1;
    r.num = -1;
    int64_t row = -1;
    if (i < 0) {
        row = ctx->n_out + i;
    } else if ((size_t) i < ctx->row_of_token.size()) {
        row = ctx->row_of_token[i];
    }
    if (row < 0 || row >= ctx->n_out) {
        log_err("llama_get_logits_ith", "no output was requested for this batch index");
        return r;
    }
    r.len = ctx->out_len;
    r.num = ctx->n_out - row;
    r.values = ctx->out_values.data() + row * ctx->out_len;
    if (r.type == LLAMA_LOGITS_TYPE_TOPK) r.indices = ctx->out_indices.data() + row * ctx->out_len;
    return r;
}

// ---- 5. KV cache -------------------------------------------------------------------------------------------------------------
bool llama_kv_cache_seq_rm(llama_context * ctx, llama_seq_id seq_id, llama_pos p0, llama_pos p1) {
    jib::PagedKv & kv = *ctx->kv;
    if (seq_id >= kv.max_seqs()) return false;
    if (seq_id >= 0) return kv.seq_rm(seq_id, p0, p1);
    bool ok = true;
    for (int s = 0; s < kv.max_seqs(); ++s) ok = kv.seq_rm(s, p0, p1) && ok;
    return ok;
}

void llama_kv_cache_seq_cp(llama_context * ctx, llama_seq_id src, llama_seq_id dst, llama_pos p0, llama_pos p1) {
    jib::PagedKv & kv = *ctx->kv;
    if (src < 0 || dst < 0 || src >= kv.max_seqs() || dst >= kv.max_seqs() || src == dst) return;
    if (!kv.seq_cp(src, dst, p0, p1)) log_err("llama_kv_cache_seq_cp", "only a prefix [0, p1) can be shared between sequences");
}

void llama_kv_cache_seq_add(llama_context *, llama_seq_id, llama_pos, llama_pos, llama_pos) {}
void llama_kv_cache_clear(llama_context * ctx) { ctx->kv->clear(); }
bool llama_kv_cache_can_shift(llama_context *) { return false; }

void llama_kv_cache_update(llama_context * ctx) {
    jib::PagedKv & kv = *ctx->kv;
    if (ctx->params.defrag_thold < 0.0f || kv.fragmentation() <= ctx->params.defrag_thold) return;
    if (!flush_block_copies(ctx)) return;          // copy-on-write copies name block ids that the plan may move
    const auto moves = kv.defrag(kv.n_blocks());
    if (moves.empty()) return;
    std::vector<int32_t> flat;
    for (const auto & m : moves) { flat.push_back(m.first); flat.push_back(m.second); }
    std::string err;
    if (!jib::PyBridge::call("copy_blocks", nullptr, &err, "(LLi)", ctx->py, (long long) (intptr_t) flat.data(), (int) moves.size()))
        log_err("llama_kv_cache_update", err);
}

llama_kv_cache_view llama_kv_cache_view_init(const llama_context * ctx, int32_t n_seq_max) {
    llama_kv_cache_view v;
    memset(&v, 0, sizeof(v));
    v.n_cells = ctx->kv->n_blocks() * ctx->kv->block_size();
    v.n_seq_max = std::max(n_seq_max, 1);
    v.cells = (llama_kv_cache_view_cell *) calloc((size_t) v.n_cells, sizeof(llama_kv_cache_view_cell));
    v.cells_sequences = (llama_seq_id *) calloc((size_t) v.n_cells * v.n_seq_max, sizeof(llama_seq_id));
    return v;
}

void llama_kv_cache_view_update(const llama_context * ctx, llama_kv_cache_view * v) {
    const jib::PagedKv & kv = *ctx->kv;
    const int bs = kv.block_size();
    if (v->n_cells != kv.n_blocks() * bs) return;
    for (int i = 0; i < v->n_cells; ++i) v->cells[i].pos = -1;
    std::fill(v->cells_sequences, v->cells_sequences + (size_t) v->n_cells * v->n_seq_max, -1);
    v->token_count = 0;
    for (int s = 0; s < kv.max_seqs(); ++s) {
        const std::vector<int32_t> & bl = kv.seq_blocks(s);
        const int len = kv.seq_len(s);
        v->token_count += len;
        for (int p = 0; p < len; ++p) {
            const int cell = bl[p / bs] * bs + p % bs;
            v->cells[cell].pos = p;
            llama_seq_id * owners = v->cells_sequences + (size_t) cell * v->n_seq_max;
            for (int k = 0; k < v->n_seq_max; ++k)
                if (owners[k] < 0) { owners[k] = s; break; }
        }
    }
    v->used_cells = 0;
    v->max_contiguous = 0;
    v->max_contiguous_idx = -1;
    int run = 0;
    for (int i = 0; i < v->n_cells; ++i) {
        if (v->cells[i].pos >= 0) { ++v->used_cells; run = 0; continue; }
        if (++run > v->max_contiguous) { v->max_contiguous = run; v->max_contiguous_idx = i - run + 1; }
    }
}

void llama_kv_cache_view_free(llama_kv_cache_view * v) {
    free(v->cells);
    free(v->cells_sequences);
    v->cells = nullptr;
    v->cells_sequences = nullptr;
}

// ---- 6. vocabulary -----------------------------------------------------------------------------------------------------------
int32_t llama_vocab_n_tokens(const llama_vocab * v) { return v->n_tokens; }
llama_token llama_vocab_bos(const llama_vocab * v) { return v->bos; }
llama_token llama_vocab_eos(const llama_vocab * v) { return v->eos; }
llama_token llama_vocab_sep(const llama_vocab * v) { return v->sep; }
bool llama_vocab_is_eog(const llama_vocab * v, llama_token t) { return v->tok ? v->tok->is_eog(t) : t == v->eos; }
bool llama_vocab_get_add_bos(const llama_vocab * v) { return v->add_bos; }
bool llama_vocab_get_add_eos(const llama_vocab * v) { return v->add_eos; }

int32_t llama_tokenize(const llama_vocab * v, const char * text, int32_t text_len, llama_token * tokens, int32_t n_max,
                       bool add_special, bool parse_special) {
    if (!v->tok) { log_err("llama_tokenize", "the model file carries no tokenizer"); return 0; }
    const std::vector<int32_t> ids = v->tok->encode(std::string(text, (size_t) std::max(text_len, 0)), add_special, parse_special);
    if ((int64_t) ids.size() > n_max) return -(int32_t) ids.size();
    std::copy(ids.begin(), ids.end(), tokens);
    return (int32_t) ids.size();
}

int32_t llama_token_to_piece(const llama_vocab * v, llama_token token, char * buf, int32_t length, int32_t lstrip, bool special) {
    if (!v->tok || token < 0 || token >= v->n_tokens) return 0;
    std::string piece = v->tok->token_to_piece(token, special);
    size_t skip = 0;
    while (skip < piece.size() && (int32_t) skip < lstrip && piece[skip] == ' ') ++skip;
    return copy_out(piece.substr(skip), buf, length);
}

int32_t llama_detokenize(const llama_vocab * v, const llama_token * tokens, int32_t n_tokens, char * text, int32_t text_len_max,
                         bool remove_special, bool unparse_special) {
    if (!v->tok) return 0;
    const std::string s = v->tok->decode(std::vector<int32_t>(tokens, tokens + std::max(n_tokens, 0)), remove_special, unparse_special);
    return copy_out(s, text, text_len_max);
}

// ---- 7. chat template --------------------------------------------------------------------------------------------------------
int32_t llama_chat_apply_template(const char * tmpl, const llama_chat_message * chat, size_t n_msg, bool add_ass, char * buf,
                                  int32_t length) {
    const std::string t = tmpl ? tmpl : "deepseek2";
    const bool known = t == "deepseek2" || t == "deepseek" || t.find("'Assistant: ' + message['content'] + eos_token") != std::string::npos;
    if (!known) return -1;
    std::string out;
    for (size_t i = 0; i < n_msg; ++i) {
        const std::string role = chat[i].role ? chat[i].role : "";
        const std::string content = chat[i].content ? chat[i].content : "";
        if (role == "system") out += content + "\n\n";
        else if (role == "user") out += "User: " + content + "\n\n";
        else if (role == "assistant") out += "Assistant: " + content + "<\xef\xbd\x9c" "end\xe2\x96\x81of\xe2\x96\x81sentence\xef\xbd\x9c>";
    }
    if (add_ass) out += "Assistant:";
    if (buf != nullptr && length > 0) memcpy(buf, out.data(), std::min((size_t) length, out.size()));
    return (int32_t) out.size();
}

// ---- 9. timings --------------------------------------------------------------------------------------------------------------
llama_perf_context_data llama_perf_context(const llama_context * ctx) {
    llama_perf_context_data d;
    d.t_start_ms = ctx->t_start_ms;
    d.t_load_ms = ctx->model->t_load_ms;
    d.t_p_eval_ms = ctx->t_p_eval_ms;
    d.t_eval_ms = ctx->t_eval_ms;
    d.n_p_eval = std::max(1, ctx->n_p_eval);
    d.n_eval = std::max(1, ctx->n_eval);
    return d;
}

void llama_perf_context_print(const llama_context * ctx) {
    const llama_perf_context_data d = llama_perf_context(ctx);
    fprintf(stderr, "load time        = %10.2f ms\n", d.t_load_ms);
    fprintf(stderr, "prompt eval time = %10.2f ms / %5d tokens (%8.2f tokens per second)\n", d.t_p_eval_ms, d.n_p_eval,
            d.t_p_eval_ms > 0 ? 1e3 * d.n_p_eval / d.t_p_eval_ms : 0.0);
    fprintf(stderr, "eval time        = %10.2f ms / %5d tokens (%8.2f tokens per second)\n", d.t_eval_ms, d.n_eval,
            d.t_eval_ms > 0 ? 1e3 * d.n_eval / d.t_eval_ms : 0.0);
    fprintf(stderr, "total time       = %10.2f ms\n", now_ms() - d.t_start_ms);
}

void llama_perf_context_reset(llama_context * ctx) {
    ctx->t_start_ms = now_ms();
    ctx->t_p_eval_ms = ctx->t_eval_ms = 0;
    ctx->n_p_eval = ctx->n_eval = 0;
}

}  // extern "C"
