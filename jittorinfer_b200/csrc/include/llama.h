/* llama.h -- public C API of jittorinfer_b200 (libllama.so).
 *
 * The entry points, structs and enum values are those of JittorInfer's include/llama.h, so that a
 * program written against that header builds against this one.  What differs:
 *
 *   - every function has C linkage, and the header is valid C as well as C++ (in C, llama_decode
 *     takes its third argument explicitly; in C++ it defaults to false);
 *   - the few ggml types the original header borrows are declared here as opaque handles or small
 *     enums: nothing of ggml exists in this library;
 *   - llama_logits is a plain struct (see below) instead of a C++ class;
 *   - the device back end is CUDA on B200 (sm_100a): `enable_cann_flash_attention`, `enable_ge`,
 *     `enable_scatter_kv`, `offload_input`, `n_threads*` are accepted and have no effect -- attention
 *     always runs the absorbed-MLA kernel over the paged latent cache and decode steps are replayed
 *     as CUDA graphs.
 *
 * Groups: 1 types, 2 parameters, 3 backend / model / context, 4 batch + decode + logits, 5 KV cache,
 * 6 vocabulary, 7 chat template, 8 samplers, 9 timings.
 */
#ifndef JITTORINFER_B200_LLAMA_H
#define JITTORINFER_B200_LLAMA_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#if defined(LLAMA_BUILD)
#    define MINI_API __attribute__((visibility("default")))
#else
#    define MINI_API
#endif
#define LLAMA_API MINI_API

#ifdef __cplusplus
#    define LLAMA_DEFAULT_ARG(v) = v
extern "C" {
#else
#    define LLAMA_DEFAULT_ARG(v)
#endif

#define LLAMA_TOKEN_NULL   (-1)
#define LLAMA_DEFAULT_SEED 0xFFFFFFFF

/* ------------------------------------------------------------------------------------------------
 * 1. types
 * ---------------------------------------------------------------------------------------------- */
struct llama_vocab;
struct llama_sampler;
struct llama_model;
struct llama_context;
struct llama_adapter_lora;
struct ggml_tensor;

typedef int32_t llama_token;
typedef int32_t llama_pos;
typedef int32_t llama_seq_id;
typedef void *  llama_sampler_context_t;

/* stand-ins for the ggml handles the original header uses in its parameter structs */
typedef struct ggml_backend_device * ggml_backend_dev_t;
typedef struct ggml_threadpool *     ggml_threadpool_t;
typedef bool (*ggml_abort_callback)(void * data);
typedef bool (*ggml_backend_sched_eval_callback)(struct ggml_tensor * t, bool ask, void * user_data);
enum ggml_type {
    GGML_TYPE_F32 = 0, GGML_TYPE_F16 = 1, GGML_TYPE_Q4_0 = 2, GGML_TYPE_Q4_1 = 3, GGML_TYPE_Q5_0 = 6, GGML_TYPE_Q5_1 = 7,
    GGML_TYPE_Q8_0 = 8, GGML_TYPE_Q8_1 = 9, GGML_TYPE_Q2_K = 10, GGML_TYPE_Q3_K = 11, GGML_TYPE_Q4_K = 12, GGML_TYPE_Q5_K = 13,
    GGML_TYPE_Q6_K = 14, GGML_TYPE_Q8_K = 15, GGML_TYPE_I8 = 24, GGML_TYPE_I16 = 25, GGML_TYPE_I32 = 26, GGML_TYPE_I64 = 27,
    GGML_TYPE_F64 = 28, GGML_TYPE_BF16 = 30,
};

enum llama_vocab_type {
    LLAMA_VOCAB_TYPE_NONE = 0, LLAMA_VOCAB_TYPE_SPM = 1, LLAMA_VOCAB_TYPE_BPE = 2, LLAMA_VOCAB_TYPE_WPM = 3,
    LLAMA_VOCAB_TYPE_UGM = 4, LLAMA_VOCAB_TYPE_RWKV = 5,
};

/* only DEFAULT and DEEPSEEK_LLM pre-tokenizers are implemented; the numbering is kept */
enum llama_vocab_pre_type {
    LLAMA_VOCAB_PRE_TYPE_DEFAULT = 0, LLAMA_VOCAB_PRE_TYPE_LLAMA3 = 1, LLAMA_VOCAB_PRE_TYPE_DEEPSEEK_LLM = 2,
    LLAMA_VOCAB_PRE_TYPE_DEEPSEEK_CODER = 3, LLAMA_VOCAB_PRE_TYPE_FALCON = 4, LLAMA_VOCAB_PRE_TYPE_MPT = 5,
    LLAMA_VOCAB_PRE_TYPE_STARCODER = 6, LLAMA_VOCAB_PRE_TYPE_GPT2 = 7, LLAMA_VOCAB_PRE_TYPE_REFACT = 8,
    LLAMA_VOCAB_PRE_TYPE_COMMAND_R = 9, LLAMA_VOCAB_PRE_TYPE_STABLELM2 = 10, LLAMA_VOCAB_PRE_TYPE_QWEN2 = 11,
    LLAMA_VOCAB_PRE_TYPE_OLMO = 12, LLAMA_VOCAB_PRE_TYPE_DBRX = 13, LLAMA_VOCAB_PRE_TYPE_SMAUG = 14,
    LLAMA_VOCAB_PRE_TYPE_PORO = 15, LLAMA_VOCAB_PRE_TYPE_CHATGLM3 = 16, LLAMA_VOCAB_PRE_TYPE_CHATGLM4 = 17,
    LLAMA_VOCAB_PRE_TYPE_VIKING = 18, LLAMA_VOCAB_PRE_TYPE_JAIS = 19, LLAMA_VOCAB_PRE_TYPE_TEKKEN = 20,
    LLAMA_VOCAB_PRE_TYPE_SMOLLM = 21, LLAMA_VOCAB_PRE_TYPE_CODESHELL = 22, LLAMA_VOCAB_PRE_TYPE_BLOOM = 23,
    LLAMA_VOCAB_PRE_TYPE_GPT3_FINNISH = 24, LLAMA_VOCAB_PRE_TYPE_EXAONE = 25, LLAMA_VOCAB_PRE_TYPE_CHAMELEON = 26,
    LLAMA_VOCAB_PRE_TYPE_MINERVA = 27, LLAMA_VOCAB_PRE_TYPE_DEEPSEEK3_LLM = 28,
};

enum llama_token_type {
    LLAMA_TOKEN_TYPE_UNDEFINED = 0, LLAMA_TOKEN_TYPE_NORMAL = 1, LLAMA_TOKEN_TYPE_UNKNOWN = 2, LLAMA_TOKEN_TYPE_CONTROL = 3,
    LLAMA_TOKEN_TYPE_USER_DEFINED = 4, LLAMA_TOKEN_TYPE_UNUSED = 5, LLAMA_TOKEN_TYPE_BYTE = 6,
};

enum llama_token_attr {
    LLAMA_TOKEN_ATTR_UNDEFINED = 0,
    LLAMA_TOKEN_ATTR_UNKNOWN = 1 << 0, LLAMA_TOKEN_ATTR_UNUSED = 1 << 1, LLAMA_TOKEN_ATTR_NORMAL = 1 << 2,
    LLAMA_TOKEN_ATTR_CONTROL = 1 << 3, LLAMA_TOKEN_ATTR_USER_DEFINED = 1 << 4, LLAMA_TOKEN_ATTR_BYTE = 1 << 5,
    LLAMA_TOKEN_ATTR_NORMALIZED = 1 << 6, LLAMA_TOKEN_ATTR_LSTRIP = 1 << 7, LLAMA_TOKEN_ATTR_RSTRIP = 1 << 8,
    LLAMA_TOKEN_ATTR_SINGLE_WORD = 1 << 9,
};

/* file types a GGUF may declare (general.file_type); F32, F16, BF16, Q8_0 and Q4_0 tensors load */
enum llama_ftype {
    LLAMA_FTYPE_ALL_F32 = 0, LLAMA_FTYPE_MOSTLY_F16 = 1, LLAMA_FTYPE_MOSTLY_Q4_0 = 2, LLAMA_FTYPE_MOSTLY_Q4_1 = 3,
    LLAMA_FTYPE_MOSTLY_Q8_0 = 7, LLAMA_FTYPE_MOSTLY_Q5_0 = 8, LLAMA_FTYPE_MOSTLY_Q5_1 = 9, LLAMA_FTYPE_MOSTLY_Q2_K = 10,
    LLAMA_FTYPE_MOSTLY_Q3_K_S = 11, LLAMA_FTYPE_MOSTLY_Q3_K_M = 12, LLAMA_FTYPE_MOSTLY_Q3_K_L = 13,
    LLAMA_FTYPE_MOSTLY_Q4_K_S = 14, LLAMA_FTYPE_MOSTLY_Q4_K_M = 15, LLAMA_FTYPE_MOSTLY_Q5_K_S = 16,
    LLAMA_FTYPE_MOSTLY_Q5_K_M = 17, LLAMA_FTYPE_MOSTLY_Q6_K = 18, LLAMA_FTYPE_MOSTLY_IQ2_XXS = 19,
    LLAMA_FTYPE_MOSTLY_IQ2_XS = 20, LLAMA_FTYPE_MOSTLY_Q2_K_S = 21, LLAMA_FTYPE_MOSTLY_IQ3_XS = 22,
    LLAMA_FTYPE_MOSTLY_IQ3_XXS = 23, LLAMA_FTYPE_MOSTLY_IQ1_S = 24, LLAMA_FTYPE_MOSTLY_IQ4_NL = 25,
    LLAMA_FTYPE_MOSTLY_IQ3_S = 26, LLAMA_FTYPE_MOSTLY_IQ3_M = 27, LLAMA_FTYPE_MOSTLY_IQ2_S = 28,
    LLAMA_FTYPE_MOSTLY_IQ2_M = 29, LLAMA_FTYPE_MOSTLY_IQ4_XS = 30, LLAMA_FTYPE_MOSTLY_IQ1_M = 31,
    LLAMA_FTYPE_MOSTLY_BF16 = 32, LLAMA_FTYPE_MOSTLY_TQ1_0 = 36, LLAMA_FTYPE_MOSTLY_TQ2_0 = 37,
    LLAMA_FTYPE_GUESSED = 1024,
};

enum llama_split_mode {
    LLAMA_SPLIT_MODE_NONE  = 0,   /* one GPU */
    LLAMA_SPLIT_MODE_LAYER = 1,   /* consecutive layer ranges on consecutive GPUs */
    LLAMA_SPLIT_MODE_ROW   = 2,   /* tensor parallel (one process per GPU) */
};

enum llama_rope_type {
    LLAMA_ROPE_TYPE_NONE = -1, LLAMA_ROPE_TYPE_NORM = 0, LLAMA_ROPE_TYPE_NEOX = 2, LLAMA_ROPE_TYPE_MROPE = 8,
    LLAMA_ROPE_TYPE_VISION = 24,
};

enum llama_rope_scaling_type {
    LLAMA_ROPE_SCALING_TYPE_UNSPECIFIED = -1, LLAMA_ROPE_SCALING_TYPE_NONE = 0, LLAMA_ROPE_SCALING_TYPE_LINEAR = 1,
    LLAMA_ROPE_SCALING_TYPE_YARN = 2, LLAMA_ROPE_SCALING_TYPE_LONGROPE = 3,
    LLAMA_ROPE_SCALING_TYPE_MAX_VALUE = LLAMA_ROPE_SCALING_TYPE_LONGROPE,
};

enum llama_pooling_type {
    LLAMA_POOLING_TYPE_UNSPECIFIED = -1, LLAMA_POOLING_TYPE_NONE = 0, LLAMA_POOLING_TYPE_MEAN = 1, LLAMA_POOLING_TYPE_CLS = 2,
    LLAMA_POOLING_TYPE_LAST = 3, LLAMA_POOLING_TYPE_RANK = 4,
};

enum llama_attention_type {
    LLAMA_ATTENTION_TYPE_UNSPECIFIED = -1, LLAMA_ATTENTION_TYPE_CAUSAL = 0, LLAMA_ATTENTION_TYPE_NON_CAUSAL = 1,
};

enum llama_model_kv_override_type {
    LLAMA_KV_OVERRIDE_TYPE_INT, LLAMA_KV_OVERRIDE_TYPE_FLOAT, LLAMA_KV_OVERRIDE_TYPE_BOOL, LLAMA_KV_OVERRIDE_TYPE_STR,
};

struct llama_model_kv_override {
    enum llama_model_kv_override_type tag;
    char key[128];                 /* an empty key ends the list */
    union {
        int64_t val_i64;
        double  val_f64;
        bool    val_bool;
        char    val_str[128];
    };
};

struct llama_chat_message {
    const char * role;
    const char * content;
};

typedef struct llama_token_data {
    llama_token id;
    float       logit;
    float       p;
} llama_token_data;

typedef struct llama_token_data_array {
    llama_token_data * data;
    size_t             size;
    int64_t            selected;   /* index into data (not a token id); -1 = nothing selected yet */
    bool               sorted;     /* data is in descending logit order */
} llama_token_data_array;

typedef struct llama_logit_bias {
    llama_token token;
    float       bias;
} llama_logit_bias;

/* A batch of tokens for llama_decode.  token[i] at position pos[i] belongs to the sequences
 * seq_id[i][0..n_seq_id[i]); logits[i] != 0 asks for that token's output row.  pos / n_seq_id / seq_id /
 * logits may be NULL (positions continue sequence 0, only the last token has an output). */
typedef struct llama_batch {
    int32_t         n_tokens;
    llama_token *   token;
    float *         embd;          /* not supported (token ids only) */
    llama_pos *     pos;
    int32_t *       n_seq_id;
    llama_seq_id ** seq_id;
    int8_t *        logits;
} llama_batch;

/* One output row.  RAW: values[0..len) are the logits of the whole vocabulary.  TOPK (context created
 * with presample_count = k > 0): values[0..len) are the k largest logits in descending order and
 * indices[0..len) their token ids -- the top-k runs on the GPU and only 12*k bytes cross PCIe. */
enum llama_logits_type { LLAMA_LOGITS_TYPE_RAW = 0, LLAMA_LOGITS_TYPE_TOPK = 1 };
typedef struct llama_logits {
    enum llama_logits_type type;
    float *   values;
    int64_t * indices;             /* NULL for RAW */
    int64_t   len;                 /* entries per row; -1 = no such row */
    int64_t   num;                 /* rows from this one to the end of the batch's outputs */
} llama_logits;

/* ------------------------------------------------------------------------------------------------
 * 2. parameters
 * ---------------------------------------------------------------------------------------------- */
typedef bool (*llama_progress_callback)(float progress, void * user_data);

struct llama_model_params {
    ggml_backend_dev_t * devices;          /* ignored: GPUs are chosen with CUDA_VISIBLE_DEVICES / main_gpu */
    int32_t n_gpu_layers;                  /* <= 0 keeps the model on the CPU (fp32 reference ops); > 0 = all layers on the GPU */
    enum llama_split_mode split_mode;
    int32_t main_gpu;
    const float * tensor_split;            /* LAYER mode: relative share of layers per GPU (NULL = even) */

    bool enable_tensor_parallel;           /* this process is rank tp_id of num_parallel (launched one per GPU) */
    bool enable_expert_parallel;           /* routed experts sharded by expert id instead of by column */
    bool enable_data_parallel;             /* attention data-parallel: every rank decodes its own batch */
    bool enable_mpi;                       /* ranks rendezvous through torch.distributed (env MASTER_ADDR/PORT) */
    bool offload_input;
    bool enable_mla;                       /* kept for source compatibility: the latent cache is always used */
    bool enable_cann_flash_attention;
    int  tp_id;
    int  num_parallel;

    llama_progress_callback progress_callback;   /* called with 0..1 while tensors load; return false to abort */
    void * progress_callback_user_data;
    const struct llama_model_kv_override * kv_overrides;

    bool vocab_only;                       /* read metadata + vocabulary only (no Python, no GPU) */
    bool use_mmap;
    bool use_mlock;
    bool check_tensors;                    /* reject NaN/Inf in the checkpoint */
    bool enable_fused_moe;
};

struct llama_context_params {
    uint32_t n_ctx;                        /* KV capacity in tokens over all sequences; 0 = model's training context */
    uint32_t n_batch;                      /* most tokens per llama_decode call */
    uint32_t n_ubatch;                     /* most tokens per forward pass (longer batches are chunked) */
    uint32_t n_seq_max;                    /* most distinct sequence ids */
    int32_t  n_threads;
    int32_t  n_threads_batch;

    enum llama_rope_scaling_type rope_scaling_type;
    enum llama_pooling_type      pooling_type;
    enum llama_attention_type    attention_type;

    float    rope_freq_base;               /* 0 = from the model */
    float    rope_freq_scale;              /* 0 = from the model */
    float    yarn_ext_factor;              /* < 0 = from the model */
    float    yarn_attn_factor;
    float    yarn_beta_fast;
    float    yarn_beta_slow;
    uint32_t yarn_orig_ctx;
    float    defrag_thold;                 /* defragment when the share of holes exceeds this; < 0 = never */

    ggml_backend_sched_eval_callback cb_eval;   /* not called: there is no per-node scheduler */
    void * cb_eval_user_data;

    enum ggml_type type_k;                 /* the latent cache is bf16 on the GPU, f32 on the CPU */
    enum ggml_type type_v;

    bool logits_all;
    bool embeddings;
    bool offload_kqv;
    bool flash_attn;
    bool no_perf;
    bool enable_ge;
    bool enable_scatter_kv;
    int  presample_count;                  /* k > 0: llama_get_logits_ith returns the top-k of each row */

    ggml_abort_callback abort_callback;    /* polled between forward chunks */
    void *              abort_callback_data;
};

MINI_API struct llama_model_params   llama_model_default_params(void);
MINI_API struct llama_context_params llama_context_default_params(void);

/* ------------------------------------------------------------------------------------------------
 * 3. backend, model, context
 * ---------------------------------------------------------------------------------------------- */
MINI_API void llama_backend_init(void);
MINI_API void llama_backend_free(void);
MINI_API bool llama_supports_gpu_offload(void);
MINI_API bool llama_supports_rpc(void);

MINI_API struct llama_model * llama_model_load_from_file(const char * path_model, struct llama_model_params params);
MINI_API void                 llama_model_free(struct llama_model * model);

MINI_API const struct llama_vocab * llama_model_get_vocab(const struct llama_model * model);
MINI_API enum llama_rope_type       llama_model_rope_type(const struct llama_model * model);
MINI_API int32_t                    llama_model_n_ctx_train(const struct llama_model * model);
MINI_API bool                       llama_model_is_recurrent(const struct llama_model * model);
MINI_API bool                       llama_model_has_encoder(const struct llama_model * model);
MINI_API bool                       llama_model_has_decoder(const struct llama_model * model);
MINI_API llama_token                llama_model_decoder_start_token(const struct llama_model * model);
/* tokenizer.chat_template (name == NULL) or tokenizer.chat_template.<name>; NULL if the file has none */
MINI_API const char *               llama_model_chat_template(const struct llama_model * model, const char * name);

MINI_API struct llama_context * llama_init_from_model(struct llama_model * model, struct llama_context_params params);
MINI_API void                   llama_free(struct llama_context * ctx);

MINI_API const struct llama_model * llama_get_model(const struct llama_context * ctx);
MINI_API uint32_t                   llama_n_ctx(const struct llama_context * ctx);
MINI_API uint32_t                   llama_n_batch(const struct llama_context * ctx);
MINI_API enum llama_pooling_type    llama_pooling_type(const struct llama_context * ctx);
MINI_API void    llama_set_embeddings(struct llama_context * ctx, bool embeddings);
MINI_API void    llama_set_abort_callback(struct llama_context * ctx, ggml_abort_callback abort_callback, void * abort_callback_data);
MINI_API void    llama_attach_threadpool(struct llama_context * ctx, ggml_threadpool_t threadpool, ggml_threadpool_t threadpool_batch);
/* LoRA adapters are not implemented (they are empty stubs in the original as well): set returns -1 */
MINI_API void    llama_clear_adapter_lora(struct llama_context * ctx);
MINI_API int32_t llama_set_adapter_lora(struct llama_context * ctx, struct llama_adapter_lora * adapter, float scale);

/* ------------------------------------------------------------------------------------------------
 * 4. batch, decode, logits
 * ---------------------------------------------------------------------------------------------- */
/* A view of `tokens` as one batch of sequence 0 continuing at its current length; nothing to free. */
MINI_API struct llama_batch llama_batch_get_one(llama_token * tokens, int32_t n_tokens);
/* Heap-allocated batch of up to n_tokens tokens (embd must be 0), each with up to n_seq_max sequence ids. */
MINI_API struct llama_batch llama_batch_init(int32_t n_tokens, int32_t embd, int32_t n_seq_max);
MINI_API void               llama_batch_free(struct llama_batch batch);

/* Runs the batch.  Tokens of one sequence must continue that sequence (pos = its current length, +1, ...).
 * Returns 0 = ok, 1 = the KV cache has no room (nothing was changed; free a sequence or shrink the batch),
 * 2 = aborted by the abort callback, < 0 = error.  sync_all_servers: data-parallel ranks step together. */
MINI_API int32_t llama_decode(struct llama_context * ctx, struct llama_batch batch, bool sync_all_servers LLAMA_DEFAULT_ARG(false));
/* There is no encoder: returns -1. */
MINI_API int32_t llama_encode(struct llama_context * ctx, struct llama_batch batch);
/* Data-parallel: join the other ranks' collectives for one step without tokens of one's own. */
MINI_API bool    llama_empty_run(struct llama_context * ctx);
/* Tokens decoded by all data-parallel ranks in the last synchronised step. */
MINI_API int     llama_all_processed_tokens(const struct llama_context * ctx);
MINI_API void    llama_synchronize(struct llama_context * ctx);
/* Output row of batch token i of the last llama_decode (negative i counts from the end of the outputs). */
MINI_API llama_logits llama_get_logits_ith(struct llama_context * ctx, int32_t i);

/* ------------------------------------------------------------------------------------------------
 * 5. KV cache.  Sequences own lists of 64-token blocks of the latent cache; sharing a prefix is a
 *    reference-count bump with copy-on-write of the one partially filled block.
 * ---------------------------------------------------------------------------------------------- */
/* Drops positions [p0, p1) of a sequence (negative bound = open; seq_id < 0 = every sequence).  Only a
 * tail range can be dropped from a paged sequence: a hole in the middle returns false. */
MINI_API bool llama_kv_cache_seq_rm(struct llama_context * ctx, llama_seq_id seq_id, llama_pos p0, llama_pos p1);
/* dst := positions [0, p1) of src (p0 must be <= 0). */
MINI_API void llama_kv_cache_seq_cp(struct llama_context * ctx, llama_seq_id seq_id_src, llama_seq_id seq_id_dst, llama_pos p0, llama_pos p1);
/* Position shifts need the cached rope part re-rotated; like the original for this architecture
 * (llama_kv_cache_can_shift == false) this is a no-op. */
MINI_API void llama_kv_cache_seq_add(struct llama_context * ctx, llama_seq_id seq_id, llama_pos p0, llama_pos p1, llama_pos delta);
MINI_API void llama_kv_cache_clear(struct llama_context * ctx);
MINI_API bool llama_kv_cache_can_shift(struct llama_context * ctx);
/* Applies a pending defragmentation if the share of holes exceeds defrag_thold. */
MINI_API void llama_kv_cache_update(struct llama_context * ctx);

struct llama_kv_cache_view_cell {
    llama_pos pos;                         /* position of the token stored in this cell, -1 = free */
};
/* Debug view: one cell per cache slot (block * 64 + offset), each with up to n_seq_max owning sequences. */
struct llama_kv_cache_view {
    int32_t n_cells;
    int32_t n_seq_max;
    int32_t token_count;                   /* sum over sequences of their lengths (shared cells count per owner) */
    int32_t used_cells;
    int32_t max_contiguous;                /* longest run of free cells */
    int32_t max_contiguous_idx;
    struct llama_kv_cache_view_cell * cells;
    llama_seq_id * cells_sequences;        /* [n_cells][n_seq_max], -1 padded */
};
MINI_API struct llama_kv_cache_view llama_kv_cache_view_init(const struct llama_context * ctx, int32_t n_seq_max);
MINI_API void llama_kv_cache_view_update(const struct llama_context * ctx, struct llama_kv_cache_view * view);
MINI_API void llama_kv_cache_view_free(struct llama_kv_cache_view * view);

/* ------------------------------------------------------------------------------------------------
 * 6. vocabulary (byte-level BPE, deepseek-llm pre-tokenizer)
 * ---------------------------------------------------------------------------------------------- */
MINI_API int32_t     llama_vocab_n_tokens(const struct llama_vocab * vocab);
MINI_API llama_token llama_vocab_bos(const struct llama_vocab * vocab);
MINI_API llama_token llama_vocab_eos(const struct llama_vocab * vocab);
MINI_API llama_token llama_vocab_sep(const struct llama_vocab * vocab);
MINI_API bool        llama_vocab_is_eog(const struct llama_vocab * vocab, llama_token token);
MINI_API bool        llama_vocab_get_add_bos(const struct llama_vocab * vocab);
MINI_API bool        llama_vocab_get_add_eos(const struct llama_vocab * vocab);

/* Returns the number of tokens written; if n_tokens_max is too small, minus the number needed. */
MINI_API int32_t llama_tokenize(const struct llama_vocab * vocab, const char * text, int32_t text_len, llama_token * tokens,
                                int32_t n_tokens_max, bool add_special, bool parse_special);
/* Bytes of one token (not NUL-terminated); lstrip = leading spaces to skip; if length is too small, minus the need. */
MINI_API int32_t llama_token_to_piece(const struct llama_vocab * vocab, llama_token token, char * buf, int32_t length,
                                      int32_t lstrip, bool special);
MINI_API int32_t llama_detokenize(const struct llama_vocab * vocab, const llama_token * tokens, int32_t n_tokens, char * text,
                                  int32_t text_len_max, bool remove_special, bool unparse_special);

/* ------------------------------------------------------------------------------------------------
 * 7. chat template.  tmpl: NULL or "deepseek2" = built-in "User: ...\n\nAssistant:" form; a Jinja source
 *    containing the DeepSeek-V2 markers is recognised as the same form.  Returns the byte count of the
 *    formatted prompt (write at most `length`), or -1 for an unknown template.
 * ---------------------------------------------------------------------------------------------- */
MINI_API int32_t llama_chat_apply_template(const char * tmpl, const struct llama_chat_message * chat, size_t n_msg, bool add_ass,
                                           char * buf, int32_t length);

/* ------------------------------------------------------------------------------------------------
 * 8. samplers.  A sampler transforms a candidate array; a chain applies its members in order and
 *    owns them.  The final member (greedy or dist) sets cur_p->selected.
 * ---------------------------------------------------------------------------------------------- */
struct llama_sampler_i {
    const char *           (*name)  (const struct llama_sampler * smpl);                                  /* may be NULL */
    void                   (*accept)(      struct llama_sampler * smpl, llama_token token);               /* may be NULL */
    void                   (*apply) (      struct llama_sampler * smpl, llama_token_data_array * cur_p);  /* required */
    void                   (*reset) (      struct llama_sampler * smpl);                                  /* may be NULL */
    struct llama_sampler * (*clone) (const struct llama_sampler * smpl);                                  /* may be NULL if ctx is NULL */
    void                   (*free)  (      struct llama_sampler * smpl);                                  /* may be NULL if ctx is NULL */
};
struct llama_sampler {
    const struct llama_sampler_i * iface;
    llama_sampler_context_t        ctx;
};
struct llama_sampler_chain_params {
    bool no_perf;
};

MINI_API struct llama_sampler * llama_sampler_init(const struct llama_sampler_i * iface, llama_sampler_context_t ctx);
MINI_API const char *           llama_sampler_name(const struct llama_sampler * smpl);
MINI_API void                   llama_sampler_accept(struct llama_sampler * smpl, llama_token token);
MINI_API void                   llama_sampler_apply(struct llama_sampler * smpl, llama_token_data_array * cur_p);
MINI_API void                   llama_sampler_reset(struct llama_sampler * smpl);
MINI_API struct llama_sampler * llama_sampler_clone(const struct llama_sampler * smpl);
MINI_API void                   llama_sampler_free(struct llama_sampler * smpl);

MINI_API struct llama_sampler_chain_params llama_sampler_chain_default_params(void);
MINI_API struct llama_sampler * llama_sampler_chain_init(struct llama_sampler_chain_params params);
MINI_API void                   llama_sampler_chain_add(struct llama_sampler * chain, struct llama_sampler * smpl);   /* takes ownership */
MINI_API struct llama_sampler * llama_sampler_chain_get(const struct llama_sampler * chain, int32_t i);
MINI_API int                    llama_sampler_chain_n(const struct llama_sampler * chain);

MINI_API struct llama_sampler * llama_sampler_init_greedy(void);
MINI_API struct llama_sampler * llama_sampler_init_dist(uint32_t seed);
MINI_API struct llama_sampler * llama_sampler_init_top_k(int32_t k);
MINI_API struct llama_sampler * llama_sampler_init_top_p(float p, size_t min_keep);
MINI_API struct llama_sampler * llama_sampler_init_min_p(float p, size_t min_keep);
MINI_API struct llama_sampler * llama_sampler_init_typical(float p, size_t min_keep);
MINI_API struct llama_sampler * llama_sampler_init_temp(float t);
/* dynamic temperature: t +- delta scaled by the normalised entropy raised to `exponent`; delta <= 0 = plain temperature */
MINI_API struct llama_sampler * llama_sampler_init_temp_ext(float t, float delta, float exponent);
/* with probability p, drop every candidate at or above threshold t except the least likely of them */
MINI_API struct llama_sampler * llama_sampler_init_xtc(float p, float t, size_t min_keep, uint32_t seed);
MINI_API struct llama_sampler * llama_sampler_init_penalties(int32_t penalty_last_n, float penalty_repeat, float penalty_freq,
                                                             float penalty_present);
/* "don't repeat yourself": penalises the token that would extend a repetition of length >= dry_allowed_length by
 * dry_multiplier * dry_base^(length - dry_allowed_length); a token whose text contains a breaker string ends a match */
MINI_API struct llama_sampler * llama_sampler_init_dry(const struct llama_vocab * vocab, int32_t n_ctx_train, float dry_multiplier,
                                                       float dry_base, int32_t dry_allowed_length, int32_t dry_penalty_last_n,
                                                       const char ** seq_breakers, size_t num_breakers);
MINI_API struct llama_sampler * llama_sampler_init_logit_bias(int32_t n_vocab, int32_t n_logit_bias, const llama_logit_bias * logit_bias);
/* Grammar-constrained sampling over a GBNF grammar (the original declares this but asserts on a non-empty grammar):
 * candidates whose text cannot continue the grammar are dropped, end-of-generation tokens are kept only where the text
 * so far is complete; if no candidate fits, one token that does is substituted.  Returns NULL if the grammar does not
 * parse.  An empty grammar gives a pass-through sampler. */
MINI_API struct llama_sampler * llama_sampler_init_grammar(const struct llama_vocab * vocab, const char * grammar_str,
                                                           const char * grammar_root);

/* ------------------------------------------------------------------------------------------------
 * 9. timings
 * ---------------------------------------------------------------------------------------------- */
struct llama_perf_context_data {
    double  t_start_ms;
    double  t_load_ms;
    double  t_p_eval_ms;                   /* batches of more than one token per sequence (prompt processing) */
    double  t_eval_ms;                     /* single-token steps */
    int32_t n_p_eval;
    int32_t n_eval;
};
struct llama_perf_sampler_data {
    double  t_sample_ms;
    int32_t n_sample;
};
MINI_API struct llama_perf_context_data llama_perf_context(const struct llama_context * ctx);
MINI_API void                           llama_perf_context_print(const struct llama_context * ctx);
MINI_API void                           llama_perf_context_reset(struct llama_context * ctx);
MINI_API struct llama_perf_sampler_data llama_perf_sampler(const struct llama_sampler * chain);
MINI_API void                           llama_perf_sampler_print(const struct llama_sampler * chain);
MINI_API void                           llama_perf_sampler_reset(struct llama_sampler * chain);

#ifdef __cplusplus
}   /* extern "C" */

#include <memory>
struct llama_model_deleter   { void operator()(llama_model * m) { llama_model_free(m); } };
struct llama_context_deleter { void operator()(llama_context * c) { llama_free(c); } };
struct llama_sampler_deleter { void operator()(llama_sampler * s) { llama_sampler_free(s); } };
typedef std::unique_ptr<llama_model, llama_model_deleter>     llama_model_ptr;
typedef std::unique_ptr<llama_context, llama_context_deleter> llama_context_ptr;
typedef std::unique_ptr<llama_sampler, llama_sampler_deleter> llama_sampler_ptr;
#endif

#endif /* JITTORINFER_B200_LLAMA_H */
