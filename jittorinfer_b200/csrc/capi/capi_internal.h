// Internals shared by the translation units of libllama.so.
#pragma once
#include "../include/llama.h"
#include "../runtime/gguf.h"
#include "../runtime/kv_paged.h"
#include "../runtime/tokenizer.h"

#include <map>
#include <memory>
#include <string>
#include <vector>

namespace jib {

// Calls into the Python package (jittorinfer_b200.capi_backend), which owns the weights, the latent cache and the
// kernels.  The interpreter is the host process's if there is one (a Python program that loaded this library through
// ctypes), otherwise one is started inside this process.
class PyBridge {
  public:
    // Empty string = ready.
    static std::string ensure();
    // fn(args...) -> integer.  fmt is a Py_BuildValue tuple format such as "(sii)".  Returns false and fills err on
    // a Python exception.
    static bool call(const char * fn, long long * result, std::string * err, const char * fmt, ...);
    static void shutdown();
};

}  // namespace jib

struct llama_vocab {
    std::unique_ptr<jib::Tokenizer> tok;     // NULL when the file carries no tokenizer
    int32_t n_tokens = 0;
    int32_t bos = 11, eos = 11, sep = -1;
    bool add_bos = false, add_eos = false;
};

struct llama_model {
    jib::GgufFile gguf;
    std::string path;
    llama_model_params params{};
    llama_vocab vocab;
    int32_t n_layer = 0, n_ctx_train = 0, n_embd = 0, kv_row = 0;
    std::map<std::string, std::string> templates;    // "" = default
    long long py = 0;                                // handle in the Python backend (0 = metadata only)
    double t_load_ms = 0;
};

struct llama_context {
    llama_model * model = nullptr;
    llama_context_params params{};
    std::unique_ptr<jib::PagedKv> kv;
    long long py = 0;
    int32_t block_size = 64;

    // outputs of the last llama_decode
    std::vector<float> out_values;
    std::vector<int64_t> out_indices;
    std::vector<int32_t> row_of_token;       // batch index -> output row or -1
    int64_t out_len = -1, n_out = 0;

    ggml_abort_callback abort_cb = nullptr;
    void * abort_data = nullptr;

    double t_start_ms = 0, t_p_eval_ms = 0, t_eval_ms = 0;
    int32_t n_p_eval = 0, n_eval = 0;
    int all_processed = 0;
};
