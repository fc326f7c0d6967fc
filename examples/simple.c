/* Minimal program against the llama.h C API of jittorinfer_b200: load a GGUF model, tokenise a prompt, decode, sample
 * with a chain (top-k, top-p, temperature, dist) and print the text.
 *
 *   python -m jittorinfer_b200.build
 *   gcc -O2 -I jittorinfer_b200/csrc/include examples/simple.c -o simple \
 *       -L jittorinfer_b200/lib -lllama -Wl,-rpath,$PWD/jittorinfer_b200/lib
 *   ./simple model.gguf "The capital of France is" 64
 *
 * The forward pass runs in the engine through an embedded interpreter: JITTORINFER_PYTHON selects the Python executable
 * (default: python3 on PATH), n_gpu_layers = 0 keeps the model on the CPU.
 */
#include "llama.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

int main(int argc, char ** argv) {
    if (argc < 3) {
        fprintf(stderr, "usage: %s model.gguf \"prompt\" [n_predict] [n_gpu_layers]\n", argv[0]);
        return 1;
    }
    const int n_predict = argc > 3 ? atoi(argv[3]) : 32;
    llama_backend_init();

    struct llama_model_params mp = llama_model_default_params();
    if (argc > 4) mp.n_gpu_layers = atoi(argv[4]);
    struct llama_model * model = llama_model_load_from_file(argv[1], mp);
    if (!model) return 2;
    const struct llama_vocab * vocab = llama_model_get_vocab(model);

    struct llama_context_params cp = llama_context_default_params();
    cp.n_ctx = 4096;
    cp.n_batch = 512;
    cp.n_seq_max = 1;
    cp.presample_count = 64;                       /* top-64 on the device: 768 bytes per step cross PCIe */
    struct llama_context * ctx = llama_init_from_model(model, cp);
    if (!ctx) return 3;

    const int n_max = (int) strlen(argv[2]) + 8;
    llama_token * tokens = malloc(sizeof(llama_token) * (size_t) n_max);
    int n = llama_tokenize(vocab, argv[2], (int) strlen(argv[2]), tokens, n_max, true, true);
    if (n <= 0) { fprintf(stderr, "cannot tokenise the prompt\n"); return 4; }

    struct llama_sampler * smpl = llama_sampler_chain_init(llama_sampler_chain_default_params());
    llama_sampler_chain_add(smpl, llama_sampler_init_top_k(40));
    llama_sampler_chain_add(smpl, llama_sampler_init_top_p(0.95f, 1));
    llama_sampler_chain_add(smpl, llama_sampler_init_temp(0.8f));
    llama_sampler_chain_add(smpl, llama_sampler_init_dist(LLAMA_DEFAULT_SEED));

    llama_token_data cand[64];
    struct llama_batch batch = llama_batch_get_one(tokens, n);
    for (int i = 0; i < n_predict; ++i) {
        const int rc = llama_decode(ctx, batch, false);
        if (rc != 0) { fprintf(stderr, "llama_decode returned %d\n", rc); break; }
        llama_logits lg = llama_get_logits_ith(ctx, -1);            /* TOPK: values + token ids, sorted */
        for (int k = 0; k < lg.len; ++k) {
            cand[k].id = (llama_token) lg.indices[k];
            cand[k].logit = lg.values[k];
            cand[k].p = 0.0f;
        }
        llama_token_data_array arr = { cand, (size_t) lg.len, -1, true };
        llama_sampler_apply(smpl, &arr);
        const llama_token tok = arr.data[arr.selected].id;
        llama_sampler_accept(smpl, tok);
        if (llama_vocab_is_eog(vocab, tok)) break;
        char piece[256];
        const int len = llama_token_to_piece(vocab, tok, piece, sizeof(piece), 0, false);
        if (len > 0) fwrite(piece, 1, (size_t) len, stdout);
        fflush(stdout);
        tokens[0] = tok;
        batch = llama_batch_get_one(tokens, 1);
    }
    printf("\n");
    llama_perf_context_print(ctx);
    llama_sampler_free(smpl);
    llama_free(ctx);
    llama_model_free(model);
    llama_backend_free();
    free(tokens);
    return 0;
}
