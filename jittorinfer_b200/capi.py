"""ctypes declarations of ``libllama.so`` (``csrc/include/llama.h``) for Python programs and tests.

``load()`` builds the library if needed and returns the ``ctypes.CDLL`` with argument / result types
set for every exported function.  Struct layouts mirror the header field by field.
"""
from __future__ import annotations

import ctypes as C

from . import build

_lib = None

llama_token = C.c_int32
llama_pos = C.c_int32
llama_seq_id = C.c_int32
progress_cb_t = C.CFUNCTYPE(C.c_bool, C.c_float, C.c_void_p)
abort_cb_t = C.CFUNCTYPE(C.c_bool, C.c_void_p)


class TokenData(C.Structure):
    _fields_ = [("id", llama_token), ("logit", C.c_float), ("p", C.c_float)]


class TokenDataArray(C.Structure):
    _fields_ = [("data", C.POINTER(TokenData)), ("size", C.c_size_t), ("selected", C.c_int64), ("sorted", C.c_bool)]


class LogitBias(C.Structure):
    _fields_ = [("token", llama_token), ("bias", C.c_float)]


class Batch(C.Structure):
    _fields_ = [("n_tokens", C.c_int32), ("token", C.POINTER(llama_token)), ("embd", C.POINTER(C.c_float)),
                ("pos", C.POINTER(llama_pos)), ("n_seq_id", C.POINTER(C.c_int32)),
                ("seq_id", C.POINTER(C.POINTER(llama_seq_id))), ("logits", C.POINTER(C.c_int8))]


class Logits(C.Structure):
    _fields_ = [("type", C.c_int), ("values", C.POINTER(C.c_float)), ("indices", C.POINTER(C.c_int64)),
                ("len", C.c_int64), ("num", C.c_int64)]


class ChatMessage(C.Structure):
    _fields_ = [("role", C.c_char_p), ("content", C.c_char_p)]


class KvOverride(C.Structure):
    class _V(C.Union):
        _fields_ = [("val_i64", C.c_int64), ("val_f64", C.c_double), ("val_bool", C.c_bool), ("val_str", C.c_char * 128)]
    _anonymous_ = ("v",)
    _fields_ = [("tag", C.c_int), ("key", C.c_char * 128), ("v", _V)]


class ModelParams(C.Structure):
    _fields_ = [("devices", C.c_void_p), ("n_gpu_layers", C.c_int32), ("split_mode", C.c_int), ("main_gpu", C.c_int32),
                ("tensor_split", C.POINTER(C.c_float)),
                ("enable_tensor_parallel", C.c_bool), ("enable_expert_parallel", C.c_bool), ("enable_data_parallel", C.c_bool),
                ("enable_mpi", C.c_bool), ("offload_input", C.c_bool), ("enable_mla", C.c_bool),
                ("enable_cann_flash_attention", C.c_bool), ("tp_id", C.c_int), ("num_parallel", C.c_int),
                ("progress_callback", progress_cb_t), ("progress_callback_user_data", C.c_void_p), ("kv_overrides", C.POINTER(KvOverride)),
                ("vocab_only", C.c_bool), ("use_mmap", C.c_bool), ("use_mlock", C.c_bool), ("check_tensors", C.c_bool),
                ("enable_fused_moe", C.c_bool)]


class ContextParams(C.Structure):
    _fields_ = [("n_ctx", C.c_uint32), ("n_batch", C.c_uint32), ("n_ubatch", C.c_uint32), ("n_seq_max", C.c_uint32),
                ("n_threads", C.c_int32), ("n_threads_batch", C.c_int32),
                ("rope_scaling_type", C.c_int), ("pooling_type", C.c_int), ("attention_type", C.c_int),
                ("rope_freq_base", C.c_float), ("rope_freq_scale", C.c_float), ("yarn_ext_factor", C.c_float),
                ("yarn_attn_factor", C.c_float), ("yarn_beta_fast", C.c_float), ("yarn_beta_slow", C.c_float),
                ("yarn_orig_ctx", C.c_uint32), ("defrag_thold", C.c_float),
                ("cb_eval", C.c_void_p), ("cb_eval_user_data", C.c_void_p), ("type_k", C.c_int), ("type_v", C.c_int),
                ("logits_all", C.c_bool), ("embeddings", C.c_bool), ("offload_kqv", C.c_bool), ("flash_attn", C.c_bool),
                ("no_perf", C.c_bool), ("enable_ge", C.c_bool), ("enable_scatter_kv", C.c_bool), ("presample_count", C.c_int),
                ("abort_callback", abort_cb_t), ("abort_callback_data", C.c_void_p)]


class KvViewCell(C.Structure):
    _fields_ = [("pos", llama_pos)]


class KvView(C.Structure):
    _fields_ = [("n_cells", C.c_int32), ("n_seq_max", C.c_int32), ("token_count", C.c_int32), ("used_cells", C.c_int32),
                ("max_contiguous", C.c_int32), ("max_contiguous_idx", C.c_int32), ("cells", C.POINTER(KvViewCell)),
                ("cells_sequences", C.POINTER(llama_seq_id))]


class SamplerChainParams(C.Structure):
    _fields_ = [("no_perf", C.c_bool)]


class PerfContext(C.Structure):
    _fields_ = [("t_start_ms", C.c_double), ("t_load_ms", C.c_double), ("t_p_eval_ms", C.c_double), ("t_eval_ms", C.c_double),
                ("n_p_eval", C.c_int32), ("n_eval", C.c_int32)]


class PerfSampler(C.Structure):
    _fields_ = [("t_sample_ms", C.c_double), ("n_sample", C.c_int32)]


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = build.build_capi()
    L = C.CDLL(path, mode=C.RTLD_GLOBAL)
    vp, i32, f32, sz, b, cp = C.c_void_p, C.c_int32, C.c_float, C.c_size_t, C.c_bool, C.c_char_p

    def sig(name, res, *args):
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = list(args)

    sig("llama_model_default_params", ModelParams)
    sig("llama_context_default_params", ContextParams)
    sig("llama_backend_init", None)
    sig("llama_backend_free", None)
    sig("llama_supports_gpu_offload", b)
    sig("llama_supports_rpc", b)
    sig("llama_model_load_from_file", vp, cp, ModelParams)
    sig("llama_model_free", None, vp)
    sig("llama_model_get_vocab", vp, vp)
    sig("llama_model_rope_type", C.c_int, vp)
    sig("llama_model_n_ctx_train", i32, vp)
    sig("llama_model_is_recurrent", b, vp)
    sig("llama_model_has_encoder", b, vp)
    sig("llama_model_has_decoder", b, vp)
    sig("llama_model_decoder_start_token", llama_token, vp)
    sig("llama_model_chat_template", cp, vp, cp)
    sig("llama_init_from_model", vp, vp, ContextParams)
    sig("llama_free", None, vp)
    sig("llama_get_model", vp, vp)
    sig("llama_n_ctx", C.c_uint32, vp)
    sig("llama_n_batch", C.c_uint32, vp)
    sig("llama_pooling_type", C.c_int, vp)
    sig("llama_set_embeddings", None, vp, b)
    sig("llama_set_abort_callback", None, vp, abort_cb_t, vp)
    sig("llama_attach_threadpool", None, vp, vp, vp)
    sig("llama_clear_adapter_lora", None, vp)
    sig("llama_set_adapter_lora", i32, vp, vp, f32)
    sig("llama_batch_get_one", Batch, C.POINTER(llama_token), i32)
    sig("llama_batch_init", Batch, i32, i32, i32)
    sig("llama_batch_free", None, Batch)
    sig("llama_decode", i32, vp, Batch, b)
    sig("llama_encode", i32, vp, Batch)
    sig("llama_empty_run", b, vp)
    sig("llama_all_processed_tokens", C.c_int, vp)
    sig("llama_synchronize", None, vp)
    sig("llama_get_logits_ith", Logits, vp, i32)
    sig("llama_kv_cache_seq_rm", b, vp, llama_seq_id, llama_pos, llama_pos)
    sig("llama_kv_cache_seq_cp", None, vp, llama_seq_id, llama_seq_id, llama_pos, llama_pos)
    sig("llama_kv_cache_seq_add", None, vp, llama_seq_id, llama_pos, llama_pos, llama_pos)
    sig("llama_kv_cache_clear", None, vp)
    sig("llama_kv_cache_can_shift", b, vp)
    sig("llama_kv_cache_update", None, vp)
    sig("llama_kv_cache_view_init", KvView, vp, i32)
    sig("llama_kv_cache_view_update", None, vp, C.POINTER(KvView))
    sig("llama_kv_cache_view_free", None, C.POINTER(KvView))
    sig("llama_vocab_n_tokens", i32, vp)
    sig("llama_vocab_bos", llama_token, vp)
    sig("llama_vocab_eos", llama_token, vp)
    sig("llama_vocab_sep", llama_token, vp)
    sig("llama_vocab_is_eog", b, vp, llama_token)
    sig("llama_vocab_get_add_bos", b, vp)
    sig("llama_vocab_get_add_eos", b, vp)
    sig("llama_tokenize", i32, vp, cp, i32, C.POINTER(llama_token), i32, b, b)
    sig("llama_token_to_piece", i32, vp, llama_token, C.c_char_p, i32, i32, b)
    sig("llama_detokenize", i32, vp, C.POINTER(llama_token), i32, C.c_char_p, i32, b, b)
    sig("llama_chat_apply_template", i32, cp, C.POINTER(ChatMessage), sz, b, C.c_char_p, i32)
    sig("llama_sampler_name", cp, vp)
    sig("llama_sampler_accept", None, vp, llama_token)
    sig("llama_sampler_apply", None, vp, C.POINTER(TokenDataArray))
    sig("llama_sampler_reset", None, vp)
    sig("llama_sampler_clone", vp, vp)
    sig("llama_sampler_free", None, vp)
    sig("llama_sampler_chain_default_params", SamplerChainParams)
    sig("llama_sampler_chain_init", vp, SamplerChainParams)
    sig("llama_sampler_chain_add", None, vp, vp)
    sig("llama_sampler_chain_get", vp, vp, i32)
    sig("llama_sampler_chain_n", C.c_int, vp)
    sig("llama_sampler_init_greedy", vp)
    sig("llama_sampler_init_dist", vp, C.c_uint32)
    sig("llama_sampler_init_top_k", vp, i32)
    sig("llama_sampler_init_top_p", vp, f32, sz)
    sig("llama_sampler_init_min_p", vp, f32, sz)
    sig("llama_sampler_init_typical", vp, f32, sz)
    sig("llama_sampler_init_temp", vp, f32)
    sig("llama_sampler_init_temp_ext", vp, f32, f32, f32)
    sig("llama_sampler_init_xtc", vp, f32, f32, sz, C.c_uint32)
    sig("llama_sampler_init_penalties", vp, i32, f32, f32, f32)
    sig("llama_sampler_init_dry", vp, vp, i32, f32, f32, i32, i32, C.POINTER(cp), sz)
    sig("llama_sampler_init_logit_bias", vp, i32, i32, C.POINTER(LogitBias))
    sig("llama_sampler_init_grammar", vp, vp, cp, cp)
    sig("jib_sampler_init_grammar_pieces", vp, C.POINTER(cp), C.POINTER(C.c_int32), i32, C.POINTER(llama_token), i32, llama_token, cp, cp)
    sig("llama_perf_context", PerfContext, vp)
    sig("llama_perf_context_print", None, vp)
    sig("llama_perf_context_reset", None, vp)
    sig("llama_perf_sampler", PerfSampler, vp)
    sig("llama_perf_sampler_print", None, vp)
    sig("llama_perf_sampler_reset", None, vp)
    _lib = L
    return L


def candidates(logits):
    """(TokenDataArray, backing array) over a list of logits, token id = index."""
    n = len(logits)
    arr = (TokenData * n)()
    for i, l in enumerate(logits):
        arr[i].id, arr[i].logit, arr[i].p = i, float(l), 0.0
    return TokenDataArray(C.cast(arr, C.POINTER(TokenData)), n, -1, False), arr
