"""libllama.so (llama.h C API) on the CPU: samplers, vocabulary, decode vs the fp32 oracle, KV operations.

The scenarios follow the reference's manual integration programs: a scripted single sequence
(tests/main/single_sequence.cpp:181-372) and several clients sharing a system prompt through
``llama_kv_cache_seq_cp`` with continuous batching and ``seq_rm`` on finish (tests/main/multi_sequence.cpp:140-566),
here with a pass/fail criterion: the greedy tokens must equal the fp32 oracle's.
"""
import ctypes as C
import math
import os
import subprocess
import sys

import pytest
import torch

from jittorinfer_b200 import build, capi
from jittorinfer_b200.models.hparams import preset
from jittorinfer_b200.models.oracle import OracleModel
from jittorinfer_b200.models.weights import random_weights, write_random_gguf
from jittorinfer_b200.tokenizer import Tokenizer


@pytest.fixture(scope="module")
def L():
    return capi.load()


@pytest.fixture(scope="module")
def gguf_path(tmp_path_factory):
    p = str(tmp_path_factory.mktemp("capi") / "tiny.gguf")
    write_random_gguf(p, preset("tiny"), seed=0)
    return p


def apply(L, smpl, logits):
    arr, keep = capi.candidates(logits)
    L.llama_sampler_apply(smpl, C.byref(arr))
    out = [(arr.data[i].id, arr.data[i].logit, arr.data[i].p) for i in range(arr.size)]
    return arr, out


# ---- samplers ---------------------------------------------------------------------------------------
def test_sampler_greedy_topk_topp_minp(L):
    logits = [0.1, 2.0, -1.0, 3.0, 1.5]
    s = L.llama_sampler_init_greedy()
    arr, _ = apply(L, s, logits)
    assert arr.data[arr.selected].id == 3
    L.llama_sampler_free(s)

    s = L.llama_sampler_init_top_k(2)
    arr, out = apply(L, s, logits)
    assert [o[0] for o in out] == [3, 1] and arr.sorted
    L.llama_sampler_free(s)

    probs = torch.softmax(torch.tensor(logits), 0)
    s = L.llama_sampler_init_top_p(0.8, 1)
    _, out = apply(L, s, logits)
    order = torch.argsort(probs, descending=True).tolist()
    cum, want = 0.0, []
    for i in order:
        want.append(i)
        cum += float(probs[i])
        if cum >= 0.8:
            break
    assert [o[0] for o in out] == want
    assert all(abs(o[2] - float(probs[o[0]])) < 1e-6 for o in out)
    L.llama_sampler_free(s)

    s = L.llama_sampler_init_min_p(0.3, 1)
    _, out = apply(L, s, logits)
    pmax = float(probs.max())
    assert sorted(o[0] for o in out) == sorted(i for i in range(5) if float(probs[i]) >= 0.3 * pmax)
    L.llama_sampler_free(s)


def test_sampler_temperature_and_dynatemp(L):
    logits = [1.0, 2.0, 4.0]
    s = L.llama_sampler_init_temp(2.0)
    _, out = apply(L, s, logits)
    assert [round(o[1], 5) for o in out] == [0.5, 1.0, 2.0]
    L.llama_sampler_free(s)
    s = L.llama_sampler_init_temp(0.0)                # collapses to the arg-max
    _, out = apply(L, s, logits)
    assert out[2][1] == 4.0 and out[0][1] == -math.inf and out[1][1] == -math.inf
    L.llama_sampler_free(s)
    # entropy-scaled temperature: uniform logits -> normalised entropy 1 -> temperature t + delta
    s = L.llama_sampler_init_temp_ext(1.0, 0.5, 1.0)
    _, out = apply(L, s, [3.0, 3.0, 3.0, 3.0])
    assert all(abs(o[1] - 2.0) < 1e-5 for o in out)
    L.llama_sampler_free(s)


def test_sampler_typical_and_xtc(L):
    logits = [5.0, 4.9, 1.0, 0.5, -3.0]
    s = L.llama_sampler_init_typical(0.5, 1)
    _, out = apply(L, s, logits)
    probs = torch.softmax(torch.tensor(logits), 0)
    ent = float(-(probs * probs.log()).sum())
    closest = min(range(5), key=lambda i: abs(-math.log(float(probs[i])) - ent))
    assert out[0][0] == closest and 1 <= len(out) < 5
    L.llama_sampler_free(s)
    # XTC with probability 1: every candidate at or above the threshold except the least likely of them goes
    s = L.llama_sampler_init_xtc(1.0, 0.1, 1, 7)
    _, out = apply(L, s, logits)
    assert [o[0] for o in out] == [1, 2, 3, 4]
    L.llama_sampler_free(s)
    s = L.llama_sampler_init_xtc(0.0, 0.1, 1, 7)      # probability 0: untouched
    _, out = apply(L, s, logits)
    assert len(out) == 5
    L.llama_sampler_free(s)


def test_sampler_penalties_bias_dry(L):
    s = L.llama_sampler_init_penalties(4, 2.0, 0.5, 0.25)
    for t in (1, 1, 2):
        L.llama_sampler_accept(s, t)
    _, out = apply(L, s, [1.0, 2.0, -2.0, 1.0])
    got = {o[0]: o[1] for o in out}
    assert abs(got[0] - 1.0) < 1e-6 and abs(got[3] - 1.0) < 1e-6
    assert abs(got[1] - (2.0 / 2.0 - 2 * 0.5 - 0.25)) < 1e-6
    assert abs(got[2] - (-2.0 * 2.0 - 1 * 0.5 - 0.25)) < 1e-6
    for t in (3, 3, 3, 3):                             # window of 4 forgets tokens 1 and 2
        L.llama_sampler_accept(s, t)
    _, out = apply(L, s, [1.0, 2.0, -2.0, 1.0])
    assert abs({o[0]: o[1] for o in out}[1] - 2.0) < 1e-6
    L.llama_sampler_free(s)

    bias = (capi.LogitBias * 2)((2, 5.0), (0, -1.0))
    s = L.llama_sampler_init_logit_bias(4, 2, bias)
    _, out = apply(L, s, [0.0, 0.0, 0.0, 0.0])
    assert [o[1] for o in out] == [-1.0, 0.0, 5.0, 0.0]
    L.llama_sampler_free(s)

    # history "7 8 9 4 7 8": token 9 would extend the repeat "7 8" (length 2)
    s = L.llama_sampler_init_dry(None, 64, 0.8, 1.75, 2, -1, None, 0)
    for t in (7, 8, 9, 4, 7, 8):
        L.llama_sampler_accept(s, t)
    _, out = apply(L, s, [0.0] * 12)
    got = {o[0]: o[1] for o in out}
    assert abs(got[9] + 0.8) < 1e-6 and all(v == 0.0 for k, v in got.items() if k != 9)
    L.llama_sampler_accept(s, 9)                        # now "7 8 9" repeats: token 4 gets multiplier * base^(3-2)
    _, out = apply(L, s, [0.0] * 12)
    assert abs({o[0]: o[1] for o in out}[4] + 0.8 * 1.75) < 1e-5
    L.llama_sampler_free(s)


def test_dry_breaker_spelled_with_several_tokens(L, gguf_path):
    """A sequence breaker that no single token contains ("ab" in the byte-level toy vocabulary) stops a repetition match like
    a one-token breaker does: the match may not reach back across the place where the token sequence "a" "b" ends."""
    mp = L.llama_model_default_params()
    mp.vocab_only = True
    model = L.llama_model_load_from_file(gguf_path.encode(), mp)
    vocab = L.llama_model_get_vocab(model)
    buf = (capi.llama_token * 16)()

    def ids(text):
        n = L.llama_tokenize(vocab, text.encode(), len(text), buf, 16, False, False)
        return list(buf[:n])
    (a, b), (q,), (x,), (y,), (z,) = ids("ab"), ids("q"), ids("x"), ids("y"), ids("z")
    hist = [q, a, b, x, y, z, q, a, b, x, y]           # "q a b x y" repeats; z followed its first occurrence
    n_vocab = L.llama_vocab_n_tokens(vocab)

    def penalty_on_z(breakers):
        arr = (C.c_char_p * len(breakers))(*[s.encode() for s in breakers]) if breakers else None
        smp = L.llama_sampler_init_dry(vocab, 64, 0.8, 1.75, 2, -1, arr, len(breakers))
        for t in hist:
            L.llama_sampler_accept(smp, t)
        _, out = apply(L, smp, [0.0] * n_vocab)
        L.llama_sampler_free(smp)
        return -{o[0]: o[1] for o in out}[z]
    assert abs(penalty_on_z([]) - 0.8 * 1.75 ** 3) < 1e-4              # repeat of length 5, allowed 2
    assert abs(penalty_on_z(["ab"]) - 0.8) < 1e-5                      # only "x y" after the breaker counts: length 2
    assert abs(penalty_on_z(["y"]) - 0.0) < 1e-6                       # a one-token breaker right at the end: no match at all
    # a breaker that begins inside a token: "ex" over the merged token "he" followed by "x"
    (he,) = ids("he")
    assert len(ids("he")) == 1 and len(ids("ex")) == 2
    hist[:] = [q, he, x, a, y, z, q, he, x, a, y]                      # "q he x a y" repeats; "ex" sits across "he" | "x"
    assert abs(penalty_on_z([]) - 0.8 * 1.75 ** 3) < 1e-4
    assert abs(penalty_on_z(["ex"]) - 0.8) < 1e-5                      # only "a y" after the breaker counts
    L.llama_model_free(model)


def test_sampler_chain_dist_clone_and_perf(L):
    p = capi.SamplerChainParams(False)
    chain = L.llama_sampler_chain_init(p)
    L.llama_sampler_chain_add(chain, L.llama_sampler_init_top_k(3))
    L.llama_sampler_chain_add(chain, L.llama_sampler_init_temp(0.7))
    L.llama_sampler_chain_add(chain, L.llama_sampler_init_dist(1234))
    assert L.llama_sampler_chain_n(chain) == 3
    assert L.llama_sampler_name(L.llama_sampler_chain_get(chain, 0)) == b"top-k"
    clone = L.llama_sampler_clone(chain)
    logits = [0.0, 1.0, 2.0, 3.0, 2.5, -1.0]
    a, b = [], []
    for _ in range(50):
        arr, _ = apply(L, chain, logits)
        a.append(arr.data[arr.selected].id)
        arr, _ = apply(L, clone, logits)
        b.append(arr.data[arr.selected].id)
        L.llama_sampler_accept(chain, a[-1])
    assert a == b and set(a) <= {2, 3, 4} and len(set(a)) > 1
    perf = L.llama_perf_sampler(chain)
    assert perf.n_sample == 50 and perf.t_sample_ms >= 0
    L.llama_sampler_reset(chain)
    assert L.llama_perf_sampler(chain).n_sample == 0
    # the same seed reproduces the stream after a reset
    c = []
    for _ in range(50):
        arr, _ = apply(L, chain, logits)
        c.append(arr.data[arr.selected].id)
    assert c == a
    L.llama_sampler_free(chain)
    L.llama_sampler_free(clone)
    assert L.llama_sampler_init_grammar(None, b"root ::= \"a\"", b"root") is None
    g = L.llama_sampler_init_grammar(None, b"", b"")
    assert L.llama_sampler_name(g) == b"grammar"
    L.llama_sampler_free(g)


# ---- model metadata, vocabulary, chat template ------------------------------------------------------------
def test_vocab_only_model_and_tokenizer_parity(L, gguf_path):
    mp = L.llama_model_default_params()
    mp.vocab_only = True
    model = L.llama_model_load_from_file(gguf_path.encode(), mp)
    assert model
    hp = preset("tiny")
    vocab = L.llama_model_get_vocab(model)
    assert L.llama_vocab_n_tokens(vocab) == hp.n_vocab
    assert L.llama_model_n_ctx_train(model) == hp.n_ctx_train
    assert L.llama_model_has_decoder(model) and not L.llama_model_has_encoder(model)
    from jittorinfer_b200.gguf.io import GGUFReader
    ref = Tokenizer.from_gguf_kv(GGUFReader(gguf_path).kv)
    text = "Hello, wörld! 你好 123 tokens\n\n  indented"
    raw = text.encode()
    buf = (capi.llama_token * 256)()
    n = L.llama_tokenize(vocab, raw, len(raw), buf, 256, False, True)
    assert n > 0 and list(buf[:n]) == ref.encode(text, add_special=False)
    assert L.llama_tokenize(vocab, raw, len(raw), buf, 2, False, True) == -n
    out = C.create_string_buffer(512)
    m = L.llama_detokenize(vocab, buf, n, out, 512, False, False)
    assert out.raw[:m].decode() == text
    piece = C.create_string_buffer(64)
    k = L.llama_token_to_piece(vocab, buf[0], piece, 64, 0, False)
    assert piece.raw[:k] == ref.piece_bytes(buf[0])
    assert L.llama_vocab_bos(vocab) == ref.bos and L.llama_vocab_eos(vocab) == ref.eos
    assert L.llama_vocab_is_eog(vocab, ref.eos)
    assert L.llama_init_from_model(model, L.llama_context_default_params()) is None      # vocab_only: no weights
    L.llama_model_free(model)
    assert L.llama_model_load_from_file(b"/nonexistent.gguf", mp) is None


def test_chat_template(L):
    msgs = (capi.ChatMessage * 3)((b"system", b"Be brief."), (b"user", b"Hi"), (b"assistant", b"Hello"))
    buf = C.create_string_buffer(256)
    n = L.llama_chat_apply_template(None, msgs, 3, True, buf, 256)
    want = "Be brief.\n\nUser: Hi\n\nAssistant: Hello<｜end▁of▁sentence｜>Assistant:"
    assert buf.raw[:n].decode() == want
    jinja = b"{{ 'Assistant: ' + message['content'] + eos_token }}"
    assert L.llama_chat_apply_template(jinja, msgs, 3, False, buf, 256) == n - len("Assistant:")
    assert L.llama_chat_apply_template(b"chatml", msgs, 3, True, buf, 256) == -1


# ---- decode ---------------------------------------------------------------------------------------------
def _greedy(L, ctx, row):
    lg = L.llama_get_logits_ith(ctx, row)
    assert lg.len > 0
    if lg.type == 1:
        return int(lg.indices[0])
    return int(torch.tensor([lg.values[i] for i in range(lg.len)]).argmax())


@pytest.fixture(scope="module")
def model(L, gguf_path):
    mp = L.llama_model_default_params()
    mp.n_gpu_layers = 0                                    # CPU: fp32 reference ops
    seen = []
    cb = capi.progress_cb_t(lambda p, ud: seen.append(p) or True)
    mp.progress_callback = cb
    m = L.llama_model_load_from_file(gguf_path.encode(), mp)
    assert m and seen[0] == 0.0 and seen[-1] == 1.0
    yield m
    L.llama_model_free(m)


def _oracle_tokens(prompt, n_new):
    hp = preset("tiny")
    return OracleModel(hp, random_weights(hp, seed=0)).generate(prompt, n_new)


def test_single_sequence_greedy_matches_oracle(L, model):
    cp = L.llama_context_default_params()
    cp.n_ctx, cp.n_batch, cp.n_ubatch, cp.n_seq_max = 256, 64, 16, 2      # prompt of 32 runs as two chunks
    ctx = L.llama_init_from_model(model, cp)
    assert ctx and L.llama_n_ctx(ctx) == 256 and L.llama_n_batch(ctx) == 64
    prompt = torch.randint(0, 1024, (32,), generator=torch.Generator().manual_seed(0)).tolist()
    want = _oracle_tokens(prompt, 32)
    toks = (capi.llama_token * 32)(*prompt)
    assert L.llama_decode(ctx, L.llama_batch_get_one(toks, 32), False) == 0
    got = []
    for _ in range(32):
        got.append(_greedy(L, ctx, -1))
        one = (capi.llama_token * 1)(got[-1])
        assert L.llama_decode(ctx, L.llama_batch_get_one(one, 1), False) == 0
    assert got == want
    perf = L.llama_perf_context(ctx)
    assert perf.n_p_eval == 32 and perf.n_eval == 32 and perf.t_eval_ms > 0
    # rewind: drop the generated tail and decode it again from the prompt
    assert L.llama_kv_cache_seq_rm(ctx, 0, 32, -1)
    assert not L.llama_kv_cache_seq_rm(ctx, 0, 3, 9)        # a hole in the middle is not representable
    one = (capi.llama_token * 1)(want[0])
    assert L.llama_decode(ctx, L.llama_batch_get_one(one, 1), False) == 0
    assert _greedy(L, ctx, 0) == want[1]
    assert not L.llama_kv_cache_can_shift(ctx)
    L.llama_free(ctx)


def test_multi_sequence_shared_prefix_topk_and_view(L, model):
    cp = L.llama_context_default_params()
    cp.n_ctx, cp.n_batch, cp.n_ubatch, cp.n_seq_max, cp.presample_count = 512, 128, 128, 4, 8
    cp.defrag_thold = 0.0
    ctx = L.llama_init_from_model(model, cp)
    g = torch.Generator().manual_seed(1)
    system = torch.randint(0, 1024, (20,), generator=g).tolist()
    tails = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (5, 9, 3)]
    n_new = 12
    want = [_oracle_tokens(system + t, n_new) for t in tails]

    # the shared prompt is decoded once in sequence 0 and aliased into sequences 1..3
    toks = (capi.llama_token * 20)(*system)
    assert L.llama_decode(ctx, L.llama_batch_get_one(toks, 20), False) == 0
    for s in (1, 2, 3):
        L.llama_kv_cache_seq_cp(ctx, 0, s, 0, -1)
    view = L.llama_kv_cache_view_init(ctx, 4)
    L.llama_kv_cache_view_update(ctx, C.byref(view))
    assert view.token_count == 80 and view.used_cells == 20
    owners = [view.cells_sequences[c * 4 + k] for c in range(view.n_cells) if view.cells[c].pos == 0 for k in range(4)]
    assert sorted(owners) == [0, 1, 2, 3]

    # one batch carries the three different tails (continuous batching), outputs only at each tail's end
    total = sum(len(t) for t in tails)
    b = L.llama_batch_init(128, 0, 1)
    k = 0
    last_idx = []
    for s, tail in zip((1, 2, 3), tails):
        for j, t in enumerate(tail):
            b.token[k], b.pos[k], b.n_seq_id[k], b.seq_id[k][0] = t, 20 + j, 1, s
            b.logits[k] = int(j == len(tail) - 1)
            k += 1
        last_idx.append(k - 1)
    b.n_tokens = total
    assert L.llama_decode(ctx, b, False) == 0
    lg = L.llama_get_logits_ith(ctx, last_idx[0])
    assert lg.type == 1 and lg.len == 8 and lg.num == 3
    assert all(lg.values[i] >= lg.values[i + 1] for i in range(7))
    got = [[_greedy(L, ctx, i)] for i in last_idx]
    lens = [20 + len(t) for t in tails]
    for step in range(1, n_new):
        for j, s in enumerate((1, 2, 3)):
            b.token[j], b.pos[j], b.n_seq_id[j], b.seq_id[j][0], b.logits[j] = got[j][-1], lens[j], 1, s, 1
            lens[j] += 1
        b.n_tokens = 3
        assert L.llama_decode(ctx, b, False) == 0
        for j in range(3):
            got[j].append(_greedy(L, ctx, j))
    assert got == want

    # finished clients free their cells; the system prompt stays while sequence 0 holds it
    for s in (1, 2, 3):
        assert L.llama_kv_cache_seq_rm(ctx, s, -1, -1)
    L.llama_kv_cache_update(ctx)                            # defrag_thold = 0: compacts if there are holes
    L.llama_kv_cache_view_update(ctx, C.byref(view))
    assert view.token_count == 20 and view.used_cells == 20
    L.llama_kv_cache_clear(ctx)
    L.llama_kv_cache_view_update(ctx, C.byref(view))
    assert view.used_cells == 0 and view.max_contiguous == view.n_cells
    L.llama_kv_cache_view_free(C.byref(view))

    # a batch that cannot fit returns 1 and leaves the cache as it was
    big = torch.randint(0, 1024, (128,), generator=g).tolist()
    for j, t in enumerate(big):
        b.token[j], b.pos[j], b.n_seq_id[j], b.seq_id[j][0], b.logits[j] = t, j, 1, 0, 0
    b.n_tokens = 128
    rcs = []
    for s in range(4):
        for j in range(128):
            b.seq_id[j][0] = s
        rcs.append(L.llama_decode(ctx, b, False))
    assert rcs == [0, 0, 0, 0]
    # n_ctx = 512 tokens is 8 blocks of 64 plus one spare block per sequence: 12 blocks, 8 are in use
    for s in (0, 1, 2):
        for j in range(128):
            b.seq_id[j][0] = s
            b.pos[j] = 128 + j
        rcs.append(L.llama_decode(ctx, b, False))
    assert rcs[4:] == [0, 0, 1]
    view = L.llama_kv_cache_view_init(ctx, 4)
    L.llama_kv_cache_view_update(ctx, C.byref(view))
    assert view.token_count == 4 * 128 + 2 * 128
    L.llama_kv_cache_view_free(C.byref(view))
    L.llama_batch_free(b)
    L.llama_free(ctx)


def test_errors_are_reported_not_fatal(L, model):
    cp = L.llama_context_default_params()
    cp.n_ctx, cp.n_batch, cp.n_seq_max = 128, 16, 1
    ctx = L.llama_init_from_model(model, cp)
    toks = (capi.llama_token * 20)(*range(20))
    assert L.llama_decode(ctx, L.llama_batch_get_one(toks, 20), False) == -1       # larger than n_batch
    bad = (capi.llama_token * 1)(5000)
    assert L.llama_decode(ctx, L.llama_batch_get_one(bad, 1), False) == -1         # token id out of range
    assert L.llama_encode(ctx, L.llama_batch_get_one(toks, 1)) == -1
    assert L.llama_get_logits_ith(ctx, 0).len == -1
    stop = capi.abort_cb_t(lambda ud: True)
    L.llama_set_abort_callback(ctx, stop, None)
    assert L.llama_decode(ctx, L.llama_batch_get_one(toks, 4), False) == 2
    L.llama_free(ctx)


# ---- a C program linked against the library (the interpreter is started by the library) -------------------------
C_PROGRAM = r"""
#include "llama.h"
#include <stdio.h>
#include <stdlib.h>
int main(int argc, char ** argv) {
    llama_backend_init();
    struct llama_model_params mp = llama_model_default_params();
    mp.n_gpu_layers = 0;
    struct llama_model * model = llama_model_load_from_file(argv[1], mp);
    if (!model) return 2;
    struct llama_context_params cp = llama_context_default_params();
    cp.n_ctx = 256; cp.n_batch = 64; cp.n_seq_max = 1;
    struct llama_context * ctx = llama_init_from_model(model, cp);
    if (!ctx) return 3;
    int n_prompt = argc - 2;
    llama_token * prompt = malloc(sizeof(llama_token) * n_prompt);
    for (int i = 0; i < n_prompt; ++i) prompt[i] = atoi(argv[2 + i]);
    struct llama_sampler * smpl = llama_sampler_chain_init(llama_sampler_chain_default_params());
    llama_sampler_chain_add(smpl, llama_sampler_init_greedy());
    int n_vocab = llama_vocab_n_tokens(llama_model_get_vocab(model));
    llama_token_data * cand = malloc(sizeof(llama_token_data) * n_vocab);
    struct llama_batch batch = llama_batch_get_one(prompt, n_prompt);
    for (int step = 0; step < 8; ++step) {
        if (llama_decode(ctx, batch, false) != 0) return 4;
        llama_logits lg = llama_get_logits_ith(ctx, -1);
        for (int i = 0; i < n_vocab; ++i) { cand[i].id = i; cand[i].logit = lg.values[i]; cand[i].p = 0; }
        llama_token_data_array arr = { cand, (size_t) n_vocab, -1, false };
        llama_sampler_apply(smpl, &arr);
        llama_token tok = arr.data[arr.selected].id;
        llama_sampler_accept(smpl, tok);
        printf("%d ", tok);
        prompt[0] = tok;
        batch = llama_batch_get_one(prompt, 1);
    }
    printf("\n");
    llama_sampler_free(smpl);
    llama_free(ctx);
    llama_model_free(model);
    llama_backend_free();
    return 0;
}
"""


def test_c_program_embeds_the_engine(L, gguf_path, tmp_path):
    src = tmp_path / "simple.c"
    src.write_text(C_PROGRAM)
    exe = str(tmp_path / "simple")
    inc = os.path.join(build.CSRC, "include")
    subprocess.run(["gcc", "-std=c11", "-O1", "-I", inc, str(src), "-o", exe, f"-L{build.LIBDIR}", "-lllama",
                    f"-Wl,-rpath,{build.LIBDIR}"], check=True)
    prompt = torch.randint(0, 1024, (16,), generator=torch.Generator().manual_seed(5)).tolist()
    env = dict(os.environ, JITTORINFER_PYTHON=sys.executable)
    r = subprocess.run([exe, gguf_path] + [str(t) for t in prompt], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(x) for x in r.stdout.split()] == _oracle_tokens(prompt, 8)


def test_engine_uses_the_native_sampler_chain():
    """The engine's per-request sampler is the C++ chain: seeded runs repeat, dry and dynatemp are honoured, and with a
    sharp distribution it agrees with the numpy chain."""
    import numpy as np
    from jittorinfer_b200.runtime.sampling import HostSampler, NativeSampler, SamplingParams, make_sampler
    sp = SamplingParams(temperature=0.8, top_k=5, top_p=0.9, min_p=0.0, seed=7)
    vals = np.array([4.0, 3.5, 1.0, 0.5, -2.0, -5.0], dtype=np.float32)
    ids = np.array([10, 11, 12, 13, 14, 15], dtype=np.int32)
    a, b = make_sampler(sp, 100), make_sampler(sp, 100)
    assert isinstance(a, NativeSampler)
    seq_a = [a.sample(vals, ids) for _ in range(40)]
    assert seq_a == [b.sample(vals, ids) for _ in range(40)] and set(seq_a) <= {10, 11} | {12} and len(set(seq_a)) > 1
    sharp = SamplingParams(temperature=0.01, top_k=0, top_p=1.0, min_p=0.0, seed=1)
    assert NativeSampler(sharp, 100).sample(vals, ids) == HostSampler(sharp).sample(vals, ids) == 10
    # penalties through accept(): token 10 was just produced twice, a strong repeat penalty moves the choice to 11
    pen = NativeSampler(SamplingParams(temperature=0.0, repeat_penalty=4.0, repeat_last_n=8), 100)
    pen.accept(10)
    pen.accept(10)
    assert pen.sample(vals, ids) == 11
    # dry: history 20 21 22 20 21 -> 22 would repeat the sequence; the penalty hands the arg-max to another token
    dry = NativeSampler(SamplingParams(temperature=0.0, dry_multiplier=5.0, dry_allowed_length=2), 100)
    for t in (20, 21, 22, 20, 21):
        dry.accept(t)
    v2 = np.array([3.0, 2.9], dtype=np.float32)
    assert dry.sample(v2, np.array([22, 23], dtype=np.int32)) == 23
    # engine end to end with a sampled request
    hp = preset("tiny")
    from jittorinfer_b200.models.deepseek2 import DeepSeek2Model
    from jittorinfer_b200.runtime.engine import EngineConfig, LLMEngine
    outs = []
    for _ in range(2):
        eng = LLMEngine(DeepSeek2Model(hp, random_weights(hp, seed=0).items(), dtype=torch.float32), EngineConfig(n_ctx=512, n_batch=32, n_parallel=2))
        outs.append(eng.generate([[1, 2, 3, 4, 5]], SamplingParams(temperature=0.9, seed=3, ignore_eos=True, dynatemp_range=0.3), max_new_tokens=8))
    assert outs[0] == outs[1] and len(outs[0][0]) == 8


def test_kv_overrides_change_the_loaded_hyperparameters(L, gguf_path):
    """llama_model_params.kv_overrides: metadata of the file is replaced before the hyper-parameters are read -- here the
    number of experts used per token, which changes the logits."""
    def first_logits(overrides):
        mp = L.llama_model_default_params()
        mp.n_gpu_layers = 0
        keep = None
        if overrides:
            keep = (capi.KvOverride * (len(overrides) + 1))()
            for i, (k, v) in enumerate(overrides.items()):
                keep[i].tag, keep[i].key, keep[i].val_i64 = 0, k.encode(), v
            mp.kv_overrides = keep
        m = L.llama_model_load_from_file(gguf_path.encode(), mp)
        assert m
        cp = L.llama_context_default_params()
        cp.n_ctx, cp.n_batch, cp.n_seq_max = 128, 32, 1
        ctx = L.llama_init_from_model(m, cp)
        toks = (capi.llama_token * 6)(3, 9, 27, 81, 243, 729)
        assert L.llama_decode(ctx, L.llama_batch_get_one(toks, 6), False) == 0
        lg = L.llama_get_logits_ith(ctx, -1)
        out = [lg.values[i] for i in range(32)]
        L.llama_free(ctx)
        L.llama_model_free(m)
        return out
    base = first_logits(None)
    same = first_logits({"deepseek2.expert_used_count": 2})       # the file's own value
    one = first_logits({"deepseek2.expert_used_count": 1})
    assert base == same and base != one


def test_context_rope_overrides(L, gguf_path):
    """llama_context_params RoPE fields: the defaults keep the model's values; a different frequency base changes the
    positions' rotation and therefore the logits of every token after the first."""
    def logits(freq_base):
        mp = L.llama_model_default_params()
        mp.n_gpu_layers = 0
        m = L.llama_model_load_from_file(gguf_path.encode(), mp)
        cp = L.llama_context_default_params()
        cp.n_ctx, cp.n_batch, cp.n_seq_max, cp.rope_freq_base = 128, 32, 1, freq_base
        ctx = L.llama_init_from_model(m, cp)
        toks = (capi.llama_token * 5)(11, 22, 33, 44, 55)
        assert L.llama_decode(ctx, L.llama_batch_get_one(toks, 5), False) == 0
        lg = L.llama_get_logits_ith(ctx, -1)
        out = [lg.values[i] for i in range(16)]
        L.llama_free(ctx)
        L.llama_model_free(m)
        return out
    assert logits(0.0) == logits(10000.0)          # 10000 is the file's own base
    assert logits(0.0) != logits(500000.0)


def test_example_program_builds_and_runs(gguf_path, tmp_path):
    """examples/simple.c (tokenise, decode with the device top-k, sampler chain, detokenise) against the tiny model."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "simple")
    subprocess.run(["gcc", "-std=c11", "-O1", "-Wall", "-Werror", "-I", os.path.join(build.CSRC, "include"),
                    os.path.join(root, "examples", "simple.c"), "-o", exe, f"-L{build.LIBDIR}", "-lllama", f"-Wl,-rpath,{build.LIBDIR}"],
                   check=True)
    env = dict(os.environ, JITTORINFER_PYTHON=sys.executable)
    r = subprocess.run([exe, gguf_path, "hello there", "6", "0"], capture_output=True, text=True, timeout=600, env=env, errors="replace")
    assert r.returncode == 0, r.stderr[-2000:]
    assert "eval time" in r.stderr and len(r.stdout) >= 1
