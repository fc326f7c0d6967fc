"""A byte-level toy vocabulary for random-init GGUF files.

Real checkpoints carry the DeepSeek BPE vocabulary (``tokenizer.ggml.*`` keys read in
src/llama-vocab.cpp:427-530).  Random-init test models get 256 byte tokens (GPT-2 byte alphabet),
a few merges and control tokens, so that the tokenizer and chat-template paths can be exercised
end to end without a real vocabulary file.
"""
from __future__ import annotations

from typing import Any, Dict


def gpt2_byte_alphabet():
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


def toy_vocab_kv(n_vocab: int, bos_id: int, eos_id: int) -> Dict[str, Any]:
    alpha = gpt2_byte_alphabet()
    tokens = [None] * n_vocab
    types = [1] * n_vocab
    specials = {bos_id: "<｜begin▁of▁sentence｜>", eos_id: "<｜end▁of▁sentence｜>"}
    byte_tokens = [alpha[b] for b in range(256)]
    merges_src = [("Ġ", "t"), ("h", "e"), ("Ġt", "he"), ("i", "n"), ("e", "r"), ("Ġ", "a"), ("o", "n"), ("r", "e")]
    pieces = byte_tokens + [a + b for a, b in merges_src]
    it = iter(pieces)
    for i in range(n_vocab):
        if i in specials:
            tokens[i] = specials[i]
            types[i] = 3
            continue
        nxt = next(it, None)
        if nxt is None:
            tokens[i] = f"<unused_{i}>"
            types[i] = 5
        else:
            tokens[i] = nxt
    merges = [f"{a} {b}" for a, b in merges_src]
    return {
        "tokenizer.ggml.model": "gpt2",
        "tokenizer.ggml.pre": "deepseek-llm",
        "tokenizer.ggml.tokens": tokens,
        "tokenizer.ggml.token_type": ("i32", types),
        "tokenizer.ggml.merges": merges,
        "tokenizer.ggml.add_bos_token": True,
        "tokenizer.ggml.add_eos_token": False,
    }
