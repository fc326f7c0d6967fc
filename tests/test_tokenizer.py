"""Native BPE tokenizer: pre-split rules, merges, specials, byte-level round trip."""
from jittorinfer_b200.tokenizer import Tokenizer
from jittorinfer_b200.utils.toy_vocab import gpt2_byte_alphabet, toy_vocab_kv


def _tok(n_vocab=512, bos=300, eos=301):
    kv = toy_vocab_kv(n_vocab, bos, eos)
    kv = {k: (v[1] if isinstance(v, tuple) else v) for k, v in kv.items()}
    kv["tokenizer.ggml.bos_token_id"] = bos
    kv["tokenizer.ggml.eos_token_id"] = eos
    return Tokenizer.from_gguf_kv(kv), kv


def test_round_trip_any_bytes_and_merges():
    tok, kv = _tok()
    for text in ["the cat in the hat", "Hello, World! 123\n\n  tabs\tand  spaces  ", "中文字符和한국어 mixed ünïcödé", "a" * 50, ""]:
        ids = tok.encode(text, add_special=False)
        assert tok.decode(ids) == text
    toks = kv["tokenizer.ggml.tokens"]
    ids = tok.encode(" the", add_special=False)
    assert [toks[i] for i in ids] == ["Ġthe"]                       # merges Ġ+t, h+e, Ġt+he applied in rank order
    ids = tok.encode("then", add_special=False)
    assert [toks[i] for i in ids] == ["t", "he", "n"]                # no 't he' merge without the leading space


def test_bos_and_special_token_partition():
    tok, kv = _tok()
    eos_text = kv["tokenizer.ggml.tokens"][301]
    ids = tok.encode("hi" + eos_text + "there", add_special=True, parse_special=True)
    assert ids[0] == 300 and 301 in ids
    ids2 = tok.encode("hi" + eos_text + "there", add_special=False, parse_special=False)
    assert 301 not in ids2 and tok.decode(ids2) == "hi" + eos_text + "there"
    assert tok.is_eog(301) and not tok.is_eog(5)
    assert tok.piece_bytes(301) == b"" and tok.piece_bytes(301, special=True) == eos_text.encode()


def test_pre_split_rules():
    tok, _ = _tok()
    # words keep one leading space; digits split from letters; newlines are single pieces; trailing spaces group
    cases = {"Hello world": ["Hello", " world"], "abc123def": ["abc", "123", "def"], "a\n\nb": ["a", "\n", "\n", "b"],
             "x  ": ["x", "  "], "wow!!! ok": ["wow", "!!!", " ok"], "数字42": ["数字", "42"]}
    toks = toy_vocab_kv(512, 300, 301)["tokenizer.ggml.tokens"]
    alpha = gpt2_byte_alphabet()
    for text, words in cases.items():
        ids = tok.encode(text, add_special=False)
        # boundaries: no token may straddle two pre-split words
        pieces = [tok.piece_bytes(i) for i in ids]
        joined = b"".join(pieces)
        assert joined == text.encode()
        cuts = set()
        pos = 0
        for p in pieces:
            pos += len(p)
            cuts.add(pos)
        pos = 0
        for w in words:
            pos += len(w.encode())
            assert pos in cuts, (text, w)


def test_incomplete_utf8_tail():
    tok, _ = _tok()
    b = "é中".encode()
    assert tok.incomplete_utf8_tail(b) == 0
    assert tok.incomplete_utf8_tail(b[:-1]) == 2 and tok.incomplete_utf8_tail(b[:1]) == 1
