"""JSON schema -> GBNF: the generated grammars accept the documents the schema allows and reject the others."""
import json

import pytest

from jittorinfer_b200.server.json_schema import (SchemaError, grammar_accepts, grammar_for_response_format,
                                                 json_schema_to_grammar)


def ok(g, doc):
    return grammar_accepts(g, json.dumps(doc) if not isinstance(doc, str) else doc)


def test_primitives_and_enum():
    g = json_schema_to_grammar({"type": "integer"})
    assert ok(g, "12") and ok(g, "-7") and not ok(g, "1.5") and not ok(g, '"1"')
    g = json_schema_to_grammar({"type": "number"})
    assert ok(g, "3.25") and ok(g, "-1e5") and not ok(g, "abc")
    g = json_schema_to_grammar({"type": "string", "minLength": 2, "maxLength": 3})
    assert ok(g, '"ab"') and ok(g, '"abc"') and not ok(g, '"a"') and not ok(g, '"abcd"')
    g = json_schema_to_grammar({"enum": ["red", "green", 3]})
    assert ok(g, '"red"') and ok(g, "3") and not ok(g, '"blue"')
    g = json_schema_to_grammar({"type": ["string", "null"]})
    assert ok(g, "null") and ok(g, '"x"') and not ok(g, "1")
    g = json_schema_to_grammar({"type": "string", "format": "date"})
    assert ok(g, '"2026-11-25"') and not ok(g, '"2026-13-01"')


def test_object_required_optional_and_nesting():
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"},
                                               "tags": {"type": "array", "items": {"type": "string"}, "minItems": 1, "maxItems": 2}},
              "required": ["name"]}
    g = json_schema_to_grammar(schema)
    assert g.startswith("root ::= ")
    assert ok(g, '{"name": "a"}') and ok(g, '{"name":"a","age":3}') and ok(g, '{"name": "a", "tags": ["x", "y"]}')
    assert ok(g, '{\n  "name": "a",\n  "age": 1,\n  "tags": ["x"]\n}')
    assert not ok(g, '{"age": 3}')                       # required member missing
    assert not ok(g, '{"name": "a", "tags": []}')        # minItems
    assert not ok(g, '{"name": "a", "tags": ["x","y","z"]}')
    assert not ok(g, '{"name": "a", "other": 1}')        # no additional properties when properties are listed
    assert not ok(g, '{"name": 5}')


def test_refs_anyof_allof_tuple_and_recursion():
    schema = {"$defs": {"node": {"type": "object", "properties": {"v": {"type": "integer"}, "next": {"anyOf": [{"$ref": "#/$defs/node"}, {"type": "null"}]}},
                                 "required": ["v", "next"]}},
              "$ref": "#/$defs/node"}
    g = json_schema_to_grammar(schema)
    assert ok(g, '{"v": 1, "next": {"v": 2, "next": null}}') and not ok(g, '{"v": 1}')
    g = json_schema_to_grammar({"prefixItems": [{"type": "integer"}, {"type": "boolean"}]})
    assert ok(g, "[1, true]") and not ok(g, "[true, 1]") and not ok(g, "[1]")
    g = json_schema_to_grammar({"allOf": [{"type": "object", "properties": {"a": {"type": "integer"}}, "required": ["a"]},
                                          {"type": "object", "properties": {"b": {"const": "x"}}, "required": ["b"]}]})
    assert ok(g, '{"a": 1, "b": "x"}') and not ok(g, '{"a": 1, "b": "y"}')
    g = json_schema_to_grammar({"type": "object", "additionalProperties": {"type": "integer"}})
    assert ok(g, '{"k": 1, "j": 2}') and ok(g, "{}") and not ok(g, '{"k": "v"}')


def test_response_format_and_errors():
    assert grammar_for_response_format(None) is None and grammar_for_response_format({"type": "text"}) is None
    g = grammar_for_response_format({"type": "json_object"})
    assert ok(g, '{"anything": [1, {"x": null}]}') and not ok(g, "[1]")
    g = grammar_for_response_format({"type": "json_schema", "json_schema": {"name": "t", "schema": {"type": "boolean"}}})
    assert ok(g, "true") and not ok(g, "1")
    with pytest.raises(SchemaError):
        grammar_for_response_format({"type": "json_schema", "json_schema": {}})
    with pytest.raises(SchemaError):
        json_schema_to_grammar({"$ref": "http://example.com/x"})
    with pytest.raises(SchemaError):
        json_schema_to_grammar({"type": "frob"})


def test_chat_request_carries_grammar_and_rejects_bad_schema():
    from jittorinfer_b200.server import protocol as P
    from jittorinfer_b200.server.chat import ChatTemplate

    class Tok:
        def encode(self, text, add_special=True, parse_special=True):
            return [1, 2, 3]

    body = {"messages": [{"role": "user", "content": "hi"}],
            "response_format": {"type": "json_schema", "json_schema": {"schema": {"type": "object", "properties": {"a": {"type": "integer"}}}}}}
    req = P.parse_chat(body, Tok(), ChatTemplate(""), "m", 16)
    assert req.grammar and grammar_accepts(req.grammar, '{"a": 4}')
    body["response_format"] = {"type": "json_schema", "json_schema": {"schema": {"type": "frob"}}}
    with pytest.raises(P.BadRequest):
        P.parse_chat(body, Tok(), ChatTemplate(""), "m", 16)


def _toy_vocab_model(tmp_path):
    from jittorinfer_b200 import capi
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.models.weights import write_random_gguf
    L = capi.load()
    p = str(tmp_path / "m.gguf")
    write_random_gguf(p, preset("tiny"), seed=0)
    mp = L.llama_model_default_params()
    mp.vocab_only = True
    model = L.llama_model_load_from_file(p.encode(), mp)
    return L, capi, model, L.llama_model_get_vocab(model)


def test_grammar_sampler_constrains_random_logits(tmp_path):
    """The C API's grammar sampler: with random logits over the whole vocabulary every generated text is a sentence of
    the grammar (here: the grammar of a JSON schema), and generation ends with an end-of-generation token."""
    import ctypes as C
    import random
    L, capi, model, vocab = _toy_vocab_model(tmp_path)
    schema = {"type": "object", "properties": {"color": {"enum": ["red", "green"]}, "n": {"type": "integer"}, "ok": {"type": "boolean"}},
              "required": ["color", "n"]}
    gbnf = json_schema_to_grammar(schema)
    assert L.llama_sampler_init_grammar(vocab, b"root ::= (", b"root") is None          # syntax error -> NULL
    V = L.llama_vocab_n_tokens(vocab)
    rng = random.Random(0)
    for trial in range(3):
        smpl = L.llama_sampler_init_grammar(vocab, gbnf.encode(), b"root")
        assert smpl
        toks = []
        for step in range(400):
            arr, keep = capi.candidates([rng.gauss(0, 1) for _ in range(V)])
            L.llama_sampler_apply(smpl, C.byref(arr))
            assert arr.size >= 1
            best = max(range(arr.size), key=lambda i: arr.data[i].logit)
            tok = arr.data[best].id
            L.llama_sampler_accept(smpl, tok)
            if L.llama_vocab_is_eog(vocab, tok):
                break
            toks.append(tok)
        else:
            raise AssertionError("generation did not finish")
        buf = C.create_string_buffer(4096)
        ids = (capi.llama_token * len(toks))(*toks)
        n = L.llama_detokenize(vocab, ids, len(toks), buf, 4096, False, False)
        text = buf.raw[:n].decode()
        doc = json.loads(text)
        assert grammar_accepts(gbnf, text), text
        assert doc["color"] in ("red", "green") and isinstance(doc["n"], int) and set(doc) <= {"color", "n", "ok"}
        clone = L.llama_sampler_clone(smpl)
        assert clone
        L.llama_sampler_free(clone)
        L.llama_sampler_free(smpl)
    L.llama_model_free(model)


def test_server_enforces_response_format():
    """Through the server: a chat request with a JSON schema gets a document that parses and fits the schema even though
    the model is random (the device top-k candidates are filtered; a dead end substitutes an admissible token)."""
    import threading
    import urllib.request
    import torch
    from jittorinfer_b200.config import ServerConfig
    from jittorinfer_b200.server.app import ServerContext, serve
    from jittorinfer_b200.server.chat import ChatTemplate
    from jittorinfer_b200.server.launch import build_from_config
    cfg = ServerConfig(random_init="tiny", n_ctx=2048, n_parallel=2, n_batch=64, port=0, enable_ge=False)
    eng, tok, tpl = build_from_config(cfg, device=torch.device("cpu"))
    ctx = ServerContext(eng, tok, cfg, ChatTemplate(tpl))
    httpd = serve(ctx, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    try:
        schema = {"type": "object", "properties": {"answer": {"enum": ["yes", "no"]}, "score": {"type": "integer"}}, "required": ["answer", "score"]}
        body = {"messages": [{"role": "user", "content": "judge"}], "max_tokens": 200, "temperature": 0.7, "seed": 5,
                "response_format": {"type": "json_schema", "json_schema": {"schema": schema}}}
        req = urllib.request.Request(f"http://127.0.0.1:{httpd.server_address[1]}/v1/chat/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        out = json.loads(urllib.request.urlopen(req, timeout=120).read())
        doc = json.loads(out["choices"][0]["message"]["content"])
        assert doc["answer"] in ("yes", "no") and isinstance(doc["score"], int)
        assert out["choices"][0]["finish_reason"] == "stop"
    finally:
        httpd.shutdown()
        httpd.server_close()
        ctx.shutdown()


def test_server_rejects_a_grammar_the_engine_cannot_build():
    import threading
    import urllib.error
    import urllib.request
    import torch
    from jittorinfer_b200.config import ServerConfig
    from jittorinfer_b200.server.app import ServerContext, serve
    from jittorinfer_b200.server.chat import ChatTemplate
    from jittorinfer_b200.server.launch import build_from_config
    cfg = ServerConfig(random_init="tiny", n_ctx=1024, n_parallel=2, n_batch=64, port=0, enable_ge=False)
    eng, tok, tpl = build_from_config(cfg, device=torch.device("cpu"))
    ctx = ServerContext(eng, tok, cfg, ChatTemplate(tpl))
    httpd = serve(ctx, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    url = f"http://127.0.0.1:{httpd.server_address[1]}/v1/chat/completions"
    try:
        body = {"messages": [{"role": "user", "content": "x"}], "max_tokens": 8,
                "response_format": {"type": "json_schema", "json_schema": {"schema": {"type": "string", "maxLength": 100000}}}}
        req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(req, timeout=60)
        assert e.value.code == 400
        body["response_format"] = {"type": "json_object"}      # the server is still healthy
        body["temperature"] = 0
        req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
        assert json.loads(urllib.request.urlopen(req, timeout=60).read())["object"] == "chat.completion"
    finally:
        httpd.shutdown()
        httpd.server_close()
        ctx.shutdown()
