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
