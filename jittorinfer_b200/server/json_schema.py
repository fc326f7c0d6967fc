"""JSON schema -> GBNF grammar text.

Counterpart of the reference's ``json_schema_to_grammar`` / ``build_grammar``
(common/json-schema-to-grammar_local.cpp:824-856): ``response_format`` of a chat request is turned into a GBNF
grammar.  As in the reference, nothing consumes the grammar at sampling time (its grammar sampler asserts on a
non-empty grammar, src/llama-sampling.cpp:313-389; ``llama_sampler_init_grammar`` here returns NULL for one): the
server attaches the grammar text to the request so that a client or an external constrained decoder can use it, and
validates the schema early so that a malformed ``response_format`` is a 400 instead of a silent no-op.

Supported: ``type`` (string, number, integer, boolean, null, object, array, and lists of types), ``enum``, ``const``,
``properties`` / ``required`` / ``additionalProperties``, ``items`` / ``prefixItems`` / ``minItems`` / ``maxItems``,
``minLength`` / ``maxLength``, ``anyOf`` / ``oneOf``, ``allOf`` of objects, local ``$ref`` (``#/definitions/..``,
``#/$defs/..``), and a small set of string ``format`` values (date, time, date-time, uuid).
"""
from __future__ import annotations

import json
import re
from typing import Any, Dict, List, Optional

SPACE = '| " " | "\\n" [ \\t]{0,20}'

PRIMITIVES = {
    "boolean": '("true" | "false") space',
    "null": '"null" space',
    "integer": '("-"? integral-part) space',
    "number": '("-"? integral-part) ("." decimal-part)? ([eE] [-+]? integral-part)? space',
    "integral-part": '[0] | [1-9] [0-9]{0,15}',
    "decimal-part": '[0-9]{1,16}',
    "char": '[^"\\\\\\x7F\\x00-\\x1F] | [\\\\] (["\\\\bfnrt] | "u" [0-9a-fA-F]{4})',
    "string": '"\\"" char* "\\"" space',
    "value": 'object | array | string | number | boolean | null',
    "object": '"{" space ( string ":" space value ("," space string ":" space value)* )? "}" space',
    "array": '"[" space ( value ("," space value)* )? "]" space',
    "uuid": '"\\"" [0-9a-fA-F]{8} "-" [0-9a-fA-F]{4} "-" [0-9a-fA-F]{4} "-" [0-9a-fA-F]{4} "-" [0-9a-fA-F]{12} "\\"" space',
    "date": '[0-9]{4} "-" ( "0" [1-9] | "1" [0-2] ) "-" ( "0" [1-9] | [1-2] [0-9] | "3" [0-1] )',
    "time": '([01] [0-9] | "2" [0-3]) ":" [0-5] [0-9] ":" [0-5] [0-9] ( "." [0-9]{3} )? ( "Z" | ( "+" | "-" ) ( [01] [0-9] | "2" [0-3] ) ":" [0-5] [0-9] )',
    "date-time": 'date "T" time',
    "date-string": '"\\"" date "\\"" space',
    "time-string": '"\\"" time "\\"" space',
    "date-time-string": '"\\"" date-time "\\"" space',
}
DEPS = {"number": ["integral-part", "decimal-part"], "integer": ["integral-part"], "string": ["char"],
        "value": ["object", "array", "string", "number", "boolean", "null"], "object": ["string", "value"], "array": ["value"],
        "date-time": ["date", "time"], "date-string": ["date"], "time-string": ["time"], "date-time-string": ["date-time"]}
FORMATS = {"date": "date-string", "time": "time-string", "date-time": "date-time-string", "uuid": "uuid"}
_BAD_NAME = re.compile(r"[^a-zA-Z0-9-]+")


class SchemaError(ValueError):
    pass


def _literal(text: str) -> str:
    esc = text.replace("\\", "\\\\").replace('"', '\\"').replace("\n", "\\n").replace("\r", "\\r")
    return f'"{esc}"'


class Converter:
    def __init__(self, schema: Any):
        self.root_schema = schema
        self.rules: Dict[str, str] = {"space": SPACE}
        self._ref_names: Dict[str, str] = {}

    # ---- rule table ------------------------------------------------------------------------------
    def _add(self, name: str, body: str) -> str:
        name = _BAD_NAME.sub("-", name).strip("-") or "r"
        base, i = name, 0
        while name in self.rules and self.rules[name] != body:
            i += 1
            name = f"{base}{i}"
        self.rules[name] = body
        return name

    def _prim(self, name: str) -> str:
        if name not in self.rules:
            self.rules[name] = PRIMITIVES[name]
            for d in DEPS.get(name, []):
                self._prim(d)
        return name

    # ---- schema walk -----------------------------------------------------------------------------
    def _resolve(self, ref: str) -> Any:
        if not ref.startswith("#/"):
            raise SchemaError(f"only local $ref is supported: {ref}")
        node = self.root_schema
        for part in ref[2:].split("/"):
            part = part.replace("~1", "/").replace("~0", "~")
            if not isinstance(node, dict) or part not in node:
                raise SchemaError(f"$ref {ref} does not resolve")
            node = node[part]
        return node

    def visit(self, schema: Any, name: str) -> str:
        if schema is True or schema == {}:
            return self._prim("value")
        if not isinstance(schema, dict):
            raise SchemaError(f"schema at {name or 'root'} must be an object")
        if "$ref" in schema:
            ref = schema["$ref"]
            if ref not in self._ref_names:
                rule = _BAD_NAME.sub("-", ref.split("/")[-1]) or "ref"
                self._ref_names[ref] = rule                   # reserve first: recursive schemas refer to themselves
                body_rule = self.visit(self._resolve(ref), rule)
                if body_rule != rule:
                    self.rules[rule] = body_rule
            return self._ref_names[ref]
        if "const" in schema:
            return self._add(name or "const", _literal(json.dumps(schema["const"], ensure_ascii=False)) + " space")
        if "enum" in schema:
            alts = " | ".join(_literal(json.dumps(v, ensure_ascii=False)) for v in schema["enum"])
            return self._add(name or "enum", f"({alts}) space")
        for key in ("anyOf", "oneOf"):
            if key in schema:
                alts = [self.visit(s, f"{name}-{i}" if name else f"alt{i}") for i, s in enumerate(schema[key])]
                return self._add(name or key.lower(), " | ".join(alts))
        if "allOf" in schema:
            merged: Dict[str, Any] = {"type": "object", "properties": {}, "required": []}
            for s in schema["allOf"]:
                s = self._resolve(s["$ref"]) if isinstance(s, dict) and "$ref" in s else s
                if not isinstance(s, dict) or s.get("type", "object") != "object":
                    raise SchemaError("allOf is supported for object schemas only")
                merged["properties"].update(s.get("properties", {}))
                merged["required"] += s.get("required", [])
            return self.visit(merged, name)
        t = schema.get("type")
        if isinstance(t, list):
            alts = [self.visit({**schema, "type": one}, f"{name}-{one}" if name else one) for one in t]
            return self._add(name or "multi", " | ".join(alts))
        if t == "object" or (t is None and ("properties" in schema or "additionalProperties" in schema)):
            return self._object(schema, name)
        if t == "array" or (t is None and ("items" in schema or "prefixItems" in schema)):
            return self._array(schema, name)
        if t == "string":
            if schema.get("format") in FORMATS:
                return self._prim(FORMATS[schema["format"]])
            lo, hi = schema.get("minLength"), schema.get("maxLength")
            if lo is None and hi is None:
                return self._prim("string")
            self._prim("char")
            rep = f"{{{lo or 0},{hi if hi is not None else ''}}}"
            return self._add(name or "string-n", f'"\\"" char{rep} "\\"" space')
        if t in ("number", "integer", "boolean", "null"):
            return self._prim(t)
        if t is None:
            return self._prim("value")
        raise SchemaError(f"unsupported type {t!r} at {name or 'root'}")

    def _object(self, schema: Dict[str, Any], name: str) -> str:
        props: Dict[str, Any] = schema.get("properties", {})
        required = set(schema.get("required", []))
        extra = schema.get("additionalProperties", False if props else True)
        kv = {}
        for key, sub in props.items():
            vr = self.visit(sub, f"{name}-{key}" if name else key)
            kv[key] = self._add(f"{name}-{key}-kv" if name else f"{key}-kv", f'{_literal(json.dumps(key))} space ":" space {vr}')
        req = [k for k in props if k in required]
        opt = [k for k in props if k not in required]
        if extra is not False and extra is not None:
            vr = self._prim("value") if extra is True or extra == {} else self.visit(extra, f"{name}-additional" if name else "additional")
            self._prim("string")
            kv["*"] = self._add(f"{name}-additional-kv" if name else "additional-kv", f'string ":" space {vr}')
            opt.append("*")
        body = '"{" space '
        body += ' "," space '.join(kv[k] for k in req)
        if opt:
            # optional members keep their declaration order; each may be followed by any later one
            def tail(ks: List[str]) -> str:
                k, rest = ks[0], ks[1:]
                me = kv[k] + (f' ( "," space {kv[k]} )*' if k == "*" else "")
                if not rest:
                    return me
                sub = self._add(f"{name}-{k}-rest" if name else f"{k}-rest", tail_alts(rest))
                return f'{me} ( "," space {sub} )?'

            def tail_alts(ks: List[str]) -> str:
                return " | ".join(tail(ks[i:]) for i in range(len(ks)))

            opt_rule = tail_alts(opt)
            body += (' ( "," space ( ' + opt_rule + ' ) )?') if req else (' ( ' + opt_rule + ' )?')
        body += ' "}" space'
        return self._add(name or "object-n", body)

    def _array(self, schema: Dict[str, Any], name: str) -> str:
        prefix = schema.get("prefixItems")
        if isinstance(schema.get("items"), list):
            prefix = schema["items"]
        if prefix:
            parts = [self.visit(s, f"{name}-tuple-{i}" if name else f"tuple-{i}") for i, s in enumerate(prefix)]
            return self._add(name or "tuple", '"[" space ' + ' "," space '.join(parts) + ' "]" space')
        item = self.visit(schema.get("items", True), f"{name}-item" if name else "item")
        lo, hi = int(schema.get("minItems", 0)), schema.get("maxItems")
        if hi is not None and int(hi) < lo:
            raise SchemaError("maxItems < minItems")
        if hi is not None and int(hi) == 0:
            return self._add(name or "array-n", '"[" space "]" space')
        more_lo = max(lo - 1, 0)
        more = f'( "," space {item} ){{{more_lo},{int(hi) - 1 if hi is not None else ""}}}'
        inner = f"{item} {more}"
        return self._add(name or "array-n", f'"[" space ( {inner} ){"" if lo > 0 else "?"} "]" space')

    def grammar(self) -> str:
        root = self.visit(self.root_schema, "")
        self.rules["root"] = root if root != "root" else self.rules["root"]
        order = ["root"] + sorted(k for k in self.rules if k != "root")
        return "\n".join(f"{k} ::= {self.rules[k]}" for k in order) + "\n"


def json_schema_to_grammar(schema: Any) -> str:
    """GBNF text whose ``root`` accepts exactly the JSON documents the schema describes (within the supported subset)."""
    if isinstance(schema, str):
        schema = json.loads(schema)
    return Converter(schema).grammar()


def grammar_for_response_format(fmt: Optional[Dict[str, Any]]) -> Optional[str]:
    """OpenAI ``response_format``: ``{"type": "json_object"}`` or ``{"type": "json_schema", "json_schema": {"schema": ...}}``
    (also the older ``{"type": "json_object", "schema": ...}``).  ``None`` / ``{"type": "text"}`` -> no grammar."""
    if not fmt:
        return None
    t = fmt.get("type", "text")
    if t == "text":
        return None
    if t == "json_object":
        return json_schema_to_grammar(fmt.get("schema") or {"type": "object", "additionalProperties": True})
    if t == "json_schema":
        js = fmt.get("json_schema") or {}
        if "schema" not in js:
            raise SchemaError("response_format.json_schema.schema is required")
        return json_schema_to_grammar(js["schema"])
    raise SchemaError(f"unknown response_format type {t!r}")


# ---- a small GBNF matcher, used by the tests to check that generated grammars accept / reject documents ------------
class _Gbnf:
    """Recursive-descent recogniser for the GBNF subset this module emits (literals, classes, groups, | * + ? {m,n})."""

    def __init__(self, text: str):
        self.rules: Dict[str, Any] = {}
        for line in text.strip().splitlines():
            name, _, body = line.partition("::=")
            self.rules[name.strip()] = self._parse_alts(_Lexer(body.strip()))

    def _parse_alts(self, lx: "_Lexer"):
        alts = [self._parse_seq(lx)]
        while lx.peek() == "|":
            lx.next()
            alts.append(self._parse_seq(lx))
        return ("alt", alts)

    def _parse_seq(self, lx: "_Lexer"):
        items = []
        while lx.peek() not in (None, "|", ")"):
            tok = lx.next()
            if tok == "(":
                node = self._parse_alts(lx)
                assert lx.next() == ")"
            elif tok[0] == '"':
                node = ("lit", json.loads(tok.replace("\\x7F", "\\u007f")))
            elif tok[0] == "[":
                node = ("cls", re.compile(tok, re.S))
            else:
                node = ("ref", tok)
            while lx.peek() in ("*", "+", "?") or (lx.peek() or "").startswith("{"):
                q = lx.next()
                if q == "*":
                    node = ("rep", node, 0, None)
                elif q == "+":
                    node = ("rep", node, 1, None)
                elif q == "?":
                    node = ("rep", node, 0, 1)
                else:
                    lo, _, hi = q[1:-1].partition(",")
                    node = ("rep", node, int(lo or 0), (int(hi) if hi else None) if "," in q else int(lo))
            items.append(node)
        return ("seq", items)

    def _match(self, node, s: str, i: int, depth: int = 0):
        """Yields every end position at which ``node`` can stop when started at ``i``."""
        kind = node[0]
        if kind == "lit":
            if s.startswith(node[1], i):
                yield i + len(node[1])
        elif kind == "cls":
            if i < len(s) and node[1].fullmatch(s[i]):
                yield i + 1
        elif kind == "ref":
            yield from self._match(self.rules[node[1]], s, i, depth + 1)
        elif kind == "alt":
            seen = set()
            for a in node[1]:
                for e in self._match(a, s, i, depth + 1):
                    if e not in seen:
                        seen.add(e)
                        yield e
        elif kind == "seq":
            ends = {i}
            for item in node[1]:
                ends = {e2 for e in ends for e2 in self._match(item, s, e, depth + 1)}
                if not ends:
                    return
            yield from ends
        elif kind == "rep":
            _, inner, lo, hi = node
            ends, n, out = {i}, 0, set()
            if lo == 0:
                out.add(i)
            while ends and (hi is None or n < hi):
                nxt = {e2 for e in ends for e2 in self._match(inner, s, e, depth + 1) if e2 > e}
                n += 1
                if n >= lo:
                    out |= nxt
                ends = nxt
            yield from out

    def accepts(self, s: str) -> bool:
        return any(e == len(s) for e in self._match(self.rules["root"], s, 0))


class _Lexer:
    TOKEN = re.compile(r'\s*("(?:[^"\\]|\\.)*"|\[(?:[^\]\\]|\\.)*\]|\{[0-9]*,?[0-9]*\}|::=|[()|*+?]|[A-Za-z0-9-]+)')

    def __init__(self, text: str):
        self.toks = self.TOKEN.findall(text)
        self.i = 0

    def peek(self):
        return self.toks[self.i] if self.i < len(self.toks) else None

    def next(self):
        t = self.toks[self.i]
        self.i += 1
        return t


def grammar_accepts(grammar: str, document: str) -> bool:
    return _Gbnf(grammar).accepts(document)
