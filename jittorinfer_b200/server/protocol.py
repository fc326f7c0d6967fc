"""OpenAI-compatible request parsing and response assembly.

Request side: what ``oaicompat_completion_params_parse`` / ``params_from_json_cmpl`` and
``tokenize_input_prompts`` do in the reference (common/utils.hpp:75-155, 218-342;
examples/server/server.cpp:84-100), except that ``max_tokens`` / ``n_predict``, ``stop``, ``seed``,
``ignore_eos`` and the penalties ARE honoured here (the reference never reads them from the request).
Response side: OAI completion / chat / chat-chunk JSON with ``usage`` on the final stream chunk and
``finish_reason`` stop|length (examples/server/server.cpp:251-346, 385-492).
"""
from __future__ import annotations

import json
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Union

from ..runtime.sampling import SamplingParams


class BadRequest(ValueError):
    pass


@dataclass
class ParsedRequest:
    prompts: List[List[int]]
    params: SamplingParams
    stream: bool
    chat: bool
    model: str
    stop: List[str] = field(default_factory=list)
    return_tokens: bool = False
    grammar: Optional[str] = None      # GBNF text derived from response_format (not enforced at sampling time)


def tokenize_mixed(tokenizer, prompt: Any, add_special: bool) -> List[int]:
    """A prompt may be a string, a list of token ids, or a list mixing strings and ids."""
    if isinstance(prompt, str):
        return tokenizer.encode(prompt, add_special=add_special, parse_special=True)
    if isinstance(prompt, list):
        if all(isinstance(x, int) for x in prompt):
            return list(prompt)
        out: List[int] = []
        first = True
        for piece in prompt:
            if isinstance(piece, str):
                out += tokenizer.encode(piece, add_special=add_special and first, parse_special=True)
                first = False
            elif isinstance(piece, int):
                out.append(piece)
            else:
                raise BadRequest("prompt list may only contain strings and token ids")
        return out
    raise BadRequest("prompt must be a string, a list of tokens, or a list mixing both")


def tokenize_prompts(tokenizer, prompt: Any) -> List[List[int]]:
    """Single prompt or a list of prompts (a list whose elements are strings/lists of ints)."""
    if isinstance(prompt, str):
        return [tokenize_mixed(tokenizer, prompt, True)]
    if isinstance(prompt, list) and prompt:
        if all(isinstance(x, int) for x in prompt):
            return [list(prompt)]
        if any(isinstance(x, list) for x in prompt) or (all(isinstance(x, str) for x in prompt) and len(prompt) > 1):
            return [tokenize_mixed(tokenizer, p, True) for p in prompt]
        return [tokenize_mixed(tokenizer, prompt, True)]
    raise BadRequest("\"prompt\" must be a non-empty string or list")


def sampling_from_body(body: Dict[str, Any], default_max: int) -> SamplingParams:
    def num(key, default, lo=None, hi=None, cast=float):
        v = body.get(key, default)
        if v is None:
            return default
        try:
            v = cast(v)
        except (TypeError, ValueError):
            raise BadRequest(f"\"{key}\" must be a number")
        if v != v or v in (float("inf"), float("-inf")):
            raise BadRequest(f"\"{key}\" must be finite")
        if (lo is not None and v < lo) or (hi is not None and v > hi):
            raise BadRequest(f"\"{key}\" out of range")
        return v

    if int(body.get("n_probs", 0) or 0) != 0:
        raise BadRequest("n_probs is not supported (use the OpenAI \"logprobs\" field)")      # as in the reference (server.cpp:1555)
    # OpenAI forms: completions "logprobs": n (0..20 alternatives per token); chat "logprobs": true + "top_logprobs": n
    lp = body.get("logprobs")
    want_lp = lp is not None and lp is not False
    n_alt = num("top_logprobs", 0, 0, 20, cast=int) if isinstance(lp, bool) or lp is None else num("logprobs", 0, 0, 20, cast=int)
    if int(body.get("n", 1) or 1) != 1:
        raise BadRequest("Only one completion choice is allowed")
    for k in ("best_of", "echo", "suffix"):
        if body.get(k):
            raise BadRequest(f"\"{k}\" is not supported")
    max_tokens = body.get("max_tokens", body.get("max_completion_tokens", body.get("n_predict", default_max)))
    bias = {}
    lb = body.get("logit_bias")
    if isinstance(lb, dict):
        bias = {int(k): float(v) for k, v in lb.items()}
    elif isinstance(lb, list):
        bias = {int(k): float(v) for k, v in lb}
    stop = body.get("stop") or []
    if isinstance(stop, str):
        stop = [stop]
    seed = body.get("seed")
    n_keep = body.get("n_keep")                # per request, as the reference reads it (examples/server/server.cpp:90, 1390-1393)
    if n_keep is not None:
        n_keep = int(num("n_keep", 0, cast=int))
    return SamplingParams(
        n_keep=n_keep,
        temperature=num("temperature", 0.8, 0.0), top_k=int(num("top_k", 40, 0, cast=int)), top_p=num("top_p", 0.95, 0.0, 1.0),
        min_p=num("min_p", 0.05, 0.0, 1.0), typical_p=num("typical_p", 1.0, 0.0, 1.0),
        xtc_probability=num("xtc_probability", 0.0, 0.0, 1.0), xtc_threshold=num("xtc_threshold", 0.1, 0.0, 1.0),
        repeat_penalty=num("repeat_penalty", 1.0, 0.0), frequency_penalty=num("frequency_penalty", 0.0),
        presence_penalty=num("presence_penalty", 0.0), repeat_last_n=int(num("repeat_last_n", 64, -1, cast=int)),
        dynatemp_range=num("dynatemp_range", 0.0, 0.0), dynatemp_exponent=num("dynatemp_exponent", 1.0, 0.0),
        dry_multiplier=num("dry_multiplier", 0.0, 0.0), dry_base=num("dry_base", 1.75, 1.0),
        dry_allowed_length=int(num("dry_allowed_length", 2, 1, cast=int)), dry_penalty_last_n=int(num("dry_penalty_last_n", -1, -1, cast=int)),
        min_keep=int(num("min_keep", 0, 0, cast=int)),
        logit_bias=bias, seed=None if seed in (None, -1) else int(seed) & 0xFFFFFFFFFFFFFFFF,
        max_tokens=-1 if max_tokens is None else int(max_tokens), ignore_eos=bool(body.get("ignore_eos", False)),
        stop=[str(s) for s in stop], logprobs=bool(want_lp), top_logprobs=int(n_alt))


def parse_completion(body: Dict[str, Any], tokenizer, model_alias: str, default_max: int) -> ParsedRequest:
    if "prompt" not in body:
        raise BadRequest("\"prompt\" is required")
    params = sampling_from_body(body, default_max)
    return ParsedRequest(tokenize_prompts(tokenizer, body["prompt"]), params, bool(body.get("stream", False)), False,
                         str(body.get("model", model_alias)), params.stop, bool(body.get("return_tokens", False)))


def parse_chat(body: Dict[str, Any], tokenizer, template, model_alias: str, default_max: int) -> ParsedRequest:
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise BadRequest("\"messages\" must be a non-empty list")
    rf = body.get("response_format")
    if isinstance(rf, dict) and rf.get("type") not in (None, "text", "json_object", "json_schema"):
        raise BadRequest("response_format type must be text, json_object or json_schema")
    try:
        prompt = template.render(msgs, tools=body.get("tools"), add_generation_prompt=True)
    except ValueError as e:
        raise BadRequest(str(e))
    grammar = None
    if isinstance(rf, dict):
        from .json_schema import SchemaError, grammar_for_response_format
        try:
            grammar = grammar_for_response_format(rf)
        except (SchemaError, ValueError) as e:
            raise BadRequest(f"response_format: {e}")
    params = sampling_from_body(body, default_max)
    return ParsedRequest([tokenizer.encode(prompt, add_special=True, parse_special=True)], params, bool(body.get("stream", False)),
                         True, str(body.get("model", model_alias)), params.stop, bool(body.get("return_tokens", False)), grammar)


# ---- responses -------------------------------------------------------------------------------------
def _usage(n_prompt: int, n_gen: int, n_cached: int = 0) -> Dict[str, Any]:
    return {"prompt_tokens": n_prompt, "completion_tokens": n_gen, "total_tokens": n_prompt + n_gen,
            "prompt_tokens_details": {"cached_tokens": n_cached}}


def new_id(chat: bool) -> str:
    return ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]


def completion_response(rid: str, model: str, text: str, finish: str, n_prompt: int, n_gen: int, index: int = 0,
                        timings: Optional[dict] = None, n_cached: int = 0) -> Dict[str, Any]:
    r = {"id": rid, "object": "text_completion", "created": int(time.time()), "model": model,
         "choices": [{"text": text, "index": index, "logprobs": None, "finish_reason": finish}], "usage": _usage(n_prompt, n_gen, n_cached)}
    if timings:
        r["timings"] = timings
    return r


def completion_chunk(rid: str, model: str, text: str, finish: Optional[str], usage: Optional[dict] = None) -> Dict[str, Any]:
    r = {"id": rid, "object": "text_completion", "created": int(time.time()), "model": model,
         "choices": [{"text": text, "index": 0, "logprobs": None, "finish_reason": finish}]}
    if usage:
        r["usage"] = usage
    return r


def chat_response(rid: str, model: str, content: str, reasoning: Optional[str], tool_call: Optional[dict], finish: str,
                  n_prompt: int, n_gen: int, timings: Optional[dict] = None, n_cached: int = 0) -> Dict[str, Any]:
    msg: Dict[str, Any] = {"role": "assistant", "content": content}
    if reasoning is not None:
        msg["reasoning_content"] = reasoning
    if tool_call is not None:
        msg["content"] = None
        msg["tool_calls"] = [dict(tool_call, id="call_" + uuid.uuid4().hex[:16])]
        finish = "tool_calls"
    r = {"id": rid, "object": "chat.completion", "created": int(time.time()), "model": model,
         "choices": [{"index": 0, "message": msg, "finish_reason": finish}], "usage": _usage(n_prompt, n_gen, n_cached)}
    if timings:
        r["timings"] = timings
    return r


def chat_chunk(rid: str, model: str, delta: Dict[str, Any], finish: Optional[str], usage: Optional[dict] = None) -> Dict[str, Any]:
    r = {"id": rid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model,
         "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}
    if usage:
        r["usage"] = usage
    return r


def completion_logprobs(entries, piece) -> Dict[str, Any]:
    """OpenAI text-completion form.  ``entries``: [(token id, logprob, [(id, logprob)])]; ``piece``: id -> text."""
    toks = [piece(t) for t, _, _ in entries]
    offs, pos = [], 0
    for t in toks:
        offs.append(pos)
        pos += len(t)
    return {"tokens": toks, "token_logprobs": [lp for _, lp, _ in entries],
            "top_logprobs": [{piece(i): v for i, v in alts} for _, _, alts in entries], "text_offset": offs}


def chat_logprobs(entries, piece) -> Dict[str, Any]:
    """OpenAI chat form: ``{"content": [{"token", "logprob", "bytes", "top_logprobs": [...]}]}``."""
    def one(i, v):
        text = piece(i)
        return {"token": text, "logprob": v, "bytes": list(text.encode("utf-8"))}
    return {"content": [dict(one(t, lp), top_logprobs=[one(i, v) for i, v in alts]) for t, lp, alts in entries]}


def sse(obj: Union[Dict[str, Any], str]) -> bytes:
    """Server-sent event framing (common/utils.hpp:348-354)."""
    payload = obj if isinstance(obj, str) else json.dumps(obj, ensure_ascii=False)
    return ("data: " + payload + "\n\n").encode("utf-8")


def error_body(message: str, code: int, etype: str = "invalid_request_error") -> Dict[str, Any]:
    return {"error": {"code": code, "message": message, "type": etype}}
