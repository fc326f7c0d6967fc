"""Chat templates and reasoning-content splitting.

The reference formats chats either with its built-in DeepSeek-2 template
(src/llama-chat.cpp:92-163: ``User: ...\\n\\nAssistant:``) or, in the servers, with the Jinja template stored
in the GGUF file / given in the config, rendered by the vendored minja engine
(common/chat_local.cpp, common/chat-template.hpp).  Here the built-in template is restated and Jinja
templates are rendered with ``jinja2`` when it is installed.  ``reasoning_format: DEEPSEEK`` splits
``<think>...</think>`` into ``reasoning_content`` (the reference parses the option but never produces
the field, common/chat_local.cpp:476-485).
"""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional, Tuple

EOS_TEXT = "<｜end▁of▁sentence｜>"
BOS_TEXT = "<｜begin▁of▁sentence｜>"


def _content_text(content: Any) -> str:
    """OpenAI message content: a string or a list of {type: text, text: ...} parts."""
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    if isinstance(content, list):
        parts = []
        for p in content:
            if isinstance(p, dict) and p.get("type") == "text":
                parts.append(str(p.get("text", "")))
            elif isinstance(p, str):
                parts.append(p)
            else:
                raise ValueError("unsupported content part (only text parts are served)")
        return "".join(parts)
    raise ValueError("message content must be a string or a list of text parts")


def apply_deepseek2(messages: List[Dict[str, Any]], add_assistant: bool = True) -> str:
    out = []
    for m in messages:
        role, text = m.get("role"), _content_text(m.get("content"))
        if role == "system":
            out.append(text + "\n\n")
        elif role == "user":
            out.append("User: " + text + "\n\n")
        elif role == "assistant":
            out.append("Assistant: " + text + EOS_TEXT)
        elif role == "tool":
            out.append("Tool: " + text + "\n\n")
        else:
            raise ValueError(f"unknown role {role!r}")
    if add_assistant:
        out.append("Assistant:")
    return "".join(out)


class ChatTemplate:
    """``source``: a Jinja template string, the name "deepseek2", or empty (= built-in)."""

    def __init__(self, source: str = "", bos_token: str = BOS_TEXT, eos_token: str = EOS_TEXT):
        self.source = source or "deepseek2"
        self.bos_token, self.eos_token = bos_token, eos_token
        self._jinja = None
        if self.source not in ("deepseek2", "deepseek"):
            try:
                from jinja2.sandbox import ImmutableSandboxedEnvironment
                env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
                env.filters.setdefault("tojson", lambda v, **kw: json.dumps(v, ensure_ascii=False))
                env.globals["raise_exception"] = self._raise
                self._jinja = env.from_string(self.source)
            except ImportError:
                raise RuntimeError("a Jinja chat template was configured but jinja2 is not installed")

    @staticmethod
    def _raise(msg):
        raise ValueError(msg)

    def render(self, messages: List[Dict[str, Any]], tools: Optional[list] = None, add_generation_prompt: bool = True) -> str:
        if self._jinja is None:
            msgs = list(messages)
            if tools:
                # generic tool-call format: describe the tools in a leading system message
                spec = json.dumps(tools, ensure_ascii=False)
                msgs = [{"role": "system", "content": "You can call these tools by answering with JSON "
                         '{"tool_call": {"name": ..., "arguments": {...}}}:\n' + spec}] + msgs
            return apply_deepseek2(msgs, add_generation_prompt)
        norm = [dict(m, content=_content_text(m.get("content"))) for m in messages]
        return self._jinja.render(messages=norm, tools=tools, add_generation_prompt=add_generation_prompt,
                                  bos_token=self.bos_token, eos_token=self.eos_token)


def split_reasoning(text: str, enabled: bool) -> Tuple[Optional[str], str]:
    """('reasoning', 'content') for DeepSeek-R1 style output; (None, text) when disabled or absent."""
    if not enabled:
        return None, text
    t = text.lstrip()
    if t.startswith("<think>"):
        body = t[len("<think>"):]
        end = body.find("</think>")
        if end < 0:
            return body.strip(), ""
        return body[:end].strip(), body[end + len("</think>"):].lstrip()
    end = t.find("</think>")                     # template already opened the think block
    if end >= 0:
        return t[:end].strip(), t[end + len("</think>"):].lstrip()
    return None, text


def parse_tool_call(content: str) -> Optional[Dict[str, Any]]:
    """Generic tool-call format: a JSON object with a "tool_call" member."""
    s = content.strip()
    if not (s.startswith("{") and s.endswith("}")):
        return None
    try:
        obj = json.loads(s)
    except json.JSONDecodeError:
        return None
    tc = obj.get("tool_call") if isinstance(obj, dict) else None
    if not isinstance(tc, dict) or "name" not in tc:
        return None
    return {"type": "function", "function": {"name": tc["name"], "arguments": json.dumps(tc.get("arguments", {}))}}
