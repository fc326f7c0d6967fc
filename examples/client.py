"""Minimal client of the OpenAI-compatible routes: prints a chat completion as it streams.

    python examples/client.py --url http://127.0.0.1:8084 "Write a haiku about NVLink"
    python examples/client.py --completion --max-tokens 32 "The capital of France is"

Standard library only.  Works against the reference's server as well (same routes, same event format:
examples/server/server.cpp:1663-1690 -- ``data: {json}`` lines, then ``data: [DONE]``).
"""
import argparse
import json
import sys
import urllib.request


def stream(url: str, body: dict, timeout: float = 600.0):
    """Yields the text pieces of a streamed completion (``choices[0].delta.content`` or ``choices[0].text``)."""
    req = urllib.request.Request(url, data=json.dumps(dict(body, stream=True)).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        for line in r:
            line = line.strip()
            if not line.startswith(b"data:"):
                continue
            payload = line[5:].strip()
            if payload == b"[DONE]":
                return
            ev = json.loads(payload)
            if "error" in ev:
                raise RuntimeError(ev["error"])
            for ch in ev.get("choices", []):
                piece = ch.get("delta", {}).get("content") if "delta" in ch else ch.get("text")
                if piece:
                    yield piece


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("prompt")
    ap.add_argument("--url", default="http://127.0.0.1:8080")
    ap.add_argument("--completion", action="store_true", help="use /v1/completions with the raw prompt instead of the chat route")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--system", default=None)
    a = ap.parse_args(argv)
    if a.completion:
        route, body = "/v1/completions", {"prompt": a.prompt}
    else:
        msgs = ([{"role": "system", "content": a.system}] if a.system else []) + [{"role": "user", "content": a.prompt}]
        route, body = "/v1/chat/completions", {"messages": msgs}
    body.update(max_tokens=a.max_tokens, temperature=a.temperature)
    for piece in stream(a.url.rstrip("/") + route, body):
        sys.stdout.write(piece)
        sys.stdout.flush()
    sys.stdout.write("\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
