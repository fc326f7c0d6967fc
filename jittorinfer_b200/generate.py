"""Command-line text generation: ``python -m jittorinfer_b200.generate -c configs/x.yaml -p "prompt"``.

The smallest end-to-end program over the engine (model from a GGUF file named in the YAML config, or ``--random-init``):
tokenises the prompt (or takes ``--tokens 1,2,3``), runs continuous batching over all prompts given, prints the
completions and a one-line timing summary -- what the reference's scripted single-sequence program does
(tests/main/single_sequence.cpp:181-372) without the hard-coded model path.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="jittorinfer_b200.generate")
    ap.add_argument("--config", "-c", default=None)
    ap.add_argument("--random-init", default=None, help="tiny | tiny-v2 | lite | v2: random weights instead of a GGUF file")
    ap.add_argument("--prompt", "-p", action="append", default=[], help="text prompt (repeatable)")
    ap.add_argument("--tokens", action="append", default=[], help="prompt as comma-separated token ids (repeatable)")
    ap.add_argument("--chat", action="store_true", help="wrap each text prompt in the chat template as a user turn")
    ap.add_argument("--max-tokens", "-n", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=40)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--device", default=None, help="cpu | cuda (default: cuda when available)")
    ap.add_argument("--json", action="store_true", help="print one JSON object instead of text")
    a = ap.parse_args(argv)
    import torch
    from .config import load_yaml
    from .runtime.sampling import SamplingParams
    from .server.chat import ChatTemplate
    from .server.launch import build_from_config
    cfg = load_yaml(a.config)
    if a.random_init:
        cfg.random_init = a.random_init
    if not cfg.model and not cfg.random_init:
        print("need a config with \"model\" or --random-init", file=sys.stderr)
        return 2
    device = torch.device(a.device) if a.device else None
    t0 = time.time()
    eng, tok, tpl = build_from_config(cfg, device=device)
    t_load = time.time() - t0
    prompts = []
    template = ChatTemplate(tpl) if a.chat else None
    for text in a.prompt:
        if template is not None:
            text = template.render([{"role": "user", "content": text}], add_generation_prompt=True)
        prompts.append(tok.encode(text, add_special=True, parse_special=True))
    for ids in a.tokens:
        prompts.append([int(x) for x in ids.split(",") if x.strip()])
    if not prompts:
        print("no prompt given (-p or --tokens)", file=sys.stderr)
        return 2
    sp = SamplingParams(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, seed=a.seed, ignore_eos=a.ignore_eos,
                        max_tokens=a.max_tokens)
    eng.warmup()
    t1 = time.time()
    outs = eng.generate(prompts, sp)
    dt = time.time() - t1
    n_out = sum(len(o) for o in outs)
    texts = [tok.decode(o) for o in outs]
    summary = {"load_s": round(t_load, 3), "generate_s": round(dt, 3), "prompt_tokens": sum(len(p) for p in prompts),
               "generated_tokens": n_out, "tokens_per_s": round(n_out / dt, 2) if dt > 0 else 0.0, "steps": eng.stats["steps"]}
    if a.json:
        print(json.dumps({"completions": [{"tokens": o, "text": t} for o, t in zip(outs, texts)], "timing": summary}))
    else:
        for i, t in enumerate(texts):
            print(f"--- completion {i} ---\n{t}")
        print(json.dumps(summary), file=sys.stderr)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
