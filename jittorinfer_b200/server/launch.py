"""Builds engine + tokenizer from a YAML config and runs the HTTP server (all ranks call this)."""
from __future__ import annotations

import argparse
import logging
import os
import sys

log = logging.getLogger("jittorinfer_b200.server")


def build_from_config(cfg, device=None, world: int = 1, rank: int = 0):
    import torch
    from ..models.hparams import preset
    from ..runtime.factory import build_engine
    from ..tokenizer import Tokenizer
    from ..utils.toy_vocab import toy_vocab_kv
    if device is None:
        device = torch.device("cuda", cfg.main_gpu if world == 1 else rank) if torch.cuda.is_available() else torch.device("cpu")
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    auto_kv = bool(getattr(cfg, "kv_cache_auto", False)) and device.type == "cuda"
    n_ctx_slot = getattr(cfg, "max_seq_len", 0) or max(cfg.kv_block_size, cfg.n_ctx // cfg.slots)
    common = dict(device=device, dtype=dtype, world=world, rank=rank, n_parallel=cfg.slots, n_ctx_slot=n_ctx_slot,
                  n_ctx=None if auto_kv else cfg.n_ctx, gpu_memory_utilization=cfg.gpu_memory_utilization if auto_kv else None,
                  n_batch=cfg.n_batch, cuda_graphs=cfg.cuda_graphs, graph_buckets=tuple(b for b in cfg.cuda_graph_buckets if b <= cfg.slots) or (1,),
                  expert_parallel=cfg.ep_size > 1, n_keep=cfg.n_keep, cont_batching=cfg.cont_batching, defrag_thold=cfg.defrag_thold,
                  presample_count=max(1, cfg.presample_count) if cfg.presample_count > 0 else 64,
                  dp_attention=bool(getattr(cfg, "attention_dp", False)) and world > 1, ep_max_tokens=getattr(cfg, "ep_max_tokens", 256),
                  run_ahead=bool(getattr(cfg, "run_ahead", False)), device_sampling=bool(getattr(cfg, "device_sampling", False)),
                  mixed_prompt_budget=int(getattr(cfg, "mixed_prompt_budget", 0)),
                  check_tensors=bool(getattr(cfg, "check_tensors", False)))
    hp_known = preset(cfg.random_init) if cfg.random_init else None
    if world == 1 and device.type == "cuda" and cfg.split_mode == "LLAMA_SPLIT_MODE_LAYER":
        n = int(getattr(cfg, "layer_split_gpus", 1))
        if n <= 0:          # automatic, as the reference spreads layers over all devices by free memory (src/llama-model.cpp:495-540)
            if hp_known is None:
                from ..gguf.io import GGUFReader
                from ..models.hparams import DeepSeek2HParams
                with GGUFReader(cfg.model) as rd:
                    hp_known = DeepSeek2HParams.from_gguf_kv(rd.kv, rd.tensors)
            free = [torch.cuda.mem_get_info(i)[0] for i in range(torch.cuda.device_count())]
            n = auto_layer_split(hp_known.n_params() * 2, free)
        n = min(max(n, 1), torch.cuda.device_count())
        if n > 1:
            common.update(layer_devices=[torch.device("cuda", (cfg.main_gpu + i) % torch.cuda.device_count()) for i in range(n)],
                          tensor_split=list(cfg.tensor_split) or None)
    if cfg.random_init:
        hp = hp_known
        eng = build_engine(hp, **common)
        kv = {k: (v[1] if isinstance(v, tuple) else v) for k, v in toy_vocab_kv(hp.n_vocab, hp.bos_id, hp.eos_id).items()}
        kv["tokenizer.ggml.bos_token_id"], kv["tokenizer.ggml.eos_token_id"] = hp.bos_id, hp.eos_id
        tok = Tokenizer.from_gguf_kv(kv)
        template_src = ""
    else:
        from ..gguf.io import GGUFReader
        reader = GGUFReader(cfg.model)
        tok = Tokenizer.from_gguf_kv(reader.kv)
        template_src = reader.kv.get("tokenizer.chat_template", "")
        reader.close()
        eng = build_engine(None, gguf_path=cfg.model, **common)
    return eng, tok, (cfg.chat_template or template_src or "")


def apply_world(cfg, world: int) -> None:
    """A configuration written for the reference has no tp_size / ep_size: started as N ranks it means what the reference's
    multi-process server forces on -- tensor parallelism plus expert parallelism over all ranks
    (examples/mpi_server/server.cpp:888-916).  Explicit sizes are kept (they must match the number of ranks)."""
    if world <= 1:
        return
    if cfg.tp_size == 1 and cfg.ep_size == 1:
        cfg.tp_size = cfg.ep_size = world
    if cfg.world_size != world:
        raise SystemExit(f"configuration asks for {cfg.world_size} ranks (tp_size / ep_size), started with {world}")


def auto_layer_split(weight_bytes: int, free_bytes, headroom: float = 0.8) -> int:
    """Smallest number of GPUs (taken in order) whose free memory, kept to ``headroom`` of it so that the cache and
    activations have room, holds the weights; all of them if even that is not enough."""
    acc = 0.0
    for n, f in enumerate(free_bytes, 1):
        acc += headroom * f
        if acc >= weight_bytes:
            return n
    return max(1, len(free_bytes))


def main(argv=None, world: int = 1, rank: int = 0, control_group=None) -> int:
    ap = argparse.ArgumentParser(prog="jittorinfer_b200.server")
    ap.add_argument("--config", "-c", default=None, help="YAML file with the reference's keys (configs/*.yaml)")
    ap.add_argument("--port", type=int, default=None)
    ap.add_argument("--host", default=None)
    ap.add_argument("--random-init", default=None, help="serve a random-init preset (tiny | lite | v2) instead of a GGUF file")
    args = ap.parse_args(argv)
    logging.basicConfig(level=os.environ.get("JITTORINFER_LOG", "INFO"), format="%(asctime)s %(levelname)s %(name)s: %(message)s")
    from ..config import load_yaml
    from .app import ServerContext, serve
    from .chat import ChatTemplate
    cfg = load_yaml(args.config)
    if args.random_init:
        cfg.random_init = args.random_init
    if args.port:
        cfg.port = args.port
    if args.host:
        cfg.hostname = args.host
    if not cfg.model and not cfg.random_init:
        print("config has no \"model\" (GGUF path) and no random_init preset", file=sys.stderr)
        return 2
    apply_world(cfg, world)
    eng, tok, template_src = build_from_config(cfg, world=world, rank=rank)
    try:
        template = ChatTemplate(template_src)
    except Exception as e:        # a template the Jinja subset cannot render: fall back to the built-in one
        log.warning("chat template rejected (%s): using the built-in deepseek2 template", e)
        template = ChatTemplate("")
    eng.warmup()
    ctx = ServerContext(eng, tok, cfg, template, rank=rank, world=world, control_group=control_group)
    watchdog = None
    if world > 1 and os.environ.get("JITTORINFER_HEARTBEAT", "1") != "0":
        # failure detection: every rank publishes heartbeats through the rendezvous store; rank 0 refuses to broadcast to
        # a dead worker (in-flight requests fail with 503), workers leave when rank 0 goes silent
        try:
            import torch.distributed as dist
            from ..parallel.health import Heartbeat, Watchdog
            store = dist.distributed_c10d._get_default_store()
            timeout = float(os.environ.get("JITTORINFER_HEARTBEAT_TIMEOUT", "30"))
            ctx.heartbeat = Heartbeat(store, rank, world, interval=1.0, timeout=timeout, prefix="jib_hb").start()
            if rank != 0:
                watchdog = Watchdog(ctx.heartbeat, [0], period=2.0).start()
        except Exception as e:      # no store (unusual launchers): serve without failure detection
            log.warning("heartbeats disabled: %s", e)
    if rank != 0:
        ctx.run()                 # worker ranks: follow rank 0's task broadcasts until told to stop
        if watchdog is not None:
            watchdog.stop()
        return 0
    httpd = serve(ctx, cfg.hostname, cfg.port, cfg.n_threads_http)
    log.info("listening on http://%s:%d  (slots=%d, n_ctx_slot=%d, kv blocks=%d)", cfg.hostname, cfg.port, eng.cfg.n_parallel,
             eng.n_ctx_slot, eng.kv.n_blocks)
    try:
        httpd.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        ctx.shutdown()
        httpd.server_close()
    return 0
