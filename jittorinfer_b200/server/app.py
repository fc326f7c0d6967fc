"""OpenAI-compatible HTTP server over the engine ("llama-server").

Same process layout as the reference (examples/server/server.cpp:646-899, 1567-1768): a pool of HTTP threads
parses requests and posts tasks to ONE engine thread through a queue; the engine thread runs the
continuous-batching loop and hands tokens back through per-request queues; responses are plain JSON or
server-sent events.  Endpoints: ``POST /v1/completions``, ``POST /v1/chat/completions`` (also without the
``/v1`` prefix), ``GET /exit`` as in the reference, plus ``/health``, ``/metrics`` (Prometheus text),
``/slots``, ``/props`` and ``/v1/models`` which the reference dropped.

With more than one rank (``mpi_server``) rank 0 owns the HTTP side and broadcasts the tasks of every loop
iteration to the other ranks before the step, the role MPI_Bcast of the serialised batch plays in
examples/mpi_server/server.cpp:928-983, 1896-1910; all ranks then run identical schedulers.
"""
from __future__ import annotations

import json
import queue
import threading
import time
from dataclasses import dataclass, field
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Dict, List, Optional

from ..runtime.sampling import SamplingParams
from . import protocol as P
from .chat import ChatTemplate, parse_tool_call, split_reasoning


@dataclass
class _Stream:
    """Server-side state of one in-flight completion."""
    rid: int = -1
    q: "queue.Queue" = field(default_factory=queue.Queue)
    n_prompt: int = 0
    n_gen: int = 0
    pending: bytes = b""           # bytes not yet emitted (incomplete UTF-8 or possible stop-word prefix)
    text: str = ""                 # everything emitted so far
    held: str = ""                 # decoded text held back because it may start a stop word
    stop: List[str] = field(default_factory=list)
    t0: float = 0.0
    t_first: float = 0.0
    done: bool = False
    tokens: List[int] = field(default_factory=list)      # generated ids (returned when the request sets return_tokens)
    logprobs: list = field(default_factory=list)          # per generated token (id, logprob, alternatives) when requested
    n_cached: int = 0                                     # prompt tokens served from the cache


class Metrics:
    BUCKETS = (0.001, 0.002, 0.005, 0.01, 0.02, 0.05, 0.1, 0.25, 1.0)

    def __init__(self):
        self.lock = threading.Lock()
        self.c = {"requests_total": 0, "requests_failed_total": 0, "prompt_tokens_total": 0, "generation_tokens_total": 0,
                  "steps_total": 0, "cancelled_total": 0}
        self.hist = [0] * (len(self.BUCKETS) + 1)
        self.step_seconds_sum = 0.0

    def inc(self, k, n=1):
        with self.lock:
            self.c[k] += n

    def observe_step(self, dt):
        with self.lock:
            self.c["steps_total"] += 1
            self.step_seconds_sum += dt
            for i, b in enumerate(self.BUCKETS):
                if dt <= b:
                    self.hist[i] += 1
                    return
            self.hist[-1] += 1

    def render(self, gauges: Dict[str, float]) -> str:
        out = []
        with self.lock:
            for k, v in self.c.items():
                out += [f"# TYPE jittorinfer_{k} counter", f"jittorinfer_{k} {v}"]
            out.append("# TYPE jittorinfer_step_seconds histogram")
            acc = 0
            for b, n in zip(self.BUCKETS, self.hist):
                acc += n
                out.append(f'jittorinfer_step_seconds_bucket{{le="{b}"}} {acc}')
            out.append(f'jittorinfer_step_seconds_bucket{{le="+Inf"}} {acc + self.hist[-1]}')
            out.append(f"jittorinfer_step_seconds_sum {self.step_seconds_sum}")
            out.append(f"jittorinfer_step_seconds_count {acc + self.hist[-1]}")
        for k, v in gauges.items():
            out += [f"# TYPE jittorinfer_{k} gauge", f"jittorinfer_{k} {v}"]
        return "\n".join(out) + "\n"


class ServerContext:
    def __init__(self, engine, tokenizer, cfg, template: Optional[ChatTemplate] = None, rank: int = 0, world: int = 1,
                 control_group=None):
        self.engine, self.tokenizer, self.cfg = engine, tokenizer, cfg
        self.template = template or ChatTemplate(getattr(cfg, "chat_template", "") or "")
        self.rank, self.world, self.group = rank, world, control_group
        self.inbox: "queue.Queue" = queue.Queue()
        self.streams: Dict[int, _Stream] = {}
        self.metrics = Metrics()
        self.engine.tokenizer_for_grammar = tokenizer         # the table of token texts is built on the first grammar request
        self.stop_flag = threading.Event()
        self.thread: Optional[threading.Thread] = None
        self.model_alias = getattr(cfg, "model_alias", "") or "deepseek2"
        self.reasoning = getattr(cfg, "reasoning_format", "") == "COMMON_REASONING_FORMAT_DEEPSEEK"
        self.default_max = getattr(cfg, "n_predict", -1)

    # ---- HTTP side ----------------------------------------------------------------------------------
    def submit(self, prompt: List[int], params: SamplingParams, stop: List[str]) -> _Stream:
        st = _Stream(n_prompt=len(prompt), stop=list(stop), t0=time.time())
        if params.seed is None and not params.greedy:
            params.seed = int.from_bytes(__import__("os").urandom(4), "little")     # fixed here so that all ranks sample alike
        self.inbox.put(("add", st, prompt, params))
        self.metrics.inc("requests_total")
        return st

    def cancel(self, st: _Stream):
        self.inbox.put(("cancel", st))

    # ---- engine thread ------------------------------------------------------------------------------
    def start(self):
        self._refresh_snapshot()
        self.thread = threading.Thread(target=self.run, name="engine", daemon=True)
        self.thread.start()

    def shutdown(self):
        self.stop_flag.set()
        self.inbox.put(("wake",))
        if self.thread:
            self.thread.join(timeout=30)

    def _collect_tasks(self, block: bool) -> list:
        tasks = []
        try:
            tasks.append(self.inbox.get(timeout=0.02 if block else 0.0))
        except queue.Empty:
            return tasks
        while True:
            try:
                tasks.append(self.inbox.get_nowait())
            except queue.Empty:
                return tasks

    def _share_tasks(self, tasks: list) -> list:
        """Rank 0 -> all ranks: (kind, local handle or None, prompt, params-dict, rid)."""
        if self.world == 1:
            return tasks
        import torch.distributed as dist
        from ..utils import fault
        fault.check("transport")
        hb = getattr(self, "heartbeat", None)
        if hb is not None:
            gone = hb.dead()
            if gone:
                raise RuntimeError(f"rank(s) {gone} stopped responding")
        wire = [None]
        if self.rank == 0:
            w = []
            for t in tasks:
                if t[0] == "add":
                    w.append(("add", t[2], t[3].__dict__))
                elif t[0] == "cancel":
                    w.append(("cancel", t[1].rid))
            wire = [(w, self.stop_flag.is_set())]
        dist.broadcast_object_list(wire, src=0, group=self.group)
        w, stop = wire[0]
        if stop:
            self.stop_flag.set()
        if self.rank == 0:
            return tasks
        out = []
        for t in w:
            if t[0] == "add":
                out.append(("add", None, t[1], SamplingParams(**t[2])))
            else:
                out.append(("cancel_rid", t[1]))
        return out

    def _prepare_grammar(self, params: SamplingParams) -> None:
        """Every rank that samples a grammar-constrained request needs the table of token texts."""
        if params.grammar and getattr(self.engine, "token_table", None) is None:
            self.engine.token_table = self.tokenizer.token_table()

    def _run_dp(self):
        """Attention data-parallel serving: rank 0 assigns every request to one rank (round robin), all ranks step
        together (a rank without tokens runs the idle forward), and every iteration the new tokens of all ranks are
        gathered to rank 0, which owns the HTTP streams.  Per iteration: one broadcast (tasks, stop, step-or-not) and
        one gather (events, has-work) on the host-side control group."""
        import torch.distributed as dist
        eng = self.engine
        gid_of: Dict[int, int] = {}                  # this rank's engine request id -> global request id
        rid_of: Dict[int, int] = {}
        next_gid, rr, global_work = 1, 0, False
        while True:
            wire = [None]
            if self.rank == 0:
                w = []
                for t in self._collect_tasks(block=not global_work):
                    if t[0] == "add":
                        _, st, prompt, params = t
                        st.rid = next_gid
                        self.streams[next_gid] = st
                        w.append(("add", next_gid, rr % self.world, prompt, params.__dict__))
                        next_gid += 1
                        rr += 1
                        self.metrics.inc("prompt_tokens_total", len(prompt))
                    elif t[0] == "cancel":
                        if t[1].rid >= 0:
                            w.append(("cancel", t[1].rid))
                        if not t[1].done:
                            self._finish(t[1], "cancelled")
                            self.metrics.inc("cancelled_total")
                wire = [(w, self.stop_flag.is_set(), global_work or bool(w))]
            dist.broadcast_object_list(wire, src=0, group=self.group)
            w, stop, run_step = wire[0]
            if stop:
                self.stop_flag.set()
                return
            for t in w:
                if t[0] == "add" and t[2] == self.rank:
                    sp = SamplingParams(**t[4])
                    self._prepare_grammar(sp)
                    rid = eng.add_request(t[3], sp)
                    gid_of[rid], rid_of[t[1]] = t[1], rid
                elif t[0] == "cancel" and t[1] in rid_of:
                    rid = rid_of.pop(t[1])
                    eng.cancel(rid)
                    eng.requests.pop(rid, None)
                    gid_of.pop(rid, None)
            events = []
            if run_step:
                t0 = time.time()
                for rid, tok, fin in eng.step():
                    gid = gid_of.get(rid)
                    if gid is None:
                        continue
                    events.append((gid, tok, fin))
                    if fin is not None:
                        eng.requests.pop(rid, None)
                        gid_of.pop(rid, None)
                        rid_of.pop(gid, None)
                self.metrics.observe_step(time.time() - t0)
                self._refresh_snapshot()
            gathered = [None] * self.world if self.rank == 0 else None
            dist.gather_object((events, eng.has_work()), gathered, dst=0, group=self.group)
            if self.rank == 0:
                global_work = any(g[1] for g in gathered)
                for evs, _ in gathered:
                    for gid, tok, fin in evs:
                        st = self.streams.get(gid)
                        if st is None or st.done:
                            continue
                        if tok >= 0:
                            self._on_token(st, tok)
                        if fin is not None and not st.done:
                            self._finish(st, "stop" if fin == "stop" else ("cancelled" if fin == "cancelled" else "length"))

    def run(self):
        eng = self.engine
        if getattr(eng, "dp", False) and self.world > 1:
            return self._run_dp()
        while not self.stop_flag.is_set():
            tasks = self._collect_tasks(block=not eng.has_work()) if self.rank == 0 else []
            tasks = self._share_tasks(tasks)
            for t in tasks:
                if t[0] == "add":
                    _, st, prompt, params = t
                    try:
                        self._prepare_grammar(params)
                        rid = eng.add_request(prompt, params)
                    except Exception as e:             # a request the engine refuses fails alone
                        if st is not None:
                            st.q.put(("error", f"request rejected: {e}"))
                            st.done = True
                        self.metrics.inc("requests_failed_total")
                        continue
                    if st is not None:
                        st.rid = rid
                        self.streams[rid] = st
                    self.metrics.inc("prompt_tokens_total", len(prompt))
                elif t[0] == "cancel":
                    if t[1].rid >= 0:
                        eng.cancel(t[1].rid)
                        eng.requests.pop(t[1].rid, None)
                    if not t[1].done:
                        self._finish(t[1], "cancelled")
                        self.metrics.inc("cancelled_total")
                elif t[0] == "cancel_rid":
                    eng.cancel(t[1])
                    eng.requests.pop(t[1], None)
            if not eng.has_work():
                if tasks:
                    self._refresh_snapshot()      # a cancel or a rejected request changed what the endpoints show
                continue
            t0 = time.time()
            try:
                events = eng.step()
            except Exception as e:       # fail the in-flight requests with 503 and keep serving (reference: abort)
                n_failed = len(self.streams)
                for st in list(self.streams.values()):
                    st.q.put(("error", f"engine step failed: {e}"))
                    st.done = True
                self.streams.clear()
                self.metrics.inc("requests_failed_total", max(n_failed, 1))
                if self.world > 1:
                    raise                # the ranks' schedulers have diverged: a coordinated restart is the launcher's job
                eng.reset()
                continue
            self.metrics.observe_step(time.time() - t0)
            self._refresh_snapshot()
            if getattr(self.cfg, "display_chat", False):
                self._display_chat()
            for rid, tok, fin in events:
                st = self.streams.get(rid)
                if st is None or st.done:
                    if fin is not None:
                        eng.requests.pop(rid, None)
                    continue
                if tok >= 0:
                    es = eng.requests.get(rid)
                    if es is not None:
                        st.n_cached = es.n_cached
                    if es is not None and es.params.logprobs and len(es.logprobs) > len(st.logprobs):
                        st.logprobs.append(es.logprobs[len(st.logprobs)])      # this rank sampled it: the entry is there
                    self._on_token(st, tok)
                if fin is not None and not st.done:
                    self._finish(st, "stop" if fin == "stop" else ("cancelled" if fin == "cancelled" else "length"))
                if fin is not None:
                    eng.requests.pop(rid, None)

    def _display_chat(self, every: float = 0.25):
        """Console view of what every active request has generated so far, redrawn a few times per second
        (the reference's display_chat: examples/server/server.cpp:1509-1520)."""
        now = time.time()
        if now - getattr(self, "_last_display", 0.0) < every:
            return
        self._last_display = now
        import sys
        lines = ["\x1b[2J\x1b[H" if sys.stderr.isatty() else "---- active requests ----"]
        for rid, st in sorted(self.streams.items()):
            tail = st.text[-200:].replace("\n", " ")
            lines.append(f"[req {rid}] prompt {st.n_prompt} tok, generated {st.n_gen}: {tail}")
        sys.stderr.write("\n".join(lines) + "\n")
        sys.stderr.flush()

    def _emit(self, st: _Stream, text: str):
        if text:
            st.text += text
            st.q.put(("text", text))

    def _on_token(self, st: _Stream, tok: int):
        st.n_gen += 1
        st.tokens.append(int(tok))
        self.metrics.inc("generation_tokens_total")
        if st.n_gen == 1:
            st.t_first = time.time()
        st.pending += self.tokenizer.piece_bytes(tok, special=getattr(self.cfg, "special", False))
        cut = len(st.pending) - self.tokenizer.incomplete_utf8_tail(st.pending)      # hold back a split code point
        chunk, st.pending = st.pending[:cut], st.pending[cut:]
        if not chunk:
            return
        st.held += chunk.decode("utf-8", errors="replace")
        if st.stop:
            for s in st.stop:
                i = st.held.find(s)
                if i >= 0:                                   # stop word: emit what precedes it and finish
                    self._emit(st, st.held[:i])
                    st.held = ""
                    self._finish(st, "stop")
                    self.inbox.put(("cancel", st))      # through the task queue, so that every rank drops it too
                    return
            keep = 0                                         # hold back a possible beginning of a stop word
            for s in st.stop:
                for k in range(min(len(s) - 1, len(st.held)), 0, -1):
                    if st.held.endswith(s[:k]):
                        keep = max(keep, k)
                        break
            out, st.held = st.held[:len(st.held) - keep], st.held[len(st.held) - keep:]
            self._emit(st, out)
        else:
            out, st.held = st.held, ""
            self._emit(st, out)

    def _finish(self, st: _Stream, reason: str):
        if st.done:
            return
        if reason != "cancelled":
            tail = st.held + st.pending.decode("utf-8", errors="replace")
            st.held, st.pending = "", b""
            if reason != "stop" or not st.stop:
                self._emit(st, tail)
        st.done = True
        now = time.time()
        gen_s = max(1e-9, now - (st.t_first or now))
        timings = {"prompt_n": st.n_prompt, "prompt_ms": 1e3 * ((st.t_first or now) - st.t0), "predicted_n": st.n_gen,
                   "predicted_ms": 1e3 * gen_s, "predicted_per_second": (st.n_gen - 1) / gen_s if st.n_gen > 1 else 0.0}
        st.q.put(("done", reason, timings))
        self.streams.pop(st.rid, None)

    # ---- introspection ------------------------------------------------------------------------------
    # The runtime objects belong to the engine thread.  HTTP threads read a snapshot that the engine thread refreshes after
    # every step (and while idle), never the live allocator / scheduler.
    def _refresh_snapshot(self) -> None:
        eng = self.engine
        self._snapshot = (self._gauges_now(), [{"id": i, "state": eng.sched.slot_state(i), "n_past": eng.kv.seq_len(i)}
                                              for i in range(eng.cfg.n_parallel)])

    def _snap(self):
        snap = getattr(self, "_snapshot", None)
        if snap is None or self.thread is None:
            self._refresh_snapshot()              # no engine thread to race with
            snap = self._snapshot
        return snap

    def gauges(self) -> Dict[str, float]:
        return self._snap()[0]

    def slots(self) -> list:
        return self._snap()[1]

    def _gauges_now(self) -> Dict[str, float]:
        eng = self.engine
        return {"requests_running": eng.sched.n_running(), "requests_waiting": eng.sched.n_waiting(),
                "kv_blocks_used": eng.kv.used_blocks, "kv_blocks_total": eng.kv.n_blocks,
                "kv_blocks_used_ratio": eng.kv.used_blocks / max(1, eng.kv.n_blocks),
                "kv_fragmentation": eng.kv.fragmentation(), "graph_steps": eng.stats["graph_steps"],
                "eager_steps": eng.stats["eager_steps"], "defrag_moves": eng.stats.get("defrag_moves", 0),
                "preemptions": eng.sched.stats().get("preemptions", 0) if hasattr(eng.sched, "stats") else 0,
                "prefix_shared": eng.sched.stats().get("prefix_shared", 0) if hasattr(eng.sched, "stats") else 0,
                "kernel_launches": eng.launches, "h2d_bytes": eng.stats["h2d_bytes"], "d2h_bytes": eng.stats["d2h_bytes"],
                "engine_resets": eng.stats.get("resets", 0), "run_ahead_steps": eng.stats.get("run_ahead_steps", 0),
                # collectives this rank took part in (in-kernel or library) and how many used the two-shot (prefill) form
                "collectives": getattr(getattr(eng.model, "comm", None), "n_collectives", 0),
                "collectives_two_shot": getattr(getattr(eng.model, "comm", None), "n_two_shot", 0)}


# =================================================================================================
MAX_BODY_BYTES = 64 << 20          # largest accepted request body


def make_handler(ctx: ServerContext):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"
        server_version = "jittorinfer_b200"

        def log_message(self, fmt, *args):      # quiet by default; errors still go to stderr
            pass

        # ---- helpers ----
        def _json(self, code: int, obj: Any):
            body = json.dumps(obj, ensure_ascii=False).encode("utf-8")
            self.send_response(code)
            self.send_header("Content-Type", "application/json; charset=utf-8")
            self.send_header("Content-Length", str(len(body)))
            self.send_header("Access-Control-Allow-Origin", "*")
            self.end_headers()
            self.wfile.write(body)

        def _text(self, code: int, text: str, ctype="text/plain; version=0.0.4"):
            body = text.encode("utf-8")
            self.send_response(code)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def _chunk(self, data: bytes):
            self.wfile.write(b"%x\r\n" % len(data) + data + b"\r\n")
            self.wfile.flush()

        # ---- GET ----
        def do_GET(self):
            path = self.path.split("?")[0]
            if path in ("/health", "/v1/health"):
                return self._json(200, {"status": "ok"})
            if path == "/metrics":
                return self._text(200, ctx.metrics.render(ctx.gauges()))
            if path in ("/v1/models", "/models"):
                return self._json(200, {"object": "list", "data": [{"id": ctx.model_alias, "object": "model", "owned_by": "jittorinfer_b200"}]})
            if path == "/slots":
                eng = ctx.engine
                return self._json(200, ctx.slots())
            if path == "/props":
                eng = ctx.engine
                return self._json(200, {"model_alias": ctx.model_alias, "n_ctx_slot": eng.n_ctx_slot, "total_slots": eng.cfg.n_parallel,
                                        "n_batch": eng.cfg.n_batch, "kv_blocks": eng.kv.n_blocks, "chat_template": ctx.template.source})
            if path == "/exit":                  # same as the reference: shut the server down
                self._json(200, {"status": "exiting"})
                threading.Thread(target=self.server.shutdown, daemon=True).start()
                return
            self._json(404, P.error_body("not found", 404, "not_found_error"))

        def do_OPTIONS(self):
            self.send_response(204)
            self.send_header("Access-Control-Allow-Origin", "*")
            self.send_header("Access-Control-Allow-Headers", "*")
            self.send_header("Content-Length", "0")
            self.end_headers()

        # ---- POST ----
        def do_POST(self):
            path = self.path.split("?")[0]
            try:
                n = int(self.headers.get("Content-Length", "0"))
                if n < 0 or n > MAX_BODY_BYTES:          # a negative length would read until the peer closes
                    self.close_connection = True
                    return self._json(413, P.error_body(f"request body must be 0..{MAX_BODY_BYTES} bytes", 413))
                body = json.loads(self.rfile.read(n) or b"{}")
                if not isinstance(body, dict):
                    raise P.BadRequest("request body must be a JSON object")
                if path in ("/v1/completions", "/completions", "/completion"):
                    req = P.parse_completion(body, ctx.tokenizer, ctx.model_alias, ctx.default_max)
                elif path in ("/v1/chat/completions", "/chat/completions"):
                    req = P.parse_chat(body, ctx.tokenizer, ctx.template, ctx.model_alias, ctx.default_max)
                elif path in ("/tokenize", "/v1/tokenize"):
                    return self._json(200, {"tokens": ctx.tokenizer.encode(str(body.get("content", "")), bool(body.get("add_special", False)))})
                elif path in ("/detokenize", "/v1/detokenize"):
                    return self._json(200, {"content": ctx.tokenizer.decode(list(body.get("tokens", [])))})
                else:
                    return self._json(404, P.error_body("not found", 404, "not_found_error"))
                n_vocab = ctx.engine.hp.n_vocab
                for p in req.prompts:
                    if not p:
                        raise P.BadRequest("empty prompt")
                    if min(p) < 0 or max(p) >= n_vocab:
                        raise P.BadRequest(f"prompt token ids must be in [0, {n_vocab})")
                if req.stream and len(req.prompts) != 1:
                    raise P.BadRequest("streaming supports a single prompt")
            except P.BadRequest as e:
                ctx.metrics.inc("requests_failed_total")
                return self._json(400, P.error_body(str(e), 400))
            except (json.JSONDecodeError, UnicodeDecodeError, ValueError) as e:
                ctx.metrics.inc("requests_failed_total")
                return self._json(400, P.error_body(f"invalid request: {e}", 400))
            if req.params.logprobs and getattr(ctx.engine, "dp", False) and ctx.world > 1:
                # with data-parallel attention a request is sampled on the rank that owns it; only ids travel back
                ctx.metrics.inc("requests_failed_total")
                return self._json(400, P.error_body("logprobs are not available with attention_dp", 400))
            if req.grammar and getattr(ctx.cfg, "enforce_response_format", True):
                req.params.grammar = req.grammar               # response_format is enforced token by token
                if getattr(ctx.engine, "token_table", None) is None:
                    ctx.engine.token_table = ctx.tokenizer.token_table()
                try:                                           # compile it here: a grammar the engine cannot build is a 400
                    from ..runtime.sampling import NativeSampler
                    NativeSampler(SamplingParams(grammar=req.grammar), token_table=ctx.engine.token_table)
                except Exception as e:
                    ctx.metrics.inc("requests_failed_total")
                    return self._json(400, P.error_body(f"response_format: {e}", 400))
            streams = [ctx.submit(p, SamplingParams(**req.params.__dict__), req.stop) for p in req.prompts]
            try:
                if req.stream:
                    self._stream(req, streams[0])
                else:
                    self._blocking(req, streams)
            except (BrokenPipeError, ConnectionResetError):
                for st in streams:               # client went away: free the slot (reference: server.cpp:1216-1220)
                    ctx.cancel(st)

        def _wait(self, st: _Stream):
            """Yields ('text', str) ... then ('done', reason, timings)."""
            while True:
                try:
                    item = st.q.get(timeout=1.0)
                except queue.Empty:
                    if ctx.stop_flag.is_set():
                        yield ("error", "server shutting down")
                        return
                    continue
                yield item
                if item[0] in ("done", "error"):
                    return

        def _blocking(self, req: P.ParsedRequest, streams: List[_Stream]):
            rid = P.new_id(req.chat)
            results = []
            for st in streams:
                text, reason, timings = "", "length", None
                for item in self._wait(st):
                    if item[0] == "text":
                        text += item[1]
                    elif item[0] == "done":
                        reason, timings = item[1], item[2]
                    else:
                        return self._json(503, P.error_body(item[1], 503, "unavailable_error"))
                results.append((st, text, reason, timings))
            piece = lambda t: ctx.tokenizer.piece_bytes(t, special=True).decode("utf-8", errors="replace")      # noqa: E731
            if req.chat:
                st, text, reason, timings = results[0]
                reasoning, content = split_reasoning(text, ctx.reasoning)
                body = P.chat_response(rid, req.model, content, reasoning, parse_tool_call(content), reason, st.n_prompt, st.n_gen, timings,
                                       st.n_cached)
                if req.params.logprobs:
                    body["choices"][0]["logprobs"] = P.chat_logprobs(st.logprobs, piece)
                return self._json(200, body)
            if len(results) == 1:
                st, text, reason, timings = results[0]
                body = P.completion_response(rid, req.model, text, reason, st.n_prompt, st.n_gen, 0, timings, st.n_cached)
                if req.return_tokens:
                    body["choices"][0]["tokens"] = list(st.tokens)
                if req.params.logprobs:
                    body["choices"][0]["logprobs"] = P.completion_logprobs(st.logprobs, piece)
                return self._json(200, body)
            out = [P.completion_response(rid, req.model, text, reason, st.n_prompt, st.n_gen, i, timings, st.n_cached)
                   for i, (st, text, reason, timings) in enumerate(results)]
            self._json(200, out)

        def _stream(self, req: P.ParsedRequest, st: _Stream):
            rid = P.new_id(req.chat)
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Transfer-Encoding", "chunked")
            self.send_header("Access-Control-Allow-Origin", "*")
            self.end_headers()
            if req.chat:
                self._chunk(P.sse(P.chat_chunk(rid, req.model, {"role": "assistant", "content": ""}, None)))
            for item in self._wait(st):
                if item[0] == "text":
                    obj = P.chat_chunk(rid, req.model, {"content": item[1]}, None) if req.chat else P.completion_chunk(rid, req.model, item[1], None)
                    self._chunk(P.sse(obj))
                elif item[0] == "done":
                    usage = {"prompt_tokens": st.n_prompt, "completion_tokens": st.n_gen, "total_tokens": st.n_prompt + st.n_gen,
                             "prompt_tokens_details": {"cached_tokens": st.n_cached}}
                    obj = P.chat_chunk(rid, req.model, {}, item[1], usage) if req.chat else P.completion_chunk(rid, req.model, "", item[1], usage)
                    obj["timings"] = item[2]
                    if req.params.logprobs:      # streamed text is cut at code-point boundaries, not token boundaries: the
                        piece = lambda t: ctx.tokenizer.piece_bytes(t, special=True).decode("utf-8", errors="replace")      # noqa: E731
                        obj["choices"][0]["logprobs"] = (P.chat_logprobs if req.chat else P.completion_logprobs)(st.logprobs, piece)
                        # per-token log-probabilities of the whole answer come with the final chunk
                    self._chunk(P.sse(obj))
                else:
                    self._chunk(P.sse(P.error_body(item[1], 503, "unavailable_error")))
            self._chunk(P.sse("[DONE]"))
            self.wfile.write(b"0\r\n\r\n")
            self.wfile.flush()

    return Handler


class PooledHTTPServer(ThreadingHTTPServer):
    """``n_threads_http`` of the configuration (reference: common_local.h, ``n_threads_http``): connections are handled by a
    fixed pool of worker threads instead of one new thread each; further connections wait in the pool's queue."""

    def __init__(self, addr, handler, n_threads: int):
        super().__init__(addr, handler)
        from concurrent.futures import ThreadPoolExecutor
        self._pool = ThreadPoolExecutor(max_workers=n_threads, thread_name_prefix="http")

    def process_request(self, request, client_address):
        self._pool.submit(self.process_request_thread, request, client_address)

    def server_close(self):
        super().server_close()
        self._pool.shutdown(wait=False, cancel_futures=True)


def serve(ctx: ServerContext, host: str, port: int, n_threads: int = -1) -> ThreadingHTTPServer:
    """Starts the engine thread and returns the (not yet serving) HTTP server; call serve_forever() on it.
    ``n_threads`` > 0 bounds the number of HTTP worker threads; otherwise every connection gets its own thread."""
    httpd = PooledHTTPServer((host, port), make_handler(ctx), n_threads) if n_threads and n_threads > 0 \
        else ThreadingHTTPServer((host, port), make_handler(ctx))
    httpd.daemon_threads = True
    ctx.start()
    return httpd
