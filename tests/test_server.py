"""OpenAI-compatible server end to end on CPU: tiny random model, toy byte-level vocabulary."""
import json
import os
import threading
import urllib.error
import urllib.request

import pytest
import torch

from jittorinfer_b200.config import ServerConfig
from jittorinfer_b200.server.app import ServerContext, serve
from jittorinfer_b200.server.chat import ChatTemplate, apply_deepseek2, split_reasoning
from jittorinfer_b200.server.launch import build_from_config


@pytest.fixture(scope="module")
def server():
    cfg = ServerConfig(random_init="tiny", n_ctx=2048, n_parallel=4, n_batch=64, port=0, enable_ge=False)
    eng, tok, tpl = build_from_config(cfg, device=torch.device("cpu"))
    ctx = ServerContext(eng, tok, cfg, ChatTemplate(tpl))
    httpd = serve(ctx, "127.0.0.1", 0)
    t = threading.Thread(target=httpd.serve_forever, daemon=True)
    t.start()
    yield f"http://127.0.0.1:{httpd.server_address[1]}", ctx
    httpd.shutdown()
    httpd.server_close()
    ctx.shutdown()


def _post(url, body, stream=False):
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=120) as r:
        data = r.read().decode()
    return data if stream else json.loads(data)


def test_completion_and_usage(server):
    url, ctx = server
    r = _post(url + "/v1/completions", {"prompt": "hello there", "max_tokens": 8, "temperature": 0, "ignore_eos": True})
    assert r["object"] == "text_completion" and r["choices"][0]["finish_reason"] == "length"
    assert r["usage"]["completion_tokens"] == 8 and r["usage"]["prompt_tokens"] == len(ctx.tokenizer.encode("hello there"))
    r2 = _post(url + "/v1/completions", {"prompt": "hello there", "max_tokens": 8, "temperature": 0, "ignore_eos": True})
    assert r2["choices"][0]["text"] == r["choices"][0]["text"]          # greedy is deterministic (and hits the prefix cache)
    assert r["usage"]["prompt_tokens_details"]["cached_tokens"] == 0
    assert r2["usage"]["prompt_tokens_details"]["cached_tokens"] == r2["usage"]["prompt_tokens"] - 1      # all but the token that yields logits
    r3 = _post(url + "/v1/completions", {"prompt": [5, 6, 7, 8], "max_tokens": 3, "temperature": 0.7, "seed": 1, "ignore_eos": True})
    assert {k: r3["usage"][k] for k in ("prompt_tokens", "completion_tokens", "total_tokens")} == \
        {"prompt_tokens": 4, "completion_tokens": 3, "total_tokens": 7}


def test_chat_and_stream(server):
    url, _ = server
    body = {"messages": [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}], "max_tokens": 6,
            "temperature": 0, "ignore_eos": True}
    r = _post(url + "/v1/chat/completions", body)
    assert r["object"] == "chat.completion" and r["choices"][0]["message"]["role"] == "assistant"
    s = _post(url + "/v1/chat/completions", dict(body, stream=True), stream=True)
    events = [json.loads(l[6:]) for l in s.split("\n") if l.startswith("data: ") and l != "data: [DONE]"]
    assert s.rstrip().endswith("data: [DONE]")
    text = "".join(e["choices"][0]["delta"].get("content", "") for e in events)
    assert text == (r["choices"][0]["message"]["content"] or "")
    assert events[-1]["choices"][0]["finish_reason"] == "length" and events[-1]["usage"]["completion_tokens"] == 6
    assert all("usage" not in e for e in events[:-1])                   # usage only on the final chunk


def test_stop_word_and_multi_prompt(server):
    url, _ = server
    full = _post(url + "/v1/completions", {"prompt": "abc", "max_tokens": 24, "temperature": 0, "ignore_eos": True})["choices"][0]["text"]
    if len(full) >= 6:
        stop = full[3:5]
        cut = _post(url + "/v1/completions", {"prompt": "abc", "max_tokens": 24, "temperature": 0, "ignore_eos": True, "stop": [stop]})
        assert cut["choices"][0]["finish_reason"] == "stop" and cut["choices"][0]["text"] == full[:full.find(stop)]
    multi = _post(url + "/v1/completions", {"prompt": ["one", "two two"], "max_tokens": 4, "temperature": 0, "ignore_eos": True})
    assert isinstance(multi, list) and len(multi) == 2


def test_errors_and_introspection(server):
    url, _ = server
    for bad in ({"prompt": "x", "n": 2}, {"prompt": "x", "n_probs": 3}, {"prompt": "x", "echo": True}, {"messages": []}, {},
                {"prompt": [5, 10 ** 9]}, {"prompt": [3, -4]}, {"prompt": "x", "temperature": float("nan")},
                {"prompt": "x", "top_p": float("inf")}, {"prompt": "x", "n_keep": "many"}):
        path = "/v1/chat/completions" if "messages" in bad else "/v1/completions"
        with pytest.raises(urllib.error.HTTPError) as e:
            _post(url + path, bad)
        assert e.value.code == 400 and "error" in json.loads(e.value.read())
    # malformed JSON and absurd body lengths are refused without touching the engine
    import http.client
    host, port = url.replace("http://", "").split(":")
    for headers, payload, want in (({"Content-Length": "7"}, b"{not js", 400), ({"Content-Length": "-5"}, b"", 413),
                                   ({"Content-Length": str(1 << 40)}, b"", 413)):
        c = http.client.HTTPConnection(host, int(port), timeout=10)
        c.putrequest("POST", "/v1/completions")
        for k, v in headers.items():
            c.putheader(k, v)
        c.endheaders()
        c.send(payload)
        r = c.getresponse()
        assert r.status == want and "error" in json.loads(r.read())
        c.close()
    assert json.loads(urllib.request.urlopen(url + "/health").read())["status"] == "ok"
    m = urllib.request.urlopen(url + "/metrics").read().decode()
    assert "jittorinfer_generation_tokens_total" in m and "jittorinfer_kv_blocks_total" in m
    assert len(json.loads(urllib.request.urlopen(url + "/slots").read())) == 4
    assert json.loads(urllib.request.urlopen(url + "/v1/models").read())["data"][0]["object"] == "model"


def test_templates_and_reasoning():
    msgs = [{"role": "system", "content": "S"}, {"role": "user", "content": "U"}, {"role": "assistant", "content": "A"},
            {"role": "user", "content": [{"type": "text", "text": "U2"}]}]
    assert apply_deepseek2(msgs) == "S\n\nUser: U\n\nAssistant: A<｜end▁of▁sentence｜>User: U2\n\nAssistant:"
    t = ChatTemplate("{% for m in messages %}[{{ m.role }}]{{ m.content }}{% endfor %}{% if add_generation_prompt %}[assistant]{% endif %}")
    assert t.render(msgs[:2]) == "[system]S[user]U[assistant]"
    assert split_reasoning("<think>why</think>answer", True) == ("why", "answer")
    assert split_reasoning("plain", True) == (None, "plain") and split_reasoning("<think>x</think>y", False) == (None, "<think>x</think>y")


def test_serving_benchmark_poisson(server):
    """The load generator against the in-process server: open-loop arrivals, streamed responses, client-side timings."""
    from jittorinfer_b200.server import bench_serving
    url, ctx = server
    res = bench_serving.run(url, rate=50.0, num_requests=10, prompt_min=4, prompt_max=40, output_len=5, max_concurrency=4,
                            n_vocab=1000, seed=1, timeout=120)
    assert res["completed"] == 10 and res["failed"] == 0 and res["errors"] == []
    assert res["output_tokens_per_s"] > 0 and res["ttft_ms"]["p50"] > 0 and res["e2e_ms"]["p99"] >= res["ttft_ms"]["p50"]
    closed = bench_serving.run(url, rate=0.0, num_requests=6, prompt_min=4, prompt_max=8, output_len=3, max_concurrency=2,
                               n_vocab=1000, seed=2, timeout=120)
    assert closed["completed"] == 6 and closed["arrivals"].startswith("closed loop")
    m = bench_serving.scrape_metrics(url)
    assert "jittorinfer_kv_blocks_used_ratio" in m and m["jittorinfer_requests_total"] >= 16
    # a common system prompt: later requests start from the blocks an earlier one computed
    shared0 = m.get("jittorinfer_prefix_shared", 0)
    sp = bench_serving.run(url, rate=0.0, num_requests=6, prompt_min=4, prompt_max=10, output_len=3, max_concurrency=2,
                           n_vocab=1000, seed=3, timeout=120, shared_prefix=150)
    assert sp["completed"] == 6 and sp["shared_prefix"] == 150
    # whether a request shares another slot's blocks or finds the prefix in its own slot's cache depends on arrival
    # timing; the engine test pins the sharing itself (test_prefix_blocks_are_shared_across_slots)
    assert bench_serving.scrape_metrics(url)["jittorinfer_prefix_shared"] >= shared0


def test_generate_cli(capsys):
    from jittorinfer_b200 import generate
    rc = generate.main(["--random-init", "tiny", "--device", "cpu", "--tokens", "5,6,7,8,9", "-p", "hello", "-n", "5", "--ignore-eos",
                        "--json"])
    assert rc == 0
    out = json.loads(capsys.readouterr().out)
    assert [len(c["tokens"]) for c in out["completions"]] == [5, 5] and out["timing"]["generated_tokens"] == 10
    assert generate.main(["--device", "cpu"]) == 2


def test_clients_that_disconnect_free_their_slots(server):
    """Streaming clients that go away mid-generation: the server cancels their requests (reference: server.cpp:1216-1220),
    the slots return to idle, and requests that stayed connected complete normally."""
    import http.client
    import concurrent.futures as cf
    import time
    url, ctx = server
    host, port = url.replace("http://", "").split(":")

    def quitter(i):
        c = http.client.HTTPConnection(host, int(port), timeout=60)
        body = json.dumps({"prompt": f"quit early {i}", "max_tokens": 400, "temperature": 0, "ignore_eos": True, "stream": True})
        c.request("POST", "/v1/completions", body=body, headers={"Content-Type": "application/json"})
        r = c.getresponse()
        r.read(40)                      # the first bytes of the stream, then hang up
        c.close()
        return True

    def stayer(i):
        return _post(url + "/v1/completions", {"prompt": f"stay {i}", "max_tokens": 12, "temperature": 0, "ignore_eos": True})

    with cf.ThreadPoolExecutor(8) as ex:
        q = [ex.submit(quitter, i) for i in range(4)]
        s = [ex.submit(stayer, i) for i in range(4)]
        assert all(f.result() for f in q)
        done = [f.result() for f in s]
    assert all(d["usage"]["completion_tokens"] == 12 for d in done)
    deadline = time.time() + 30
    while time.time() < deadline:
        slots = json.loads(urllib.request.urlopen(url + "/slots", timeout=10).read())
        if all(sl["state"] == "IDLE" for sl in slots) and not ctx.streams:
            break
        time.sleep(0.1)
    assert all(sl["state"] == "IDLE" for sl in slots) and not ctx.streams
    assert ctx.engine.kv.check()
    assert _post(url + "/v1/completions", {"prompt": "after", "max_tokens": 3, "temperature": 0, "ignore_eos": True})["usage"]["completion_tokens"] == 3


def test_bounded_http_worker_pool():
    """n_threads_http > 0: a fixed pool of HTTP workers; more simultaneous requests than workers still all complete."""
    from concurrent.futures import ThreadPoolExecutor

    from jittorinfer_b200.server.app import PooledHTTPServer
    cfg = ServerConfig(random_init="tiny", n_ctx=1024, n_parallel=4, n_batch=64, port=0, enable_ge=False, n_threads_http=2)
    eng, tok, tpl = build_from_config(cfg, device=torch.device("cpu"))
    ctx = ServerContext(eng, tok, cfg, ChatTemplate(tpl))
    httpd = serve(ctx, "127.0.0.1", 0, cfg.n_threads_http)
    assert isinstance(httpd, PooledHTTPServer)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    url = f"http://127.0.0.1:{httpd.server_address[1]}"
    try:
        with ThreadPoolExecutor(6) as ex:
            outs = list(ex.map(lambda i: _post(url + "/v1/completions", {"prompt": f"p{i}", "max_tokens": 4, "temperature": 0, "ignore_eos": True}), range(6)))
        assert all(o["usage"]["completion_tokens"] == 4 for o in outs)
        assert sum(t.name.startswith("http") for t in threading.enumerate()) <= 2
    finally:
        httpd.shutdown()
        httpd.server_close()
        ctx.shutdown()


def test_logprobs_in_completions_and_chat(server):
    url, ctx = server
    r = _post(url + "/v1/completions", {"prompt": "hello", "max_tokens": 5, "temperature": 0, "ignore_eos": True, "logprobs": 3,
                                        "return_tokens": True})
    lp = r["choices"][0]["logprobs"]
    assert len(lp["tokens"]) == len(lp["token_logprobs"]) == len(lp["top_logprobs"]) == len(lp["text_offset"]) == 5
    assert all(v <= 1e-6 for v in lp["token_logprobs"]) and all(len(d) <= 3 for d in lp["top_logprobs"])
    for t, v, alts in zip(lp["tokens"], lp["token_logprobs"], lp["top_logprobs"]):      # greedy: the token is the best alternative
        assert abs(max(alts.values()) - v) < 1e-6
    c = _post(url + "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "temperature": 0,
                                             "ignore_eos": True, "logprobs": True, "top_logprobs": 2})
    content = c["choices"][0]["logprobs"]["content"]
    assert len(content) == 4 and all(len(e["top_logprobs"]) == 2 and e["logprob"] <= 1e-6 and isinstance(e["bytes"], list) for e in content)
    plain = _post(url + "/v1/completions", {"prompt": "hello", "max_tokens": 5, "temperature": 0, "ignore_eos": True})
    assert plain["choices"][0]["logprobs"] is None and plain["choices"][0]["text"] == r["choices"][0]["text"]
    s = _post(url + "/v1/completions", {"prompt": "hello", "max_tokens": 3, "temperature": 0, "ignore_eos": True, "logprobs": 1,
                                        "stream": True}, stream=True)
    chunks = [json.loads(ln[6:]) for ln in s.splitlines() if ln.startswith("data: {")]
    assert len(chunks[-1]["choices"][0]["logprobs"]["tokens"]) == 3
    with pytest.raises(urllib.error.HTTPError) as e:
        _post(url + "/v1/completions", {"prompt": "x", "logprobs": 50})
    assert e.value.code == 400


def test_request_fields_of_the_reference_server_are_parsed():
    """``n_keep`` is read per request, as the reference's server reads it; ``id_slot`` / ``post_sampling_probs`` are accepted
    (slots are chosen by prefix match here, and probabilities come through the OpenAI ``logprobs`` field)."""
    from jittorinfer_b200.server.protocol import sampling_from_body
    assert sampling_from_body({"n_keep": 7}, 16).n_keep == 7
    assert sampling_from_body({"n_keep": -1}, 16).n_keep == -1
    assert sampling_from_body({}, 16).n_keep is None
    p = sampling_from_body({"id_slot": 3, "post_sampling_probs": True, "temperature": 0.5}, 16)
    assert p.n_keep is None and p.temperature == 0.5
    from jittorinfer_b200.runtime.sampling import SamplingParams
    assert SamplingParams(**p.__dict__) == p                      # what the data-parallel server sends to the owning rank


def test_example_client_streams_both_routes(server, capsys):
    import importlib.util
    url, _ = server
    spec = importlib.util.spec_from_file_location("example_client", os.path.join(os.path.dirname(__file__), "..", "examples", "client.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    pieces = list(mod.stream(url + "/v1/completions", {"prompt": "the", "max_tokens": 6, "temperature": 0, "ignore_eos": True}))
    whole = _post(url + "/v1/completions", {"prompt": "the", "max_tokens": 6, "temperature": 0, "ignore_eos": True})
    assert "".join(pieces) == whole["choices"][0]["text"]
    assert mod.main(["--url", url, "--max-tokens", "5", "--temperature", "0", "hello"]) == 0
    assert capsys.readouterr().out.endswith("\n")
