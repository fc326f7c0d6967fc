"""The CUDA branch of the op front-end without a GPU: every call the model makes through ``ops`` must fit the signature
of the function in ``ops.native`` that it reaches on a GPU.  A stand-in for the native module checks each call against
the real signature (``inspect.signature(...).bind``) and then computes the result with the reference op, so a bf16 model
pass through the "native" branch must equal the same pass through the reference branch."""
import inspect
import types

import pytest
import torch

from jittorinfer_b200 import ops
from jittorinfer_b200.models.deepseek2 import DeepSeek2Model
from jittorinfer_b200.models.hparams import preset
from jittorinfer_b200.models.weights import random_weights
from jittorinfer_b200.ops import native
from jittorinfer_b200.ops import reference as ref
from jittorinfer_b200.runtime.engine import EngineConfig, LLMEngine
from jittorinfer_b200.runtime.sampling import SamplingParams


def _stand_in(calls, fused_norm):
    def make(name):
        nsig = inspect.signature(getattr(native, name))
        rfn = getattr(ref, name)
        n_ref = len(inspect.signature(rfn).parameters)

        def f(*a, **k):
            ba = nsig.bind(*a, **k)                     # TypeError here = the front-end does not fit the native signature
            ba.apply_defaults()
            calls.append(name)
            vals = list(ba.arguments.values())
            if name == "moe_gate" and ba.arguments.get("pre_norm") is not None:
                w, eps = ba.arguments["pre_norm"]             # the router launch normalises its input rows itself
                gn = ref.rmsnorm(vals[0], w, eps)[0]
                ids, wts = rfn(gn, *vals[1:n_ref])
                return ids, wts, gn
            out = rfn(*vals[:n_ref])
            if name == "moe_ffn" and ba.arguments.get("norm") is not None:
                w, eps = ba.arguments["norm"]
                return out, ref.rmsnorm(out, w, eps)[0]
            return out
        return f
    names = [n for n in dir(native) if not n.startswith("_") and inspect.isfunction(getattr(native, n)) and hasattr(ref, n)]
    fns = {n: make(n) for n in names}

    def gather_rows(*a, **k):                           # the one front-end target without a reference twin
        ba = inspect.signature(native.gather_rows).bind(*a, **k)
        calls.append("gather_rows")
        x, rows = list(ba.arguments.values())[:2]
        return x[rows.long()].contiguous()
    fns["gather_rows"] = gather_rows
    # the per-head prompt attention needs real kernels: the stand-in declines it, prompts take the absorbed form
    return types.SimpleNamespace(FUSED_COMBINE_NORM=fused_norm, mha_prefill_ok=lambda *a, **k: False, **fns), names


@pytest.mark.parametrize("fused_norm", [False, True])
@pytest.mark.parametrize("name", ["tiny", "tiny-v2", "tiny-v3"])
def test_model_calls_fit_the_native_signatures(monkeypatch, name, fused_norm):
    hp = preset(name)
    w = random_weights(hp, seed=0)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, hp.n_vocab, (n,), generator=g).tolist() for n in (9, 30)]

    def run():
        m = DeepSeek2Model(hp, w.items(), dtype=torch.bfloat16)
        eng = LLMEngine(m, EngineConfig(n_ctx=512, n_batch=32, n_parallel=2, n_ctx_slot=128, device_sampling=True))
        a = eng.add_request(prompts[0], SamplingParams(ignore_eos=True, max_tokens=4))
        b = eng.add_request(prompts[1], SamplingParams(ignore_eos=True, max_tokens=4, temperature=0.9, seed=2))
        while eng.has_work():
            eng.step()
        return eng.requests[a].output, eng.requests[b].output

    want = run()                                          # reference branch, bf16
    calls = []
    fake, names = _stand_in(calls, fused_norm)
    monkeypatch.setattr(ops, "_native", fake)
    monkeypatch.setattr(ops, "use_native", lambda t: True)
    got = run()
    assert got == want
    used = set(calls)
    assert {"rmsnorm", "linear", "mla_qkv_post", "q_absorb", "mla_attention", "v_up", "moe_gate", "moe_ffn", "argmax", "topk_logits",
            "sample_topk", "embed_gather"} <= used, sorted(used)


def test_prompt_attention_form_is_chosen_by_what_would_be_expanded():
    """The per-head prompt attention expands the cached rows of every sequence of the step: it is taken for prompt chunks, not
    for small batches, other head sizes, or mixed steps whose rows are mostly the contexts of sequences that only decode."""
    ok = native.mha_prefill_ok
    dims = (128, 64, 128, 512, 64)
    assert ok(2048, *dims, {"total_kv": 2048, "n_q_tiles": 16})
    assert ok(2048, *dims, {"total_kv": 2048 + 30000, "n_q_tiles": 16, "kv_decode": 0})          # a chunk deep into a long prompt
    assert ok(2048, *dims, {"total_kv": 2048 + 1500, "n_q_tiles": 17, "kv_decode": 1500})        # one decoding neighbour
    assert not ok(2048, *dims, {"total_kv": 2048 + 64 * 4000, "n_q_tiles": 80, "kv_decode": 64 * 4000})
    assert not ok(32, *dims, {"total_kv": 32, "n_q_tiles": 1})                                    # below the size that pays
    assert not ok(2048, 32, 16, 32, 64, 64, {"total_kv": 2048, "n_q_tiles": 16})                  # not the DeepSeek head sizes
    assert not ok(2048, *dims, None)
