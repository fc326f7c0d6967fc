"""The package's fp32 oracle and engine against logits computed by the reference's own CPU code.

``tests/data/reference_cpu_logits.npz`` holds, for two small models, the logits that the reference's loader + graph builder +
ggml CPU kernels produced for a 32-token sequence from a GGUF file written by this package (made by
``python -m jittorinfer_b200.utils.ref_cpu_oracle``; that module says what had to be stood in for).  The files are recreated
here from the same seeds, so a change of the writer, of the tensor layouts or of the forward pass shows up against numbers
this package did not produce.  With ``JITTORINFER_REFERENCE_DIR`` pointing at a checkout of the reference the stubbed build
is also redone and compared live."""
import os

import numpy as np
import pytest
import torch

from jittorinfer_b200.models.oracle import OracleModel
from jittorinfer_b200.models.weights import random_weights
from jittorinfer_b200.utils import ref_cpu_oracle as R

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "reference_cpu_logits.npz")


@pytest.mark.parametrize("name", ["v2", "lite"])
def test_oracle_matches_the_reference_cpu_logits(name):
    gold = np.load(GOLD)
    hp = R.case(name)
    toks = R.case_tokens(hp)
    assert toks == gold[f"{name}_tokens"].tolist()
    ref = gold[f"{name}_logits"]
    mine = OracleModel(hp, random_weights(hp, seed=0, std=0.05)).forward(torch.tensor(toks)).numpy()
    assert ref.shape == mine.shape == (len(toks), hp.n_vocab)
    # the reference keeps its cache and its norm weights in half precision: a few 1e-3 of the largest logit (measured 4.0e-3 at 3
    # layers, 7.8e-3 at 27)
    assert np.abs(ref - mine).max() <= 1e-2 * max(1.0, float(np.abs(mine).max()))
    assert (ref.argmax(-1) == mine.argmax(-1)).all()


def test_engine_continues_as_the_reference_would():
    """The serving engine (CPU, fp32, chunked prefill through the paged cache) picks, after every prefix, the token the
    reference's logits rank first."""
    from jittorinfer_b200.models.deepseek2 import DeepSeek2Model
    from jittorinfer_b200.runtime.engine import EngineConfig, LLMEngine
    from jittorinfer_b200.runtime.sampling import SamplingParams
    gold = np.load(GOLD)
    hp = R.case("v2")
    toks = gold["v2_tokens"].tolist()
    ref_next = gold["v2_logits"].argmax(-1)
    m = DeepSeek2Model(hp, random_weights(hp, seed=0, std=0.05).items(), dtype=torch.float32)
    eng = LLMEngine(m, EngineConfig(n_ctx=512, n_batch=16, n_parallel=4, n_ctx_slot=128, cuda_graphs=False))
    prefixes = [5, 16, 17, 32]
    outs = eng.generate([toks[:n] for n in prefixes], SamplingParams(ignore_eos=True), max_new_tokens=1)
    assert [o[0] for o in outs] == [int(ref_next[n - 1]) for n in prefixes]


@pytest.mark.skipif(not os.environ.get("JITTORINFER_REFERENCE_DIR"), reason="set JITTORINFER_REFERENCE_DIR to a checkout of the reference")
def test_stubbed_build_of_the_reference_reproduces_the_stored_logits(tmp_path):
    exe = R.build(os.environ["JITTORINFER_REFERENCE_DIR"], str(tmp_path))
    from jittorinfer_b200.models.weights import write_random_gguf
    gold = np.load(GOLD)
    hp = R.case("v2")
    path = str(tmp_path / "m.gguf")
    write_random_gguf(path, hp, seed=0, std=0.05)
    live = R.reference_logits(exe, path, gold["v2_tokens"].tolist(), str(tmp_path))
    assert np.abs(live - gold["v2_logits"]).max() <= 1e-4
    # and back: the reference's GGUF writer re-emits the file byte for byte
    import filecmp
    import subprocess
    back = str(tmp_path / "back.gguf")
    subprocess.run([R.build_rewriter(str(tmp_path)), path, back], check=True)
    assert filecmp.cmp(path, back, shallow=False)
