"""Block-quantised checkpoint types: the numpy and the native expanders agree bit for bit on random blocks, the quantisers
round-trip within the resolution of each type, shards of quantised tensors equal slices of the whole tensor, and a model
loaded from a quantised file computes what the same weights stored as fp32 compute."""
import ctypes as C

import numpy as np
import pytest
import torch

from jittorinfer_b200.gguf import format as F
from jittorinfer_b200.gguf import quants as Q
from jittorinfer_b200.gguf.io import GGUFReader, GGUFWriter

TYPES = sorted(Q.TRAITS)
# offsets of the half-precision fields of each block (random bytes there would make infinities and NaNs)
HALF_FIELDS = {Q.Q4_0: [0], Q.Q4_1: [0, 2], Q.Q5_0: [0], Q.Q5_1: [0, 2], Q.Q8_0: [0], Q.Q2_K: [80, 82], Q.Q3_K: [108],
               Q.Q4_K: [0, 2], Q.Q5_K: [0, 2], Q.Q6_K: [208]}


def random_blocks(t, n, seed):
    rng = np.random.default_rng(seed)
    blk, bsz = Q.TRAITS[t]
    b = rng.integers(0, 256, size=(n, bsz), dtype=np.uint8)
    for off in HALF_FIELDS.get(t, []):
        b[:, off:off + 2] = rng.uniform(-2, 2, size=(n, 1)).astype(np.float16).view(np.uint8)
    if t == Q.Q8_K:
        b[:, 0:4] = rng.uniform(-2, 2, size=(n, 1)).astype("<f4").view(np.uint8)
    return b


def native(t, blocks, bf16=False, threads=0):
    from jittorinfer_b200.runtime.native_rt import lib
    L = lib()
    L.jib_dequantize.restype = C.c_int
    L.jib_dequantize.argtypes = [C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p, C.c_int, C.c_int]
    n = blocks.shape[0] * Q.TRAITS[t][0]
    out = torch.empty(n, dtype=torch.bfloat16 if bf16 else torch.float32)
    flat = np.ascontiguousarray(blocks)
    assert L.jib_dequantize(t, flat.ctypes.data, n, out.data_ptr(), int(bf16), threads) == 0
    return out


@pytest.mark.parametrize("t", TYPES, ids=[Q.NAMES[t] for t in TYPES])
def test_numpy_and_native_expanders_agree_on_random_blocks(t):
    """Two implementations written differently (array reshapes here, per-element index arithmetic in C++) read every bit
    pattern alike -- every code, every scale nibble and every high-bit plane is exercised by random bytes."""
    blocks = random_blocks(t, 257, seed=t)
    ref = Q.DEQUANT[t](blocks).reshape(-1)
    assert np.isfinite(ref).all()
    got = native(t, blocks).numpy()
    np.testing.assert_allclose(got, ref, rtol=1e-6, atol=1e-7)
    many = native(t, blocks, threads=5).numpy()                    # block ranges over threads, uneven split
    np.testing.assert_array_equal(many, got)
    bf = native(t, blocks, bf16=True)
    assert torch.equal(bf, torch.from_numpy(got).to(torch.bfloat16))            # same rounding as the framework's cast


def test_native_expander_rejects_what_it_cannot_do():
    from jittorinfer_b200.runtime.native_rt import lib
    L = lib()
    L.jib_dequantize.restype = C.c_int
    L.jib_dequantize.argtypes = [C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p, C.c_int, C.c_int]
    buf = (C.c_uint8 * 512)()
    out = (C.c_float * 512)()
    assert L.jib_dequantize(16, buf, 256, out, 0, 1) == -1         # IQ2_XXS: a codebook type
    assert L.jib_dequantize(Q.Q4_K, buf, 100, out, 0, 1) == -2     # not a whole block
    assert L.jib_dequantize(Q.Q4_K, None, 256, out, 0, 1) == -3
    assert L.jib_dequantize(Q.Q4_K, buf, 0, out, 0, 1) == 0
    L.jib_quant_block_bytes.restype = C.c_uint64
    for t, (blk, bsz) in Q.TRAITS.items():
        assert L.jib_quant_block_bytes(C.c_uint32(t)) == bsz and F.TYPE_TRAITS[t] == (blk, bsz)


def test_half_subnormals_and_specials_convert_like_numpy():
    halves = np.array([0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x3C00, 0xBC00, 0x7BFF, 0x0200, 0x8001], dtype=np.uint16)
    blocks = np.zeros((halves.size, 34), dtype=np.uint8)
    blocks[:, 0:2] = halves.view(np.uint8).reshape(-1, 2)
    blocks[:, 2] = 1                                               # first code 1: the element is the scale itself
    got = native(Q.Q8_0, blocks).numpy().reshape(-1, 32)[:, 0]
    np.testing.assert_array_equal(got, halves.view(np.float16).astype(np.float32))


# relative rms error a round-to-nearest encoder reaches on unit normal data (generous: an encoder that packs a field into
# the wrong bits is off by ~1)
RMS_BOUND = {Q.Q4_0: 0.12, Q.Q4_1: 0.11, Q.Q5_0: 0.06, Q.Q5_1: 0.055, Q.Q8_0: 0.008, Q.Q2_K: 0.45, Q.Q3_K: 0.22, Q.Q4_K: 0.11,
             Q.Q5_K: 0.055, Q.Q6_K: 0.03, Q.Q8_K: 0.01}


@pytest.mark.parametrize("t", TYPES, ids=[Q.NAMES[t] for t in TYPES])
def test_quantise_expand_round_trip(t):
    rng = np.random.default_rng(100 + t)
    x = rng.standard_normal(256 * 40).astype(np.float32)
    x[:256] = 0.0                                                  # an all-zero block must not divide by zero
    x[256:512] = np.abs(x[256:512])                                # one-sided data: the offset types clamp their minimum at 0
    raw = Q.quantize(t, x)
    assert raw.size == x.size // Q.TRAITS[t][0] * Q.TRAITS[t][1]
    y = Q.dequantize(t, raw, x.size)
    assert np.isfinite(y).all() and (y[:256] == 0).all()
    rms = float(np.sqrt(((y - x) ** 2).mean()))
    assert rms < RMS_BOUND[t], (Q.NAMES[t], rms)
    again = Q.dequantize(t, Q.quantize(t, y), x.size)              # codes of expanded values are (nearly) a fixed point
    assert float(np.sqrt(((again - y) ** 2).mean())) < 0.6 * RMS_BOUND[t]


def test_legacy_helpers_match_the_table_driven_ones():
    x = np.random.default_rng(0).standard_normal(32 * 50).astype(np.float32)
    for t, qf, df in ((Q.Q8_0, F.quantize_q8_0, F.dequantize_q8_0), (Q.Q4_0, F.quantize_q4_0, F.dequantize_q4_0)):
        raw = qf(x)
        np.testing.assert_array_equal(raw, Q.quantize(t, x))
        np.testing.assert_array_equal(df(raw, x.size), Q.dequantize(t, raw, x.size))


@pytest.mark.parametrize("native_reader", [False, True], ids=["python", "native"])
def test_shards_of_quantised_tensors(tmp_path, native_reader):
    """Cuts along an outer dimension, along the row dimension on a block boundary and off it (the last falls back to
    expanding the whole tensor) all equal the slice of the whole expanded tensor; the 3-D expert layout included."""
    rng = np.random.default_rng(3)
    p = str(tmp_path / "q.gguf")
    w = GGUFWriter(p)
    mats = {}
    for t in TYPES:
        a = rng.standard_normal((4, 6, 512)).astype(np.float32)
        mats[Q.NAMES[t]] = a
        w.add_tensor(Q.NAMES[t], a, t)
    with pytest.raises(ValueError):
        w.add_tensor("bad", rng.standard_normal((4, 100)).astype(np.float32), Q.Q4_K)
    w.write()
    if native_reader:
        from jittorinfer_b200.gguf.native_reader import NativeGGUFReader as Reader
    else:
        Reader = GGUFReader
    rd = Reader(p)
    for t in TYPES:
        name = Q.NAMES[t]
        whole = rd.tensor(name)
        assert whole.shape == (4, 6, 512) and whole.dtype == torch.float32
        ref = torch.from_numpy(Q.dequantize(t, Q.quantize(t, mats[name]), mats[name].size)).view(4, 6, 512)
        assert torch.equal(whole, ref)
        for dim, count in ((0, 2), (0, 4), (1, 3), (2, 2), (-1, 2), (2, 16), (2, 32)):
            for index in (0, count - 1):
                got = rd.tensor_slice(name, dim, index, count)
                step = whole.shape[dim] // count
                assert torch.equal(got, whole.narrow(dim, index * step, step)), (name, dim, count, index)
        with pytest.raises(ValueError):
            rd.tensor_slice(name, 1, 0, 4)                         # 6 rows do not split four ways
    rd.quant_out_dtype = torch.bfloat16
    assert torch.equal(rd.tensor("Q6_K"), ref_bf16(rd, "Q6_K"))
    rd.close()


def ref_bf16(rd, name):
    keep, rd.quant_out_dtype = rd.quant_out_dtype, None
    try:
        return rd.tensor(name).to(torch.bfloat16)
    finally:
        rd.quant_out_dtype = keep


@pytest.mark.parametrize("quant", [Q.Q4_K, Q.Q6_K, Q.Q5_0], ids=["Q4_K", "Q6_K", "Q5_0"])
def test_model_from_quantised_file_equals_model_from_its_expanded_weights(tmp_path, quant):
    """A quantised checkpoint generates exactly what an fp32 checkpoint holding the expanded weights generates, and the
    tensor-parallel shards of the quantised file are the shards of the expanded one."""
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.models.weights import ShardSpec, iter_gguf, write_random_gguf
    from jittorinfer_b200.runtime.factory import build_engine
    from jittorinfer_b200.runtime.sampling import SamplingParams
    hp = preset("tiny")
    pq, pf = str(tmp_path / "q.gguf"), str(tmp_path / "f.gguf")
    write_random_gguf(pq, hp, seed=5, std=0.05, quant=quant)
    rq = GGUFReader(pq)
    kinds = {ti.ggml_type for ti in rq.tensors.values()}
    assert quant in kinds and F.GGML_F32 in kinds                  # matrices quantised, norms and router not
    if quant in (Q.Q4_K, Q.Q6_K):
        assert F.GGML_Q8_0 in kinds                                # rows of 128 fall back
    w = GGUFWriter(pf)
    for k, v in rq.kv.items():
        w.add(k, v)
    for name in rq.tensors:
        w.add_tensor(name, rq.tensor(name).to(torch.float32))
    w.write()
    rf = GGUFReader(pf)
    for rank in range(2):
        spec = ShardSpec(rank, 2, True)
        a = dict(iter_gguf(rq, hp, spec))
        b = dict(iter_gguf(rf, hp, spec))
        assert a.keys() == b.keys()
        for name in a:
            assert torch.equal(a[name].to(torch.float32), b[name].to(torch.float32)), name
    rq.close()
    rf.close()
    prompt = [[3, 9, 27, 81, 243, 5]]
    outs = []
    for path in (pq, pf):
        eng = build_engine(None, gguf_path=path, device="cpu", dtype=torch.float32, n_parallel=2, n_ctx_slot=64, cuda_graphs=False)
        outs.append(eng.generate(prompt, SamplingParams(ignore_eos=True), max_new_tokens=8))
    assert outs[0] == outs[1]


def test_requantise_keeps_keys_and_re_encodes_tensors(tmp_path):
    from jittorinfer_b200.gguf.requant import main, requantize
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.models.weights import write_random_gguf
    src, q, back = str(tmp_path / "a.gguf"), str(tmp_path / "q.gguf"), str(tmp_path / "b.gguf")
    write_random_gguf(src, preset("tiny"), seed=1, std=0.05)
    names = []
    n = requantize(src, q, "q5_k", progress=names.append)
    with GGUFReader(src) as a, GGUFReader(q) as b:
        assert list(a.kv) == list(b.kv) and a.kv_types == b.kv_types and a.kv_elem_types == b.kv_elem_types
        for k in a.kv:
            va, vb = a.kv[k], b.kv[k]
            assert (list(va) == list(vb)) if isinstance(va, (list, np.ndarray)) else (va == vb), k
        assert list(a.tensors) == list(b.tensors) == names
        kinds = {ti.ggml_type for ti in b.tensors.values()}
        assert kinds == {F.GGML_F32, F.GGML_Q5_K, F.GGML_Q8_0} and 0 < n < len(names)
        for name, ti in a.tensors.items():
            x, y = a.tensor(name), b.tensor(name)
            if b.tensors[name].ggml_type == F.GGML_F32:
                assert torch.equal(x, y)                              # norms and the router: byte for byte
            else:
                assert (x - y).abs().max().item() < 0.05 * x.abs().max().item() + 1e-6
    assert main([q, back, "--type", "bf16", "-q"]) == 0               # expanded once: a plain view of the file from then on
    with GGUFReader(q) as b, GGUFReader(back) as c:
        for name in b.tensors:
            if c.tensors[name].ggml_type == F.GGML_BF16:
                assert torch.equal(c.tensor(name), b.tensor(name).to(torch.bfloat16)), name
    with pytest.raises(ValueError):
        requantize(src, q + "x", "q8_k")


@pytest.mark.parametrize("t", TYPES, ids=[Q.NAMES[t] for t in TYPES])
def test_layout_function_shared_with_device_code_equals_the_block_expanders(t):
    """``jib_quant_elem`` (csrc/include/jib_quant_layout.h) is what the device kernel evaluates per element; on the host it
    gives exactly what the per-block expanders give, for every element of random blocks."""
    from jittorinfer_b200.runtime.native_rt import lib
    L = lib()
    L.jib_dequantize_elementwise.restype = C.c_int
    L.jib_dequantize_elementwise.argtypes = [C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p]
    blocks = random_blocks(t, 97, seed=50 + t)
    n = blocks.shape[0] * Q.TRAITS[t][0]
    out = np.empty(n, dtype=np.float32)
    assert L.jib_dequantize_elementwise(t, blocks.ctypes.data, n, out.ctypes.data) == 0
    np.testing.assert_array_equal(out, native(t, blocks).numpy())
    assert L.jib_dequantize_elementwise(16, blocks.ctypes.data, n, out.ctypes.data) == -1
