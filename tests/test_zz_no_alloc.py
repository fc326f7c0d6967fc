"""The allocation-free split-K GEMM entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they need a GEMM: the engine has
already given almost all of HBM to the KV cache, or the embedding program forbids allocations on
its latency-critical thread.  ``jib_gemm_bf16_noalloc`` serves them from a scratch array built into
the library.  This test calls it twice in a row (the second call finds the array as the first left
it) and checks both results against the regular entry point, which gets its scratch from the
caller.  The file sorts last so that a run that stops at the first failure has already run every
other test; it also passes when run alone in a fresh process.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

JIB_E_NOALLOC_TOO_LARGE = -7


def _lib():
    from jittorinfer_b200 import build
    from jittorinfer_b200.ops import native
    native.load()                                   # builds the library if needed
    L = C.CDLL(build.KERNELS_SO)
    L.jib_gemm_bf16_noalloc.restype = C.c_int
    L.jib_gemm_bf16_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    L.jib_gemm_bf16_noalloc_need.restype = C.c_size_t
    L.jib_gemm_bf16_noalloc_need.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int]
    L.jib_gemm_bf16_noalloc_status.restype = C.c_int
    L.jib_gemm_bf16_noalloc_status.argtypes = [C.c_void_p, C.c_void_p]
    return L, native


def _rand(shape, scale, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).bfloat16().cuda()


@pytest.mark.parametrize("T,N,K,splits", [(1, 2048, 2048, 8), (8, 3648, 2048, 4), (40, 384, 1408, 2), (8, 512, 2048, 0), (5, 640, 512, 1),
                                          (64, 1024, 2048, 4), (200, 512, 1400, 3), (200, 640, 2048, 0)])
def test_noalloc_matches_regular_entry_point_twice(T, N, K, splits):
    L, native = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                            # second call reuses the array the first one dirtied
        x, w = _rand((T, K), 1.0, 10 * call + 1), _rand((N, K), 0.05, 10 * call + 2)
        out = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
        rc = L.jib_gemm_bf16_noalloc(x.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, splits, stream)
        assert rc == 0, f"jib_gemm_bf16_noalloc returned {rc}"
        ref = native.gemm(x, w, splits=splits)       # regular entry point, caller-provided scratch
        torch.cuda.synchronize()
        exact = x.float() @ w.float().T
        mag = exact.abs().max().item() + 1e-6
        assert (out.float() - ref.float()).abs().max().item() <= 2e-2 * mag
        assert (out.float() - exact).abs().max().item() <= 2e-2 * mag
        # faults the kernel itself found (a wait that ran out, an index out of range) are only visible here
        status = torch.zeros(4, dtype=torch.int32).pin_memory()
        assert L.jib_gemm_bf16_noalloc_status(status.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert status.tolist() == [0, 0, 0, 0]
    native.check_status()


def test_noalloc_rejects_sizes_beyond_its_array():
    L, _ = _lib()
    x, w = _rand((8, 4096), 1.0, 1), _rand((256, 4096), 0.05, 2)
    out = torch.empty(8, 256, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # 256 token columns x 8192 tiles worth of partials cannot fit: ask for it through the size helper first
    assert L.jib_gemm_bf16_noalloc_need(256, 128 * 400, 4096, 16) > (8 << 20)
    big_w = C.c_void_p(w.data_ptr())                 # never dereferenced: the call must be refused before any launch
    rc = L.jib_gemm_bf16_noalloc(x.data_ptr(), big_w, out.data_ptr(), 256, 128 * 400, 4096, 16, stream)
    assert rc == JIB_E_NOALLOC_TOO_LARGE
    torch.cuda.synchronize()
