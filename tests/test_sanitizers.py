"""The host runtime (KV allocator, scheduler, tokenizer, GGUF reader) under AddressSanitizer + UBSan.

The reference declares sanitizer options in CMake but never wires them (CMakeLists.txt:59-61, 101).  Here the runtime is
rebuilt with -fsanitize=address,undefined and its unit tests run again in a child process against that library; any
report makes the child fail.  Device code has no such tool on this class of machine, which is why kernels carry their own
bounds checks and status words.
"""
import os
import subprocess
import sys

import pytest

from jittorinfer_b200 import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _san_runtime(name):
    r = subprocess.run(["gcc", f"-print-file-name={name}"], capture_output=True, text=True)
    p = r.stdout.strip()
    return p if os.path.isabs(p) and os.path.exists(p) else None


@pytest.mark.timeout(900)
def test_runtime_tests_pass_under_asan_ubsan():
    asan = _san_runtime("libasan.so")
    if asan is None:
        pytest.skip("no libasan in this toolchain")
    so = build.build_runtime(sanitize="address,undefined")
    env = dict(os.environ, JITTORINFER_RUNTIME_SO=so, LD_PRELOAD=asan,
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=1:halt_on_error=1", UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider", "tests/test_runtime_native.py",
                        "tests/test_tokenizer.py"], cwd=ROOT, env=env, capture_output=True, text=True, timeout=800)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert "ERROR: AddressSanitizer" not in tail and "runtime error:" not in tail
