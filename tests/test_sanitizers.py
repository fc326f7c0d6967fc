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
                        "tests/test_tokenizer.py", "tests/test_quants.py"], cwd=ROOT, env=env, capture_output=True, text=True, timeout=800)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert "ERROR: AddressSanitizer" not in tail and "runtime error:" not in tail


GRAMMAR_HARNESS = r"""
#include "grammar.h"
#include <cstdio>
#include <fstream>
#include <sstream>
// argv[1]: file with a GBNF grammar, argv[2]: file with a text.  Prints "parse-error", "accept" or "reject".
int main(int argc, char ** argv) {
    if (argc < 3) return 2;
    std::stringstream g, t;
    g << std::ifstream(argv[1]).rdbuf();
    t << std::ifstream(argv[2]).rdbuf();
    jib::Grammar grammar;
    if (!grammar.parse(g.str(), "root").empty()) { puts("parse-error"); return 0; }
    jib::GrammarMatcher m(&grammar);
    std::vector<uint32_t> cps;
    jib::Utf8Tail tail;
    jib::utf8_decode(t.str(), cps, tail);
    for (uint32_t cp : cps)
        if (!m.accept(cp)) { puts("reject"); return 0; }
    puts(m.complete() ? "accept" : "reject");
    return 0;
}
"""


@pytest.mark.timeout(900)
def test_grammar_engine_under_asan_with_hostile_input(tmp_path):
    """Grammar text arrives in requests: the parser and matcher run under ASan + UBSan over valid grammars, truncated
    and mutated ones and random bytes; they must answer (accept / reject / parse-error) and never trip a sanitizer."""
    import random
    from jittorinfer_b200.server.json_schema import grammar_accepts, json_schema_to_grammar
    if _san_runtime("libasan.so") is None:
        pytest.skip("no libasan in this toolchain")
    src = tmp_path / "harness.cpp"
    src.write_text(GRAMMAR_HARNESS)
    exe = str(tmp_path / "harness")
    capi_dir = os.path.join(build.CSRC, "capi")
    subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-I", capi_dir,
                    str(src), os.path.join(capi_dir, "grammar.cpp"), "-o", exe], check=True)
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=1", UBSAN_OPTIONS="halt_on_error=1")

    def run(grammar: bytes, text: bytes) -> str:
        (tmp_path / "g.txt").write_bytes(grammar)
        (tmp_path / "t.txt").write_bytes(text)
        r = subprocess.run([exe, str(tmp_path / "g.txt"), str(tmp_path / "t.txt")], capture_output=True, text=True, env=env, timeout=60)
        assert r.returncode == 0, r.stderr[-2000:]
        return r.stdout.strip()

    schema = {"type": "object", "properties": {"name": {"type": "string", "maxLength": 8}, "tags": {"type": "array", "items": {"enum": ["a", "b"]}},
                                               "n": {"type": "number"}}, "required": ["name"]}
    g = json_schema_to_grammar(schema)
    docs = ['{"name": "x"}', '{"name":"é✓","tags":["a","b"],"n":-1.5e3}', '{"tags": []}', '{"name": "toolongname"}', '[1]', '']
    for d in docs:                                        # the C++ matcher agrees with the Python one
        assert run(g.encode(), d.encode()) == ("accept" if grammar_accepts(g, d) else "reject"), d
    rng = random.Random(0)
    raw = g.encode()
    for _ in range(40):                                   # truncations, byte flips, random bytes
        kind = rng.randrange(3)
        if kind == 0:
            bad = raw[: rng.randrange(len(raw))]
        elif kind == 1:
            b = bytearray(raw)
            for _ in range(rng.randrange(1, 6)):
                b[rng.randrange(len(b))] = rng.randrange(256)
            bad = bytes(b)
        else:
            bad = bytes(rng.randrange(256) for _ in range(rng.randrange(1, 200)))
        assert run(bad, b'{"name": "x"}') in ("accept", "reject", "parse-error")
    assert run(b'root ::= root "a" | "a"', b"aaa") in ("accept", "reject")       # left recursion: bounded, no crash
    assert run(b'root ::= ("a" | "b"){2,3} [^x-z]* "\\u00e9"', "abqé".encode()) == "accept"


GGUF_HARNESS = r"""
#include "gguf.h"
#include <cstdio>
// argv[1]: a file that claims to be GGUF.  Opens it, walks the metadata and the tensor table, touches the first and last
// byte of every tensor.  Prints "ok <n_kv> <n_tensors>" or "error: ...".
int main(int argc, char ** argv) {
    if (argc < 2) return 2;
    jib::GgufFile f;
    const std::string err = f.open(argv[1], false);
    if (!err.empty()) { printf("error: %s\n", err.c_str()); return 0; }
    unsigned long long sum = 0;
    for (const auto & kv : f.kv()) {
        sum += kv.first.size() + (unsigned long long) kv.second.as_i64() + kv.second.s.size() + kv.second.arr_s.size();
        if (kv.second.type == jib::GT_ARR && kv.second.arr_type != jib::GT_STR && kv.second.arr_n > 0) sum += kv.second.arr_data[0];
    }
    for (const auto & t : f.tensors()) {
        const uint8_t * p = f.tensor_data(t);
        if (t.nbytes > 0) sum += p[0] + p[t.nbytes - 1];
    }
    printf("ok %zu %zu %llu\n", f.kv().size(), f.tensors().size(), sum & 1);
    return 0;
}
"""


@pytest.mark.timeout(900)
def test_gguf_reader_under_asan_with_hostile_files(tmp_path):
    """Checkpoints come from outside: the C++ GGUF reader runs under ASan + UBSan over a valid file, truncations of it and
    copies with mutated header bytes (counts, lengths, types, offsets); every case must end in "ok" or an error string."""
    import random

    import torch
    from jittorinfer_b200.models.hparams import preset
    from jittorinfer_b200.models.weights import write_random_gguf
    if _san_runtime("libasan.so") is None:
        pytest.skip("no libasan in this toolchain")
    rt_dir = os.path.join(build.CSRC, "runtime")
    src = tmp_path / "gguf_harness.cpp"
    src.write_text(GGUF_HARNESS)
    exe = str(tmp_path / "gguf_harness")
    subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-I", rt_dir, str(src),
                    os.path.join(rt_dir, "gguf.cpp"), "-o", exe], check=True)
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=1", UBSAN_OPTIONS="halt_on_error=1")
    good = tmp_path / "good.gguf"
    write_random_gguf(str(good), preset("tiny"), dtype=torch.float16)
    raw = good.read_bytes()

    def run(data: bytes) -> str:
        f = tmp_path / "case.gguf"
        f.write_bytes(data)
        r = subprocess.run([exe, str(f)], capture_output=True, text=True, env=env, timeout=120)
        assert r.returncode == 0, r.stderr[-2000:]
        return r.stdout.strip()

    assert run(raw).startswith("ok ")
    rng = random.Random(1)
    header = min(len(raw), 1 << 15)                       # metadata and tensor table live here
    seen_error = 0
    for i in range(60):
        kind = i % 3
        if kind == 0:
            bad = raw[: rng.randrange(header)]
        elif kind == 1:
            b = bytearray(raw)
            for _ in range(rng.randrange(1, 4)):
                b[rng.randrange(4, header)] = rng.randrange(256)
            bad = bytes(b)
        else:                                             # a 64-bit field blown up: counts, string lengths, dims, offsets
            b = bytearray(raw)
            at = rng.randrange(8, header - 8) & ~3
            b[at:at + 8] = rng.choice([b"\xff" * 8, (1 << 60).to_bytes(8, "little"), (1 << 33).to_bytes(8, "little")])
            bad = bytes(b)
        out = run(bad)
        assert out.startswith("ok ") or out.startswith("error: "), out
        seen_error += out.startswith("error: ")
    assert seen_error > 10

    # directed cases: the fields whose blow-up used to matter
    def patched(at: int, value: int) -> bytes:
        b = bytearray(raw)
        b[at:at + 8] = value.to_bytes(8, "little")
        return bytes(b)

    assert run(patched(8, 1 << 60)).startswith("error: ")                   # tensor count
    assert run(patched(16, 1 << 60)).startswith("error: ")                  # metadata count
    name = b"token_embd.weight"
    at = raw.rfind(name) + len(name)                                         # the tensor table entry: n_dims, dims, type, offset
    assert at > len(name) and int.from_bytes(raw[at:at + 4], "little") == 2
    both = bytearray(raw)
    both[at + 4:at + 12] = (1 << 40).to_bytes(8, "little")
    both[at + 12:at + 20] = (1 << 40).to_bytes(8, "little")
    assert run(bytes(both)).startswith("error: ")                           # element count that wraps 64 bits
    assert run(patched(at + 24, (1 << 64) - 32)).startswith("error: ")      # data offset that wraps the bounds check
    assert run(patched(at + 24, 1 << 50)).startswith("error: ")             # data offset past the end
