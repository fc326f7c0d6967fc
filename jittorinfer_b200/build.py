"""In-tree native builds: host runtime (g++) and sm_100a CUDA kernels (nvcc).

The reference builds with CMake against CANN (CMakeLists.txt, ggml/src/ggml-cann/CMakeLists.txt);
here two shared libraries are produced next to the Python package so that they travel with a
source snapshot and are loaded with ctypes:

* ``lib/libjib200_runtime.so`` — paged-KV allocator, scheduler, GGUF, tokenizer, samplers, llama.h C API
* ``lib/libjib200_kernels.so`` — every CUDA kernel, compiled for ``sm_100a`` only

``python -m jittorinfer_b200.build`` builds both; each library is rebuilt only when a source is
newer than the output.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
import sysconfig
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
RUNTIME_SO = os.path.join(LIBDIR, "libjib200_runtime.so")
KERNELS_SO = os.path.join(LIBDIR, "libjib200_kernels.so")
LLAMA_SO = os.path.join(LIBDIR, "libllama.so")

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _newer(srcs: List[str], out: str) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in srcs)


def _run(cmd: List[str], verbose: bool):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError(f"build failed: {' '.join(cmd[:3])} ...")
    if verbose and r.stdout.strip():
        print(r.stdout)
    return r.stdout


def nvcc_path() -> str:
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found")
    return p


def build_runtime(force: bool = False, verbose: bool = False, sanitize: str = "") -> str:
    """``sanitize``: e.g. "address,undefined" or "thread" builds a separate instrumented library
    (libjib200_runtime_<san>.so) for running the host-side tests under the sanitizers; load it by pointing
    JITTORINFER_RUNTIME_SO at it and preloading the sanitizer runtime (``gcc -print-file-name=libasan.so``)."""
    srcs = sorted(glob.glob(os.path.join(CSRC, "runtime", "*.cpp")))
    deps = srcs + glob.glob(os.path.join(CSRC, "runtime", "*.h")) + glob.glob(os.path.join(CSRC, "include", "*.h"))
    os.makedirs(LIBDIR, exist_ok=True)
    if sanitize:
        tag = sanitize.replace(",", "_")
        out = os.path.join(LIBDIR, f"libjib200_runtime_{tag}.so")
        if force or _newer(deps, out):
            _run(["g++", "-std=c++17", "-O1", "-g", "-fPIC", "-fno-omit-frame-pointer", f"-fsanitize={sanitize}", "-fvisibility=hidden",
                  "-I", os.path.join(CSRC, "include"), "-I", os.path.join(CSRC, "runtime"), "-shared", "-o", out] + srcs +
                 ["-lpthread", "-ldl"], verbose)
        return out
    if force or _newer(deps, RUNTIME_SO):
        objs = []
        objdir = os.path.join(LIBDIR, "obj")
        os.makedirs(objdir, exist_ok=True)
        procs = []
        for s in srcs:
            o = os.path.join(objdir, os.path.basename(s) + ".o")
            objs.append(o)
            if force or _newer([s] + [d for d in deps if d.endswith(".h")], o):
                cmd = ["g++", "-std=c++17", "-O2", "-g", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function",
                       "-I", os.path.join(CSRC, "include"), "-I", os.path.join(CSRC, "runtime"), "-c", s, "-o", o]
                if verbose:
                    print(" ".join(cmd), flush=True)
                procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        for cmd, p in procs:
            out, _ = p.communicate()
            if p.returncode != 0:
                sys.stderr.write(out)
                raise RuntimeError(f"build failed: {cmd[-3]}")
        _run(["g++", "-shared", "-o", RUNTIME_SO] + objs + ["-lpthread", "-ldl"], verbose)
    return RUNTIME_SO


def python_embed_flags() -> tuple:
    """(include flags, link flags) for embedding the interpreter this module runs under."""
    import sysconfig
    inc = ["-I", sysconfig.get_paths()["include"]]
    libdir = sysconfig.get_config_var("LIBDIR") or ""
    ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    link = ([f"-L{libdir}", f"-Wl,-rpath,{libdir}"] if libdir else []) + [f"-lpython{ver}"]
    return inc, link


def build_capi(force: bool = False, verbose: bool = False) -> str:
    """libllama.so: the llama.h C API (native GGUF / tokenizer / samplers / KV bookkeeping + the embedded-Python bridge)."""
    rt = [os.path.join(CSRC, "runtime", f) for f in ("gguf.cpp", "kv_paged.cpp", "tokenizer.cpp")]
    srcs = sorted(glob.glob(os.path.join(CSRC, "capi", "*.cpp"))) + rt
    deps = srcs + glob.glob(os.path.join(CSRC, "capi", "*.h")) + glob.glob(os.path.join(CSRC, "runtime", "*.h")) + \
        glob.glob(os.path.join(CSRC, "runtime", "*.inc")) + glob.glob(os.path.join(CSRC, "include", "*.h"))
    os.makedirs(LIBDIR, exist_ok=True)
    if force or _newer(deps, LLAMA_SO):
        inc, link = python_embed_flags()
        objdir = os.path.join(LIBDIR, "obj_capi")
        os.makedirs(objdir, exist_ok=True)
        objs, procs = [], []
        for s in srcs:
            o = os.path.join(objdir, os.path.basename(s) + ".o")
            objs.append(o)
            cmd = ["g++", "-std=c++17", "-O2", "-g", "-fPIC", "-fvisibility=hidden", "-DLLAMA_BUILD", "-Wall", "-Wno-unused-function",
                   "-I", os.path.join(CSRC, "include"), "-I", os.path.join(CSRC, "runtime"), *inc, "-c", s, "-o", o]
            if verbose:
                print(" ".join(cmd), flush=True)
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        for cmd, p in procs:
            out, _ = p.communicate()
            if p.returncode != 0:
                sys.stderr.write(out)
                raise RuntimeError(f"build failed: {cmd[-3]}")
        _run(["g++", "-shared", "-o", LLAMA_SO] + objs + link + ["-lpthread", "-ldl"], verbose)
    return LLAMA_SO


def _build_kernels_variant(define: str, suffix: str, force: bool, verbose: bool) -> str:
    srcs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "kernels", "*.cuh")) + glob.glob(os.path.join(CSRC, "kernels", "*.h")) + \
        [os.path.join(CSRC, "include", "jib_quant_layout.h")]
    out = os.path.join(LIBDIR, f"libjib200_kernels_{suffix}.so")
    if force or _newer(srcs + hdrs, out):
        objdir = os.path.join(LIBDIR, "obj_" + suffix)
        os.makedirs(objdir, exist_ok=True)
        nvcc = nvcc_path()
        objs, procs = [], []
        for s in srcs:
            o = os.path.join(objdir, os.path.basename(s) + ".o")
            objs.append(o)
            cmd = [nvcc, "-std=c++17", "-O3", "-lineinfo", *NVCC_ARCH, "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
                   *["-D" + d for d in define.split(",")], "-I", os.path.join(CSRC, "kernels"), "-I", os.path.join(CSRC, "include"), "-c", s, "-o", o]
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        for cmd, p in procs:
            o, _ = p.communicate()
            if p.returncode != 0:
                sys.stderr.write(o)
                raise RuntimeError(f"build failed: {cmd[-3]}")
        _run([nvcc, "-shared", *NVCC_ARCH, "-o", out] + objs, verbose)
    return out


def build_kernels_bounds_check(force: bool = False, verbose: bool = False) -> str:
    """The kernels with -DJIB_BOUNDS_CHECK (see csrc/kernels/bounds_check.cuh) as libjib200_kernels_bc.so; select it with
    JITTORINFER_KERNELS_SO=<path>."""
    return _build_kernels_variant("JIB_BOUNDS_CHECK", "bc", force, verbose)


def build_kernels_timeline(force: bool = False, verbose: bool = False) -> str:
    """The kernels with -DJIB_TIMELINE (device time stamps of the collective phases, csrc/kernels/timeline.cuh) as
    libjib200_kernels_tl.so; select it with JITTORINFER_KERNELS_SO=<path> and read the stamps with parallel/timeline.py."""
    return _build_kernels_variant("JIB_TIMELINE", "tl", force, verbose)


def build_kernels_pdl_late(force: bool = False, verbose: bool = False, timeline: bool = False) -> str:
    """The kernels with -DJIB_PDL_LATE (csrc/kernels/pdl.cuh: dependents are released once a kernel's loads are in flight instead
    of first thing) as libjib200_kernels_late.so, for A/B measurements; ``timeline=True`` adds the time stamps (…_late_tl.so)."""
    return _build_kernels_variant("JIB_PDL_LATE,JIB_TIMELINE" if timeline else "JIB_PDL_LATE", "late_tl" if timeline else "late", force, verbose)


def build_kernels_poll(force: bool = False, verbose: bool = False) -> str:
    """The kernels with -DJIB_SUSPEND_NS=0 (csrc/kernels/sm100.cuh: mbarrier waits poll with test_wait and never suspend the
    thread) as libjib200_kernels_poll.so, to compare the wake-up latency of a suspended wait against polling."""
    return _build_kernels_variant("JIB_SUSPEND_NS=0", "poll", force, verbose)


def build_kernels(force: bool = False, verbose: bool = False, extra_flags: List[str] = ()) -> str:
    srcs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "kernels", "*.cuh")) + glob.glob(os.path.join(CSRC, "kernels", "*.h")) + \
        [os.path.join(CSRC, "include", "jib_quant_layout.h")]
    os.makedirs(LIBDIR, exist_ok=True)
    if not srcs:
        raise RuntimeError("no CUDA sources found")
    if force or _newer(srcs + hdrs, KERNELS_SO):
        nvcc = nvcc_path()
        objdir = os.path.join(LIBDIR, "obj")
        os.makedirs(objdir, exist_ok=True)
        objs, procs = [], []
        for s in srcs:
            o = os.path.join(objdir, os.path.basename(s) + ".o")
            objs.append(o)
            if force or _newer([s] + hdrs, o):
                cmd = [nvcc, "-std=c++17", "-O3", "-lineinfo", *NVCC_ARCH, "-Xcompiler", "-fPIC,-fvisibility=hidden",
                       "--expt-relaxed-constexpr", "-Xptxas", "-v", *extra_flags,
                       "-I", os.path.join(CSRC, "kernels"), "-I", os.path.join(CSRC, "include"), "-c", s, "-o", o]
                if verbose:
                    print(" ".join(cmd), flush=True)
                procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        log = []
        for s, p in procs:
            out, _ = p.communicate()
            log.append(f"==== {os.path.basename(s)}\n{out}")
            if p.returncode != 0:
                sys.stderr.write(out)
                raise RuntimeError(f"nvcc failed on {s}")
        if log:
            with open(os.path.join(LIBDIR, "ptxas.log"), "w") as f:
                f.write("\n".join(log))
        _run([nvcc, "-shared", *NVCC_ARCH, "-o", KERNELS_SO] + objs, verbose)
    return KERNELS_SO


def build_all(force: bool = False, verbose: bool = False):
    return build_runtime(force, verbose), build_kernels(force, verbose), build_capi(force, verbose)


if __name__ == "__main__":
    f = "--force" in sys.argv
    v = "-v" in sys.argv or "--verbose" in sys.argv
    for p in build_all(f, v):
        print("built", p)
