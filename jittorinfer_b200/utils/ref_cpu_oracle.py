"""A second oracle: the reference's OWN CPU code run on a GGUF file this package wrote.

The reference's only device back end is an NPU one, but its model loader, graph builder and ggml CPU kernels are plain
C/C++.  This tool builds them outside the product tree from a checkout of the reference (no MPI, no device back end),
loads a GGUF written by ``models/weights.py:write_random_gguf`` with the reference's loader (which asserts the tensor
count and names, src/llama-model-loader.cpp:871-876), decodes a token sequence through ``llama_decode`` on the CPU and
compares the logits of every position with ``models/oracle.py``.

    python -m jittorinfer_b200.utils.ref_cpu_oracle --reference <checkout> --workdir <scratch dir> [--cases v2,lite] [--save logits.npz]

(``tests/data/reference_cpu_logits.npz`` was written by this command; ``tests/test_reference_cpu_oracle.py`` compares against it.)

What has to be stood in for, and how (nothing of the checkout is modified; a COPY under the work directory is):

* ``ggml-cann.h`` / ``ggml_backend_cann_presample`` (src/llama-execute-decode.cpp:4,148): a header and an aborting
  definition; raw logits are requested (``presample_count = -1``), so it is never called.
* MPI: the guard macro stays undefined; two calls outside the guard (src/llama-context-load-utils.cpp:377,
  src/llama-context.cpp:545) get single-process inline stand-ins.
* Three graph nodes without a CPU kernel: ``GGML_OP_GET_SLICE`` (top-k of the router's argsort, src/llama-graph-ffn.cpp:175),
  ``GGML_OP_RMS_NORM_FUSED``, and ``MUL`` of an f32 activation with an f16 norm weight (src/llama-graph-utils.cpp:93-95 casts
  every norm weight to half precision for the device).  Each gets a plain loop in the copied ``ggml-cpu.c``.

The other direction is checked too: ``ref_rewrite`` passes the file through the reference's GGUF reader and writer, and the
result is byte-identical to what this package wrote (same key order, tensor order, alignment and padding).

Known difference that the comparison has to avoid: the reference ranks ALL experts and ignores ``n_group`` / ``topk_group``
(src/llama-graph-ffn.cpp:173-176), so a configuration with group-limited routing is compared with ``n_group = 1``.
The f16 cache and f16 norm weights of the reference bound the agreement at a few 1e-3 of the largest logit.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import shutil
import subprocess
import sys
from typing import List

import numpy as np

STUB_CANN_H = r'''#pragma once
#include "ggml.h"
#include "ggml-backend.h"
#ifdef __cplusplus
extern "C" {
#endif
void ggml_backend_cann_presample(ggml_backend_t backend, const struct ggml_tensor * logits, struct ggml_tensor * values,
                                 struct ggml_tensor * indices, int64_t k);
#ifdef __cplusplus
}
#endif
'''

STUB_CPP = r'''#include <cstdio>
#include <cstdlib>
#include "ggml-cann.h"
extern "C" void ggml_backend_cann_presample(ggml_backend_t, const struct ggml_tensor *, struct ggml_tensor *, struct ggml_tensor *, int64_t) {
    fprintf(stderr, "presample: no device back end in this build\n");
    abort();
}
'''

STUB_MPI_H = r'''#pragma once
#define MPI_CHAR 1
#define MPI_INT 2
#define MPI_COMM_WORLD 0
static inline int MPI_Bcast(void *, int, int, int, int) { return 0; }
static inline int MPI_Allgather(const void * s, int n, int, void * r, int, int, int) { for (int i = 0; i < n; ++i) ((int *) r)[i] = ((const int *) s)[i]; return 0; }
'''

CPU_KERNELS = r'''
// ---- oracle build only: plain CPU forms of graph nodes that only the device back end implements -----------------------
static void oracle_get_slice(struct ggml_compute_params * params, struct ggml_tensor * dst) {
    if (params->ith != 0) return;
    const struct ggml_tensor * a = dst->src[0];
    const int64_t * op = (const int64_t *) dst->op_params;
    const int64_t fr = op[0]; const int axis = (int) op[2];
    const size_t ts = ggml_type_size(a->type);
    GGML_ASSERT(ggml_blck_size(a->type) == 1);
    for (int64_t i3 = 0; i3 < dst->ne[3]; ++i3) for (int64_t i2 = 0; i2 < dst->ne[2]; ++i2)
    for (int64_t i1 = 0; i1 < dst->ne[1]; ++i1) for (int64_t i0 = 0; i0 < dst->ne[0]; ++i0) {
        int64_t j[4] = { i0, i1, i2, i3 };
        j[axis] += fr;
        memcpy((char *) dst->data + i0 * dst->nb[0] + i1 * dst->nb[1] + i2 * dst->nb[2] + i3 * dst->nb[3],
               (const char *) a->data + j[0] * a->nb[0] + j[1] * a->nb[1] + j[2] * a->nb[2] + j[3] * a->nb[3], ts);
    }
}
static void oracle_rms_norm_fused(struct ggml_compute_params * params, struct ggml_tensor * dst) {
    if (params->ith != 0) return;
    const struct ggml_tensor * a = dst->src[0];
    const struct ggml_tensor * w = dst->src[1];
    float eps; memcpy(&eps, dst->op_params, sizeof(float));
    GGML_ASSERT(a->type == GGML_TYPE_F32 && w->type == GGML_TYPE_F32);
    const int64_t n = a->ne[0];
    for (int64_t i3 = 0; i3 < a->ne[3]; ++i3) for (int64_t i2 = 0; i2 < a->ne[2]; ++i2) for (int64_t i1 = 0; i1 < a->ne[1]; ++i1) {
        const float * x = (const float *) ((const char *) a->data + i1 * a->nb[1] + i2 * a->nb[2] + i3 * a->nb[3]);
        float * y = (float *) ((char *) dst->data + i1 * dst->nb[1] + i2 * dst->nb[2] + i3 * dst->nb[3]);
        double ss = 0.0;
        for (int64_t i = 0; i < n; ++i) ss += (double) x[i] * x[i];
        const float sc = 1.0f / sqrtf((float) (ss / n) + eps);
        for (int64_t i = 0; i < n; ++i) y[i] = x[i] * sc * ((const float *) w->data)[i];
    }
}
static void oracle_mul_f16(struct ggml_compute_params * params, struct ggml_tensor * dst) {
    if (params->ith != 0) return;
    const struct ggml_tensor * a = dst->src[0];
    const struct ggml_tensor * w = dst->src[1];
    GGML_ASSERT(a->type == GGML_TYPE_F32 && dst->type == GGML_TYPE_F32 && ggml_is_contiguous(w));
    for (int64_t i3 = 0; i3 < a->ne[3]; ++i3) for (int64_t i2 = 0; i2 < a->ne[2]; ++i2) for (int64_t i1 = 0; i1 < a->ne[1]; ++i1) {
        const float * x = (const float *) ((const char *) a->data + i1 * a->nb[1] + i2 * a->nb[2] + i3 * a->nb[3]);
        float * y = (float *) ((char *) dst->data + i1 * dst->nb[1] + i2 * dst->nb[2] + i3 * dst->nb[3]);
        const ggml_fp16_t * wr = (const ggml_fp16_t *) ((const char *) w->data + (i1 % w->ne[1]) * w->nb[1] + (i2 % w->ne[2]) * w->nb[2] + (i3 % w->ne[3]) * w->nb[3]);
        for (int64_t i = 0; i < a->ne[0]; ++i) y[i] = x[i] * GGML_FP16_TO_FP32(wr[i % w->ne[0]]);
    }
}
'''

DRIVER_CPP = r'''// usage: ref_logits model.gguf tokens.txt out.bin -- logits of every position, raw float32 [n_tokens][n_vocab]
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "llama.h"
#include "llama-context.h"
int main(int argc, char ** argv) {
    if (argc < 4) return 2;
    std::vector<llama_token> toks;
    { FILE * f = fopen(argv[2], "r"); if (!f) return 2; int t; while (fscanf(f, "%d", &t) == 1) toks.push_back(t); fclose(f); }
    llama_backend_init();
    llama_model_params mp = llama_model_default_params();
    mp.n_gpu_layers = 0; mp.use_mmap = true; mp.enable_mla = false; mp.enable_mpi = false; mp.enable_tensor_parallel = false;
    mp.enable_expert_parallel = false; mp.enable_data_parallel = false; mp.enable_fused_moe = false; mp.enable_cann_flash_attention = false;
    mp.num_parallel = 1; mp.tp_id = 0;
    llama_model * model = llama_model_load_from_file(argv[1], mp);
    if (!model) { fprintf(stderr, "load failed\n"); return 1; }
    llama_context_params cp = llama_context_default_params();
    cp.n_ctx = 256; cp.n_batch = 64; cp.n_ubatch = 64; cp.n_seq_max = 1; cp.n_threads = 8; cp.n_threads_batch = 8;
    cp.flash_attn = false; cp.enable_ge = false; cp.presample_count = -1; cp.no_perf = true;
    llama_context * ctx = llama_init_from_model(model, cp);
    if (!ctx) { fprintf(stderr, "context failed\n"); return 1; }
    const int n = (int) toks.size();
    const int V = llama_vocab_n_tokens(llama_model_get_vocab(model));
    llama_batch b = llama_batch_init(n, 0, 1);
    b.n_tokens = n;
    for (int i = 0; i < n; ++i) { b.token[i] = toks[i]; b.pos[i] = i; b.n_seq_id[i] = 1; b.seq_id[i][0] = 0; b.logits[i] = 1; }
    const int rc = llama_decode(ctx, b);
    if (rc != 0) { fprintf(stderr, "decode rc=%d\n", rc); return 1; }
    FILE * o = fopen(argv[3], "wb");
    for (int i = 0; i < n; ++i) {
        llama_logits l = llama_get_logits_ith(ctx, i);
        if (l.values == nullptr || l.len != V) { fprintf(stderr, "logits %d: len %lld\n", i, (long long) l.len); return 1; }
        fwrite(l.values, sizeof(float), V, o);
    }
    fclose(o);
    return 0;
}
'''


REWRITE_CPP = r'''// usage: ref_rewrite in.gguf out.gguf -- read a file with the reference's GGUF reader, write it back with its writer
#include <cstdio>
#include "ggml.h"
#include "gguf.h"
int main(int argc, char ** argv) {
    if (argc < 3) return 2;
    struct ggml_context * data = nullptr;
    struct gguf_init_params p = { /*no_alloc=*/false, /*ctx=*/&data };
    struct gguf_context * g = gguf_init_from_file(argv[1], p);
    if (!g) { fprintf(stderr, "read failed\n"); return 1; }
    // a fresh writer context: the keys copied over, the tensors added in file order from the loaded data (the tensor records of
    // a context that was READ carry an uninitialised buffer field, which the writer would follow)
    struct gguf_context * w = gguf_init_empty();
    gguf_set_kv(w, g);
    for (int64_t i = 0; i < gguf_get_n_tensors(g); ++i) {
        struct ggml_tensor * t = ggml_get_tensor(data, gguf_get_tensor_name(g, i));
        if (!t) { fprintf(stderr, "tensor %lld missing\n", (long long) i); return 1; }
        gguf_add_tensor(w, t);
    }
    if (!gguf_write_to_file(w, argv[2], false)) { fprintf(stderr, "write failed\n"); return 1; }
    gguf_free(w);
    gguf_free(g);
    ggml_free(data);
    return 0;
}
'''


def build_rewriter(workdir: str) -> str:
    """``ref_rewrite``: the reference's GGUF reader + writer as a filter (after ``build``, which made the objects)."""
    open(os.path.join(workdir, "ref_rewrite.cpp"), "w").write(REWRITE_CPP)
    objs = [os.path.relpath(o, workdir) for o in sorted(glob.glob(os.path.join(workdir, "obj", "ggml_*.o")))]
    subprocess.run(["g++", "-std=c++17", "-O1", "-w", "-Iggml/include", "-Iggml/src", "ref_rewrite.cpp", *objs, "-o", "ref_rewrite",
                    "-lpthread", "-ldl", "-lm", "-fopenmp"], cwd=workdir, check=True)
    return os.path.join(workdir, "ref_rewrite")


def _patch_cpu_dispatch(path: str) -> None:
    """Adds the three plain kernels to the COPIED ggml-cpu.c and routes their ops to them."""
    s = open(path).read()
    if "oracle_get_slice" in s:
        return
    anchor = "static void ggml_compute_forward(struct ggml_compute_params * params, struct ggml_tensor * tensor) {"
    fwd_old = "        case GGML_OP_MUL:\n            {\n                ggml_compute_forward_mul(params, tensor);\n            }\n            break;"
    fwd_new = ("        case GGML_OP_GET_SLICE:\n            oracle_get_slice(params, tensor);\n            break;\n"
               "        case GGML_OP_RMS_NORM_FUSED:\n            oracle_rms_norm_fused(params, tensor);\n            break;\n"
               "        case GGML_OP_MUL:\n            {\n"
               "                if (tensor->src[1]->type == GGML_TYPE_F16 && tensor->src[0]->type == GGML_TYPE_F32) oracle_mul_f16(params, tensor);\n"
               "                else ggml_compute_forward_mul(params, tensor);\n            }\n            break;")
    tasks_old = "        case GGML_OP_NONE:\n            {\n                n_tasks = 1;\n            }\n            break;"
    tasks_new = "        case GGML_OP_GET_SLICE:\n        case GGML_OP_RMS_NORM_FUSED:\n" + tasks_old
    for needle in (anchor, fwd_old, tasks_old):
        if needle not in s:
            raise RuntimeError("the reference's ggml-cpu.c does not look as expected: " + needle.splitlines()[0].strip())
    s = s.replace(anchor, CPU_KERNELS + anchor, 1).replace(fwd_old, fwd_new, 1).replace(tasks_old, tasks_new, 1)
    open(path, "w").write(s)


def build(reference: str, workdir: str, jobs: int = 8) -> str:
    """Copies ggml/, src/ and include/ of the checkout into ``workdir``, adds the stand-ins and builds ``ref_logits``."""
    os.makedirs(workdir, exist_ok=True)
    for d in ("ggml", "src", "include"):
        dst = os.path.join(workdir, d)
        if not os.path.isdir(dst):
            shutil.copytree(os.path.join(reference, d), dst)
    stub = os.path.join(workdir, "stub")
    os.makedirs(stub, exist_ok=True)
    for name, text in (("ggml-cann.h", STUB_CANN_H), ("stubs.cpp", STUB_CPP), ("mpi_stub.h", STUB_MPI_H)):
        open(os.path.join(stub, name), "w").write(text)
    open(os.path.join(workdir, "ref_logits.cpp"), "w").write(DRIVER_CPP)
    _patch_cpu_dispatch(os.path.join(workdir, "ggml", "src", "ggml-cpu", "ggml-cpu.c"))
    obj = os.path.join(workdir, "obj")
    os.makedirs(obj, exist_ok=True)
    inc = ["-Iggml/include", "-Iggml/src", "-Iggml/src/ggml-cpu", "-Iinclude", "-Isrc", "-Istub"]
    defs = ["-DGGML_USE_CPU", "-D_GNU_SOURCE", '-DGGML_VERSION="ref"', '-DGGML_COMMIT="ref"']
    flags = ["-O2", "-fPIC", "-march=native", "-w"]
    c_srcs = ["ggml/src/ggml.c", "ggml/src/ggml-alloc.c", "ggml/src/ggml-quants.c", "ggml/src/ggml-cpu/ggml-cpu.c",
              "ggml/src/ggml-cpu/ggml-cpu-quants.c"]
    cpp_srcs = ["ggml/src/ggml-backend.cpp", "ggml/src/ggml-backend-reg.cpp", "ggml/src/ggml-threading.cpp", "ggml/src/gguf.cpp",
                "ggml/src/ggml-cpu/ggml-cpu.cpp", "ggml/src/ggml-cpu/ggml-cpu-aarch64.cpp", "ggml/src/ggml-cpu/ggml-cpu-traits.cpp",
                "ggml/src/ggml-cpu/ggml-cpu-hbm.cpp", "ggml/src/ggml-cpu/amx/amx.cpp", "ggml/src/ggml-cpu/amx/mmq.cpp", "stub/stubs.cpp"]
    cpp_srcs += sorted(os.path.relpath(p, workdir) for p in glob.glob(os.path.join(workdir, "src", "*.cpp")))
    cmds: List[List[str]] = []
    objs = []
    for src in c_srcs + cpp_srcs:
        o = os.path.join("obj", src.replace("/", "_") + ".o")
        objs.append(o)
        if os.path.exists(os.path.join(workdir, o)) and os.path.getmtime(os.path.join(workdir, o)) >= os.path.getmtime(os.path.join(workdir, src)):
            continue
        if src.endswith(".c"):
            cmds.append(["gcc", "-std=c11", *flags, *defs, *inc, "-c", src, "-o", o])
        else:     # <unordered_map> is used without its include in one file; the MPI names outside the guard in two
            cmds.append(["g++", "-std=c++17", *flags, *defs, *inc, "-include", "unordered_map", "-include", "stub/mpi_stub.h", "-c", src, "-o", o])
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        list(pool.map(lambda cmd: subprocess.run(cmd, cwd=workdir, stderr=subprocess.DEVNULL), cmds))
    missing = [o for o in objs if not os.path.exists(os.path.join(workdir, o))]
    if missing:
        raise RuntimeError(f"the stubbed build failed for {missing[:3]} ...")
    exe = os.path.join(workdir, "ref_logits")
    subprocess.run(["g++", "-std=c++17", "-O1", "-w", *inc, "-include", "unordered_map", "-DGGML_USE_CPU", "ref_logits.cpp", *objs, "-o",
                    "ref_logits", "-lpthread", "-ldl", "-lm", "-fopenmp"], cwd=workdir, check=True)
    return exe


def reference_logits(exe: str, gguf_path: str, tokens: List[int], workdir: str) -> np.ndarray:
    tok_file, out_file = os.path.join(workdir, "tokens.txt"), os.path.join(workdir, "logits.bin")
    open(tok_file, "w").write(" ".join(str(int(t)) for t in tokens))
    r = subprocess.run([exe, gguf_path, tok_file, out_file], stdout=subprocess.DEVNULL, stderr=subprocess.PIPE)
    if r.returncode != 0:
        raise RuntimeError("the reference's CPU path failed: " + r.stderr.decode("utf-8", errors="replace")[-400:])
    return np.fromfile(out_file, dtype=np.float32).reshape(len(tokens), -1)


def case(name: str):
    """The two structures the reference distinguishes (by layer count, src/llama-model.cpp): 27 layers without a low-rank query
    projection (V2-Lite) and anything else with one (V2).  Small dimensions; group-limited routing off (see the module text)."""
    from ..models.hparams import preset
    if name == "v2":
        return preset("tiny-v2").replace(n_group=1, topk_group=1)
    if name == "lite":
        return preset("tiny").replace(n_layer=27, n_group=1, topk_group=1)
    raise ValueError(name)


def case_tokens(hp, n: int = 32) -> List[int]:
    import torch
    return torch.randint(2, hp.n_vocab, (n,), generator=torch.Generator().manual_seed(3)).tolist()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--reference", required=True, help="checkout of the reference (read only)")
    ap.add_argument("--workdir", required=True, help="scratch directory for the copied sources, objects and files")
    ap.add_argument("--cases", default="v2,lite")
    ap.add_argument("--save", default=None, help="write tokens and reference logits of every case to this .npz")
    args = ap.parse_args(argv)
    import torch
    from ..models.oracle import OracleModel
    from ..models.weights import random_weights, write_random_gguf
    exe = build(args.reference, args.workdir)
    saved, rc = {}, 0
    for name in args.cases.split(","):
        hp = case(name)
        path = os.path.join(args.workdir, f"case_{name}.gguf")
        write_random_gguf(path, hp, seed=0, std=0.05)
        toks = case_tokens(hp)
        ref = reference_logits(exe, path, toks, args.workdir)
        mine = OracleModel(hp, random_weights(hp, seed=0, std=0.05)).forward(torch.tensor(toks)).numpy()
        err = float(np.abs(ref - mine).max())
        mag = float(np.abs(mine).max())
        agree = float((ref.argmax(-1) == mine.argmax(-1)).mean())
        print(json.dumps({"case": name, "layers": hp.n_layer, "positions": len(toks), "max_abs_diff": round(err, 5), "largest_logit": round(mag, 4),
                          "argmax_agreement": agree}))
        rc |= int(err > 1e-2 * max(mag, 1.0) or agree < 1.0)
        # the other direction: the reference's GGUF writer re-emits the file; this package's reader must see the same tensors
        back = os.path.join(args.workdir, f"case_{name}_rewritten.gguf")
        subprocess.run([build_rewriter(args.workdir), path, back], check=True, stderr=subprocess.DEVNULL)
        import filecmp
        print(json.dumps({"case": name, "rewritten_by_the_reference_writer": "byte-identical" if filecmp.cmp(path, back, shallow=False) else "differs"}))
        saved[f"{name}_tokens"] = np.asarray(toks, dtype=np.int32)
        saved[f"{name}_logits"] = ref
    if args.save:
        np.savez_compressed(args.save, **saved)
    return rc


if __name__ == "__main__":
    sys.exit(main())
