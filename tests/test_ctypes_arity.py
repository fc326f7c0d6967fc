"""Arity of the ctypes bindings of the CUDA library, checked without loading it: for every ``jib_*`` entry point the number
of parameters in the C prototype (``csrc/kernels/*.h``, ``*.cu``), the number of declared ctypes argument types and the
number of arguments at every call site in the Python wrappers must agree.  (A mismatch would otherwise only show as a
TypeError on a machine with a GPU.)"""
import ast
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "jittorinfer_b200")


def _c_prototypes():
    protos = {}
    files = glob.glob(os.path.join(PKG, "csrc", "kernels", "*.h")) + glob.glob(os.path.join(PKG, "csrc", "kernels", "*.cu")) + \
        glob.glob(os.path.join(PKG, "csrc", "kernels", "*.cuh"))
    for f in files:
        src = re.sub(r"//[^\n]*", "", open(f).read())
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        for m in re.finditer(r"\b(jib_[a-z0-9_]+)\s*\(([^;{)]*)\)\s*[;{]", src):
            name, params = m.group(1), m.group(2).strip()
            if not re.search(r"\b(int|void|float|const|size_t|unsigned|long|JibArCtx|JibEpCtx|jib_gemm_desc)\b", params) and params != "":
                continue                                  # a call, not a prototype
            n = 0 if params in ("", "void") else params.count(",") + 1
            protos.setdefault(name, set()).add(n)
    return protos


def _python_bindings():
    declared, calls = {}, {}
    for f in glob.glob(os.path.join(PKG, "**", "*.py"), recursive=True):
        tree = ast.parse(open(f).read())
        for node in ast.walk(tree):
            if isinstance(node, ast.Call):
                fn = node.func
                # sig("jib_x", res?, *argtypes): native.py passes (name, *argtypes) with int result implied
                if isinstance(fn, ast.Name) and fn.id == "sig" and node.args and isinstance(node.args[0], ast.Constant) \
                        and str(node.args[0].value).startswith("jib_") and f.endswith(os.path.join("ops", "native.py")):
                    declared[node.args[0].value] = len(node.args) - 1
                if isinstance(fn, ast.Attribute) and fn.attr.startswith("jib_") and not any(isinstance(a, ast.Starred) for a in node.args):
                    calls.setdefault(fn.attr, set()).add((len(node.args), os.path.relpath(f, ROOT), node.lineno))
            # ("jib_name", [argtypes...]) tuples in comm.py / ep.py
            if isinstance(node, ast.Tuple) and len(node.elts) == 2 and isinstance(node.elts[0], ast.Constant) \
                    and str(node.elts[0].value).startswith("jib_") and isinstance(node.elts[1], ast.List):
                declared[node.elts[0].value] = len(node.elts[1].elts)
    return declared, calls


def test_ctypes_declarations_and_call_sites_match_the_c_prototypes():
    protos = _c_prototypes()
    declared, calls = _python_bindings()
    assert len(declared) > 25 and "jib_moe_route_fused" in declared and "jib_gemm_bf16" in declared
    problems = []
    for name, n_decl in declared.items():
        if name not in protos:
            problems.append(f"{name}: declared in Python, no C prototype found")
        elif n_decl not in protos[name]:
            problems.append(f"{name}: {n_decl} ctypes argument types, C prototype has {sorted(protos[name])}")
    for name, sites in calls.items():
        want = protos.get(name)
        for n, f, line in sites:
            if want is not None and n not in want:
                problems.append(f"{f}:{line}: {name} called with {n} arguments, C prototype has {sorted(want)}")
    assert not problems, "\n".join(problems)


def test_descriptor_field_names_exist():
    """ctypes structures accept assignments to names that are not fields (they become plain attributes and never reach the
    library): every ``d.<name> = ...`` on a GEMM descriptor and every ``ctx.<name>`` write on the communicator / dispatcher
    contexts must name a declared field."""
    from jittorinfer_b200.ops.native import GemmDesc
    from jittorinfer_b200.parallel.comm import ArCtx
    from jittorinfer_b200.parallel.ep import EpCtx
    checks = [(os.path.join(PKG, "ops", "native.py"), "d", {n for n, _ in GemmDesc._fields_}),
              (os.path.join(PKG, "parallel", "comm.py"), "ctx", {n for n, _ in ArCtx._fields_}),
              (os.path.join(PKG, "parallel", "ep.py"), "ctx", {n for n, _ in EpCtx._fields_})]
    bad = []
    for path, var, fields in checks:
        tree = ast.parse(open(path).read())
        n_seen = 0
        for node in ast.walk(tree):
            targets = []
            if isinstance(node, ast.Assign):
                for t in node.targets:
                    targets += list(t.elts) if isinstance(t, ast.Tuple) else [t]
            elif isinstance(node, ast.AugAssign):
                targets = [node.target]
            for t in targets:
                base = t.value if isinstance(t, ast.Attribute) else (t.value.value if isinstance(t, ast.Subscript) and isinstance(t.value, ast.Attribute) else None)
                attr = t.attr if isinstance(t, ast.Attribute) else (t.value.attr if isinstance(t, ast.Subscript) and isinstance(t.value, ast.Attribute) else None)
                if attr is None:
                    continue
                owner = base
                name = owner.id if isinstance(owner, ast.Name) else (owner.attr if isinstance(owner, ast.Attribute) else None)
                if name == var:
                    n_seen += 1
                    if attr not in fields:
                        bad.append(f"{os.path.relpath(path, ROOT)}:{t.lineno}: {var}.{attr} is not a field")
        assert n_seen > 5, path
    assert not bad, "\n".join(bad)
