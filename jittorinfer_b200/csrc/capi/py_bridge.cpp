// Embedded-CPython bridge of libllama.so: the C API's model forward runs in the Python package.
//
// The reference links its C API straight onto the ggml graph executor (src/llama-execute-decode.cpp:156-344); here the
// model graph is a PyTorch module that launches the sm_100a kernels, so llama_decode hands one packed step descriptor
// to Python and gets the logits back in a caller-owned buffer.  Everything else of the C API (GGUF metadata, tokenizer,
// samplers, KV bookkeeping) is native and never enters Python.
#include "capi_internal.h"

#define PY_SSIZE_T_CLEAN
#include <Python.h>

#include <cstdarg>
#include <cstdlib>
#include <dlfcn.h>
#include <mutex>
#include <unistd.h>

namespace jib {

namespace {

std::mutex g_mu;
bool g_ready = false, g_owns_interpreter = false;
PyObject * g_module = nullptr;

std::string fetch_error() {
    PyObject *type = nullptr, *value = nullptr, *tb = nullptr;
    PyErr_Fetch(&type, &value, &tb);
    PyErr_NormalizeException(&type, &value, &tb);
    std::string msg = "python error";
    if (value != nullptr) {
        PyObject * s = PyObject_Str(value);
        if (s != nullptr) {
            const char * c = PyUnicode_AsUTF8(s);
            if (c != nullptr) msg = c;
            Py_DECREF(s);
        }
    }
    if (type != nullptr) {
        PyObject * n = PyObject_GetAttrString(type, "__name__");
        if (n != nullptr) {
            const char * c = PyUnicode_AsUTF8(n);
            if (c != nullptr) msg = std::string(c) + ": " + msg;
            Py_DECREF(n);
        }
    }
    Py_XDECREF(type);
    Py_XDECREF(value);
    Py_XDECREF(tb);
    return msg;
}

// directory that contains the package = two levels above this shared object (<root>/jittorinfer_b200/lib/libllama.so)
std::string package_root() {
    Dl_info info;
    if (dladdr((void *) &package_root, &info) == 0 || info.dli_fname == nullptr) return "";
    std::string p = info.dli_fname;
    for (int up = 0; up < 3; ++up) {
        const size_t pos = p.find_last_of('/');
        if (pos == std::string::npos) return "";
        p.erase(pos);
    }
    return p;
}

std::string find_in_path(const char * name) {
    const char * path = getenv("PATH");
    if (path == nullptr) return "";
    std::string all(path);
    size_t start = 0;
    while (start <= all.size()) {
        size_t end = all.find(':', start);
        if (end == std::string::npos) end = all.size();
        const std::string cand = all.substr(start, end - start) + "/" + name;
        if (access(cand.c_str(), X_OK) == 0) return cand;
        start = end + 1;
    }
    return "";
}

}  // namespace

std::string PyBridge::ensure() {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_ready) return "";
    if (!Py_IsInitialized()) {
        // Start an interpreter that resolves site-packages the way `python3` on PATH does (virtual environments are
        // found through the executable's pyvenv.cfg).  JITTORINFER_PYTHON overrides the executable.
        PyConfig cfg;
        PyConfig_InitPythonConfig(&cfg);
        const char * exe_env = getenv("JITTORINFER_PYTHON");
        std::string exe = exe_env != nullptr ? exe_env : find_in_path("python3");
        if (!exe.empty()) {
            PyStatus st = PyConfig_SetBytesString(&cfg, &cfg.executable, exe.c_str());
            if (PyStatus_Exception(st)) { PyConfig_Clear(&cfg); return "cannot set the Python executable"; }
            PyConfig_SetBytesString(&cfg, &cfg.program_name, exe.c_str());
        }
        cfg.install_signal_handlers = 0;
        PyStatus st = Py_InitializeFromConfig(&cfg);
        PyConfig_Clear(&cfg);
        if (PyStatus_Exception(st)) return std::string("Python failed to start: ") + (st.err_msg ? st.err_msg : "?");
        g_owns_interpreter = true;
        PyEval_SaveThread();          // drop the GIL; every call below takes it through PyGILState_Ensure
    }
    PyGILState_STATE gs = PyGILState_Ensure();
    std::string err;
    const std::string root = package_root();
    if (!root.empty()) {
        PyObject * sys_path = PySys_GetObject("path");       // borrowed
        PyObject * r = PyUnicode_FromString(root.c_str());
        if (sys_path != nullptr && r != nullptr && PySequence_Contains(sys_path, r) == 0) PyList_Insert(sys_path, 0, r);
        Py_XDECREF(r);
    }
    g_module = PyImport_ImportModule("jittorinfer_b200.capi_backend");
    if (g_module == nullptr) err = "cannot import jittorinfer_b200.capi_backend: " + fetch_error();
    PyGILState_Release(gs);
    if (err.empty()) g_ready = true;
    return err;
}

bool PyBridge::call(const char * fn, long long * result, std::string * err, const char * fmt, ...) {
    const std::string e = ensure();
    if (!e.empty()) {
        if (err) *err = e;
        return false;
    }
    PyGILState_STATE gs = PyGILState_Ensure();
    bool ok = false;
    va_list ap;
    va_start(ap, fmt);
    PyObject * args = Py_VaBuildValue(fmt, ap);
    va_end(ap);
    PyObject * f = args != nullptr ? PyObject_GetAttrString(g_module, fn) : nullptr;
    PyObject * r = f != nullptr ? PyObject_CallObject(f, args) : nullptr;
    if (r != nullptr) {
        const long long v = r == Py_None ? 0 : PyLong_AsLongLong(r);
        if (!PyErr_Occurred()) {
            if (result) *result = v;
            ok = true;
        }
    }
    if (!ok && err) *err = std::string(fn) + ": " + fetch_error();
    if (!ok) PyErr_Clear();
    Py_XDECREF(r);
    Py_XDECREF(f);
    Py_XDECREF(args);
    PyGILState_Release(gs);
    return ok;
}

void PyBridge::shutdown() {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_ready) return;
    PyGILState_STATE gs = PyGILState_Ensure();
    Py_CLEAR(g_module);
    g_ready = false;
    if (g_owns_interpreter) {
        // Finalising an interpreter that holds CUDA state from a library destructor is fragile; the
        // process is about to exit, so the interpreter is left to the operating system.
        PyGILState_Release(gs);
        return;
    }
    PyGILState_Release(gs);
}

}  // namespace jib
