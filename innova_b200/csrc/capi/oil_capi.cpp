// liboil_capi.so: the reference's C entry points (include/oil/production.h:134-141, src/production_core.cpp:37-224)
// over this package's generator. See oil_capi.h for the contract.
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <dlfcn.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "oil_capi.h"

struct OilModel {
  long handle;
};

namespace {
thread_local std::string g_error;
std::once_flag g_once;
bool g_started_here = false;
PyObject* g_module = nullptr;   // innova_b200.serving.capi, owned for the life of the process

std::string package_root() {
  if (const char* r = std::getenv("INNOVA_B200_ROOT")) return r;
  Dl_info info;
  if (dladdr(reinterpret_cast<void*>(&package_root), &info) && info.dli_fname) {
    std::string p = info.dli_fname;              // <root>/innova_b200/lib/liboil_capi.so
    for (int up = 0; up < 3; ++up) {
      const size_t k = p.find_last_of('/');
      if (k == std::string::npos) return ".";
      p.erase(k);
    }
    return p.empty() ? "/" : p;
  }
  return ".";
}

std::string find_python() {
  if (const char* e = std::getenv("INNOVA_B200_PYTHON")) return e;
  const char* path = std::getenv("PATH");
  std::string dirs = path ? path : "/usr/bin";
  size_t a = 0;
  while (a <= dirs.size()) {
    size_t b = dirs.find(':', a);
    if (b == std::string::npos) b = dirs.size();
    const std::string cand = dirs.substr(a, b - a) + "/python3";
    if (access(cand.c_str(), X_OK) == 0) return cand;
    a = b + 1;
  }
  return "python3";
}

void start_python() {
  if (!Py_IsInitialized()) {
    PyConfig cfg;
    PyConfig_InitPythonConfig(&cfg);
    const std::string exe = find_python();
    PyConfig_SetBytesString(&cfg, &cfg.executable, exe.c_str());   // a venv's python brings its own site-packages
    cfg.install_signal_handlers = 0;
    PyStatus st = Py_InitializeFromConfig(&cfg);
    PyConfig_Clear(&cfg);
    if (PyStatus_Exception(st)) return;
    g_started_here = true;
  }
  PyGILState_STATE gs = g_started_here ? PyGILState_UNLOCKED : PyGILState_Ensure();
  {
    PyObject* sys_path = PySys_GetObject("path");   // borrowed
    PyObject* root = PyUnicode_FromString(package_root().c_str());
    if (sys_path && root) PyList_Insert(sys_path, 0, root);
    Py_XDECREF(root);
    g_module = PyImport_ImportModule("innova_b200.serving.capi");
    if (!g_module) PyErr_Clear();
  }
  if (g_started_here) PyEval_SaveThread();   // leave the interpreter unlocked: every call takes the lock itself
  else PyGILState_Release(gs);
}

void set_error_from_python(const char* what) {
  PyObject *t = nullptr, *v = nullptr, *tb = nullptr;
  PyErr_Fetch(&t, &v, &tb);
  g_error = what;
  if (v) {
    PyObject* s = PyObject_Str(v);
    if (s) {
      const char* c = PyUnicode_AsUTF8(s);
      if (c) g_error += std::string(": ") + c;
      Py_DECREF(s);
    }
  }
  Py_XDECREF(t);
  Py_XDECREF(v);
  Py_XDECREF(tb);
  PyErr_Clear();
}

// Calls capi.<name>(*args); returns a new reference or nullptr with g_error set. GIL must be held.
PyObject* call(const char* name, PyObject* args) {
  if (!g_module) {
    g_error = "the Python package innova_b200 could not be imported (set INNOVA_B200_ROOT / INNOVA_B200_PYTHON)";
    Py_XDECREF(args);
    return nullptr;
  }
  PyObject* fn = PyObject_GetAttrString(g_module, name);
  PyObject* out = fn ? PyObject_CallObject(fn, args) : nullptr;
  Py_XDECREF(fn);
  Py_XDECREF(args);
  if (!out) set_error_from_python(name);
  return out;
}

std::string python_last_error() {   // GIL held
  PyObject* r = call("oil_last_error", nullptr);
  std::string s;
  if (r) {
    const char* c = PyUnicode_AsUTF8(r);
    if (c) s = c;
    Py_DECREF(r);
  }
  return s;
}
}  // namespace

extern "C" {

const char* oil_last_error(void) { return g_error.c_str(); }

OilModel* oil_model_load(const char* path) {
  g_error.clear();
  if (path == nullptr) {
    g_error = "oil_model_load: null path";
    return nullptr;
  }
  std::call_once(g_once, start_python);
  if (!Py_IsInitialized()) {
    g_error = "oil_model_load: the Python interpreter could not be started";
    return nullptr;
  }
  PyGILState_STATE gs = PyGILState_Ensure();
  OilModel* m = nullptr;
  PyObject* r = call("oil_model_load", Py_BuildValue("(s)", path));
  if (r) {
    const long h = PyLong_AsLong(r);
    Py_DECREF(r);
    if (h > 0) {
      m = static_cast<OilModel*>(std::malloc(sizeof(OilModel)));
      if (m) m->handle = h;
      else g_error = "oil_model_load: out of memory";
    } else {
      g_error = python_last_error();
      if (g_error.empty()) g_error = "oil_model_load: failed";
    }
  }
  PyGILState_Release(gs);
  return m;
}

void oil_model_free(OilModel* model) {
  if (model == nullptr) return;
  if (Py_IsInitialized()) {
    PyGILState_STATE gs = PyGILState_Ensure();
    PyObject* r = call("oil_model_free", Py_BuildValue("(l)", model->handle));
    Py_XDECREF(r);
    PyGILState_Release(gs);
  }
  std::free(model);
}

char* oil_generate(OilModel* model, const char* prompt, int max_tokens) {
  g_error.clear();
  if (model == nullptr || prompt == nullptr) {
    g_error = "oil_generate: null model or prompt";
    return nullptr;
  }
  if (!Py_IsInitialized()) {
    g_error = "oil_generate: no interpreter";
    return nullptr;
  }
  PyGILState_STATE gs = PyGILState_Ensure();
  char* out = nullptr;
  PyObject* r = call("oil_generate", Py_BuildValue("(lsi)", model->handle, prompt, max_tokens));
  if (r) {
    if (r == Py_None) {
      g_error = python_last_error();
      if (g_error.empty()) g_error = "oil_generate: failed";
    } else {
      Py_ssize_t n = 0;
      const char* c = PyUnicode_AsUTF8AndSize(r, &n);
      if (c) {
        out = static_cast<char*>(std::malloc((size_t)n + 1));
        if (out) {
          std::memcpy(out, c, (size_t)n);
          out[n] = 0;
        } else {
          g_error = "oil_generate: out of memory";
        }
      } else {
        set_error_from_python("oil_generate");
      }
    }
    Py_DECREF(r);
  }
  PyGILState_Release(gs);
  return out;
}

void oil_free_string(char* s) { std::free(s); }

}  // extern "C"
