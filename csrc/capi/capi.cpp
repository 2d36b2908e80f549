// C interface over the Python engine (see onnx_genai_b200.h).  The reference implements the same
// surface in Rust over its engine crate (crates/onnx-genai-capi/src/lib.rs); here the engine lives in
// Python, so this file is a CPython embedding: it attaches to a running interpreter or starts one,
// and forwards every call to onnx_genai_b200.capi_bridge under the interpreter lock.
#include <Python.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "onnx_genai_b200.h"

#ifndef OGB_DEFAULT_PYTHON
#define OGB_DEFAULT_PYTHON ""
#endif
#ifndef OGB_DEFAULT_ROOT
#define OGB_DEFAULT_ROOT ""
#endif

struct OgeEngine {
  PyObject* engine;   // onnx_genai_b200.engine.api.Engine
};

struct OgeSampler {
  OgeSamplerVTable vt;
  std::string name;
};

namespace {

thread_local std::string g_error;
thread_local bool g_has_error = false;
std::once_flag g_init_once;
bool g_init_ok = false;
std::string g_init_error;

void set_error(const std::string& msg) {
  g_error = msg;
  g_has_error = true;
}

void clear_error() { g_has_error = false; }

// Turns the pending Python exception into the thread's error message.
void take_python_error(const char* what) {
  PyObject *type = nullptr, *value = nullptr, *tb = nullptr;
  PyErr_Fetch(&type, &value, &tb);
  PyErr_NormalizeException(&type, &value, &tb);
  std::string msg = what;
  if (value != nullptr) {
    PyObject* s = PyObject_Str(value);
    if (s != nullptr) {
      const char* c = PyUnicode_AsUTF8(s);
      if (c != nullptr) msg += std::string(": ") + c;
      Py_DECREF(s);
    }
  }
  PyErr_Clear();
  Py_XDECREF(type);
  Py_XDECREF(value);
  Py_XDECREF(tb);
  set_error(msg);
}

void start_interpreter() {
  if (Py_IsInitialized()) {   // loaded into a Python process: use its interpreter
    g_init_ok = true;
    return;
  }
  PyConfig config;
  PyConfig_InitPythonConfig(&config);
  const char* exe = std::getenv("ONNX_GENAI_B200_PYTHON");
  if (exe == nullptr || *exe == '\0') exe = OGB_DEFAULT_PYTHON;
  PyStatus st;
  if (*exe != '\0') {
    // naming the interpreter of a virtual environment makes its site-packages importable
    st = PyConfig_SetBytesString(&config, &config.program_name, exe);
    if (PyStatus_Exception(st)) { g_init_error = "cannot set the interpreter path"; PyConfig_Clear(&config); return; }
    st = PyConfig_SetBytesString(&config, &config.executable, exe);
    if (PyStatus_Exception(st)) { g_init_error = "cannot set the interpreter path"; PyConfig_Clear(&config); return; }
  }
  st = Py_InitializeFromConfig(&config);
  PyConfig_Clear(&config);
  if (PyStatus_Exception(st)) {
    g_init_error = std::string("Python could not start: ") + (st.err_msg ? st.err_msg : "unknown error");
    return;
  }
  const char* root = std::getenv("ONNX_GENAI_B200_ROOT");
  if (root == nullptr || *root == '\0') root = OGB_DEFAULT_ROOT;
  if (*root != '\0') {
    PyObject* path = PySys_GetObject("path");   // borrowed
    PyObject* entry = PyUnicode_FromString(root);
    if (path != nullptr && entry != nullptr) PyList_Insert(path, 0, entry);
    Py_XDECREF(entry);
  }
  g_init_ok = true;
  PyEval_SaveThread();   // release the lock; every call re-acquires it with PyGILState_Ensure
}

bool ready() {
  std::call_once(g_init_once, start_interpreter);
  if (!g_init_ok) set_error(g_init_error.empty() ? "Python interpreter unavailable" : g_init_error);
  return g_init_ok;
}

struct Gil {
  PyGILState_STATE state;
  Gil() : state(PyGILState_Ensure()) {}
  ~Gil() { PyGILState_Release(state); }
};

PyObject* bridge() {   // new reference or nullptr (error set)
  PyObject* mod = PyImport_ImportModule("onnx_genai_b200.capi_bridge");
  if (mod == nullptr) take_python_error("cannot import onnx_genai_b200.capi_bridge (set ONNX_GENAI_B200_ROOT and ONNX_GENAI_B200_PYTHON)");
  return mod;
}

char* dup_utf8(PyObject* str) {
  Py_ssize_t n = 0;
  const char* c = PyUnicode_AsUTF8AndSize(str, &n);
  if (c == nullptr) return nullptr;
  char* out = static_cast<char*>(std::malloc(static_cast<size_t>(n) + 1));
  if (out == nullptr) return nullptr;
  std::memcpy(out, c, static_cast<size_t>(n));
  out[n] = '\0';
  return out;
}

void destroy_sampler(OgeSampler* s) {
  if (s == nullptr) return;
  if (s->vt.free != nullptr) s->vt.free(s->vt.user_data);
  delete s;
}

char* generate(OgeEngine* engine, const char* prompt, size_t max_new_tokens, OgeSampler* sampler) {
  if (engine == nullptr || engine->engine == nullptr) { set_error("engine is NULL"); return nullptr; }
  if (prompt == nullptr) { set_error("prompt is NULL"); return nullptr; }
  Gil gil;
  PyObject* mod = bridge();
  if (mod == nullptr) return nullptr;
  PyObject* res = PyObject_CallMethod(
      mod, "generate", "OsnKKs", engine->engine, prompt, static_cast<Py_ssize_t>(max_new_tokens),
      static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(sampler ? reinterpret_cast<void*>(sampler->vt.sample) : nullptr)),
      static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(sampler ? sampler->vt.user_data : nullptr)),
      sampler ? sampler->name.c_str() : "");
  Py_DECREF(mod);
  if (res == nullptr) { take_python_error("generation failed"); return nullptr; }
  char* out = dup_utf8(res);
  Py_DECREF(res);
  if (out == nullptr) { PyErr_Clear(); set_error("generation returned text that is not valid UTF-8 or memory ran out"); }
  return out;
}

}  // namespace

extern "C" {

OgeSampler* oge_sampler_new(OgeSamplerVTable vtable) {
  clear_error();
  if (vtable.sample == nullptr) { set_error("OgeSamplerVTable.sample is required"); return nullptr; }
  OgeSampler* s = new (std::nothrow) OgeSampler();
  if (s == nullptr) { set_error("out of memory"); return nullptr; }
  s->vt = vtable;
  s->name = vtable.name != nullptr ? vtable.name : "foreign";
  s->vt.name = nullptr;   // the caller's string may go away; the copy above is what is used
  return s;
}

void oge_sampler_free(OgeSampler* sampler) { destroy_sampler(sampler); }

OgeEngine* oge_engine_load(const char* model_dir) {
  clear_error();
  if (model_dir == nullptr) { set_error("model_dir is NULL"); return nullptr; }
  if (!ready()) return nullptr;
  Gil gil;
  PyObject* mod = bridge();
  if (mod == nullptr) return nullptr;
  PyObject* eng = PyObject_CallMethod(mod, "load", "s", model_dir);
  Py_DECREF(mod);
  if (eng == nullptr) { take_python_error("cannot load the model directory"); return nullptr; }
  OgeEngine* out = new (std::nothrow) OgeEngine();
  if (out == nullptr) { Py_DECREF(eng); set_error("out of memory"); return nullptr; }
  out->engine = eng;
  return out;
}

void oge_engine_free(OgeEngine* engine) {
  if (engine == nullptr) return;
  if (engine->engine != nullptr && Py_IsInitialized()) {
    Gil gil;
    Py_DECREF(engine->engine);
  }
  delete engine;
}

char* oge_engine_generate(OgeEngine* engine, const char* prompt, size_t max_new_tokens) {
  clear_error();
  if (!ready()) return nullptr;
  return generate(engine, prompt, max_new_tokens, nullptr);
}

char* oge_engine_generate_with_sampler(OgeEngine* engine, const char* prompt, size_t max_new_tokens, OgeSampler* sampler) {
  clear_error();
  if (sampler == nullptr) { set_error("sampler is NULL"); return nullptr; }
  char* out = ready() ? generate(engine, prompt, max_new_tokens, sampler) : nullptr;
  destroy_sampler(sampler);   // consumed on success and on failure
  return out;
}

void oge_string_free(char* text) { std::free(text); }

const char* oge_last_error(void) { return g_has_error ? g_error.c_str() : nullptr; }

}  // extern "C"
